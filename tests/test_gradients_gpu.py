"""Backward pass of the dense FFN on CudaMeshImpl against the oracle backend:
the gradient graph built by mtf.gradients lowers through the same kernels as
the forward pass (einsums with permuted roles, ReLU mask, allreduces over the
split dims), so the same graph on the same mesh must give the same numbers."""

import numpy as np
import pytest

from mesh_b200 import mtf
from helpers import rel_err, rng

pytestmark = pytest.mark.gpu


def _ffn_grads(impl, dtype, b=8, l=32, d=128, f=512):
  r = rng(41)
  g = mtf.Graph()
  mesh = mtf.Mesh(g, "m")
  x = r.standard_normal((b, l, d)).astype(np.float32)
  wi = (r.standard_normal((d, f)) / np.sqrt(d)).astype(np.float32)
  wo = (r.standard_normal((f, d)) / np.sqrt(f)).astype(np.float32)
  dy = r.standard_normal((b, l, d)).astype(np.float32)
  X = mtf.import_tf_tensor(mesh, x, "batch:%d,length:%d,d_model:%d" % (b, l, d), dtype=dtype)
  WI = mtf.import_tf_tensor(mesh, wi, "d_model:%d,d_ff:%d" % (d, f), dtype=dtype)
  WO = mtf.import_tf_tensor(mesh, wo, "d_ff:%d,d_model:%d" % (f, d), dtype=dtype)
  DY = mtf.import_tf_tensor(mesh, dy, "batch:%d,length:%d,d_model:%d" % (b, l, d), dtype=dtype)
  y = mtf.layers.dense_relu_dense(X, mtf.Dimension("d_ff", f), wi=WI, wo=WO)
  grads = mtf.gradients([y], [X, WI, WO], grad_ys=[DY])
  low = mtf.Lowering(g, {mesh: impl})
  return [low.export_to_tf_tensor(t) for t in [y] + grads], low


@pytest.mark.parametrize("mesh_shape,layout", [
    ("", ""), ("rows:2,cols:2", "batch:rows;d_ff:cols"), ("all:4", "d_model:all")])
@pytest.mark.parametrize("dtype,tol", [(mtf.float32, 1e-4), (mtf.bfloat16, 2e-2)])
def test_ffn_backward(cuda_device, mesh_shape, layout, dtype, tol):
  from mesh_b200.cuda_mesh_impl import CudaMeshImpl
  from oracle.numpy_mesh_impl import NumpyMeshImpl
  n = mtf.convert_to_shape(mesh_shape).size if mesh_shape else 1
  got, low = _ffn_grads(CudaMeshImpl(mesh_shape or "all:1", layout, [0] * n), dtype)
  ref, low_ref = _ffn_grads(NumpyMeshImpl(mesh_shape or "all:1", layout), dtype)
  # With d_model split, the pre-activation is an allreduce of bf16 partial sums:
  # the two backends add them in different orders, a value next to zero can land
  # on either side of it, and that flips single entries of the ReLU mask.  Each
  # flip moves a gradient entry by about |dy . wo| |wi|, a few percent of the
  # largest entry, and a row can collect several; the bulk of the entries must
  # still agree to bf16 accuracy (the median check below).
  flips = dtype == mtf.bfloat16 and "d_model" in layout
  for name, a, b_ in zip(("y", "dx", "dwi", "dwo"), got, ref):
    assert a.shape == b_.shape
    err = rel_err(a, b_)
    assert err < (0.25 if flips else tol), (name, err)
    scale = float(np.max(np.abs(b_)))
    assert float(np.median(np.abs(np.asarray(a, np.float64) - b_))) < tol * scale / 4, name
  assert low.counter_totals() == low_ref.counter_totals()
