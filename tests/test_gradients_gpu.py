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
@pytest.mark.parametrize("dtype,tol", [(mtf.float32, 1e-5), (mtf.bfloat16, 2e-2)])
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


def test_golden_gradients_on_device(cuda_device):
  """The reference's two pinned gradient vectors (top-k on a 2x2 mesh with the
  reduced dim split; recompute_grad on two processors) through the CUDA backend."""
  import json
  import os
  from mesh_b200.cuda_mesh_impl import CudaMeshImpl
  from test_oracle import golden_recompute_grad, golden_top_k_gradient
  golden = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.json")))
  v = golden["top_k"]
  got, expected = golden_top_k_gradient(CudaMeshImpl(v["mesh"], v["layout"], [0] * 4))
  np.testing.assert_array_equal(got, expected)
  v = golden["recompute_grad"]
  got, expected = golden_recompute_grad(CudaMeshImpl(v["mesh"], v["layout"], [0] * 2))
  np.testing.assert_array_equal(got[0], expected[0])
  np.testing.assert_array_equal(got[1], expected[1])


def _moe_grads(impl, fused, dtype):
  r = rng(43)
  b, l, d, f, e = 4, 64, 64, 128, 8
  g = mtf.Graph()
  mesh = mtf.Mesh(g, "m")
  x = r.standard_normal((b, l, d)).astype(np.float32)
  wg = (r.standard_normal((d, e)) / np.sqrt(d)).astype(np.float32)
  wi = (r.standard_normal((e, d, f)) / np.sqrt(d)).astype(np.float32)
  wo = (r.standard_normal((e, f, d)) / np.sqrt(f)).astype(np.float32)
  dy = r.standard_normal((b, l, d)).astype(np.float32)
  X = mtf.import_tf_tensor(mesh, x, "batch:%d,length:%d,d_model:%d" % (b, l, d), dtype=dtype)
  WG = mtf.import_tf_tensor(mesh, wg, "d_model:%d,expert_unsplit:%d" % (d, e), dtype=mtf.float32)
  WI = mtf.import_tf_tensor(mesh, wi, "experts:%d,d_model:%d,d_ff:%d" % (e, d, f), dtype=dtype)
  WO = mtf.import_tf_tensor(mesh, wo, "experts:%d,d_ff:%d,d_model:%d" % (e, f, d), dtype=dtype)
  DY = mtf.import_tf_tensor(mesh, dy, "batch:%d,length:%d,d_model:%d" % (b, l, d), dtype=dtype)
  hp = mtf.moe.HParams(moe_group_size=l, moe_second_policy_train="all", moe_use_fused_kernels=fused)
  out, loss = mtf.moe.transformer_moe_layer_v1(
      X, mtf.Dimension("d_model", d), hp, True, "all:2", "batch:all;experts:all", WG, WI, WO)
  total = mtf.reduce_sum(mtf.cast(out * DY, mtf.float32)) + mtf.cast(loss, mtf.float32) * 10.0
  grads = mtf.gradients([total], [X, WG, WI, WO])
  low = mtf.Lowering(g, {mesh: impl})
  return [low.export_to_tf_tensor(t) for t in [out] + grads]


@pytest.mark.parametrize("dtype,tol", [(mtf.float32, 1e-4), (mtf.bfloat16, 3e-2)])
def test_moe_backward_fused_kernels(cuda_device, dtype, tol):
  """Forward + backward of the top-2 MoE layer with the fused gating / dispatch /
  combine kernels (and their backward kernels) on a mesh that splits groups and
  experts, against the oracle lowering the reference's op-by-op chain."""
  from mesh_b200.cuda_mesh_impl import CudaMeshImpl
  from oracle.numpy_mesh_impl import NumpyMeshImpl
  layout = "batch:all;experts:all"
  got = _moe_grads(CudaMeshImpl("all:2", layout, [0, 0]), True, dtype)
  ref = _moe_grads(NumpyMeshImpl("all:2", layout), False, dtype)
  for name, a, b_ in zip(("out", "dx", "dwg", "dwi", "dwo"), got, ref):
    assert a.shape == b_.shape
    assert rel_err(a, b_) < tol, (name, rel_err(a, b_))


def test_attention_backward_on_device(cuda_device):
  """Gradient of the fused attention operation (the backward pass runs the
  op-by-op chain) against the oracle differentiating the chain."""
  from mesh_b200.cuda_mesh_impl import CudaMeshImpl
  from oracle.numpy_mesh_impl import NumpyMeshImpl
  r = rng(44)
  b, h, l, d = 2, 4, 128, 64
  vals = [(r.standard_normal((b, h, l, d)) * s).astype(np.float32) for s in (0.35, 0.35, 1.0, 1.0)]

  def run(impl, fused):
    g = mtf.Graph()
    m = mtf.Mesh(g, "m")
    q = mtf.import_tf_tensor(m, vals[0], "batch:2,heads:4,length:128,d_kv:64", dtype=mtf.bfloat16)
    k = mtf.import_tf_tensor(m, vals[1], "batch:2,heads:4,memory_length:128,d_kv:64", dtype=mtf.bfloat16)
    v = mtf.import_tf_tensor(m, vals[2], "batch:2,heads:4,memory_length:128,d_kv:64", dtype=mtf.bfloat16)
    do = mtf.import_tf_tensor(m, vals[3], "batch:2,heads:4,length:128,d_kv:64", dtype=mtf.bfloat16)
    mask = mtf.layers.attention_mask_autoregressive(mtf.mtf_range(m, q.shape.dims[2], mtf.float32))
    o = mtf.layers.dot_product_attention(q, k, v, mask, fused=fused)
    grads = mtf.gradients([o], [q, k, v], [do])
    low = mtf.Lowering(g, {m: impl})
    return [low.export_to_tf_tensor(t) for t in [o] + grads], low
  got, low = run(CudaMeshImpl("all:2", "heads:all", [0, 0]), True)
  ref, _ = run(NumpyMeshImpl("all:2", "heads:all"), False)
  assert any(k == "output/FusedAttentionOperation" for k in low.counter_totals())
  for name, a, b_ in zip(("o", "dq", "dk", "dv"), got, ref):
    assert rel_err(a, b_) < 2e-2, (name, rel_err(a, b_))
