"""Laid-out einsum, dense FFN and attention lowered on CudaMeshImpl against the
oracle backend: same graph, same mesh, same layout rules, same seeded inputs."""

import numpy as np
import pytest

from mesh_b200 import mtf
from helpers import rel_err, rng

pytestmark = pytest.mark.gpu


def _impls(mesh_shape, layout):
  from mesh_b200.cuda_mesh_impl import CudaMeshImpl
  from oracle.numpy_mesh_impl import NumpyMeshImpl
  n = mtf.convert_to_shape(mesh_shape).size
  return CudaMeshImpl(mesh_shape, layout, [0] * n), NumpyMeshImpl(mesh_shape, layout)


def _einsum_graph(impl, layout_dtype):
  r = rng(31)
  g = mtf.Graph()
  mesh = mtf.Mesh(g, "m")
  x = r.standard_normal((256, 128)).astype(np.float32)
  w = (r.standard_normal((128, 512)) / np.sqrt(128)).astype(np.float32)
  X = mtf.import_tf_tensor(mesh, x, "batch:256,d_model:128", dtype=layout_dtype)
  W = mtf.import_tf_tensor(mesh, w, "d_model:128,d_ff:512", dtype=layout_dtype)
  y = mtf.einsum([X, W], mtf.Shape([X.shape.dims[0], W.shape.dims[1]]))
  low = mtf.Lowering(g, {mesh: impl})
  return low.export_to_tf_tensor(y), low


@pytest.mark.parametrize("layout", ["batch:all", "d_model:all", "d_ff:all", ""])
@pytest.mark.parametrize("dtype,tol", [(mtf.float32, 1e-5), (mtf.bfloat16, 2e-2)])
def test_laid_out_einsum(cuda_device, layout, dtype, tol):
  """cfg-1 pattern: batch split (no communication) and contracted dim split (allreduce)."""
  cuda, ora = _impls("all:4", layout)
  got, low = _einsum_graph(cuda, dtype)
  ref, _ = _einsum_graph(ora, dtype)
  assert rel_err(got, ref) < tol
  has_allreduce = any(k.startswith("allreduce") for k in low.counter_totals())
  assert has_allreduce == (layout == "d_model:all")


def _ffn_graph(impl, dtype, b=8, l=32, d=128, f=512):
  r = rng(32)
  g = mtf.Graph()
  mesh = mtf.Mesh(g, "m")
  x = r.standard_normal((b, l, d)).astype(np.float32)
  wi = (r.standard_normal((d, f)) / np.sqrt(d)).astype(np.float32)
  wo = (r.standard_normal((f, d)) / np.sqrt(f)).astype(np.float32)
  X = mtf.import_tf_tensor(mesh, x, "batch:%d,length:%d,d_model:%d" % (b, l, d), dtype=dtype)
  WI = mtf.import_tf_tensor(mesh, wi, "d_model:%d,d_ff:%d" % (d, f), dtype=dtype)
  WO = mtf.import_tf_tensor(mesh, wo, "d_ff:%d,d_model:%d" % (f, d), dtype=dtype)
  y = mtf.layers.dense_relu_dense(X, mtf.Dimension("d_ff", f), wi=WI, wo=WO)
  low = mtf.Lowering(g, {mesh: impl})
  return low.export_to_tf_tensor(y), low


@pytest.mark.parametrize("mesh_shape,layout", [("", ""), ("rows:2,cols:4", "batch:rows;d_ff:cols"),
                                               ("rows:2,cols:2", "batch:rows;d_model:cols")])
@pytest.mark.parametrize("dtype,tol", [(mtf.float32, 1e-5), (mtf.bfloat16, 2e-2)])
def test_dense_relu_dense(cuda_device, mesh_shape, layout, dtype, tol):
  cuda, ora = _impls(mesh_shape, layout)
  got, low = _ffn_graph(cuda, dtype)
  ref, low_ref = _ffn_graph(ora, dtype)
  assert rel_err(got, ref) < tol
  assert low.counter_totals() == low_ref.counter_totals()


def _attention_graph(impl, dtype, b=2, l=64, d=128, h=4, kv=32):
  r = rng(33)
  g = mtf.Graph()
  mesh = mtf.Mesh(g, "m")
  x = r.standard_normal((b, l, d)).astype(np.float32)
  X = mtf.import_tf_tensor(mesh, x, "batch:%d,length:%d,d_model:%d" % (b, l, d), dtype=dtype)
  heads, kvd = mtf.Dimension("heads", h), mtf.Dimension("d_kv", kv)
  ws = mtf.layers.WeightSource(seed=5)
  params = mtf.layers.multihead_attention_params(mesh, heads, X.shape.dims[-1], kvd, ws, dtype)
  pos = mtf.mtf_range(mesh, X.shape.dims[1], mtf.float32)
  mask = mtf.layers.attention_mask_autoregressive(pos, dtype=mtf.float32)
  y = mtf.layers.multihead_attention(X, None, mask, kvd, heads, params=params)
  low = mtf.Lowering(g, {mesh: impl})
  return low.export_to_tf_tensor(y), low


@pytest.mark.parametrize("mesh_shape,layout", [("", ""), ("all:4", "heads:all"), ("all:2", "batch:all")])
@pytest.mark.parametrize("dtype,tol", [(mtf.float32, 2e-5), (mtf.bfloat16, 2e-2)])
def test_multihead_attention(cuda_device, mesh_shape, layout, dtype, tol):
  cuda, ora = _impls(mesh_shape, layout)
  got, low = _attention_graph(cuda, dtype)
  ref, _ = _attention_graph(ora, dtype)
  assert rel_err(got, ref) < tol
  if layout == "heads:all":
    assert any(k.startswith("allreduce") for k in low.counter_totals())


def test_topk_on_split_dim(cuda_device):
  cuda, ora = _impls("rows:2,cols:2", "a:rows;b:cols")

  def run(impl):
    r = rng(34)
    g = mtf.Graph()
    mesh = mtf.Mesh(g, "m")
    x = r.standard_normal((4, 8)).astype(np.float32)
    X = mtf.import_tf_tensor(mesh, x, "a:4,b:8")
    v, i = mtf.top_k(X, X.shape.dims[1], mtf.Dimension("k", 5))
    v1, i1 = mtf.top_1(X, X.shape.dims[1])
    low = mtf.Lowering(g, {mesh: impl})
    return [low.export_to_tf_tensor(t) for t in (v, i, v1, i1)]
  for got, ref in zip(run(cuda), run(ora)):
    np.testing.assert_array_equal(got, ref)


def test_reshape_collectives_and_shift(cuda_device):
  cuda, ora = _impls("all:4", "a:all;c:all")

  def run(impl):
    r = rng(35)
    g = mtf.Graph()
    mesh = mtf.Mesh(g, "m")
    x = r.standard_normal((8, 4, 12)).astype(np.float32)
    X = mtf.import_tf_tensor(mesh, x, "a:8,b:4,x:12")      # split on a
    y1 = mtf.reshape(X, "a2:8,b:4,c:12")                    # alltoall a -> c
    y2 = mtf.reshape(X, "a2:8,b:4,x:12")                    # allconcat
    y3 = mtf.reshape(y2, "a:8,b:4,x:12")                    # allsplit
    y4 = mtf.shift(X, 3, X.shape.dims[0], wrap=False)
    y5 = mtf.shift(X, -2, X.shape.dims[0], wrap=True)
    low = mtf.Lowering(g, {mesh: impl})
    return [low.export_to_tf_tensor(t) for t in (y1, y2, y3, y4, y5)], low.counter_totals()
  (got, cg), (ref, cr) = run(cuda), run(ora)
  for a, b in zip(got, ref):
    np.testing.assert_array_equal(a, b)
  assert cg == cr


def test_variable_on_device(cuda_device):
  cuda, _ = _impls("rows:2,cols:2", "a:rows;b:cols")
  w0 = rng(36).standard_normal((8, 6)).astype(np.float32)
  g = mtf.Graph()
  mesh = mtf.Mesh(g, "m")
  w = mtf.get_variable(mesh, "w", "a:8,b:6", initial_value=w0)
  y = w * 2.0
  low = mtf.Lowering(g, {mesh: cuda})
  np.testing.assert_array_equal(low.export_to_tf_tensor(y), w0 * 2)
  lov = low.variables[w.operation]
  ops = cuda.slice_ops
  lov.assign_to_slices(lambda var, old, value: ops.binary("add", old, value), [1.0] * 4)
  lov.copy_slices_to_master()
  np.testing.assert_array_equal(w.operation.get_master(), w0 + 1)
  w.operation.assign_to_master(w0 * 3)
  lov.copy_master_to_slices()
  np.testing.assert_array_equal(cuda.export_to_tf_tensor(w, lov.laid_out_tensor), w0 * 3)


@pytest.mark.parametrize("mesh_shape,layout,splits", [("all:1", "", 1), ("all:2", "length:all", 2)])
def test_local_attention_matches_oracle(cuda_device, mesh_shape, layout, splits):
  """local_attention_1d (halo exchange over receive, blocked logits) on the device kernels
  against the oracle lowering of the same graph."""
  from mesh_b200.cuda_mesh_impl import CudaMeshImpl
  from oracle.numpy_mesh_impl import NumpyMeshImpl

  def run(impl):
    r = rng(71)
    g = mtf.Graph()
    m = mtf.Mesh(g, "m")
    q, k = [r.standard_normal((2, 256, 16)).astype(np.float32) for _ in range(2)]
    v = r.standard_normal((2, 256, 8)).astype(np.float32)
    Q = mtf.import_tf_tensor(m, q, "batch:2,length:256,d_k:16")
    K = mtf.import_tf_tensor(m, k, "batch:2,length:256,d_k:16")
    V = mtf.import_tf_tensor(m, v, "batch:2,length:256,d_v:8")
    out = mtf.layers.local_attention_1d(Q, K, V, mtf.Dimension("length", 256), mtf.Dimension("d_k", 16),
                                        mtf.Dimension("d_v", 8), fully_autoregressive=False,
                                        length_dim_num_splits=splits, radius=24)
    return mtf.Lowering(g, {m: impl}).export_to_tf_tensor(out)
  n = mtf.convert_to_shape(mesh_shape).size
  assert rel_err(run(CudaMeshImpl(mesh_shape, layout, [0] * n)), run(NumpyMeshImpl(mesh_shape, layout))) < 1e-5
