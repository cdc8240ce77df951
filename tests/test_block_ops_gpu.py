"""Row kernels for layer / RMS norm, embedding gather and softmax cross-entropy
on the device against the oracle's direct formulas, and the graph operations on
CudaMeshImpl against NumpyMeshImpl over split meshes."""

import numpy as np
import pytest

from mesh_b200 import mtf
from helpers import rel_err, rng

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def both(cuda_device):
  from mesh_b200.device_ops import DeviceOps
  from oracle.numpy_ops import NumpyOps
  return DeviceOps(cuda_device), NumpyOps()


@pytest.mark.parametrize("dtype,tol", [(mtf.float32, 1e-5), (mtf.bfloat16, 2e-2)])
@pytest.mark.parametrize("rows,cols", [(4096, 1024), (33, 2048), (7, 100), (5, 4096), (1, 8), (300, 520)])
@pytest.mark.parametrize("centered", [True, False])
def test_norm_rows(both, rows, cols, centered, dtype, tol):
  dev, ora = both
  r = rng(81)
  x = (r.standard_normal((rows, cols)) * 3 + 1).astype(np.float32)
  sc = (1 + 0.2 * r.standard_normal(cols)).astype(np.float32)
  bi = (0.3 * r.standard_normal(cols)).astype(np.float32)
  args = lambda ops: (ops.from_host(x, dtype), ops.from_host(sc, dtype),
                      ops.from_host(bi, dtype) if centered else None)
  got = dev.to_host(dev.norm_rows(*args(dev), 1e-6, centered))
  ref = ora.to_host(ora.norm_rows(*args(ora), 1e-6, centered))
  assert rel_err(got, ref) < tol


@pytest.mark.parametrize("dtype", [mtf.float32, mtf.bfloat16])
def test_gather_rows(both, dtype):
  dev, ora = both
  r = rng(82)
  table = r.standard_normal((1000, 256)).astype(np.float32)
  idx = r.integers(-50, 1100, size=(7, 300)).astype(np.int32)   # some rows fall outside the slice
  for first in (0, 200):
    got = dev.to_host(dev.gather_rows(dev.from_host(table, dtype), dev.from_host(idx, mtf.int32), first))
    ref = ora.to_host(ora.gather_rows(ora.from_host(table, dtype), ora.from_host(idx, mtf.int32), first))
    np.testing.assert_array_equal(got, ref)


@pytest.mark.parametrize("dtype,tol", [(mtf.float32, 1e-5), (mtf.bfloat16, 1e-5)])
@pytest.mark.parametrize("rows,cols", [(64, 32768), (1000, 1000), (3, 7), (256, 4096)])
def test_xent_stats_and_grad(both, rows, cols, dtype, tol):
  dev, ora = both
  r = rng(83)
  x = (r.standard_normal((rows, cols)) * 4).astype(np.float32)
  t = r.integers(0, 2 * cols, size=(rows,)).astype(np.int32)   # half the targets lie in "another slice"
  first = cols // 2
  dx, dt = dev.from_host(x, dtype), dev.from_host(t, mtf.int32)
  ox, ot = ora.from_host(x, dtype), ora.from_host(t, mtf.int32)
  got = [dev.to_host(v) for v in dev.xent_stats(dx, dt, first)]
  ref = [ora.to_host(v) for v in ora.xent_stats(ox, ot, first)]
  np.testing.assert_array_equal(got[0], ref[0])                 # row max: exact
  assert rel_err(got[1], ref[1]) < tol                          # inputs identical, fp32 statistics
  np.testing.assert_array_equal(got[2], ref[2])                 # picked logit: a copy
  log_z = (np.log(ref[1].astype(np.float64)) + ref[0]).astype(np.float32)
  dloss = r.standard_normal(rows).astype(np.float32)
  gtol = 1e-5 if dtype == mtf.float32 else 2e-2
  got_g = dev.to_host(dev.xent_grad(dx, dt, dev.from_host(log_z, mtf.float32),
                                    dev.from_host(dloss, mtf.float32), 1e-3, first))
  ref_g = ora.to_host(ora.xent_grad(ox, ot, ora.from_host(log_z, mtf.float32),
                                    ora.from_host(dloss, mtf.float32), 1e-3, first))
  assert rel_err(got_g, ref_g) < gtol


def _block(impl, dtype):
  """Embedding -> layer norm -> logits -> cross-entropy, with gradients."""
  r = rng(84)
  b, l, d, v = 4, 32, 128, 512
  table = r.standard_normal((v, d)).astype(np.float32)
  ids = r.integers(0, v, size=(b, l)).astype(np.int32)
  targets = r.integers(0, v, size=(b, l)).astype(np.int32)
  sc = (1 + 0.1 * r.standard_normal(d)).astype(np.float32)
  bi = (0.1 * r.standard_normal(d)).astype(np.float32)
  g = mtf.Graph()
  mesh = mtf.Mesh(g, "m")
  W = mtf.import_tf_tensor(mesh, table, "vocab:%d,d_model:%d" % (v, d), dtype=dtype)
  I = mtf.import_tf_tensor(mesh, ids, "batch:%d,length:%d" % (b, l), dtype=mtf.int32)
  T = mtf.import_tf_tensor(mesh, targets, "batch:%d,length:%d" % (b, l), dtype=mtf.int32)
  S = mtf.import_tf_tensor(mesh, sc, "d_model:%d" % d, dtype=dtype)
  B = mtf.import_tf_tensor(mesh, bi, "d_model:%d" % d, dtype=dtype)
  x = mtf.layers.embedding(I, W.shape.dims[0], W.shape.dims[1], dtype, table=W)
  h = mtf.layers.layer_norm(x, x.shape.dims[-1], scale=S, bias=B)
  h = mtf.layers.rms_norm(h, h.shape.dims[-1], scale=S)
  logits = mtf.einsum([h, W], output_shape=mtf.Shape(h.shape.dims[:-1] + [W.shape.dims[0]]))
  loss = mtf.layers.softmax_cross_entropy_with_logits(logits, T, W.shape.dims[0], z_loss=1e-4)
  total = mtf.reduce_mean(mtf.cast(loss, mtf.float32))
  grads = mtf.gradients([total], [W, S, B])
  low = mtf.Lowering(g, {mesh: impl})
  return [low.export_to_tf_tensor(t) for t in [x, h, loss, total] + grads], low


@pytest.mark.parametrize("mesh_shape,layout", [("all:1", ""), ("a:2,b:2", "batch:a;vocab:b"),
                                               ("all:2", "d_model:all")])
@pytest.mark.parametrize("dtype,tol", [(mtf.float32, 2e-5), (mtf.bfloat16, 3e-2)])
def test_block_on_device(cuda_device, mesh_shape, layout, dtype, tol):
  from mesh_b200.cuda_mesh_impl import CudaMeshImpl
  from oracle.numpy_mesh_impl import NumpyMeshImpl
  n = mtf.convert_to_shape(mesh_shape).size
  got, low = _block(CudaMeshImpl(mesh_shape, layout, [0] * n), dtype)
  ref, low_ref = _block(NumpyMeshImpl(mesh_shape, layout), dtype)
  for name, a, b_ in zip(("embedding", "norms", "loss", "mean loss", "dW", "dscale", "dbias"), got, ref):
    assert np.shape(a) == np.shape(b_)
    assert rel_err(a, b_) < tol, (name, rel_err(a, b_))
  np.testing.assert_array_equal(got[0], ref[0])   # the gather is exact
  assert low.counter_totals() == low_ref.counter_totals()


@pytest.mark.parametrize("dtype", [mtf.float32, mtf.bfloat16])
def test_random_matches_the_restated_generator(both, dtype):
  """The device's Philox4x32-10 stream equals the oracle's numpy restatement:
  uniform draws bit for bit, normal draws to float rounding of log / sin / cos."""
  dev, ora = both
  for n, seed in ((1001, 12345678901234567), (4096, 7), (3, 2 ** 63 + 5)):
    got = dev.to_host(dev.random([n], "uniform", seed, dtype, -2.0, 5.0))
    ref = ora.to_host(ora.random([n], "uniform", seed, dtype, -2.0, 5.0))
    np.testing.assert_array_equal(got, ref)
    got = dev.to_host(dev.random([n], "normal", seed, dtype, 0.5, 2.0))
    ref = ora.to_host(ora.random([n], "normal", seed, dtype, 0.5, 2.0))
    assert np.max(np.abs(got - ref)) < (2e-5 if dtype == mtf.float32 else 5e-2)


def test_random_operation_on_device(cuda_device):
  from mesh_b200.cuda_mesh_impl import CudaMeshImpl
  from oracle.numpy_mesh_impl import NumpyMeshImpl
  outs = []
  for impl in (CudaMeshImpl("a:2,b:2", "batch:a", [0] * 4), NumpyMeshImpl("a:2,b:2", "batch:a")):
    g = mtf.Graph()
    mesh = mtf.Mesh(g, "m")
    u = mtf.random_uniform(mesh, "batch:8,d_model:32", minval=0.0, maxval=1.0)
    low = mtf.Lowering(g, {mesh: impl})
    outs.append(low.export_to_tf_tensor(u))
  np.testing.assert_array_equal(outs[0], outs[1])
