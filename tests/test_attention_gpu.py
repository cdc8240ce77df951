"""Fused attention kernel (mtfc_attention_fwd) against the oracle's op chain."""

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


@pytest.fixture(params=[1, 2], ids=["one-tile", "two-tile"])
def variant(request):
  """Runs a test under each kernel variant (one / two query tiles per CTA)."""
  from mesh_b200 import _native as nat
  nat.check(nat.lib().mtfc_attention_set_variant(request.param))
  yield request.param
  nat.check(nat.lib().mtfc_attention_set_variant(0))


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("b,h,lq,lk,d", [(1, 1, 128, 128, 128), (2, 3, 256, 256, 128),
                                         (1, 2, 300, 300, 64), (2, 2, 512, 512, 128),
                                         (1, 2, 96, 200, 128), (1, 1, 1024, 1024, 64)])
def test_attention_kernel(both, variant, b, h, lq, lk, d, causal):
  dev, ora = both
  if causal and lq != lk:
    pytest.skip("causal mask is defined for self-attention lengths")
  r = rng(51)
  q = (r.standard_normal((b, h, lq, d)) * d ** -0.25).astype(np.float32)
  k = (r.standard_normal((b, h, lk, d)) * d ** -0.25).astype(np.float32)
  v = r.standard_normal((b, h, lk, d)).astype(np.float32)
  dq, dk, dv = [dev.from_host(t, mtf.bfloat16) for t in (q, k, v)]
  oq, ok_, ov = [ora.from_host(t, mtf.bfloat16) for t in (q, k, v)]
  from mesh_b200 import _native as nat
  launches = nat.launch_count()
  out = dev.attention(dq, dk, dv, causal)
  assert nat.launch_count() - launches == 1   # one fused kernel, nothing else
  got = dev.to_host(out)
  ref = ora.to_host(ora.attention(oq, ok_, ov, causal))
  assert got.shape == ref.shape
  assert rel_err(got, ref) < 2e-2
  nat.device_status()


def test_attention_reads_blhd_storage_in_place(both, variant):
  """[batch, length, heads, d] storage viewed as [batch, heads, length, d]."""
  dev, ora = both
  r = rng(52)
  b, l, h, d = 2, 256, 4, 128
  qs, ks, vs = [r.standard_normal((b, l, h, d)).astype(np.float32) * 0.3 for _ in range(3)]
  view = lambda ops, t: ops.transpose(ops.from_host(t, mtf.bfloat16), [0, 2, 1, 3])
  got = dev.to_host(dev.attention(view(dev, qs), view(dev, ks), view(dev, vs), True))
  ref = ora.to_host(ora.attention(view(ora, qs), view(ora, ks), view(ora, vs), True))
  assert rel_err(got, ref) < 2e-2


def test_attention_fallback_small_head(both):
  dev, ora = both
  r = rng(53)
  q, k, v = [r.standard_normal((2, 2, 40, 32)).astype(np.float32) * 0.4 for _ in range(3)]
  for dt, tol in ((mtf.bfloat16, 2e-2), (mtf.float32, 2e-5)):
    got = dev.to_host(dev.attention(*[dev.from_host(t, dt) for t in (q, k, v)], True))
    ref = ora.to_host(ora.attention(*[ora.from_host(t, dt) for t in (q, k, v)], True))
    assert rel_err(got, ref) < tol


def _layer(impl, fused, b=2, l=256, d=256, h=4, kv=64):
  r = rng(54)
  g = mtf.Graph()
  mesh = mtf.Mesh(g, "m")
  x = r.standard_normal((b, l, d)).astype(np.float32)
  X = mtf.import_tf_tensor(mesh, x, "batch:%d,length:%d,d_model:%d" % (b, l, d), dtype=mtf.bfloat16)
  heads, kvd = mtf.Dimension("heads", h), mtf.Dimension("d_kv", kv)
  params = mtf.layers.multihead_attention_params(mesh, heads, X.shape.dims[-1], kvd,
                                                 mtf.layers.WeightSource(5), mtf.bfloat16)
  pos = mtf.mtf_range(mesh, X.shape.dims[1], mtf.float32)
  mask = mtf.layers.attention_mask_autoregressive(pos)
  y = mtf.layers.multihead_attention(X, None, mask, kvd, heads, params=params, fused=fused)
  low = mtf.Lowering(g, {mesh: impl})
  return low.export_to_tf_tensor(y), low


@pytest.mark.parametrize("mesh_shape,layout", [("", ""), ("all:4", "heads:all"), ("all:2", "batch:all")])
def test_multihead_attention_fused_layer(cuda_device, mesh_shape, layout):
  from mesh_b200.cuda_mesh_impl import CudaMeshImpl
  from oracle.numpy_mesh_impl import NumpyMeshImpl
  n = mtf.convert_to_shape(mesh_shape).size
  got, low = _layer(CudaMeshImpl(mesh_shape, layout, [0] * n), fused=None)
  ref, _ = _layer(NumpyMeshImpl(mesh_shape, layout), fused=False)
  assert any(k == "output/FusedAttentionOperation" for k in low.counter_totals())
  assert rel_err(got, ref) < 2e-2


def test_fused_attention_rejects_split_length(cuda_device):
  from mesh_b200.cuda_mesh_impl import CudaMeshImpl
  with pytest.raises(ValueError):
    _layer(CudaMeshImpl("all:2", "memory_length:all", [0, 0]), fused=True)
