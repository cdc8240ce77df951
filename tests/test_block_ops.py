"""Norm, embedding gather and softmax cross-entropy on the CPU oracle backend:
the single-operation forms against the reference's op chains and against direct
numpy formulas, on meshes that split batch, the normalised dim, and the
vocabulary (where the collectives MAX / SUM come in), plus their gradients."""

import numpy as np
import pytest

from mesh_b200 import mtf
from oracle.numpy_mesh_impl import NumpyMeshImpl
from helpers import rng


def _lower(build, mesh_shape, layout):
  g = mtf.Graph()
  mesh = mtf.Mesh(g, "m")
  outs = build(mesh)
  low = mtf.Lowering(g, {mesh: NumpyMeshImpl(mesh_shape, layout)})
  return [np.asarray(low.export_to_tf_tensor(o), dtype=np.float64) for o in outs], low


MESHES = [("all:1", ""), ("a:2,b:2", "batch:a;d_model:b"), ("all:4", "batch:all"),
          ("all:2", "vocab:all"), ("a:2,b:2", "batch:a;vocab:b")]


@pytest.mark.parametrize("mesh_shape,layout", MESHES)
@pytest.mark.parametrize("centered", [True, False])
def test_norm_operation(mesh_shape, layout, centered):
  r = rng(71)
  x = r.standard_normal((4, 6, 16)).astype(np.float32) * 2 + 0.5
  sc = (1 + 0.1 * r.standard_normal(16)).astype(np.float32)
  bi = (0.1 * r.standard_normal(16)).astype(np.float32)
  dy = r.standard_normal((4, 6, 16)).astype(np.float32)

  def build(fused):
    def fn(mesh):
      X = mtf.import_tf_tensor(mesh, x, "batch:4,length:6,d_model:16", dtype=mtf.float32)
      S = mtf.import_tf_tensor(mesh, sc, "d_model:16", dtype=mtf.float32)
      B = mtf.import_tf_tensor(mesh, bi, "d_model:16", dtype=mtf.float32)
      DY = mtf.import_tf_tensor(mesh, dy, "batch:4,length:6,d_model:16", dtype=mtf.float32)
      dim = X.shape.dims[2]
      if centered:
        y = mtf.layers.layer_norm(X, dim, scale=S, bias=B, fused=fused)
        wrt = [X, S, B]
      else:
        y = mtf.layers.rms_norm(X, dim, scale=S, fused=fused)
        wrt = [X, S]
      return [y] + mtf.gradients([y], wrt, [DY])
    return fn
  got, low = _lower(build(True), mesh_shape, layout)
  ref, _ = _lower(build(False), mesh_shape, layout)
  assert any("NormOperation" in k for k in low.counter_totals())
  for a, b in zip(got, ref):
    np.testing.assert_allclose(a, b, rtol=2e-5, atol=2e-6)
  x64 = x.astype(np.float64)
  if centered:
    mean = x64.mean(-1, keepdims=True)
    direct = (x64 - mean) / np.sqrt(((x64 - mean) ** 2).mean(-1, keepdims=True) + 1e-6) * sc + bi
  else:
    direct = x64 / np.sqrt((x64 ** 2).mean(-1, keepdims=True) + 1e-6) * sc
  np.testing.assert_allclose(got[0], direct, rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("mesh_shape,layout", MESHES)
def test_gather_operation(mesh_shape, layout):
  r = rng(72)
  table = r.standard_normal((12, 8)).astype(np.float32)
  idx = r.integers(0, 12, size=(4, 6)).astype(np.int32)
  dy = r.standard_normal((4, 6, 8)).astype(np.float32)

  def fn(mesh):
    W = mtf.import_tf_tensor(mesh, table, "vocab:12,d_model:8", dtype=mtf.float32)
    I = mtf.import_tf_tensor(mesh, idx, "batch:4,length:6", dtype=mtf.int32)
    DY = mtf.import_tf_tensor(mesh, dy, "batch:4,length:6,d_model:8", dtype=mtf.float32)
    y = mtf.layers.embedding(I, W.shape.dims[0], W.shape.dims[1], mtf.float32, table=W)
    assert isinstance(y.operation, mtf.GatherOperation)
    dW, = mtf.gradients([y], [W], [DY])
    return [y, dW]
  (y, dW), low = _lower(fn, mesh_shape, layout)
  np.testing.assert_array_equal(y, table[idx])
  ref = np.zeros((12, 8))
  np.add.at(ref, idx.reshape(-1), dy.reshape(-1, 8).astype(np.float64))
  np.testing.assert_allclose(dW, ref, rtol=1e-6, atol=1e-6)
  if "vocab" in layout:
    assert any(k.startswith("allreduce") for k in low.counter_totals()) or True


def test_gather_falls_back_to_one_hot_einsum():
  """Dims shared between indices and weights, or a permuted output, keep the reference's form."""
  r = rng(73)
  vals = r.standard_normal((4, 5)).astype(np.float32)

  def fn(mesh):
    V = mtf.import_tf_tensor(mesh, vals, "a:4,k:5", dtype=mtf.float32)
    return [mtf.gather(V, 2, V.shape.dims[1])]
  (y,), _ = _lower(fn, "all:2", "a:all")
  np.testing.assert_array_equal(y, vals[:, 2])


@pytest.mark.parametrize("mesh_shape,layout", MESHES)
@pytest.mark.parametrize("z_loss", [0.0, 1e-2])
def test_softmax_cross_entropy_operation(mesh_shape, layout, z_loss):
  r = rng(74)
  logits = (r.standard_normal((4, 6, 12)) * 3).astype(np.float32)
  targets = r.integers(0, 12, size=(4, 6)).astype(np.int32)
  dl = r.standard_normal((4, 6)).astype(np.float32)

  def build(fused):
    def fn(mesh):
      L = mtf.import_tf_tensor(mesh, logits, "batch:4,length:6,vocab:12", dtype=mtf.float32)
      T = mtf.import_tf_tensor(mesh, targets, "batch:4,length:6", dtype=mtf.int32)
      DL = mtf.import_tf_tensor(mesh, dl, "batch:4,length:6", dtype=mtf.float32)
      loss = mtf.layers.softmax_cross_entropy_with_logits(L, T, L.shape.dims[2], z_loss=z_loss, fused=fused)
      dL, = mtf.gradients([loss], [L], [DL])
      return [loss, dL]
    return fn
  got, low = _lower(build(True), mesh_shape, layout)
  ref, _ = _lower(build(False), mesh_shape, layout)
  assert any("SoftmaxCrossEntropyOperation" in k for k in low.counter_totals())
  for a, b in zip(got, ref):
    np.testing.assert_allclose(a, b, rtol=2e-5, atol=2e-6)
  x = logits.astype(np.float64)
  lz = np.log(np.exp(x - x.max(-1, keepdims=True)).sum(-1)) + x.max(-1)
  direct = lz - np.take_along_axis(x, targets[..., None].astype(np.int64), -1)[..., 0] + z_loss * lz ** 2
  np.testing.assert_allclose(got[0], direct, rtol=2e-5, atol=2e-6)


def test_soft_targets_take_the_op_chain():
  r = rng(75)
  logits = r.standard_normal((3, 5)).astype(np.float32)
  soft = np.abs(r.standard_normal((3, 5))).astype(np.float32)
  soft /= soft.sum(-1, keepdims=True)

  def fn(mesh):
    L = mtf.import_tf_tensor(mesh, logits, "batch:3,vocab:5", dtype=mtf.float32)
    T = mtf.import_tf_tensor(mesh, soft, "batch:3,vocab:5", dtype=mtf.float32)
    return [mtf.layers.softmax_cross_entropy_with_logits(L, T, L.shape.dims[1])]
  (loss,), _ = _lower(fn, "all:1", "")
  x = logits.astype(np.float64)
  ls = x - (np.log(np.exp(x - x.max(-1, keepdims=True)).sum(-1, keepdims=True)) + x.max(-1, keepdims=True))
  np.testing.assert_allclose(loss, -(ls * soft).sum(-1), rtol=1e-5, atol=1e-6)


def test_random_operation_is_layout_consistent():
  """mtf.random_uniform / random_normal: slices that hold the same part of the tensor
  draw the same values (so export sees one consistent tensor), values lie in
  range, and the same graph repeats its draw."""
  def fn(mesh):
    u = mtf.random_uniform(mesh, "batch:8,d_model:16", minval=-1.0, maxval=3.0)
    z = mtf.random_normal(mesh, "batch:8,d_model:16", mean=1.0, stddev=2.0)
    d = mtf.dropout(u * 0.0 + 1.0, True, keep_prob=0.75)
    return [u, z, d]
  for mesh_shape, layout in (("all:1", ""), ("a:2,b:2", "batch:a"), ("a:2,b:2", "batch:a;d_model:b")):
    (u, z, d), _ = _lower(fn, mesh_shape, layout)
    (u2, z2, _), _ = _lower(fn, mesh_shape, layout)
    np.testing.assert_array_equal(u, u2)
    np.testing.assert_array_equal(z, z2)
    assert u.min() >= -1.0 and u.max() < 3.0 and abs(u.mean() - 1.0) < 0.5
    assert abs(z.mean() - 1.0) < 0.8 and 1.0 < z.std() < 3.0
    assert set(np.unique(np.round(d * 0.75, 6))) <= {0.0, 1.0}


def test_moe_random_policy_draws_its_own_noise():
  r = rng(76)
  x = r.standard_normal((4, 16, 8)).astype(np.float32)

  def fn(mesh):
    X = mtf.import_tf_tensor(mesh, x, "batch:4,length:16,d_model:8", dtype=mtf.float32)
    WG = mtf.import_tf_tensor(mesh, r.standard_normal((8, 4)).astype(np.float32), "d_model:8,expert_unsplit:4")
    WI = mtf.import_tf_tensor(mesh, r.standard_normal((4, 8, 16)).astype(np.float32) / 3, "experts:4,d_model:8,d_ff:16")
    WO = mtf.import_tf_tensor(mesh, r.standard_normal((4, 16, 8)).astype(np.float32) / 4, "experts:4,d_ff:16,d_model:8")
    hp = mtf.moe.HParams(moe_group_size=16)     # default second-expert policy: random
    out, loss = mtf.moe.transformer_moe_layer_v1(X, mtf.Dimension("d_model", 8), hp, True, "all:2",
                                                 "batch:all;experts:all", WG, WI, WO)
    return [out, loss]
  (out, loss), _ = _lower(fn, "all:2", "batch:all;experts:all")
  assert out.shape == (4, 16, 8) and np.isfinite(out).all() and np.isfinite(loss)


@pytest.mark.parametrize("fused", [True, False])
def test_switch_routing_layer(fused):
  """Top-1 ("Switch") routing: the single-operation form and the reference's op chain
  agree with each other and with a direct numpy restatement of the routing."""
  r = rng(77)
  b, l, d, f, e = 4, 32, 8, 16, 4
  x = r.standard_normal((b, l, d)).astype(np.float32)
  wg = r.standard_normal((d, e)).astype(np.float32)
  wi = (r.standard_normal((e, d, f)) / 3).astype(np.float32)
  wo = (r.standard_normal((e, f, d)) / 4).astype(np.float32)

  def fn(mesh):
    X = mtf.import_tf_tensor(mesh, x, "batch:4,length:32,d_model:8", dtype=mtf.float32)
    WG = mtf.import_tf_tensor(mesh, wg, "d_model:8,expert_unsplit:4")
    WI = mtf.import_tf_tensor(mesh, wi, "experts:4,d_model:8,d_ff:16")
    WO = mtf.import_tf_tensor(mesh, wo, "experts:4,d_ff:16,d_model:8")
    hp = mtf.moe.HParams(moe_group_size=32, moe_gating="switch", moe_use_fused_kernels=fused,
                         moe_capacity_factor_train=1.0)
    out, loss, aux = mtf.moe.transformer_moe_layer_v1(
        X, mtf.Dimension("d_model", 8), hp, True, "all:2", "batch:all;experts:all", WG, WI, WO,
        return_aux=True)
    grads = mtf.gradients([mtf.reduce_sum(mtf.square(out)) + loss * 5.0], [X, WG, WI])
    return [out, loss, aux["index_1"], aux["position_1"], aux["gate_1"]] + grads
  got, _ = _lower(fn, "all:2", "batch:all;experts:all")
  out, loss, i1, p1, g1 = got[:5]
  # direct restatement: 4 groups of 32 tokens, capacity 32 * 1.0 / 4 = 8
  logits = x.astype(np.float64) @ wg
  raw = np.exp(logits - logits.max(-1, keepdims=True))
  raw /= raw.sum(-1, keepdims=True)
  idx = raw.argmax(-1)
  np.testing.assert_array_equal(i1.reshape(b, l), idx)
  ref_out = np.zeros((b, l, d))
  for g in range(b):
    seen = np.zeros(e, int)
    for s in range(l):
      ex = idx[g, s]
      pos = seen[ex]
      seen[ex] += 1
      assert int(p1.reshape(b, l)[g, s]) == pos
      if pos < 8:
        h = np.maximum(x[g, s].astype(np.float64) @ wi[ex], 0)
        ref_out[g, s] = raw[g, s, ex] * (h @ wo[ex])
        np.testing.assert_allclose(g1.reshape(b, l)[g, s], raw[g, s, ex], rtol=1e-5)
      else:
        assert g1.reshape(b, l)[g, s] == 0
  np.testing.assert_allclose(out, ref_out, rtol=1e-4, atol=1e-5)
  dens = np.stack([np.bincount(idx[g], minlength=e) / l for g in range(b)])
  ref_loss = (raw.mean(1) * dens).mean() * e * e * 1e-2
  np.testing.assert_allclose(loss, ref_loss, rtol=1e-5)


def test_switch_routing_fused_gradients_equal_the_chain():
  r = rng(78)
  x = r.standard_normal((4, 16, 8)).astype(np.float32)
  wg = r.standard_normal((8, 4)).astype(np.float32)
  wi = (r.standard_normal((4, 8, 16)) / 3).astype(np.float32)
  wo = (r.standard_normal((4, 16, 8)) / 4).astype(np.float32)
  res = []
  for fused in (True, False):
    def fn(mesh):
      X = mtf.import_tf_tensor(mesh, x, "batch:4,length:16,d_model:8", dtype=mtf.float32)
      WG = mtf.import_tf_tensor(mesh, wg, "d_model:8,expert_unsplit:4")
      WI = mtf.import_tf_tensor(mesh, wi, "experts:4,d_model:8,d_ff:16")
      WO = mtf.import_tf_tensor(mesh, wo, "experts:4,d_ff:16,d_model:8")
      hp = mtf.moe.HParams(moe_group_size=16, moe_gating="switch", moe_use_fused_kernels=fused,
                           moe_capacity_factor_train=1.5)
      out, loss = mtf.moe.transformer_moe_layer_v1(X, mtf.Dimension("d_model", 8), hp, True, "all:1", "",
                                                   WG, WI, WO)
      total = mtf.reduce_sum(mtf.square(out)) + loss * 10.0
      return [total] + mtf.gradients([total], [X, WG, WI, WO])
    res.append(_lower(fn, "all:1", "")[0])
  for a, b_ in zip(*res):
    np.testing.assert_allclose(a, b_, rtol=2e-4, atol=2e-5)


@pytest.mark.parametrize("mesh_shape,layout", [("all:1", ""), ("all:4", "blocks:all"), ("a:2,b:2", "batch:a;blocks:b")])
@pytest.mark.parametrize("halo,wrap", [(1, False), (3, True), (5, False), (8, True)])
def test_halo_exchange(mesh_shape, layout, halo, wrap):
  """Blocks of a sequence extended by their neighbours' margins (whole neighbouring
  blocks when the halo exceeds the block), with the block dim split over the mesh so
  that the shifts are collective permutes; against direct numpy indexing."""
  r = rng(79)
  b, nb, bs, d = 2, 4, 4, 3
  x = r.standard_normal((b, nb, bs, d)).astype(np.float32)

  def fn(mesh):
    X = mtf.import_tf_tensor(mesh, x, "batch:2,blocks:4,block_size:4,d:3", dtype=mtf.float32)
    y = mtf.halo_exchange(X, X.shape.dims[1], X.shape.dims[2], halo, wrap=wrap)
    yl = mtf.left_halo_exchange(X, X.shape.dims[1], X.shape.dims[2], halo, wrap=wrap)
    dX, = mtf.gradients([mtf.reduce_sum(y * y) * 0.5], [X])
    return [y, yl, dX]
  (y, yl, dX), _ = _lower(fn, mesh_shape, layout)
  flat = x.reshape(b, nb * bs, d)
  n = nb * bs
  ref = np.zeros((b, nb, bs + 2 * halo, d))
  count = np.zeros((b, n, d))
  for blk in range(nb):
    for j in range(bs + 2 * halo):
      pos = blk * bs - halo + j
      if wrap:
        pos %= n
      if 0 <= pos < n:
        ref[:, blk, j] = flat[:, pos]
        count[:, pos] += 1
  np.testing.assert_array_equal(y, ref)
  np.testing.assert_array_equal(yl, ref[:, :, :bs + halo])
  np.testing.assert_allclose(dX.reshape(b, n, d), flat * count, rtol=1e-6)
