"""mtf.gradients on the CPU oracle backend: analytic gradients against central
finite differences, on meshes that split batch and contracted dims (the
gradient einsums then carry their own allreduces), and the operation-level
rules of mesh_tensorflow/ops.py:6493-6586 (no gradient through integer
outputs, stop_gradient, None for unreachable inputs)."""

import numpy as np
import pytest

from mesh_b200 import mtf
from oracle.numpy_mesh_impl import NumpyMeshImpl
from helpers import rng


def _lower(graph, mesh, outs, mesh_shape, layout):
  low = mtf.Lowering(graph, {mesh: NumpyMeshImpl(mesh_shape, layout)})
  return [np.asarray(low.export_to_tf_tensor(o), dtype=np.float64) for o in outs]


def _ffn_loss(arrays):
  x, wi, wo, b = arrays
  g = mtf.Graph()
  m = mtf.Mesh(g, "m")
  X = mtf.import_tf_tensor(m, x, "batch:4,d_model:8", dtype=mtf.float32)
  WI = mtf.import_tf_tensor(m, wi, "d_model:8,d_ff:16", dtype=mtf.float32)
  WO = mtf.import_tf_tensor(m, wo, "d_ff:16,d_model:8", dtype=mtf.float32)
  B = mtf.import_tf_tensor(m, b, "d_model:8", dtype=mtf.float32)
  h = mtf.relu(mtf.einsum([X, WI], output_shape="batch:4,d_ff:16"))
  y = mtf.einsum([h, WO], output_shape="batch:4,d_model:8") + B      # broadcast add
  p = mtf.softmax(y, y.shape.dims[1])
  top, _ = mtf.top_k(y, y.shape.dims[1], mtf.Dimension("k", 2))
  loss = (mtf.reduce_sum(mtf.square(p) * mtf.tanh(y)) + mtf.reduce_sum(mtf.reduce_max(y, reduced_dim=y.shape.dims[1]))
          + mtf.reduce_sum(top) * 0.5 + mtf.reduce_sum(mtf.maximum(y, B)) - mtf.reduce_sum(mtf.sigmoid(y) / (mtf.exp(B) + 1.0)))
  return g, m, [X, WI, WO, B], loss


@pytest.mark.parametrize("mesh_shape,layout", [
    ("all:1", ""), ("a:2,b:2", "batch:a;d_ff:b"), ("a:4", "d_model:a")])
def test_gradients_match_finite_differences(mesh_shape, layout):
  r = rng(11)
  arrays = [r.standard_normal((4, 8)).astype(np.float32),
            (r.standard_normal((8, 16)) / 3).astype(np.float32),
            (r.standard_normal((16, 8)) / 4).astype(np.float32),
            r.standard_normal((8,)).astype(np.float32)]
  g, m, ins, loss = _ffn_loss(arrays)
  grads = mtf.gradients([loss], ins)
  vals = _lower(g, m, [loss] + grads, mesh_shape, layout)

  def loss_at(which, idx, delta):
    a = [v.copy() for v in arrays]
    a[which][idx] += delta
    g2, m2, _, l2 = _ffn_loss(a)
    return float(_lower(g2, m2, [l2], "all:1", "")[0])
  eps = 2e-3
  for which, arr in enumerate(arrays):
    assert vals[1 + which].shape == arr.shape
    for _ in range(4):
      idx = tuple(int(r.integers(0, s)) for s in arr.shape)
      fd = (loss_at(which, idx, eps) - loss_at(which, idx, -eps)) / (2 * eps)
      assert abs(vals[1 + which][idx] - fd) < 2e-3 + 2e-2 * abs(fd), (which, idx)


def test_gradient_rules():
  g = mtf.Graph()
  m = mtf.Mesh(g, "m")
  x = mtf.import_tf_tensor(m, np.arange(6, dtype=np.float32).reshape(2, 3), "a:2,b:3", dtype=mtf.float32)
  w = mtf.import_tf_tensor(m, np.ones((3,), np.float32), "b:3", dtype=mtf.float32)
  unused = mtf.import_tf_tensor(m, np.ones((3,), np.float32), "b:3", dtype=mtf.float32)
  y = mtf.reduce_sum(mtf.stop_gradient(x) * w) + mtf.reduce_sum(mtf.reshape(x, "c:6") * 2.0)
  dx, dw, du = mtf.gradients([y], [x, w, unused])
  assert du is None
  vx, vw = _lower(g, m, [dx, dw], "all:1", "")
  np.testing.assert_allclose(vx, np.full((2, 3), 2.0))          # only the reshape branch
  np.testing.assert_allclose(vw, np.arange(6).reshape(2, 3).sum(0))
  idx = mtf.argmax(x, x.shape.dims[1])
  assert not idx.operation.has_gradient or idx.dtype.is_integer
  ds, = mtf.gradients([mtf.reduce_sum(mtf.stack([x, x * 3.0], "s"))], [x])
  np.testing.assert_allclose(_lower(g, m, [ds], "all:1", "")[0], np.full((2, 3), 4.0))
  dsh, = mtf.gradients([mtf.reduce_sum(mtf.shift(x, 1, x.shape.dims[1], False) * w)], [x])
  np.testing.assert_allclose(_lower(g, m, [dsh], "all:1", "")[0], [[1, 1, 0], [1, 1, 0]])


def _moe_total(arrays, mesh_shape, layout, grads, fused=False, **hparams):
  x, wg, wi, wo = arrays
  g = mtf.Graph()
  m = mtf.Mesh(g, "m")
  X = mtf.import_tf_tensor(m, x, "batch:4,length:16,d_model:8", dtype=mtf.float32)
  WG = mtf.import_tf_tensor(m, wg, "d_model:8,expert_unsplit:4", dtype=mtf.float32)
  WI = mtf.import_tf_tensor(m, wi, "experts:4,d_model:8,d_ff:16", dtype=mtf.float32)
  WO = mtf.import_tf_tensor(m, wo, "experts:4,d_ff:16,d_model:8", dtype=mtf.float32)
  settings = dict(moe_group_size=16, moe_second_policy_train="all", moe_use_fused_kernels=fused,
                  moe_capacity_factor_train=1.5)
  settings.update(hparams)
  hp = mtf.moe.HParams(**settings)
  out, loss = mtf.moe.transformer_moe_layer_v1(
      X, mtf.Dimension("d_model", 8), hp, True, mesh_shape, layout, WG, WI, WO)
  total = mtf.reduce_sum(mtf.square(out)) + loss * 10.0
  outs = [total] + (mtf.gradients([total], [X, WG, WI, WO]) if grads else [])
  return _lower(g, m, outs, mesh_shape, layout)


def test_moe_layer_gradients_match_finite_differences():
  """The op-by-op top-2 MoE layer differentiates end to end: through the gates
  (softmax, renormalisation, the auxiliary loss) but not the integer routing
  decisions, through the dispatch / combine einsums and the two reshapes that
  lower to alltoalls (experts split over the mesh)."""
  r = rng(13)
  arrays = [r.standard_normal((4, 16, 8)).astype(np.float32),
            (r.standard_normal((8, 4)) / 2).astype(np.float32),
            (r.standard_normal((4, 8, 16)) / 3).astype(np.float32),
            (r.standard_normal((4, 16, 8)) / 4).astype(np.float32)]
  mesh_shape, layout = "all:2", "batch:all;experts:all"
  vals = _moe_total(arrays, mesh_shape, layout, True)
  eps = 1e-3
  for which, arr in enumerate(arrays):
    assert vals[1 + which].shape == arr.shape
    for _ in range(3):
      idx = tuple(int(r.integers(0, s)) for s in arr.shape)
      a = [v.copy() for v in arrays]
      a[which][idx] += eps
      up = float(_moe_total(a, mesh_shape, layout, False)[0])
      a[which][idx] -= 2 * eps
      down = float(_moe_total(a, mesh_shape, layout, False)[0])
      fd = (up - down) / (2 * eps)
      assert abs(vals[1 + which][idx] - fd) < 2e-2 + 2e-2 * abs(fd), (which, idx)


def test_fused_moe_gradients_equal_the_op_chain():
  """The fused gating / dispatch / combine operations differentiate to the same
  gradients as the reference's op chain (capacity tight enough to drop tokens),
  on one processor and with groups and experts split."""
  r = rng(14)
  arrays = [r.standard_normal((4, 16, 8)).astype(np.float32),
            (r.standard_normal((8, 4)) / 2).astype(np.float32),
            (r.standard_normal((4, 8, 16)) / 3).astype(np.float32),
            (r.standard_normal((4, 16, 8)) / 4).astype(np.float32)]
  for mesh_shape, layout in (("all:1", ""), ("all:2", "batch:all;experts:all")):
    ref = _moe_total(arrays, mesh_shape, layout, True, fused=False)
    got = _moe_total(arrays, mesh_shape, layout, True, fused=True)
    for a, b in zip(got, ref):
      np.testing.assert_allclose(a, b, rtol=2e-4, atol=2e-5)


@pytest.mark.parametrize("hparams", [dict(moe_gating="switch"),
                                     dict(moe_second_policy_train="threshold", moe_second_threshold_train=0.3),
                                     dict(moe_second_policy_train="none")])
def test_fused_gating_gradient_for_other_policies(hparams):
  """The gating backward operation (softmax backward of the picked, renormalised gates
  and of the loss) against the differentiated op chain for top-1 routing and for
  second-expert policies that drop second choices."""
  r = rng(15)
  arrays = [r.standard_normal((4, 16, 8)).astype(np.float32),
            (r.standard_normal((8, 4)) / 2).astype(np.float32),
            (r.standard_normal((4, 8, 16)) / 3).astype(np.float32),
            (r.standard_normal((4, 16, 8)) / 4).astype(np.float32)]
  for mesh_shape, layout in (("all:1", ""), ("all:2", "batch:all;experts:all")):
    ref = _moe_total(arrays, mesh_shape, layout, True, fused=False, **hparams)
    got = _moe_total(arrays, mesh_shape, layout, True, fused=True, **hparams)
    for a, b in zip(got, ref):
      np.testing.assert_allclose(a, b, rtol=2e-4, atol=2e-5)
  # ... and against the restated chain the operation replaced
  saved = mtf.moe.Top2GatingOperation.fused_gradient
  try:
    mtf.moe.Top2GatingOperation.fused_gradient = False
    chain = _moe_total(arrays, "all:1", "", True, fused=True, **hparams)
  finally:
    mtf.moe.Top2GatingOperation.fused_gradient = saved
  for a, b in zip(_moe_total(arrays, "all:1", "", True, fused=True, **hparams), chain):
    np.testing.assert_allclose(a, b, rtol=2e-4, atol=2e-5)


def test_fused_attention_gradient_equals_the_op_chain():
  r = rng(15)
  b, h, l, d = 2, 2, 8, 4
  vals = [r.standard_normal((b, h, l, d)).astype(np.float32) for _ in range(3)]
  outs = []
  for fused in (True, False):
    g = mtf.Graph()
    m = mtf.Mesh(g, "m")
    q = mtf.import_tf_tensor(m, vals[0], "batch:2,heads:2,length:8,d_kv:4", dtype=mtf.float32)
    k = mtf.import_tf_tensor(m, vals[1], "batch:2,heads:2,memory_length:8,d_kv:4", dtype=mtf.float32)
    v = mtf.import_tf_tensor(m, vals[2], "batch:2,heads:2,memory_length:8,d_kv:4", dtype=mtf.float32)
    pos = mtf.mtf_range(m, q.shape.dims[2], mtf.float32)
    mask = mtf.layers.attention_mask_autoregressive(pos)
    o = mtf.layers.dot_product_attention(q, k, v, mask, fused=fused)
    loss = mtf.reduce_sum(mtf.square(o) * 0.5 + o)
    outs.append(_lower(g, m, [loss] + mtf.gradients([loss], [q, k, v]), "all:2", "heads:all"))
  for a, b in zip(*outs):
    np.testing.assert_allclose(a, b, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("mesh_shape,layout", [("all:1", ""), ("a:2,b:2", "batch:a;d_ff:b")])
def test_sgd_step_on_variables(mesh_shape, layout):
  """gradients + assign: one SGD step lowers in a single pass and lands in the
  variables' master copies; two steps reduce a least-squares loss."""
  r = rng(17)
  x = r.standard_normal((8, 8)).astype(np.float32)
  target = r.standard_normal((8, 4)).astype(np.float32)
  w0 = (r.standard_normal((8, 16)) / 3).astype(np.float32)
  v0 = (r.standard_normal((16, 4)) / 4).astype(np.float32)
  g = mtf.Graph()
  m = mtf.Mesh(g, "m")
  X = mtf.import_tf_tensor(m, x, "batch:8,d_model:8", dtype=mtf.float32)
  T = mtf.import_tf_tensor(m, target, "batch:8,out:4", dtype=mtf.float32)
  W = mtf.get_variable(m, "w", "d_model:8,d_ff:16", initial_value=w0)
  V = mtf.get_variable(m, "v", "d_ff:16,out:4", initial_value=v0)
  h = mtf.relu(mtf.einsum([X, W], output_shape="batch:8,d_ff:16"))
  loss = mtf.reduce_sum(mtf.square(mtf.einsum([h, V], output_shape="batch:8,out:4") - T))
  dW, dV = mtf.gradients([loss], [W, V])
  mtf.assign(W, W - dW * 0.01)
  mtf.assign(V, V - dV * 0.01)
  impl = NumpyMeshImpl(mesh_shape, layout)
  losses = []
  for _ in range(3):
    low = mtf.Lowering(g, {m: impl})
    losses.append(float(np.asarray(low.export_to_tf_tensor(loss))))
  assert losses[2] < losses[1] < losses[0]
  # the first step, by hand
  hh = np.maximum(x @ w0, 0)
  e = hh @ v0 - target
  np.testing.assert_allclose(losses[0], float((e * e).sum()), rtol=1e-5)
  dv = 2 * hh.T @ e
  dw = x.T @ ((2 * e @ v0.T) * (hh > 0))
  w1 = w0 - 0.01 * dw
  # after three lowerings the master holds the third update; re-derive the first from a fresh graph
  gg = mtf.Graph()
  mm = mtf.Mesh(gg, "m")
  X2 = mtf.import_tf_tensor(mm, x, "batch:8,d_model:8", dtype=mtf.float32)
  T2 = mtf.import_tf_tensor(mm, target, "batch:8,out:4", dtype=mtf.float32)
  W2 = mtf.get_variable(mm, "w", "d_model:8,d_ff:16", initial_value=w0)
  V2 = mtf.get_variable(mm, "v", "d_ff:16,out:4", initial_value=v0)
  h2 = mtf.relu(mtf.einsum([X2, W2], output_shape="batch:8,d_ff:16"))
  l2 = mtf.reduce_sum(mtf.square(mtf.einsum([h2, V2], output_shape="batch:8,out:4") - T2))
  dW2, dV2 = mtf.gradients([l2], [W2, V2])
  mtf.assign(W2, W2 - dW2 * 0.01)
  mtf.assign(V2, V2 - dV2 * 0.01)
  mtf.Lowering(gg, {mm: NumpyMeshImpl(mesh_shape, layout)})
  np.testing.assert_allclose(W2.operation.get_master(), w1, rtol=1e-4, atol=1e-5)
  np.testing.assert_allclose(V2.operation.get_master(), v0 - 0.01 * dv, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("mesh_shape,layout", [("all:1", ""), ("a:2,b:2", "batch:a;d_ff:b")])
def test_serialize_training_step_accumulates_with_one_allreduce(mesh_shape, layout):
  """Microbatched gradients equal the full-batch gradients, and each variable's
  data-parallel allreduce runs once, after the last microbatch, not once per microbatch."""
  r = rng(19)
  x = r.standard_normal((8, 6)).astype(np.float32)
  target = r.standard_normal((8, 3)).astype(np.float32)
  w0 = (r.standard_normal((6, 10)) / 3).astype(np.float32)
  v0 = (r.standard_normal((10, 3)) / 3).astype(np.float32)

  def build(num_splits):
    g = mtf.Graph()
    m = mtf.Mesh(g, "m")
    X = mtf.import_tf_tensor(m, x, "batch:8,d_model:6", dtype=mtf.float32)
    T = mtf.import_tf_tensor(m, target, "batch:8,out:3", dtype=mtf.float32)
    W = mtf.get_variable(m, "w", "d_model:6,d_ff:10", initial_value=w0)
    V = mtf.get_variable(m, "v", "d_ff:10,out:3", initial_value=v0)

    def model_fn(features):
      h = mtf.relu(mtf.einsum([features["x"], W], output_shape=mtf.Shape([features["x"].shape.dims[0], W.shape.dims[1]])))
      y = mtf.einsum([h, V], output_shape=mtf.Shape([h.shape.dims[0], V.shape.dims[1]]))
      return {"loss": mtf.reduce_sum(mtf.square(y - features["t"])), "y": y}
    if num_splits == 1:
      out = model_fn({"x": X, "t": T})
      grads = mtf.gradients([out["loss"]], [W, V])
    else:
      grads, out = mtf.serialize_training_step({"x": X, "t": T}, model_fn, X.shape.dims[0], num_splits, [W, V])
    low = mtf.Lowering(g, {m: NumpyMeshImpl(mesh_shape, layout)})
    vals = [np.asarray(low.export_to_tf_tensor(t), np.float64) for t in grads + [out["loss"], out["y"]]]
    return vals, low.counter_totals()
  full, c_full = build(1)
  micro, c_micro = build(4)
  for a, b in zip(micro, full):
    np.testing.assert_allclose(a, b, rtol=1e-5, atol=1e-5)
  if "batch" in layout:
    key = [k for k in c_full if k.startswith("allreduce") and k.endswith("einsum_op")]
    assert key
    for k in key:   # same allreduce volume as the un-split step: the microbatch sums stayed lazy
      assert c_micro.get(k, 0) == c_full[k], (k, c_micro.get(k), c_full[k])
