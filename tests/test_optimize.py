"""Adafactor and SGD as graph operations on the CPU oracle backend, against a
direct numpy restatement of mesh_tensorflow/optimize.py:294-379; variables and
optimizer slots persist on the backend across lowerings; checkpoint round trip."""

import os

import numpy as np
import pytest

from mesh_b200 import mtf
from oracle.numpy_mesh_impl import NumpyMeshImpl
from helpers import rng


def adafactor_step_numpy(w, g, state, lr, decay, factored, eps1=1e-30, eps2=1e-3, clip=1.0):
  g = g.astype(np.float64)
  g2 = g * g + eps1
  scale = max(np.sqrt(np.mean(w.astype(np.float64) ** 2)), eps2) * lr
  if factored:
    # the two largest dims are reduced: vr keeps dim 1's complement, vc dim 0's
    vr = state.get("vr", np.zeros(w.shape[1])) * decay + g2.mean(0) * (1 - decay)
    vc = state.get("vc", np.zeros(w.shape[0])) * decay + g2.mean(1) * (1 - decay)
    state["vr"], state["vc"] = vr, vc
    return vr, vc, scale, g
  v = state.get("v", np.zeros(w.shape)) * decay + g2 * (1 - decay)
  state["v"] = v
  x = g / np.sqrt(v)
  x = x / max(1.0, np.sqrt(np.mean(x * x)) / clip)
  return w - x * scale


@pytest.mark.parametrize("mesh_shape,layout", [("all:1", ""), ("a:2,b:2", "d_model:a;d_ff:b")])
def test_adafactor_unfactored_matches_numpy(mesh_shape, layout):
  r = rng(91)
  w0 = (r.standard_normal((8, 12)) / 3).astype(np.float32)
  x = r.standard_normal((16, 8)).astype(np.float32)
  t = r.standard_normal((16, 12)).astype(np.float32)
  g = mtf.Graph()
  m = mtf.Mesh(g, "m")
  X = mtf.import_tf_tensor(m, x, "batch:16,d_model:8", dtype=mtf.float32)
  T = mtf.import_tf_tensor(m, t, "batch:16,d_ff:12", dtype=mtf.float32)
  W = mtf.get_variable(m, "w", "d_model:8,d_ff:12", initial_value=w0)
  loss = mtf.reduce_sum(mtf.square(mtf.einsum([X, W], output_shape="batch:16,d_ff:12") - T))
  dW, = mtf.gradients([loss], [W])
  opt = mtf.optimize.AdafactorOptimizer(learning_rate=0.05, decay_rate=0.8, min_dim_size_to_factor=128)
  opt.apply_grads([dW], [W])
  impl = NumpyMeshImpl(mesh_shape, layout)
  ref, state, losses = w0.astype(np.float64), {}, []
  for _ in range(3):
    low = mtf.Lowering(g, {m: impl})
    losses.append(float(np.asarray(low.export_to_tf_tensor(loss))))
    grad = 2 * x.astype(np.float64).T @ (x.astype(np.float64) @ ref - t)
    ref = adafactor_step_numpy(ref, grad, state, 0.05, 0.8, False)
  assert losses[2] < losses[1] < losses[0]
  # weights and slots stayed on the backend; bring them to the host now
  np.testing.assert_array_equal(W.operation.get_master(), w0)
  low.copy_slices_to_masters()
  np.testing.assert_allclose(W.operation.get_master(), ref, rtol=2e-4, atol=2e-5)
  slot = [v for v in g.all_variables if v.name.endswith("_slot_v")][0]
  np.testing.assert_allclose(slot.get_master(), state["v"], rtol=2e-4, atol=1e-7)


def test_adafactor_factored_and_momentum():
  r = rng(92)
  w0 = (r.standard_normal((8, 12)) / 3).astype(np.float32)
  grad = r.standard_normal((8, 12)).astype(np.float32)
  g = mtf.Graph()
  m = mtf.Mesh(g, "m")
  W = mtf.get_variable(m, "w", "d_model:8,d_ff:12", initial_value=w0)
  G_ = mtf.import_tf_tensor(m, grad, "d_model:8,d_ff:12", dtype=mtf.float32)
  opt = mtf.optimize.AdafactorOptimizer(learning_rate=0.1, decay_rate=0.5, min_dim_size_to_factor=4,
                                        beta1=0.9, copy_to_master=True)
  opt.apply_grads([G_], [W])
  mtf.Lowering(g, {m: NumpyMeshImpl("all:2", "d_ff:all")})
  g64 = grad.astype(np.float64)
  g2 = g64 * g64 + 1e-30
  # d0 = d_ff (largest), d1 = d_model: vr has shape var - d0 = [d_model], vc = var - d1 = [d_ff]
  vr = g2.mean(1) * 0.5
  vc = g2.mean(0) * 0.5
  r_factor = 1 / np.sqrt(vr / vr.mean())
  c_factor = 1 / np.sqrt(vc)
  xx = g64 * r_factor[:, None] * c_factor[None, :]
  xx = xx / max(1.0, np.sqrt(np.mean(xx * xx)))
  scale = max(np.sqrt(np.mean(w0.astype(np.float64) ** 2)), 1e-3) * 0.1
  new_m = xx * scale * 0.1
  np.testing.assert_allclose(W.operation.get_master(), w0 - new_m, rtol=2e-4, atol=2e-6)
  names = sorted(v.name for v in g.all_variables)
  assert names == ["w", "w_slot_m", "w_slot_vc", "w_slot_vr"]


def test_checkpoint_round_trip(tmp_path):
  r = rng(93)
  w0 = r.standard_normal((4, 6)).astype(np.float32)
  g = mtf.Graph()
  m = mtf.Mesh(g, "m")
  W = mtf.get_variable(m, "w", "a:4,b:6", initial_value=w0)
  G_ = mtf.import_tf_tensor(m, np.ones((4, 6), np.float32), "a:4,b:6", dtype=mtf.float32)
  mtf.optimize.SgdOptimizer(0.5).apply_grads([G_], [W])
  impl = NumpyMeshImpl("all:2", "a:all")
  low = mtf.Lowering(g, {m: impl})
  path = os.path.join(str(tmp_path), "ckpt.npz")
  mtf.save_checkpoint(path, [W], lowering=low)           # copies slices to masters first
  np.testing.assert_allclose(W.operation.get_master(), w0 - 0.5)
  W.operation.assign_to_master(np.zeros((4, 6), np.float32))
  mtf.restore_checkpoint(path, [W])
  low = mtf.Lowering(g, {m: impl})                       # lays the restored master out, then steps
  low.copy_slices_to_masters()
  np.testing.assert_allclose(W.operation.get_master(), w0 - 1.0)
  with pytest.raises(KeyError):
    mtf.restore_checkpoint(path, [mtf.get_variable(m, "other", "a:4", initial_value=np.zeros(4, np.float32))])
