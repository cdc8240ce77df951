"""The two-level MoE layer (an outer router over expert groups, one inner router per
group) on the oracle backend against the whole layer written out in numpy: both
routing levels with the importance rule between them, the expert FFNs, both
combines.  One processor, and a mesh that splits the groups / the expert groups."""

import numpy as np
import pytest

from mesh_b200 import mtf
from oracle.numpy_mesh_impl import NumpyMeshImpl
from helpers import rel_err, rng

B, L, M, X, Y, F = 4, 16, 8, 2, 2, 12


def _softmax(z):
  z = z - z.max(axis=-1, keepdims=True)
  e = np.exp(z)
  return e / e.sum(axis=-1, keepdims=True)


def _route(raw, capacity, importance=None):
  """Top-2 routing of one group: combine [S, E, C] and the balancing loss."""
  raw = raw.astype(np.float32)
  S, E = raw.shape
  rows = np.arange(S)
  one_hot = lambda idx: np.eye(E, dtype=np.float32)[idx]
  i1 = raw.argmax(-1)
  g1 = raw[rows, i1]
  mask1, proxy = one_hot(i1), raw.copy()
  if importance is not None:
    full = (importance == 1.0).astype(np.float32)
    mask1, g1, proxy = mask1 * full[:, None], g1 * full, proxy * full[:, None]
  without = raw * (1 - mask1)
  i2 = without.argmax(-1)
  g2 = without[rows, i2]
  mask2 = one_hot(i2)
  if importance is not None:
    mask2 = mask2 * (importance > 0)[:, None]
  denom = g1 + g2 + np.float32(1e-9)
  g1, g2 = g1 / denom, g2 / denom
  loss = float((proxy.mean(0) * mask1.mean(0)).mean() * E * E)
  pos1 = (np.cumsum(mask1, 0) - mask1) * mask1
  mask1 = mask1 * (pos1 < capacity)
  count1, flat1, p1 = mask1.sum(0), mask1.sum(1), pos1.sum(1).astype(int)
  pos2 = ((np.cumsum(mask2, 0) - mask2) + count1) * mask2
  mask2 = mask2 * (pos2 < capacity)
  flat2, p2 = mask2.sum(1), pos2.sum(1).astype(int)
  combine = np.zeros((S, E, capacity), np.float32)
  for s_ in range(S):
    if flat1[s_]:
      combine[s_, i1[s_], p1[s_]] += g1[s_] * flat1[s_]
    if flat2[s_]:
      combine[s_, i2[s_], p2[s_]] += g2[s_] * flat2[s_]
  return combine, loss


def _numpy_layer(x, wg_outer, wg_inner, wi, wo, c, h_groups, t, d, nonpadding=None):
  G, S = B, L
  xs = x.reshape(G, S, M)
  routed = [_route(_softmax(xs[g] @ wg_outer), c, None if nonpadding is None else nonpadding[g])
            for g in range(G)]
  combine_x = np.stack([r[0] for r in routed])                       # [G, S, X, C]
  loss_outer = np.mean([r[1] for r in routed])
  expert_in = np.einsum("gsm,gsxc->xgcm", xs, (combine_x != 0).astype(np.float32))
  weight = combine_x.sum(1).transpose(1, 0, 2)                        # [X, G, C]
  importance = 0.5 * ((weight > 0.5).astype(np.float32) + (weight > 0).astype(np.float32))
  inputs_y = expert_in.reshape(X, h_groups, t, M)
  importance = importance.reshape(X, h_groups, t)
  combine_y = np.zeros((X, h_groups, t, Y, d), np.float32)
  inner_losses = []
  for e in range(X):
    for hh in range(h_groups):
      raw = _softmax(inputs_y[e, hh] @ wg_inner[e])
      combine_y[e, hh], lo = _route(raw, d, importance[e, hh])
      inner_losses.append(lo)
  expert_in_y = np.einsum("xhtm,xhtyd->yxhdm", inputs_y, (combine_y != 0).astype(np.float32))
  hidden = np.maximum(np.einsum("yxhdm,yxmf->yxhdf", expert_in_y, wi), 0)
  out_y = np.einsum("yxhdf,yxfn->yxhdn", hidden, wo)
  output_y = np.einsum("yxhdn,xhtyd->xhtn", out_y, combine_y).reshape(X, G, c, M)
  output = np.einsum("xgcn,gsxc->gsn", output_y, combine_x)
  return output.reshape(B, L, M), (loss_outer + np.mean(inner_losses)) * 1e-2


@pytest.mark.parametrize("padded", [False, True])
@pytest.mark.parametrize("mesh_shape,layout", [("all:1", ""), ("all:2", "batch:all;expert_x:all")])
def test_two_level_layer_matches_its_numpy_restatement(mesh_shape, layout, padded):
  r = rng(41)
  mask = (r.uniform(size=(B, L)) > 0.25).astype(np.float32) if padded else None
  x = r.standard_normal((B, L, M)).astype(np.float32)
  wg_outer = (r.standard_normal((M, X)) * 0.8).astype(np.float32)
  wg_inner = (r.standard_normal((X, M, Y)) * 0.8).astype(np.float32)
  wi = (r.standard_normal((Y, X, M, F)) / 3).astype(np.float32)
  wo = (r.standard_normal((Y, X, F, M)) / 3).astype(np.float32)
  g = mtf.Graph()
  m = mtf.Mesh(g, "m")
  Xt = mtf.import_tf_tensor(m, x, "batch:%d,length:%d,d_model:%d" % (B, L, M))
  WGO = mtf.import_tf_tensor(m, wg_outer, "d_model:%d,expert_x_unsplit:%d" % (M, X))
  WGI = mtf.import_tf_tensor(m, wg_inner, "expert_x:%d,d_model:%d,expert_y_unsplit:%d" % (X, M, Y))
  WI = mtf.import_tf_tensor(m, wi, "expert_y:%d,expert_x:%d,d_model:%d,expert_hidden:%d" % (Y, X, M, F))
  WO = mtf.import_tf_tensor(m, wo, "expert_y:%d,expert_x:%d,expert_hidden:%d,d_model:%d" % (Y, X, F, M))
  hparams = mtf.moe.HParams(moe_num_experts=[X, Y], moe_group_size=L, moe_capacity_factor_train=1.0,
                            moe_capacity_factor_second_level=1.0, moe_min_expert_capacity=2,
                            moe_second_policy_train="all")
  NP = None if mask is None else mtf.import_tf_tensor(m, mask, "batch:%d,length:%d" % (B, L))
  out, loss = mtf.moe.transformer_moe_layer_v2(
      Xt, mtf.Dimension("d_model", M), hparams, True, mesh_shape, layout, WGO, WGI, WI, WO,
      nonpadding=NP)
  low = mtf.Lowering(g, {m: NumpyMeshImpl(mesh_shape, layout)})
  got, got_loss = low.export_to_tf_tensor(out), float(low.export_to_tf_tensor(loss))
  c = max(min(L, int(L * 1.0 / X)), 2)
  slots = B * c                      # per expert group
  h_groups, t = slots // L, L        # inner groups of moe_group_size slots
  d = max(min(t, int(t * 1.0 / Y)), 2)
  want, want_loss = _numpy_layer(x, wg_outer, wg_inner, wi, wo, c, h_groups, t, d, mask)
  assert np.abs(want).max() > 0.05
  if padded:
    assert np.all(got[mask == 0] == 0)
  assert rel_err(got, want) < 1e-5
  assert abs(got_loss - want_loss) < 1e-6
  if mesh_shape != "all:1":
    totals = low.counter_totals()
    assert sum(v for k, v in totals.items() if k.startswith("alltoall")) > 0


def test_two_level_layer_argument_errors():
  g = mtf.Graph()
  m = mtf.Mesh(g, "m")
  x = mtf.import_tf_tensor(m, np.zeros((2, 4, 4), np.float32), "batch:2,length:4,d_model:4")
  bad = mtf.moe.HParams(moe_num_experts=4)
  with pytest.raises(ValueError):
    mtf.moe.transformer_moe_layer_v2(x, mtf.Dimension("d_model", 4), bad, True, "all:1", "", None, None, None, None)
  bad = mtf.moe.HParams(moe_num_experts=[2, 2], moe_gating="switch")
  with pytest.raises(ValueError):
    mtf.moe.transformer_moe_layer_v2(x, mtf.Dimension("d_model", 4), bad, True, "all:1", "", None, None, None, None)
