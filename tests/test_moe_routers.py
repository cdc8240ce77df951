"""The further routers of the MoE layer (no-token-left-behind, switch-max, expert
selection) as op chains on the oracle backend, each against its routing rule
written out directly in numpy, on one processor and on a mesh that splits the
groups."""

import numpy as np
import pytest

from mesh_b200 import mtf
from oracle.numpy_mesh_impl import NumpyMeshImpl
from helpers import rel_err, rng

B, L, M, E, H = 4, 16, 8, 4, 12      # 4 groups of 16 tokens


def _softmax(z, axis):
  z = z - z.max(axis=axis, keepdims=True)
  e = np.exp(z)
  return e / e.sum(axis=axis, keepdims=True)


def _layer(gating, mesh_shape, layout, seed, **hp):
  r = rng(seed)
  x = r.standard_normal((B, L, M)).astype(np.float32)
  wg = (r.standard_normal((M, E)) * 0.7).astype(np.float32)
  wi = (r.standard_normal((E, M, H)) / 3).astype(np.float32)
  wo = (r.standard_normal((E, H, M)) / 3).astype(np.float32)
  g = mtf.Graph()
  m = mtf.Mesh(g, "m")
  X = mtf.import_tf_tensor(m, x, "batch:%d,length:%d,d_model:%d" % (B, L, M))
  WG = mtf.import_tf_tensor(m, wg, "d_model:%d,expert_unsplit:%d" % (M, E))
  WI = mtf.import_tf_tensor(m, wi, "experts:%d,d_model:%d,d_ff:%d" % (E, M, H))
  WO = mtf.import_tf_tensor(m, wo, "experts:%d,d_ff:%d,d_model:%d" % (E, H, M))
  hparams = mtf.moe.HParams(moe_gating=gating, moe_group_size=L, moe_capacity_factor_train=1.0,
                            moe_min_expert_capacity=2, **hp)
  out, loss, aux = mtf.moe.transformer_moe_layer_v1(
      X, mtf.Dimension("d_model", M), hparams, True, mesh_shape, layout, WG, WI, WO, return_aux=True)
  low = mtf.Lowering(g, {m: NumpyMeshImpl(mesh_shape, layout)})
  combine = aux["combine_tensor"]
  names = [d.name for d in combine.shape.dims]
  return dict(x=x, wg=wg, wi=wi, wo=wo, out=low.export_to_tf_tensor(out),
              loss=float(low.export_to_tf_tensor(loss)), combine=low.export_to_tf_tensor(combine),
              dispatch=low.export_to_tf_tensor(aux["dispatch_tensor"]), names=names)


def _as_gsec(res):
  """combine / dispatch as [group, token, expert, slot] whatever dim order the router built."""
  order = [res["names"].index(n) for n in ("outer_batch", "batch", "group", "expert_unsplit", "expert_capacity")]
  return (np.transpose(res["combine"], order)[0], np.transpose(res["dispatch"], order)[0])


def _expected_output(res, combine):
  """sum over (expert, slot) of combine x FFN_expert(the token dispatched to the slot)."""
  x = res["x"].reshape(B, L, M)          # one group per batch row
  dispatch = (combine != 0).astype(np.float64)
  expert_in = np.einsum("gsm,gsec->egcm", x, dispatch)
  h = np.maximum(np.einsum("egcm,emh->egch", expert_in, res["wi"]), 0)
  y = np.einsum("egch,ehm->egcm", h, res["wo"])
  return np.einsum("egcm,gsec->gsm", y, combine)


def _balance_loss(raw, first_choice):
  density = np.stack([(first_choice == e).mean(axis=1) for e in range(E)], axis=-1)
  return float((raw.mean(axis=1) * density).mean() * E * E) * 1e-2


MESHES = [("all:1", ""), ("all:2", "batch:all;experts:all")]


@pytest.mark.parametrize("mesh_shape,layout", MESHES)
def test_ntlb_routes_leftover_tokens_to_their_next_choices(mesh_shape, layout):
  res = _layer("ntlb", mesh_shape, layout, 11, moe_ntlb_top_k=3)
  combine, dispatch = _as_gsec(res)
  C = combine.shape[-1]
  raw = _softmax(res["x"].reshape(B, L, M) @ res["wg"], -1)
  want = np.zeros_like(combine)
  for g in range(B):
    ranked = np.argsort(-raw[g], axis=-1, kind="stable")[:, :3]
    taken = np.zeros(E, int)
    unrouted = np.ones(L, bool)
    for i in range(3):
      arrivals = taken.copy()
      placed_now = np.zeros(E, int)
      for s in range(L):
        if not unrouted[s]:
          continue
        e = ranked[s, i]
        arrivals[e] += 1                     # every candidate counts, placed or not
        if arrivals[e] <= C:
          want[g, s, e, arrivals[e] - 1] = raw[g, s, e]
          unrouted[s] = False
          placed_now[e] += 1
      taken += placed_now
  np.testing.assert_allclose(combine, want, rtol=1e-5, atol=1e-7)
  np.testing.assert_array_equal(dispatch, (want != 0).astype(np.float32))
  assert (want != 0).sum(axis=(2, 3)).max() == 1                 # a token is routed once at most
  # the loss averages over the three ranked choices as well (the mask keeps its k dim)
  ranked_all = np.argsort(-raw, axis=-1, kind="stable")[..., :3]                   # [g, s, i]
  density = np.stack([(ranked_all == e).mean(axis=1) for e in range(E)], axis=-1)   # [g, i, e]
  want_loss = float((raw.mean(axis=1)[:, None, :] * density).mean() * E * E) * 1e-2
  assert abs(res["loss"] - want_loss) < 1e-6
  assert rel_err(res["out"].reshape(B, L, M), _expected_output(res, want)) < 1e-5


@pytest.mark.parametrize("mesh_shape,layout", MESHES)
def test_switch_max_keeps_the_highest_gates_of_an_over_full_expert(mesh_shape, layout):
  res = _layer("switch_max", mesh_shape, layout, 12)
  combine, dispatch = _as_gsec(res)
  C = combine.shape[-1]
  raw = _softmax(res["x"].reshape(B, L, M) @ res["wg"], -1)
  choice = raw.argmax(-1)
  want = np.zeros_like(combine)
  for g in range(B):
    for e in range(E):
      score = np.where(choice[g] == e, raw[g, :, e], 0.0)
      keep = np.argsort(-score, kind="stable")[:C]
      for c, s in enumerate(keep):
        want[g, s, e, c] = score[s]
  np.testing.assert_allclose(combine, want, rtol=1e-5, atol=1e-7)
  np.testing.assert_array_equal(dispatch, (want != 0).astype(np.float32))
  assert abs(res["loss"] - _balance_loss(raw, choice)) < 1e-6
  assert rel_err(res["out"].reshape(B, L, M), _expected_output(res, want)) < 1e-5


@pytest.mark.parametrize("mesh_shape,layout", MESHES)
def test_expert_selection_lets_every_expert_take_its_best_tokens(mesh_shape, layout):
  res = _layer("expert_selection", mesh_shape, layout, 13)
  combine, dispatch = _as_gsec(res)
  C = combine.shape[-1]
  prob = _softmax(res["x"].reshape(B, L, M) @ res["wg"], 1)      # over the tokens of a group
  taken = np.zeros_like(combine)
  for g in range(B):
    for e in range(E):
      for c, s in enumerate(np.argsort(-prob[g, :, e], kind="stable")[:C]):
        taken[g, s, e, c] = 1.0
  times = np.maximum(taken.sum(axis=(2, 3), keepdims=True), 1.0)
  want = taken * prob[:, :, :, None] / times
  np.testing.assert_allclose(combine, want, rtol=1e-5, atol=1e-8)
  np.testing.assert_array_equal(dispatch, taken.astype(np.float32))
  mean_prob = prob.mean(-1)
  assert abs(res["loss"] - float((mean_prob * mean_prob * L).mean() * L) * 1e-2) < 1e-6
  assert rel_err(res["out"].reshape(B, L, M), _expected_output(res, want)) < 1e-5


def test_unknown_router_is_refused():
  with pytest.raises(ValueError):
    _layer("no_such_router", "all:1", "", 1)


def _v1(gating, seed, nonpadding=None, **hp):
  """The one-level layer on one processor; returns inputs, combine [g, s, e, c], loss, aux."""
  r = rng(seed)
  x = r.standard_normal((B, L, M)).astype(np.float32)
  wg = (r.standard_normal((M, E)) * 0.7).astype(np.float32)
  wi = (r.standard_normal((E, M, H)) / 3).astype(np.float32)
  wo = (r.standard_normal((E, H, M)) / 3).astype(np.float32)
  g = mtf.Graph()
  m = mtf.Mesh(g, "m")
  X = mtf.import_tf_tensor(m, x, "batch:%d,length:%d,d_model:%d" % (B, L, M))
  WG = mtf.import_tf_tensor(m, wg, "d_model:%d,expert_unsplit:%d" % (M, E))
  WI = mtf.import_tf_tensor(m, wi, "experts:%d,d_model:%d,d_ff:%d" % (E, M, H))
  WO = mtf.import_tf_tensor(m, wo, "experts:%d,d_ff:%d,d_model:%d" % (E, H, M))
  NP = None if nonpadding is None else mtf.import_tf_tensor(m, nonpadding, "batch:%d,length:%d" % (B, L))
  hparams = mtf.moe.HParams(moe_gating=gating, moe_group_size=L, moe_capacity_factor_train=1.0,
                            moe_min_expert_capacity=2, moe_second_policy_train="all",
                            moe_use_fused_kernels=False, **hp)
  out, loss, aux = mtf.moe.transformer_moe_layer_v1(
      X, mtf.Dimension("d_model", M), hparams, True, "all:1", "", WG, WI, WO, return_aux=True,
      nonpadding=NP)
  low = mtf.Lowering(g, {m: NumpyMeshImpl("all:1", "")})
  names = [d.name for d in aux["combine_tensor"].shape.dims]
  order = [names.index(n) for n in ("outer_batch", "batch", "group", "expert_unsplit", "expert_capacity")]
  combine = np.transpose(low.export_to_tf_tensor(aux["combine_tensor"]), order)[0]
  res = dict(x=x, wg=wg, wi=wi, wo=wo, out=low.export_to_tf_tensor(out))
  return res, combine, float(low.export_to_tf_tensor(loss)), {k: low.export_to_tf_tensor(v) for k, v in aux.items()}


def test_padding_is_not_routed_by_top_2_gating():
  from test_moe_v2 import _route
  mask = (rng(21).uniform(size=(B, L)) > 0.3).astype(np.float32)
  res, combine, loss, _ = _v1("top_2", 22, nonpadding=mask)
  raw = _softmax(res["x"] @ res["wg"], -1)
  routed = [_route(raw[g], combine.shape[-1], mask[g]) for g in range(B)]
  want = np.stack([r[0] for r in routed])
  np.testing.assert_allclose(combine, want, rtol=1e-5, atol=1e-7)
  assert np.all(combine[mask == 0] == 0) and np.any(combine[mask == 1] != 0)
  assert abs(loss - np.mean([r[1] for r in routed]) * 1e-2) < 1e-6
  assert rel_err(res["out"], _expected_output(res, want)) < 1e-5
  assert np.all(res["out"][mask == 0] == 0)            # a padded position gets no expert output


def test_padding_is_not_routed_by_switch_gating():
  mask = (rng(23).uniform(size=(B, L)) > 0.3).astype(np.float32)
  res, combine, loss, _ = _v1("switch", 24, nonpadding=mask)
  raw = _softmax(res["x"] @ res["wg"], -1)
  C = combine.shape[-1]
  want = np.zeros_like(combine)
  for g in range(B):
    seen = np.zeros(E, int)
    for s in range(L):
      if mask[g, s] == 0:
        continue
      e = raw[g, s].argmax()
      if seen[e] < C:
        want[g, s, e, seen[e]] = raw[g, s, e]
      seen[e] += 1
  np.testing.assert_allclose(combine, want, rtol=1e-5, atol=1e-7)
  # the loss as the reference forms it (moe.py:1226-1236): the fraction of positions choosing
  # an expert counts padding too, and the group's mean gates are scaled by the group's
  # share of real positions (the mask meets the already averaged gates and broadcasts)
  choice = raw.argmax(-1)
  density = np.stack([(choice == e).mean(axis=1) for e in range(E)], axis=-1)
  proxy = raw.mean(axis=1) * mask.mean(axis=1, keepdims=True)
  assert abs(loss - float((proxy * density).mean() * E * E) * 1e-2) < 1e-6


def test_sampled_switch_routing():
  # temperature 0: the draw is the argmax
  _, combine_argmax, loss_argmax, _ = _v1("switch", 25)
  _, combine_t0, loss_t0, _ = _v1("switch", 25, moe_switch_policy_train="sample", moe_switch_temperature=0.0)
  np.testing.assert_array_equal(combine_t0, combine_argmax)
  assert loss_t0 == loss_argmax
  # temperature 1: every routed position carries the probability of the expert drawn for it,
  # experts other than the most probable one are drawn too, and the draw repeats (seeded by name)
  res, combine, _, aux = _v1("switch", 25, moe_switch_policy_train="sample")
  raw = _softmax(res["x"] @ res["wg"], -1)
  index = aux["index_1"].reshape(B, L)
  assert index.min() >= 0 and index.max() < E
  assert (index != raw.argmax(-1)).mean() > 0.1
  for g, s in zip(*np.nonzero(combine.sum(axis=(2, 3)))):
    e = index[g, s]
    assert abs(combine[g, s, e].sum() - raw[g, s, e]) < 1e-6 and combine[g, s].sum() == combine[g, s, e].sum()
  _, again, _, _ = _v1("switch", 25, moe_switch_policy_train="sample")
  np.testing.assert_array_equal(again, combine)


def test_padding_with_the_further_routers():
  mask = (rng(27).uniform(size=(B, L)) > 0.3).astype(np.float32)
  # no token left behind: padded positions are never candidates
  res, combine, _, _ = _v1("ntlb", 28, nonpadding=mask, moe_ntlb_top_k=3)
  raw = _softmax(res["x"] @ res["wg"], -1)
  C = combine.shape[-1]
  want = np.zeros_like(combine)
  for g in range(B):
    ranked = np.argsort(-raw[g], axis=-1, kind="stable")[:, :3]
    taken, unrouted = np.zeros(E, int), mask[g] == 1
    for i in range(3):
      arrivals, placed_now = taken.copy(), np.zeros(E, int)
      for s in range(L):
        if unrouted[s]:
          e = ranked[s, i]
          arrivals[e] += 1
          if arrivals[e] <= C:
            want[g, s, e, arrivals[e] - 1] = raw[g, s, e]
            unrouted[s] = False
            placed_now[e] += 1
      taken += placed_now
  np.testing.assert_allclose(combine, want, rtol=1e-5, atol=1e-7)
  assert np.all(combine[mask == 0] == 0)
  # switch-max: an expert ranks the real positions that chose it
  res, combine, _, _ = _v1("switch_max", 29, nonpadding=mask)
  raw = _softmax(res["x"] @ res["wg"], -1)
  choice = raw.argmax(-1)
  want = np.zeros_like(combine)
  for g in range(B):
    for e in range(E):
      score = np.where((choice[g] == e) & (mask[g] == 1), raw[g, :, e], 0.0)
      for c, s in enumerate(np.argsort(-score, kind="stable")[:C]):
        want[g, s, e, c] = score[s]
  np.testing.assert_allclose(combine, want, rtol=1e-5, atol=1e-7)
  # expert selection: padding is out of the softmax over the group
  res, combine, loss, _ = _v1("expert_selection", 30, nonpadding=mask)
  logits = res["x"] @ res["wg"] + (mask == 0)[..., None] * np.float32(-1e9)
  prob = _softmax(logits, 1)
  taken = np.zeros_like(combine)
  for g in range(B):
    for e in range(E):
      for c, s in enumerate(np.argsort(-prob[g, :, e], kind="stable")[:C]):
        taken[g, s, e, c] = 1.0
  want = taken * prob[:, :, :, None] / np.maximum(taken.sum(axis=(2, 3), keepdims=True), 1.0)
  np.testing.assert_allclose(combine, want, rtol=1e-5, atol=1e-8)
  assert np.all(combine[mask == 0] == 0)
  mean_prob = prob.mean(-1) * mask
  want_loss = float((mean_prob * mean_prob * mask.sum(axis=1, keepdims=True)).mean() * L) * 1e-2
  assert abs(loss - want_loss) < 1e-6


def test_second_place_loss_of_top_2_gating():
  res, _, loss_plain, aux = _v1("top_2", 31)
  _, _, loss_both, _ = _v1("top_2", 31, moe_use_second_place_loss=True)
  raw = _softmax(res["x"] @ res["wg"], -1).astype(np.float32)
  i1 = raw.argmax(-1)
  without = raw * (1 - np.eye(E, dtype=np.float32)[i1])
  i2 = without.argmax(-1)
  density_2 = np.stack([(i2 == e).mean(axis=1) for e in range(E)], axis=-1)
  proxy_2 = (without / (without.sum(-1, keepdims=True) + 1e-9)).mean(axis=1)
  second = float((proxy_2 * density_2).mean() * E * E)
  assert abs((loss_both - loss_plain) - 0.5 * second * 1e-2) < 1e-6
  # the fused kernels do not form it
  with pytest.raises(ValueError):
    g = mtf.Graph()
    m = mtf.Mesh(g, "m")
    X = mtf.import_tf_tensor(m, res["x"], "batch:%d,length:%d,d_model:%d" % (B, L, M))
    WG = mtf.import_tf_tensor(m, res["wg"], "d_model:%d,expert_unsplit:%d" % (M, E))
    WI = mtf.import_tf_tensor(m, res["wi"], "experts:%d,d_model:%d,d_ff:%d" % (E, M, H))
    WO = mtf.import_tf_tensor(m, res["wo"], "experts:%d,d_ff:%d,d_model:%d" % (E, H, M))
    mtf.moe.transformer_moe_layer_v1(X, mtf.Dimension("d_model", M),
                                     mtf.moe.HParams(moe_use_second_place_loss=True, moe_group_size=L,
                                                     moe_second_policy_train="all"),
                                     True, "all:1", "", WG, WI, WO)
