"""The oracle itself: reference-held vectors, self-consistency across meshes,
the two MoE formulations against each other, allreduce association order."""

import json
import os

import numpy as np
import pytest

from mesh_b200 import mtf
from oracle import moe_spec
from oracle.numpy_mesh_impl import NumpyMeshImpl, allreduce_ring, allreduce_single_shard
from oracle.numpy_ops import Arr, NumpyOps, round_to_bf16
from helpers import rel_err, rng

GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.json")))


def _lower(build, mesh_shape, layout):
  g = mtf.Graph()
  mesh = mtf.Mesh(g, "my_mesh")
  outs = build(mesh)
  low = mtf.Lowering(g, {mesh: NumpyMeshImpl(mesh_shape, layout)})
  return [low.export_to_tf_tensor(t) for t in outs], low


def test_golden_nth_largest():
  v = GOLDEN["nth_largest"]

  def build(mesh):
    x = mtf.import_tf_tensor(mesh, np.array(v["inputs"], dtype=np.int32), v["shape"])
    return [mtf.nth_largest_element(x, v["n"], x.shape.get_dim_by_name(v["reduced_dim"]))]
  (out,), _ = _lower(build, v["mesh"], v["layout"])
  np.testing.assert_array_equal(out, v["expected"])


def test_golden_nth_smallest():
  v = GOLDEN["nth_smallest_second_dim"]

  def build(mesh):
    x = mtf.import_tf_tensor(mesh, np.array(v["inputs"], dtype=np.int32), v["shape"])
    return [mtf.nth_smallest_element(x, v["n"], x.shape.get_dim_by_name(v["reduced_dim"]))]
  (out,), _ = _lower(build, v["mesh"], v["layout"])
  np.testing.assert_array_equal(out, v["expected"])


def test_golden_top_k_on_split_dim():
  v = GOLDEN["top_k"]

  def build(mesh):
    x = mtf.import_tf_tensor(mesh, np.array(v["inputs"], dtype=np.float32), v["shape"])
    return list(mtf.top_k(x, x.shape.get_dim_by_name(v["reduced_dim"]), mtf.Dimension("k", v["k"]))) + [x]
  (values, indices, x), _ = _lower(build, v["mesh"], v["layout"])
  np.testing.assert_array_equal(x, v["inputs"])
  np.testing.assert_array_equal(values, v["expected_values"])
  np.testing.assert_array_equal(indices, v["expected_indices"])


def golden_top_k_gradient(impl):
  """The reference's pinned top-k gradient (ops_test.py:606-611, 636-640)."""
  v = GOLDEN["top_k"]
  g = mtf.Graph()
  mesh = mtf.Mesh(g, "my_mesh")
  x = mtf.import_fully_replicated(mesh, np.array(v["inputs"], dtype=np.float32), v["shape"])
  d_values = mtf.import_tf_tensor(mesh, np.array(v["d_values"], dtype=np.float32), "b:2,k:2")
  values, _ = mtf.top_k(x, x.shape.get_dim_by_name(v["reduced_dim"]), mtf.Dimension("k", v["k"]))
  d_inputs, = mtf.gradients([values], [x], [d_values])
  low = mtf.Lowering(g, {mesh: impl})
  return low.export_to_tf_tensor(d_inputs), v["expected_d_inputs"]


def golden_recompute_grad(impl):
  """The reference's pinned recompute_grad case (ops_test.py:645-671)."""
  v = GOLDEN["recompute_grad"]
  g = mtf.Graph()
  mesh = mtf.Mesh(g, "my_mesh")
  x = mtf.import_fully_replicated(mesh, np.array(v["x"], dtype=np.float32), v["shape"])
  dy = mtf.import_tf_tensor(mesh, np.array(v["dy"], dtype=np.float32), v["shape"])
  y = mtf.recompute_grad(lambda t: t * t + t, [x])
  dx, = mtf.gradients([y], [x], [dy])
  low = mtf.Lowering(g, {mesh: impl})
  return (low.export_to_tf_tensor(y), low.export_to_tf_tensor(dx)), (v["expected_y"], v["expected_dx"])


def test_golden_top_k_gradient():
  v = GOLDEN["top_k"]
  got, expected = golden_top_k_gradient(NumpyMeshImpl(v["mesh"], v["layout"]))
  np.testing.assert_array_equal(got, expected)


def test_golden_recompute_grad():
  v = GOLDEN["recompute_grad"]
  got, expected = golden_recompute_grad(NumpyMeshImpl(v["mesh"], v["layout"]))
  np.testing.assert_array_equal(got[0], expected[0])
  np.testing.assert_array_equal(got[1], expected[1])


def test_top_k_operation_large_k_on_split_dim():
  """k >= 5 takes the TopKOperation path: local top-k, allconcat, global top-k."""
  x = rng(1).standard_normal((4, 16)).astype(np.float32)

  def build(mesh):
    t = mtf.import_tf_tensor(mesh, x, "a:4,b:16")
    return list(mtf.top_k(t, t.shape.dims[1], mtf.Dimension("k", 6)))
  (v, i), low = _lower(build, "all:4", "b:all")
  order = np.argsort(-x, axis=1, kind="stable")[:, :6]
  np.testing.assert_array_equal(i, order)
  np.testing.assert_array_equal(v, np.take_along_axis(x, order, 1))
  assert any(k.startswith("output/TopKOperation") for k in low.counter_totals())


def test_bf16_rounding_is_nearest_even():
  x = np.array([1.0, 1.00390625, 1.01171875, -1.00390625, 3.0e38, 1e-40, 0.0], dtype=np.float32)
  got = round_to_bf16(x)
  assert got[0] == 1.0
  assert got[1] == 1.0            # exactly halfway between 1.0 and 1.0078125 -> even mantissa
  assert got[2] == np.float32(1.015625)
  assert got[3] == -1.0
  assert np.isfinite(got[4]) and got[6] == 0.0
  assert round_to_bf16(np.float32(2.5)).shape == ()


def test_allreduce_association_order():
  """n = 4 single shard is (x0 + x1) + (x2 + x3) (placement_mesh_impl.py:378-397)."""
  vals = [np.float32(1e8), np.float32(1.0), np.float32(-1e8), np.float32(1.0)]
  got = allreduce_single_shard([np.array([v]) for v in vals], "SUM", mtf.float32)[0]
  assert got == (vals[0] + vals[1]) + (vals[2] + vals[3])
  # 5 members: (x0 + x1 + x2) + (x3 + x4) with the right sum built right-to-left
  v5 = [np.float32(x) for x in (1e8, 1.0, 2.0, -1e8, 3.0)]
  got = allreduce_single_shard([np.array([v]) for v in v5], "SUM", mtf.float32)[0]
  assert got == ((v5[0] + v5[1]) + v5[2]) + (v5[3] + v5[4])
  # sharded path rotates the member list per shard; all members get identical results
  r = rng(2)
  xs = [Arr(r.standard_normal(2048).astype(np.float32), mtf.float32) for _ in range(4)]
  out = allreduce_ring(xs, "SUM")
  for o in out[1:]:
    np.testing.assert_array_equal(o.a, out[0].a)
  assert rel_err(out[0].a, sum(x.a.astype(np.float64) for x in xs)) < 1e-6


def _ffn(mesh_shape, layout, dtype):
  r = rng(3)
  x = r.standard_normal((4, 8, 16)).astype(np.float32)
  wi = (r.standard_normal((16, 32)) / 4).astype(np.float32)
  wo = (r.standard_normal((32, 16)) / 6).astype(np.float32)

  def build(mesh):
    X = mtf.import_tf_tensor(mesh, x, "batch:4,length:8,d_model:16", dtype=dtype)
    WI = mtf.import_tf_tensor(mesh, wi, "d_model:16,d_ff:32", dtype=dtype)
    WO = mtf.import_tf_tensor(mesh, wo, "d_ff:32,d_model:16", dtype=dtype)
    return [mtf.layers.dense_relu_dense(X, mtf.Dimension("d_ff", 32), wi=WI, wo=WO)]
  (y,), low = _lower(build, mesh_shape, layout)
  return y, low, (x, wi, wo)


def test_ffn_same_on_every_mesh():
  y1, _, (x, wi, wo) = _ffn("", "", mtf.float32)
  ref = np.maximum(x.astype(np.float64) @ wi, 0) @ wo
  assert rel_err(y1, ref) < 1e-6
  for mesh_shape, layout in [("rows:2,cols:4", "batch:rows;d_ff:cols"), ("all:4", "d_model:all"),
                             ("all:2", "length:all")]:
    y, low, _ = _ffn(mesh_shape, layout, mtf.float32)
    assert rel_err(y, y1) < 1e-6
  _, low, _ = _ffn("rows:2,cols:4", "batch:rows;d_ff:cols", mtf.float32)
  assert low.counter_totals()["allreduce/[1]/einsum_op"] == 4 * 8 * 16 // 2 * 8


def test_lazy_allreduce_adds_before_reducing():
  x = rng(4).standard_normal((8, 16)).astype(np.float32)
  w = rng(5).standard_normal((16, 4)).astype(np.float32)

  def build(mesh):
    X = mtf.import_tf_tensor(mesh, x, "b:8,k:16")
    W = mtf.import_tf_tensor(mesh, w, "k:16,n:4")
    y = mtf.einsum([X, W], "b:8,n:4")
    return [y + y]
  (out,), low = _lower(build, "all:4", "k:all")
  assert rel_err(out, 2 * (x.astype(np.float64) @ w)) < 1e-6
  assert low.counter_totals()["allreduce/[0]/einsum_op"] == 8 * 4 * 4   # one allreduce, not two


def _moe(mesh_shape, fused, policy="all", noise=None):
  r = rng(6)
  b, l, d, f, e = 8, 32, 16, 32, 8
  x = r.standard_normal((b, l, d)).astype(np.float32)
  wg = (r.standard_normal((d, e)) / 4).astype(np.float32)
  wi = (r.standard_normal((e, d, f)) / 4).astype(np.float32)
  wo = (r.standard_normal((e, f, d)) / 6).astype(np.float32)
  layout = "batch:all;experts:all"
  aux_out = {}

  def build(mesh):
    X = mtf.import_tf_tensor(mesh, x, "batch:8,length:32,d_model:16", dtype=mtf.bfloat16)
    WG = mtf.import_tf_tensor(mesh, wg, "d_model:16,expert_unsplit:8", dtype=mtf.float32)
    WI = mtf.import_tf_tensor(mesh, wi, "experts:8,d_model:16,d_ff:32", dtype=mtf.bfloat16)
    WO = mtf.import_tf_tensor(mesh, wo, "experts:8,d_ff:32,d_model:16", dtype=mtf.bfloat16)
    N = None
    if noise is not None:
      N = mtf.import_tf_tensor(mesh, noise, "batch:8,length:32", dtype=mtf.float32)
    hp = mtf.moe.HParams(moe_group_size=32, moe_second_policy_train=policy,
                         moe_second_threshold_train=0.3, moe_use_fused_kernels=fused)
    out, loss, aux = mtf.moe.transformer_moe_layer_v1(
        X, mtf.Dimension("d_model", d), hp, True, mesh_shape, layout, WG, WI, WO,
        second_noise=N, return_aux=True)
    keys = sorted(k for k in aux if k != "raw_gates")
    aux_out["keys"] = keys
    return [out, loss] + [aux[k] for k in keys]
  outs, low = _lower(build, mesh_shape, layout)
  return outs[0], outs[1], dict(zip(aux_out["keys"], outs[2:])), low


@pytest.mark.parametrize("policy", ["all", "none", "threshold", "random"])
def test_moe_unfused_graph_equals_spec(policy):
  noise = rng(7).random((8, 32)).astype(np.float32) if policy == "random" else None
  o_u, l_u, a_u, _ = _moe("all:1", False, policy, noise)
  o_f, l_f, a_f, _ = _moe("all:1", True, policy, noise)
  for k in ("index_1", "index_2", "position_1", "position_2"):
    np.testing.assert_array_equal(a_u[k], a_f[k], err_msg=k)
  for k in ("gate_1", "gate_2"):
    assert np.max(np.abs(a_u[k] - a_f[k])) < 1e-6
  assert rel_err(o_f, o_u) < 1e-6
  assert abs(float(l_u) - float(l_f)) < 1e-6


@pytest.mark.parametrize("fused", [True, False])
def test_moe_same_on_every_mesh(fused):
  o1, l1, a1, _ = _moe("all:1", fused)
  for n in (2, 4, 8):
    o, l, a, low = _moe("all:%d" % n, fused)
    np.testing.assert_array_equal(o, o1)
    for k in a1:
      np.testing.assert_array_equal(a[k], a1[k])
    assert abs(float(l) - float(l1)) < 1e-7
    assert low.counter_totals()["alltoall/0/reshape_op"] == 2 * 8 * 8 * 5 * 16


def test_moe_overflow_drops_tokens():
  """All tokens prefer expert 0: only `capacity` keep their first choice."""
  s, e, cap = 16, 4, 5
  raw = np.tile(np.array([0.7, 0.2, 0.06, 0.04], dtype=np.float32), (1, s, 1))
  r = moe_spec.gating_from_raw(raw, cap)
  np.testing.assert_array_equal(r["position_1"][0], np.arange(s))
  assert r["keep_1"][0].sum() == cap and r["keep_2"][0].sum() == cap
  np.testing.assert_array_equal(r["position_2"][0], np.arange(s))   # expert 1 had no first choices
  x = rng(8).standard_normal((1, s, 8)).astype(np.float32)
  d = moe_spec.dispatch(x, r["index_1"], r["index_2"], r["position_1"], r["position_2"],
                        r["gate_1"], r["gate_2"], e, cap)
  np.testing.assert_array_equal(d[0, 0], x[0, :cap])
  np.testing.assert_array_equal(d[0, 1], x[0, :cap])
  assert not d[0, 2:].any()


def test_second_choice_positions_follow_first_choice_counts():
  raw = np.zeros((1, 6, 3), dtype=np.float32)
  raw[0, :, :] = [[.6, .3, .1], [.3, .6, .1], [.6, .3, .1], [.1, .6, .3], [.6, .1, .3], [.3, .1, .6]]
  r = moe_spec.gating_from_raw(raw, 2)
  np.testing.assert_array_equal(r["index_1"][0], [0, 1, 0, 1, 0, 2])
  np.testing.assert_array_equal(r["position_1"][0], [0, 0, 1, 1, 2, 0])
  np.testing.assert_array_equal(r["keep_1"][0], [1, 1, 1, 1, 0, 1])
  np.testing.assert_array_equal(r["index_2"][0], [1, 0, 1, 2, 2, 0])
  # kept first-choice counts: e0=2, e1=2, e2=1 -> second choices start there
  np.testing.assert_array_equal(r["position_2"][0], [2, 2, 3, 1, 2, 3])
  np.testing.assert_array_equal(r["keep_2"][0], [0, 0, 0, 1, 0, 0])


def test_attention_causal_mask():
  r = rng(9)
  x = r.standard_normal((2, 8, 16)).astype(np.float32)

  def build(mesh):
    X = mtf.import_tf_tensor(mesh, x, "batch:2,length:8,d_model:16")
    heads, kv = mtf.Dimension("heads", 2), mtf.Dimension("d_kv", 4)
    ws = mtf.layers.WeightSource(seed=3)
    params = mtf.layers.multihead_attention_params(mesh, heads, X.shape.dims[-1], kv, ws, mtf.float32)
    pos = mtf.mtf_range(mesh, X.shape.dims[1], mtf.float32)
    mask = mtf.layers.attention_mask_autoregressive(pos)
    return [mtf.layers.multihead_attention(X, None, mask, kv, heads, params=params)] + params
  (y, wq, wk, wv, wo), _ = _lower(build, "all:2", "heads:all")
  q = np.einsum("bld,hdk->bhlk", x, wq)
  k = np.einsum("bld,hdk->bhlk", x, wk)
  v = np.einsum("bld,hdk->bhlk", x, wv)
  logits = np.einsum("bhlk,bhmk->bhlm", q, k) + np.triu(np.full((8, 8), -1e9), 1)
  p = np.exp(logits - logits.max(-1, keepdims=True))
  p /= p.sum(-1, keepdims=True)
  ref = np.einsum("bhlk,hdk->bld", np.einsum("bhlm,bhmk->bhlk", p, v), wo)
  assert rel_err(y, ref) < 1e-5


def test_variable_master_and_slices_round_trip():
  w0 = rng(10).standard_normal((8, 6)).astype(np.float32)
  g = mtf.Graph()
  mesh = mtf.Mesh(g, "my_mesh")
  w = mtf.get_variable(mesh, "w", "a:8,b:6", initial_value=w0)
  y = w * 2.0
  impl = NumpyMeshImpl("rows:2,cols:2", "a:rows;b:cols")
  low = mtf.Lowering(g, {mesh: impl})
  np.testing.assert_array_equal(low.export_to_tf_tensor(y), w0 * 2)
  lov = low.variables[w.operation]
  assert lov.laid_out_tensor.slice_shape == [4, 3]
  ops = impl.slice_ops
  lov.assign_to_slices(lambda var, old, value: ops.binary("add", old, value),
                       [ops.fill([4, 3], 1.0, mtf.float32)] * 4)
  lov.copy_slices_to_master()
  np.testing.assert_array_equal(w.operation.get_master(), w0 + 1)
  w.operation.assign_to_master(w0 * 3)
  lov.copy_master_to_slices()
  np.testing.assert_array_equal(impl.export_to_tf_tensor(w, lov.laid_out_tensor), w0 * 3)


def _attention_layer(mesh_shape, layout, fused, dtype=mtf.bfloat16):
  r = rng(11)
  x = r.standard_normal((2, 32, 64)).astype(np.float32)

  def build(mesh):
    X = mtf.import_tf_tensor(mesh, x, "batch:2,length:32,d_model:64", dtype=dtype)
    heads, kv = mtf.Dimension("heads", 4), mtf.Dimension("d_kv", 16)
    params = mtf.layers.multihead_attention_params(mesh, heads, X.shape.dims[-1], kv,
                                                   mtf.layers.WeightSource(3), dtype)
    pos = mtf.mtf_range(mesh, X.shape.dims[1], mtf.float32)
    mask = mtf.layers.attention_mask_autoregressive(pos)
    assert getattr(mask, "causal_hint", False)
    return [mtf.layers.multihead_attention(X, None, mask, kv, heads, params=params, fused=fused)]
  (y,), low = _lower(build, mesh_shape, layout)
  return y, low


def test_fused_attention_operation_matches_op_chain():
  ref, low_ref = _attention_layer("", "", fused=False)
  for mesh_shape, layout in [("", ""), ("all:4", "heads:all"), ("all:2", "batch:all")]:
    got, low = _attention_layer(mesh_shape, layout, fused=None)   # bfloat16 + causal mask: fuses
    assert "output/FusedAttentionOperation" in low.counter_totals()
    assert rel_err(got, ref) < 2e-2
  assert "output/FusedAttentionOperation" not in low_ref.counter_totals()
  # float32 stays on the op chain by default
  _, low32 = _attention_layer("", "", fused=None, dtype=mtf.float32)
  assert "output/FusedAttentionOperation" not in low32.counter_totals()
  with pytest.raises(ValueError):
    _attention_layer("all:2", "memory_length:all", fused=True)


def test_bf16_rounding_fast_path_equals_definition():
  """round_to_bf16 uses torch for large arrays: the same bits as the numpy definition,
  including ties, subnormals, infinities and values that round up to infinity."""
  import torch
  from oracle.numpy_ops import round_to_bf16_numpy
  r = np.random.Generator(np.random.PCG64(3))
  bits = r.integers(0, 2 ** 32, size=1 << 20, dtype=np.uint64).astype(np.uint32)
  special = np.array([0x3F808000, 0x3F818000, 0x3F80FFFF, 0x7F7FFFFF, 0x7F800000, 0xFF800000,
                      0x00000001, 0x00008000, 0x80008000, 0x0000FFFF], dtype=np.uint32)
  x = np.concatenate([bits, special]).view(np.float32)
  x = x[~np.isnan(x)]
  a = round_to_bf16_numpy(x)
  b = torch.from_numpy(x.copy()).to(torch.bfloat16).to(torch.float32).numpy()
  np.testing.assert_array_equal(a.view(np.uint32), b.view(np.uint32))
