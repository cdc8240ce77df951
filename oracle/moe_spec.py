"""Per-group specification of top-2 gating, dispatch and combine.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

A direct restatement of what mesh_tensorflow/transformer/moe.py computes for
one group of S tokens (`_top_2_gating` 1380-1513, the dispatch einsum 443-447
and the combine einsum 509-510), in float32 numpy with the reference's order
of operations: softmax as exp(x - logsumexp(x)) (ops.py:5493-5541), argmax
ties to the lowest index (ops.py:4937-4940), gates renormalised with the
reciprocal-then-multiply form of mtf's "/" (ops.py:5156-5172), positions from
exclusive prefix counts of the pre-capacity masks, combine weights rounded to
the activation dtype (bfloat16) before use, dispatch = (rounded weight != 0).
"""

from __future__ import annotations

import numpy as np

from oracle.numpy_ops import round_to_bf16


def softmax_f32(logits):
  """exp(l - (log(sum(exp(l - max))) + max)), all in float32."""
  logits = logits.astype(np.float32)
  mx = np.max(logits, axis=-1, keepdims=True)
  shifted = logits - mx
  sum_exp = np.sum(np.exp(shifted, dtype=np.float32), axis=-1, keepdims=True, dtype=np.float32)
  lse = np.log(sum_exp, dtype=np.float32) + mx
  return np.exp(logits - lse, dtype=np.float32)


def gating_from_raw(raw, capacity, policy="all", threshold=0.2, noise=None):
  """raw: [G, S, E] float32 softmax outputs -> routing for every group."""
  g_, s_, e_ = raw.shape
  raw = raw.astype(np.float32)
  i1 = np.argmax(raw, axis=-1).astype(np.int32)
  g1 = np.take_along_axis(raw, i1[..., None].astype(np.int64), axis=-1)[..., 0]
  mask1 = (np.arange(e_)[None, None, :] == i1[..., None])
  raw2 = raw * (np.float32(1.0) + (-mask1.astype(np.float32)))
  i2 = np.argmax(raw2, axis=-1).astype(np.int32)
  g2 = np.take_along_axis(raw2, i2[..., None].astype(np.int64), axis=-1)[..., 0]
  if policy == "switch":
    # top-1 routing (_switch_gating, moe.py:1184-1309): the raw gate, no second expert
    g2 = np.zeros_like(g2)
  else:
    denom = (g1 + g2) + np.float32(1e-9)
    recip = np.float32(1.0) / denom
    g1 = g1 * recip
    g2 = g2 * recip

  # load-balancing loss per group (moe.py:1420-1424), on pre-capacity masks
  density = np.sum(mask1.astype(np.float32), axis=1, dtype=np.float32) * np.float32(1.0 / s_)
  proxy = np.sum(raw.astype(np.float64), axis=1).astype(np.float32) * np.float32(1.0 / s_)
  loss = (np.sum((proxy * density).astype(np.float64), axis=-1) / e_).astype(np.float32) \
      * np.float32(e_ * e_)

  if policy == "all":
    m2 = np.ones((g_, s_), dtype=bool)
  elif policy in ("none", "switch"):
    m2 = np.zeros((g_, s_), dtype=bool)
  elif policy == "threshold":
    m2 = g2 > np.float32(threshold)
  elif policy == "random":
    m2 = noise.astype(np.float32) < g2 * np.float32(1.0 / max(threshold, 1e-9))
  else:
    raise ValueError("Unknown policy %s" % policy)

  p1 = np.zeros((g_, s_), dtype=np.int32)
  p2 = np.zeros((g_, s_), dtype=np.int32)
  for g in range(g_):
    seen = np.zeros(e_, dtype=np.int32)
    for s in range(s_):
      p1[g, s] = seen[i1[g, s]]
      seen[i1[g, s]] += 1
    cnt1 = np.minimum(seen, capacity)
    seen2 = np.zeros(e_, dtype=np.int32)
    for s in range(s_):
      if m2[g, s]:
        p2[g, s] = seen2[i2[g, s]] + cnt1[i2[g, s]]
        seen2[i2[g, s]] += 1
  keep1 = p1 < capacity
  keep2 = m2 & (p2 < capacity)
  gate1 = np.where(keep1, g1, np.float32(0)).astype(np.float32)
  gate2 = np.where(keep2, g2, np.float32(0)).astype(np.float32)
  return dict(index_1=i1, index_2=i2, position_1=p1, position_2=p2, gate_1=gate1, gate_2=gate2,
              keep_1=keep1, keep_2=keep2, loss_per_group=loss, raw_gates=raw)


def top2_gating(x, w, capacity, policy="all", threshold=0.2, noise=None):
  """x: [G, S, M] float32 (already widened), w: [M, E] float32."""
  logits = np.einsum("gsm,me->gse", x.astype(np.float64), w.astype(np.float64)).astype(np.float32)
  out = gating_from_raw(softmax_f32(logits), capacity, policy, threshold, noise)
  out["logits"] = logits
  return out


def combine_weights(gate, bf16=True):
  """Gate as it enters the combine tensor: cast to the activation dtype
  (moe.py:1507) — rounded to bfloat16 for bfloat16 activations, unchanged for float32."""
  return round_to_bf16(gate) if bf16 else np.asarray(gate, dtype=np.float32)


def slot_table(i1, i2, p1, p2, g1, g2, num_experts, capacity, bf16=True):
  """[G, E, C] int32: the token that occupies each expert slot, -1 for none."""
  g_, s_ = i1.shape
  table = np.full((g_, num_experts, capacity), -1, dtype=np.int32)
  w1, w2 = combine_weights(g1, bf16), combine_weights(g2, bf16)
  for g in range(g_):
    for s in range(s_):
      if w1[g, s] != 0 and p1[g, s] < capacity:
        table[g, i1[g, s], p1[g, s]] = s
      if w2[g, s] != 0 and p2[g, s] < capacity:
        table[g, i2[g, s], p2[g, s]] = s
  return table


def dispatch(x, i1, i2, p1, p2, g1, g2, num_experts, capacity, bf16=True):
  """x [G,S,M] -> expert inputs [G,E,C,M]; a slot holds at most one token."""
  g_, s_, m_ = x.shape
  out = np.zeros((g_, num_experts, capacity, m_), dtype=np.float32)
  w1, w2 = combine_weights(g1, bf16), combine_weights(g2, bf16)
  for g in range(g_):
    for s in range(s_):
      if w1[g, s] != 0 and p1[g, s] < capacity:
        out[g, i1[g, s], p1[g, s]] += x[g, s]
      if w2[g, s] != 0 and p2[g, s] < capacity:
        out[g, i2[g, s], p2[g, s]] += x[g, s]
  return out


def combine(y, i1, i2, p1, p2, g1, g2, bf16=True):
  """y [G,E,C,M] -> [G,S,M]: w1*y[i1,p1] + w2*y[i2,p2] in float32 (caller rounds)."""
  g_, e_, c_, m_ = y.shape
  s_ = i1.shape[-1]
  out = np.zeros((g_, s_, m_), dtype=np.float32)
  w1, w2 = combine_weights(g1, bf16), combine_weights(g2, bf16)
  y = y.astype(np.float32)
  for g in range(g_):
    for s in range(s_):
      acc = np.zeros(m_, dtype=np.float32)
      if w1[g, s] != 0 and p1[g, s] < c_:
        acc = acc + w1[g, s] * y[g, i1[g, s], p1[g, s]]
      if w2[g, s] != 0 and p2[g, s] < c_:
        acc = acc + w2[g, s] * y[g, i2[g, s], p2[g, s]]
      out[g, s] = acc
  return out


def dispatch_weighted(x, i1, i2, p1, p2, g1, g2, num_experts, capacity, bf16=True):
  """Transpose of combine w.r.t. the expert outputs: slot (e, c) receives
  w * x[s] for the token s that occupies it through either choice."""
  g_, s_, m_ = x.shape
  out = np.zeros((g_, num_experts, capacity, m_), dtype=np.float32)
  w1, w2 = combine_weights(g1, bf16), combine_weights(g2, bf16)
  for g in range(g_):
    for s in range(s_):
      if w1[g, s] != 0 and p1[g, s] < capacity:
        out[g, i1[g, s], p1[g, s]] += w1[g, s] * x[g, s]
      if w2[g, s] != 0 and p2[g, s] < capacity:
        out[g, i2[g, s], p2[g, s]] += w2[g, s] * x[g, s]
  return out


def combine_gate_grad(y, dout, i1, i2, p1, p2, g1, g2, bf16=True):
  """Gradient of combine w.r.t. the gates: <dout[s], y[i_k, p_k]> per kept choice."""
  g_, e_, c_, m_ = y.shape
  s_ = i1.shape[-1]
  d1 = np.zeros((g_, s_), dtype=np.float32)
  d2 = np.zeros((g_, s_), dtype=np.float32)
  w1, w2 = combine_weights(g1, bf16), combine_weights(g2, bf16)
  y64, d64 = y.astype(np.float64), dout.astype(np.float64)
  for g in range(g_):
    for s in range(s_):
      if w1[g, s] != 0 and p1[g, s] < c_:
        d1[g, s] = np.dot(d64[g, s], y64[g, i1[g, s], p1[g, s]])
      if w2[g, s] != 0 and p2[g, s] < c_:
        d2[g, s] = np.dot(d64[g, s], y64[g, i2[g, s], p2[g, s]])
  return d1, d2
