"""numpy restatement of the TensorFlow slice arithmetic the reference calls.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Each function states which tf op it stands for and where the reference calls
it (mesh_tensorflow/ops.py unless noted).  TensorFlow (an un-vendored
dependency, `tensorflow>=1.15`, setup.py:26-30) is not installed here, so the
semantics below are TensorFlow's published ones:

  * bfloat16 tensors are float32 arrays holding bfloat16-representable values;
    every bfloat16 op computes in float32 and rounds once, to nearest-even;
  * einsum accumulates in float32 (float64 is used here for float32 inputs to
    make the oracle's own rounding negligible next to the 1e-5 tolerance);
  * argmax / top_k ties go to the lowest index;
  * one_hot of an index outside [0, depth) is an all-`off` row;
  * float -> int32 casts truncate; casts to bool are `!= 0`.
"""

from __future__ import annotations

import numpy as np

from mesh_b200 import mtf


def round_to_bf16(x):
  """float32 -> nearest-even bfloat16, returned as float32.

  Arrays of a million elements or more go through torch's float32 -> bfloat16
  conversion, which is the same round-to-nearest-even (tests/test_oracle.py
  holds the two against each other bit for bit); the numpy form below is the
  definition."""
  if np.size(x) >= (1 << 20):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32))
    return t.to(torch.bfloat16).to(torch.float32).numpy()
  return round_to_bf16_numpy(x)


def round_to_bf16_numpy(x):
  """The definition: add 0x7FFF plus the lowest kept bit, truncate 16 bits."""
  shape = np.shape(x)
  x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
  u = x.view(np.uint32)
  bias = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
  r = ((u + bias) & np.uint32(0xFFFF0000)).astype(np.uint32)
  out = r.view(np.float32).copy()
  nan = np.isnan(x)
  if nan.any():
    out[nan] = np.nan
  return out.reshape(shape)


class Arr(object):
  """A slice: numpy storage plus the mtf dtype it represents."""
  __slots__ = ("a", "dtype")

  def __init__(self, a, dtype):
    self.a = a
    self.dtype = dtype

  @property
  def shape(self):
    return tuple(self.a.shape)

  def __repr__(self):
    return "Arr(%s, %s)" % (self.a.shape, self.dtype)


def _storage(dtype):
  if dtype.is_floating:
    return np.float32
  if dtype.is_bool:
    return np.bool_
  return np.int32


def _finish(a, dtype):
  """Applies the dtype's storage type and rounding to a computed array."""
  a = np.asarray(a)
  if dtype == mtf.bfloat16:
    return Arr(round_to_bf16(a.astype(np.float32)), dtype)
  return Arr(a.astype(_storage(dtype), copy=False), dtype)


class NumpyOps(object):
  """The `slice_ops` array library of the oracle's mesh backend.

  `fast=True` is the timed CPU-baseline flavour: floating einsums run as
  float32 torch CPU contractions on all host threads (what TensorFlow's
  Eigen/MKL kernels would do) instead of float64 numpy; everything else is
  unchanged.  Parity checks use the default (float64 accumulate) flavour.
  """

  def __init__(self, fast=False):
    self._fast = fast

  # ---- host transfer
  def from_host(self, value, dtype):
    return _finish(np.array(value), dtype)

  def to_host(self, x):
    return np.array(x.a)

  # ---- metadata
  def shape(self, x):
    return tuple(x.a.shape)

  def dtype(self, x):
    return x.dtype

  def contiguous(self, x):
    return Arr(np.ascontiguousarray(x.a), x.dtype)

  # ---- layout ops: tf.slice / concat / transpose / expand_dims / reshape
  def slice(self, x, begin, size):
    idx = tuple(slice(b, b + s) for b, s in zip(begin, size))
    return Arr(np.ascontiguousarray(x.a[idx]), x.dtype)

  def concat(self, xs, axis):
    return Arr(np.concatenate([x.a for x in xs], axis=axis), xs[0].dtype)

  def transpose(self, x, perm):
    return Arr(np.transpose(x.a, perm), x.dtype)

  def expand_dims(self, x, axis):
    return Arr(np.expand_dims(x.a, axis), x.dtype)

  def reshape(self, x, shape):
    return Arr(np.reshape(x.a, shape), x.dtype)

  def broadcast_to(self, x, shape):
    return Arr(np.ascontiguousarray(np.broadcast_to(x.a, shape)), x.dtype)

  # ---- creation: tf.zeros / tf.constant / tf.range
  def fill(self, shape, value, dtype):
    return _finish(np.full(shape, value), dtype)

  def range(self, n, dtype):
    return _finish(np.arange(n), dtype)

  # ---- tf.cast (ops.py:1945-1950)
  def cast(self, x, dtype):
    a = x.a
    if dtype.is_bool:
      return Arr(a != 0, dtype)
    if dtype.is_integer:
      return Arr(np.trunc(a).astype(np.int32) if x.dtype.is_floating else a.astype(np.int32), dtype)
    return _finish(a.astype(np.float32), dtype)

  # ---- tf.nn.relu, tf.exp, ... via cwise (ops.py:1727-1943)
  def unary(self, name, x):
    a = x.a
    with np.errstate(all="ignore"):
      if name == "relu":
        r = np.maximum(a, 0)
      elif name == "exp":
        r = np.exp(a.astype(np.float32))
      elif name == "log":
        r = np.log(a.astype(np.float32))
      elif name == "negative":
        r = -a
      elif name == "reciprocal":
        r = np.float32(1.0) / a.astype(np.float32)
      elif name == "sqrt":
        r = np.sqrt(a.astype(np.float32))
      elif name == "rsqrt":
        r = np.float32(1.0) / np.sqrt(a.astype(np.float32))
      elif name == "square":
        r = a * a
      elif name == "tanh":
        r = np.tanh(a.astype(np.float32))
      elif name == "sigmoid":
        r = np.float32(1.0) / (np.float32(1.0) + np.exp(-a.astype(np.float32)))
      elif name == "sign":
        r = np.sign(a)
      elif name == "logical_not":
        return Arr(~(a != 0), mtf.bool_)
      elif name == "identity":
        r = a
      else:
        raise ValueError("unknown unary op %s" % name)
    return _finish(r, x.dtype)

  # ---- tf.add / multiply / less ... (ops.py:2044-2200)
  def binary(self, name, a, b):
    ref = a if isinstance(a, Arr) else b
    av = a.a if isinstance(a, Arr) else np.asarray(a, dtype=_storage(ref.dtype))
    bv = b.a if isinstance(b, Arr) else np.asarray(b, dtype=_storage(ref.dtype))
    with np.errstate(all="ignore"):
      if name == "add":
        r = av + bv
      elif name == "sub":
        r = av - bv
      elif name == "multiply":
        r = av * bv
      elif name == "divide":
        r = av / bv
      elif name == "maximum":
        r = np.maximum(av, bv)
      elif name == "minimum":
        r = np.minimum(av, bv)
      elif name == "floordiv":
        r = np.floor_divide(av, bv)
      elif name == "mod":
        r = np.mod(av, bv)
      elif name in ("less", "greater", "less_equal", "greater_equal", "equal", "not_equal"):
        fn = {"less": np.less, "greater": np.greater, "less_equal": np.less_equal,
              "greater_equal": np.greater_equal, "equal": np.equal,
              "not_equal": np.not_equal}[name]
        return Arr(fn(av, bv), mtf.bool_)
      elif name == "logical_and":
        return Arr((av != 0) & (bv != 0), mtf.bool_)
      elif name == "logical_or":
        return Arr((av != 0) | (bv != 0), mtf.bool_)
      elif name == "select_positive":
        r = np.where(bv > 0, av, np.zeros_like(av))
      else:
        raise ValueError("unknown binary op %s" % name)
    return _finish(r, ref.dtype)

  # ---- tf.reduce_sum / max / min (ops.py:5698-5706)
  def reduce(self, name, x, axes):
    axes = tuple(axes)
    if name == "SUM":
      if x.dtype.is_floating:
        r = np.sum(x.a.astype(np.float64), axis=axes).astype(np.float32)
      else:
        r = np.sum(x.a.astype(np.int64), axis=axes)
    elif name == "MAX":
      r = np.max(x.a, axis=axes)
    elif name == "MIN":
      r = np.min(x.a, axis=axes)
    else:
      raise ValueError("unknown reduction %s" % name)
    return _finish(r, x.dtype)

  # ---- tf.math.argmax / top_k / gather (ops.py:4937-4958)
  def argmax(self, x):
    return Arr(np.argmax(x.a, axis=-1).astype(np.int32), mtf.int32)

  def top_k(self, x, k):
    order = np.argsort(-x.a, axis=-1, kind="stable")[..., :k]
    return (Arr(np.take_along_axis(x.a, order, axis=-1), x.dtype),
            Arr(order.astype(np.int32), mtf.int32))

  def gather_last(self, values, indices):
    return Arr(np.take_along_axis(values.a, indices.a.astype(np.int64), axis=-1), values.dtype)

  # ---- tf.one_hot (ops.py:3843-3848)
  def one_hot(self, indices, depth, on_value, off_value, dtype):
    hit = indices.a[..., None] == np.arange(depth, dtype=np.int64)
    return _finish(np.where(hit, on_value, off_value), dtype)

  # ---- tf.einsum (ops.py:1340) and the broadcast-multiply-reduce form (2805-2814)
  def einsum(self, equation, *xs):
    dtype = xs[0].dtype
    if dtype.is_floating and self._fast:
      import torch
      r = torch.einsum(equation, *[torch.from_numpy(np.ascontiguousarray(x.a, dtype=np.float32))
                                   for x in xs]).numpy()
      return _finish(r, dtype)
    if dtype.is_floating:
      r = np.einsum(equation, *[x.a.astype(np.float64) for x in xs], optimize=True)
      return _finish(r.astype(np.float32), dtype)
    r = np.einsum(equation, *[x.a.astype(np.int64) for x in xs], optimize=True)
    return _finish(r, dtype)

  def einsum_naive(self, equation, *xs):
    return self.einsum(equation, *xs)

  # ---- fused attention entry point: the op chain of layers.py:1640-1652 with
  # float32 logits and softmax (transformer/attention.py:71-88), in one call
  def attention(self, q, k, v, causal):
    qf, kf = q.a.astype(np.float64), k.a.astype(np.float64)
    logits = np.einsum("...xd,...yd->...xy", qf, kf).astype(np.float32)
    if causal:
      lq, lk = logits.shape[-2:]
      logits = logits + np.where(np.arange(lq)[:, None] < np.arange(lk)[None, :],
                                 np.float32(-1e9), np.float32(0))
    mx = logits.max(axis=-1, keepdims=True)
    lse = np.log(np.sum(np.exp(logits - mx), axis=-1, keepdims=True)) + mx
    w = _finish(np.exp(logits - lse), v.dtype).a
    out = np.einsum("...xy,...ye->...xe", w.astype(np.float64), v.a.astype(np.float64))
    return _finish(out.astype(np.float32), v.dtype)

  # ---- random fill: Philox4x32-10, the generator the device kernel restates
  def random(self, shape, kind, seed, dtype, a, b):
    n = int(np.prod(shape)) if len(shape) else 1
    blocks = (n + 3) // 4
    q = np.arange(blocks, dtype=np.uint64)
    c = [(q & np.uint64(0xFFFFFFFF)).astype(np.uint64), (q >> np.uint64(32)).astype(np.uint64),
         np.zeros(blocks, np.uint64), np.zeros(blocks, np.uint64)]
    k0, k1 = np.uint64(seed & 0xFFFFFFFF), np.uint64((seed >> 32) & 0xFFFFFFFF)
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
      p0 = np.uint64(0xD2511F53) * c[0]
      p1 = np.uint64(0xCD9E8D57) * c[2]
      n0 = ((p1 >> np.uint64(32)) ^ c[1] ^ k0) & mask
      n2 = ((p0 >> np.uint64(32)) ^ c[3] ^ k1) & mask
      c = [n0, p1 & mask, n2, p0 & mask]
      k0 = (k0 + np.uint64(0x9E3779B9)) & mask
      k1 = (k1 + np.uint64(0xBB67AE85)) & mask
    u = [(w >> np.uint64(8)).astype(np.float32) * np.float32(1.0 / 16777216.0) for w in c]
    if kind == "normal":
      vals = []
      for h in range(2):
        r = np.sqrt(np.float32(-2.0) * np.log(np.float32(1.0) - u[2 * h], dtype=np.float32), dtype=np.float32)
        ang = np.float32(6.283185307179586) * u[2 * h + 1]
        vals += [np.float32(a) + np.float32(b) * (r * np.cos(ang, dtype=np.float32)),
                 np.float32(a) + np.float32(b) * (r * np.sin(ang, dtype=np.float32))]
    else:
      vals = [np.float32(a) + (np.float32(b) - np.float32(a)) * w for w in u]
    flat = np.stack(vals, axis=1).reshape(-1)[:n]
    return _finish(flat.reshape(shape), dtype)

  # ---- row kernels of the rest of a transformer block: direct formulas
  def norm_rows(self, x, scale, bias, epsilon, centered):
    """layer_norm (layers.py:950-979) / rms norm (transformer.py:493-516) on the
    last axis, in float64, rounded once."""
    a = x.a.astype(np.float64)
    if centered:
      mean = a.mean(-1, keepdims=True)
      var = ((a - mean) ** 2).mean(-1, keepdims=True)
      out = (a - mean) / np.sqrt(var + epsilon)
    else:
      out = a / np.sqrt((a * a).mean(-1, keepdims=True) + epsilon)
    if scale is not None:
      out = out * scale.a.astype(np.float64)
    if bias is not None:
      out = out + bias.a.astype(np.float64)
    return _finish(out.astype(np.float32), x.dtype)

  def gather_rows(self, table, indices, first_row):
    idx = indices.a.astype(np.int64) - first_row
    ok = (idx >= 0) & (idx < table.a.shape[0])
    out = table.a[np.where(ok, idx, 0)]
    out = np.where(ok.reshape(ok.shape + (1,) * (table.a.ndim - 1)), out, 0)
    return Arr(out.astype(table.a.dtype), table.dtype)

  def xent_stats(self, logits, targets, first_col):
    a = logits.a.astype(np.float64)
    m = a.max(-1)
    s = np.exp(a - m[..., None]).sum(-1)
    c = targets.a.astype(np.int64) - first_col
    ok = (c >= 0) & (c < a.shape[-1])
    picked = np.where(ok, np.take_along_axis(a, np.where(ok, c, 0)[..., None], -1)[..., 0], 0.0)
    return tuple(Arr(v.astype(np.float32), mtf.float32) for v in (m, s, picked))

  def xent_grad(self, logits, targets, log_z, dloss, z_loss, first_col):
    a = logits.a.astype(np.float64)
    lz = log_z.a.astype(np.float64)[..., None]
    hot = (np.arange(a.shape[-1]) + first_col) == targets.a[..., None]
    out = dloss.a.astype(np.float64)[..., None] * ((1 + 2 * z_loss * lz) * np.exp(a - lz) - hot)
    return _finish(out.astype(np.float32), logits.dtype)

  # ---- fused MoE entry points: the scalar specification
  def moe_top2_gating(self, x, w, capacity, policy, threshold, noise, num_groups_total,
                      want_table=False, want_raw=False):
    from oracle import moe_spec
    lead = x.a.shape[:-2]
    s, m = x.a.shape[-2:]
    xg = x.a.reshape((-1, s, m)).astype(np.float32)
    ng = None if noise is None else noise.a.reshape((-1, s)).astype(np.float32)
    r = moe_spec.top2_gating(xg, w.a.astype(np.float32), capacity, policy, threshold, ng)
    tok = lead + (s,)
    outs = [Arr(r[k].reshape(tok), mtf.int32) for k in ("index_1", "index_2", "position_1",
                                                        "position_2")]
    outs += [Arr(r[k].reshape(tok), mtf.float32) for k in ("gate_1", "gate_2")]
    loss = np.float32(np.sum(r["loss_per_group"].astype(np.float64)) / num_groups_total)
    outs.append(Arr(np.asarray(loss, dtype=np.float32), mtf.float32))
    if want_table:
      e = w.a.shape[-1]
      table = moe_spec.slot_table(*[r[k] for k in ("index_1", "index_2", "position_1", "position_2",
                                                    "gate_1", "gate_2")], e, capacity,
                                  bf16=(x.dtype == mtf.bfloat16))
      outs.append(Arr(table.reshape(lead + (e, capacity)), mtf.int32))
    if want_raw:
      outs.append(Arr(r["raw_gates"].reshape(tok + (w.a.shape[-1],)), mtf.float32))
    return tuple(outs)

  def moe_dispatch(self, x, i1, i2, p1, p2, g1, g2, num_experts, capacity, table=None):
    """`table`, when given, must be what the routing implies; the rows are
    placed from the routing itself."""
    from oracle import moe_spec
    o, g, s, m = x.a.shape
    out = moe_spec.dispatch(x.a.reshape(o * g, s, m), i1.a.reshape(-1, s), i2.a.reshape(-1, s),
                            p1.a.reshape(-1, s), p2.a.reshape(-1, s), g1.a.reshape(-1, s),
                            g2.a.reshape(-1, s), num_experts, capacity,
                            bf16=(x.dtype == mtf.bfloat16))  # [OG, E, C, M]
    out = out.reshape(o, g, num_experts, capacity, m).transpose(0, 2, 1, 3, 4)
    return Arr(np.ascontiguousarray(out), x.dtype)

  def moe_dispatch_weighted(self, x, i1, i2, p1, p2, g1, g2, num_experts, capacity, table=None):
    from oracle import moe_spec
    o, g, s, m = x.a.shape
    out = moe_spec.dispatch_weighted(
        x.a.reshape(o * g, s, m), i1.a.reshape(-1, s), i2.a.reshape(-1, s), p1.a.reshape(-1, s),
        p2.a.reshape(-1, s), g1.a.reshape(-1, s), g2.a.reshape(-1, s), num_experts, capacity,
        bf16=(x.dtype == mtf.bfloat16))
    out = out.reshape(o, g, num_experts, capacity, m).transpose(0, 2, 1, 3, 4)
    return _finish(np.ascontiguousarray(out), x.dtype)

  def moe_gate_grad(self, logits, i1, i2, g1, g2, dg1, dg2, dloss, num_groups_total, top1_only):
    """d logits of the gating (moe.py:1384-1424, 1485-1494 differentiated by hand):
    softmax backward of d raw, where d raw gathers the loss's mean-gate factor and
    the two picked, renormalised gates; routing decisions are constants."""
    z = logits.a.astype(np.float64)
    s, e = z.shape[-2:]
    z = z.reshape(-1, s, e)
    raw = np.exp(z - z.max(-1, keepdims=True))
    raw /= raw.sum(-1, keepdims=True)
    a1, a2 = i1.a.reshape(-1, s), i2.a.reshape(-1, s)
    k1 = (g1.a.reshape(-1, s) != 0).astype(np.float64)
    k2 = (g2.a.reshape(-1, s) != 0).astype(np.float64)
    d1 = (np.zeros_like(k1) if dg1 is None else dg1.a.reshape(-1, s).astype(np.float64)) * k1
    d2 = (np.zeros_like(k2) if dg2 is None else dg2.a.reshape(-1, s).astype(np.float64)) * k2
    dl = 0.0 if dloss is None else float(np.asarray(dloss.a).reshape(()))
    density = np.stack([(a1 == j).mean(axis=1) for j in range(e)], axis=-1)          # [G, E]
    draw = np.repeat((dl * e / (num_groups_total * s) * density)[:, None, :], s, axis=1)
    gi, si = np.meshgrid(np.arange(z.shape[0]), np.arange(s), indexing="ij")
    b1, b2 = raw[gi, si, a1], raw[gi, si, a2]
    if top1_only:
      at1, at2 = d1, np.zeros_like(d2)
    else:
      den = b1 + b2 + 1e-9
      at1 = d1 * (1 / den - b1 / den ** 2) - d2 * b2 / den ** 2
      at2 = d2 * (1 / den - b2 / den ** 2) - d1 * b1 / den ** 2
    np.add.at(draw, (gi, si, a1), at1)
    np.add.at(draw, (gi, si, a2), at2)
    dz = raw * (draw - (raw * draw).sum(-1, keepdims=True))
    return Arr(dz.reshape(logits.a.shape).astype(np.float32), mtf.float32)

  def moe_combine_gate_grad(self, y, dout, i1, i2, p1, p2, g1, g2):
    from oracle import moe_spec
    o, e, g, c, m = y.a.shape
    s = i1.a.shape[-1]
    yg = np.ascontiguousarray(y.a.transpose(0, 2, 1, 3, 4)).reshape(o * g, e, c, m)
    d1, d2 = moe_spec.combine_gate_grad(
        yg, dout.a.reshape(o * g, s, m), i1.a.reshape(-1, s), i2.a.reshape(-1, s),
        p1.a.reshape(-1, s), p2.a.reshape(-1, s), g1.a.reshape(-1, s), g2.a.reshape(-1, s),
        bf16=(y.dtype == mtf.bfloat16))
    return Arr(d1.reshape(o, g, s), mtf.float32), Arr(d2.reshape(o, g, s), mtf.float32)

  def moe_combine(self, y, i1, i2, p1, p2, g1, g2):
    from oracle import moe_spec
    o, e, g, c, m = y.a.shape
    s = i1.a.shape[-1]
    yg = np.ascontiguousarray(y.a.transpose(0, 2, 1, 3, 4)).reshape(o * g, e, c, m)
    out = moe_spec.combine(yg, i1.a.reshape(-1, s), i2.a.reshape(-1, s), p1.a.reshape(-1, s),
                           p2.a.reshape(-1, s), g1.a.reshape(-1, s), g2.a.reshape(-1, s),
                           bf16=(y.dtype == mtf.bfloat16))
    out = out.reshape(o, g, s, m)
    return _finish(out, y.dtype)
