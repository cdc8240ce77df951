"""DeviceOps: the array library CudaMeshImpl computes its slices with.

Plays the role `tf.*` plays inside the reference's slicewise closures
(mesh_tensorflow/ops.py) but every operation is a libmtfc kernel reached
through the C ABI of include/mtfc.h.  PyTorch appears only as the owner of
device memory (torch.empty), the source of the current stream, and for
host<->device copies; no torch compute op is on any path here.  A missing or
failing library raises — there is no CPU fallback.

A slice is a DeviceArray: a strided view (shape, element strides, offset) of
a flat torch buffer.  transpose / expand_dims / slice / broadcast_to only
rewrite the view; kernels that take strides (binary, broadcast_reduce, GEMM,
strided copy) read views in place, the others get a packed copy first.
"""

from __future__ import annotations

import ctypes

import numpy as np
import torch

from mesh_b200 import _native as nat
from mesh_b200.mtf import graph as G

_TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32,
          "bool": torch.int32}
_CODE = {"float32": nat.F32, "bfloat16": nat.BF16, "int32": nat.I32, "bool": nat.I32}

_UNARY = {"identity": 0, "relu": 1, "exp": 2, "log": 3, "negative": 4, "reciprocal": 5,
          "sqrt": 6, "rsqrt": 7, "square": 8, "tanh": 9, "sigmoid": 10, "sign": 11,
          "logical_not": 12, "nonzero": 13}
_BINARY = {"add": 0, "sub": 1, "multiply": 2, "divide": 3, "maximum": 4, "minimum": 5,
           "floordiv": 6, "mod": 7, "less": 8, "greater": 9, "less_equal": 10,
           "greater_equal": 11, "equal": 12, "not_equal": 13, "logical_and": 14,
           "logical_or": 15, "select_positive": 16}
_COMPARISONS = frozenset(["less", "greater", "less_equal", "greater_equal", "equal",
                          "not_equal", "logical_and", "logical_or"])
_REDUCE = {"SUM": 0, "MAX": 1, "MIN": 2}
_POLICY = {"all": 0, "none": 1, "threshold": 2, "random": 3, "switch": 4}


def _contiguous_strides(shape):
  strides, acc = [], 1
  for s in reversed(shape):
    strides.append(acc)
    acc *= s
  return tuple(reversed(strides))


def _volume(shape):
  n = 1
  for s in shape:
    n *= s
  return n


class HookDeclined(Exception):
  """einsum(..., gemm_hook=...) did not come down to a launch the hook took;
  nothing has been launched."""


class DeviceArray(object):
  """A strided view of a flat device buffer with an mtf dtype."""
  __slots__ = ("buf", "shape", "strides", "offset", "dtype", "origin")

  def __init__(self, buf, shape, dtype, strides=None, offset=0):
    self.buf = buf
    self.shape = tuple(int(s) for s in shape)
    self.strides = tuple(strides) if strides is not None else _contiguous_strides(self.shape)
    self.offset = offset
    self.dtype = dtype
    # for a float32 array that is a widened bfloat16 array: that array (same shape and
    # strides), whose values it holds exactly; None otherwise
    self.origin = None

  @property
  def size(self):
    return _volume(self.shape)

  @property
  def ptr(self):
    return self.buf.data_ptr() + self.offset * self.dtype.itemsize

  @property
  def device(self):
    return self.buf.device

  @property
  def is_contiguous(self):
    expect = 1
    for s, st in zip(reversed(self.shape), reversed(self.strides)):
      if s != 1 and st != expect:
        return False
      expect *= s
    return True

  def __repr__(self):
    return "DeviceArray(%s, %s, %s)" % (list(self.shape), self.dtype.name, self.device)


def _i64(values):
  return (ctypes.c_int64 * max(1, len(values)))(*values)


class DeviceOps(object):
  """libmtfc-backed array operations on one CUDA device."""

  # fp32 contractions with at least this many multiply-adds go to the tensor
  # cores as 3-term bf16 splits; smaller ones stay on the FFMA kernel
  FP32_TENSOR_CORE_MIN_WORK = 1 << 22
  # longer contractions stay on the FFMA kernel: the tensor core truncates on
  # every accumulation, and beyond this many terms that bias nears 1e-5
  FP32_TENSOR_CORE_MAX_K = 2048
  # products narrower than this waste most of the GEMM kernel's 256-wide tile
  MIN_GEMM_N = 256

  def __init__(self, device):
    self._lib = nat.lib()
    self.device = device

  # ---------------------------------------------------------------- plumbing
  @property
  def device(self):
    return self._device

  @device.setter
  def device(self, value):
    dev = torch.device(value)
    if dev.type != "cuda":
      raise nat.MtfcError(nat.ERR_CUDA, "DeviceOps needs a CUDA device, got %s" % (value,))
    self._device = dev
    self._index = dev.index if dev.index is not None else torch.cuda.current_device()

  def _activate(self):
    """Makes this object's device the current CUDA device (libmtfc works on the
    current device).  A plain check-and-set: entering a torch.cuda.device context
    on every call costs milliseconds of host time per operation."""
    if torch.cuda.current_device() != self._index:
      torch.cuda.set_device(self._index)

  def _stream(self):
    self._activate()
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

  def _empty(self, shape, dtype):
    n = max(1, _volume(shape))
    buf = torch.empty(n, dtype=_TORCH[dtype.name], device=self.device)
    return DeviceArray(buf, shape, dtype)

  def _call(self, fn, *args):
    self._activate()
    nat.check(fn(*args))

  def contiguous(self, x):
    if x.is_contiguous:
      if x.strides == _contiguous_strides(x.shape):
        return x
      return DeviceArray(x.buf, x.shape, x.dtype, offset=x.offset)
    out = self._empty(x.shape, x.dtype)
    self._copy(x, out)
    return out

  def _copy(self, src, dst):
    """dst view <- src view (same shape)."""
    assert src.shape == dst.shape, (src.shape, dst.shape)
    if src.size == 0:
      return
    self._call(self._lib.mtfc_copy_strided, ctypes.c_void_p(src.ptr), _i64(src.strides),
               ctypes.c_void_p(dst.ptr), _i64(dst.strides), len(src.shape), _i64(src.shape),
               src.dtype.itemsize, self._stream())

  # ---------------------------------------------------------------- host I/O
  def from_host(self, value, dtype):
    """Uploads a host array.  A torch CPU tensor (e.g. pinned memory already in
    the target dtype) is copied as it is, asynchronously on the current stream;
    anything else goes through numpy and is converted on the host first."""
    if isinstance(value, torch.Tensor):
      t = value if value.dtype == _TORCH[dtype.name] else value.to(_TORCH[dtype.name])
      t = t.contiguous().reshape(-1)
      self._activate()
      buf = t.to(self.device, non_blocking=True) if t.numel() else torch.empty(
          1, dtype=_TORCH[dtype.name], device=self.device)
      return DeviceArray(buf, tuple(value.shape), dtype)
    shape = np.shape(value)
    a = np.ascontiguousarray(np.asarray(value)).reshape(-1)
    if dtype.is_floating:
      t = torch.from_numpy(a.astype(np.float32, copy=False)).to(_TORCH[dtype.name])
    elif dtype.is_bool:
      t = torch.from_numpy((a != 0).astype(np.int32))
    else:
      t = torch.from_numpy(a.astype(np.int32, copy=False))
    buf = t.reshape(-1).to(self.device) if t.numel() else torch.empty(
        1, dtype=_TORCH[dtype.name], device=self.device)
    return DeviceArray(buf, shape, dtype)

  def to_host_tensor(self, x, out=None):
    """Downloads a slice into a torch CPU tensor of the slice's own dtype
    (bfloat16 stays bfloat16).  With `out` (ideally pinned) the copy is
    asynchronous on the current stream; synchronise before reading it."""
    x = self.contiguous(x)
    flat = x.buf[x.offset:x.offset + x.size]
    if out is None:
      return flat.cpu().reshape(x.shape)
    self._activate()
    out.reshape(-1).copy_(flat, non_blocking=True)
    return out

  def to_host(self, x):
    x = self.contiguous(x)
    n = x.size
    flat = x.buf[x.offset:x.offset + n].cpu()
    if x.dtype.name == "bfloat16":
      flat = flat.float()
    a = flat.numpy().reshape(x.shape)
    if x.dtype.is_bool:
      a = a != 0
    return a

  # ---------------------------------------------------------------- metadata
  def shape(self, x):
    return x.shape

  def dtype(self, x):
    return x.dtype

  # ---------------------------------------------------------------- views
  def transpose(self, x, perm):
    return DeviceArray(x.buf, [x.shape[p] for p in perm], x.dtype,
                       strides=[x.strides[p] for p in perm], offset=x.offset)

  def expand_dims(self, x, axis):
    shape, strides = list(x.shape), list(x.strides)
    shape.insert(axis, 1)
    strides.insert(axis, 0)
    return DeviceArray(x.buf, shape, x.dtype, strides=strides, offset=x.offset)

  def slice(self, x, begin, size):
    offset = x.offset + sum(b * st for b, st in zip(begin, x.strides))
    return DeviceArray(x.buf, size, x.dtype, strides=x.strides, offset=offset)

  def broadcast_to(self, x, shape):
    shape = tuple(shape)
    pad = len(shape) - len(x.shape)
    strides = [0] * pad + [0 if (s == 1 and t != 1) else st
                           for s, st, t in zip(x.shape, x.strides, shape[pad:])]
    return DeviceArray(x.buf, shape, x.dtype, strides=strides, offset=x.offset)

  def reshape(self, x, shape):
    shape = tuple(int(s) for s in shape)
    if _volume(shape) != x.size:
      raise ValueError("cannot reshape %s to %s" % (x.shape, shape))
    x = self.contiguous(x)
    return DeviceArray(x.buf, shape, x.dtype, offset=x.offset)

  def concat(self, xs, axis):
    shape = list(xs[0].shape)
    shape[axis] = sum(x.shape[axis] for x in xs)
    out = self._empty(shape, xs[0].dtype)
    at = 0
    for x in xs:
      begin = [0] * len(shape)
      begin[axis] = at
      self._copy(x, self.slice(out, begin, x.shape))
      at += x.shape[axis]
    return out

  # ---------------------------------------------------------------- creation
  def fill(self, shape, value, dtype):
    out = self._empty(shape, dtype)
    self._call(self._lib.mtfc_fill, ctypes.c_void_p(out.ptr), _CODE[dtype.name], out.size,
               ctypes.c_float(float(value)), ctypes.c_float(0.0), self._stream())
    return out

  def range(self, n, dtype):
    out = self._empty([n], dtype)
    self._call(self._lib.mtfc_fill, ctypes.c_void_p(out.ptr), _CODE[dtype.name], n,
               ctypes.c_float(0.0), ctypes.c_float(1.0), self._stream())
    return out

  def random(self, shape, kind, seed, dtype, a, b):
    """Philox-keyed fill: kind "uniform" in [a, b) or "normal" with mean a, stddev b."""
    out = self._empty(shape, dtype)
    self._call(self._lib.mtfc_random, ctypes.c_void_p(out.ptr), _CODE[dtype.name], out.size,
               1 if kind == "normal" else 0, ctypes.c_uint64(seed & 0xFFFFFFFFFFFFFFFF),
               ctypes.c_float(a), ctypes.c_float(b), self._stream())
    return out

  # ---------------------------------------------------------------- maps
  def _unary_code(self, code, x, out_dtype):
    x = self.contiguous(x)
    out = self._empty(x.shape, out_dtype)
    self._call(self._lib.mtfc_unary, code, ctypes.c_void_p(x.ptr), _CODE[x.dtype.name],
               ctypes.c_void_p(out.ptr), _CODE[out_dtype.name], x.size, self._stream())
    return out

  def unary(self, name, x):
    out_dtype = G.bool_ if name == "logical_not" else x.dtype
    return self._unary_code(_UNARY[name], x, out_dtype)

  def cast(self, x, dtype):
    if dtype == x.dtype:
      return x
    if dtype.is_bool:
      return self._unary_code(_UNARY["nonzero"], x, dtype)
    out = self._unary_code(_UNARY["identity"], x, dtype)
    if (x.dtype.name == "bfloat16" and dtype.name == "float32" and x.is_contiguous
        and out.shape == x.shape and out.strides == x.strides):
      out.origin = x      # an fp32 einsum can take the bf16 values as they are
    return out

  def binary(self, name, a, b):
    if not isinstance(a, DeviceArray):
      # scalar on the left: only commutative ops arrive this way
      if name in ("add", "multiply", "maximum", "minimum", "equal", "not_equal"):
        a, b = b, a
      else:
        a = self.fill([], a, b.dtype)
    out_dtype = G.bool_ if name in _COMPARISONS else a.dtype
    if isinstance(b, DeviceArray):
      if _CODE[a.dtype.name] != _CODE[b.dtype.name]:
        raise ValueError("binary %s: dtypes differ (%s, %s)" % (name, a.dtype, b.dtype))
      nd = max(len(a.shape), len(b.shape))
      sa = (1,) * (nd - len(a.shape)) + a.shape
      sb = (1,) * (nd - len(b.shape)) + b.shape
      shape = []
      for x, y in zip(sa, sb):
        if x != y and x != 1 and y != 1:
          raise ValueError("binary %s: shapes %s and %s do not broadcast" % (name, a.shape, b.shape))
        shape.append(max(x, y) if min(x, y) != 0 else 0)
      av, bv = self.broadcast_to(a, shape), self.broadcast_to(b, shape)
      b_ptr, b_str, scalar = ctypes.c_void_p(bv.ptr), _i64(bv.strides), 0.0
    else:
      shape = list(a.shape)
      av = a
      b_ptr, b_str, scalar = ctypes.c_void_p(0), _i64([0] * len(shape)), float(b)
    if len(shape) > nat.MAX_DIMS:
      raise ValueError("binary %s: rank %d exceeds %d" % (name, len(shape), nat.MAX_DIMS))
    out = self._empty(shape, out_dtype)
    self._call(self._lib.mtfc_binary, _BINARY[name], ctypes.c_void_p(av.ptr), _i64(av.strides),
               b_ptr, b_str, ctypes.c_double(scalar), ctypes.c_void_p(out.ptr),
               _CODE[a.dtype.name], _CODE[out_dtype.name], len(shape), _i64(shape),
               self._stream())
    return out

  # ---------------------------------------------------------------- reductions
  def _broadcast_reduce(self, op, xs, out_shape, out_strides, red_shape, red_strides, out_dtype):
    n = len(xs)
    ptrs = (ctypes.c_void_p * n)(*[x.ptr for x in xs])
    keep = [_i64(s) for s in out_strides] + [_i64(s) for s in red_strides]
    o_arr = (ctypes.POINTER(ctypes.c_int64) * n)(
        *[ctypes.cast(k, ctypes.POINTER(ctypes.c_int64)) for k in keep[:n]])
    r_arr = (ctypes.POINTER(ctypes.c_int64) * n)(
        *[ctypes.cast(k, ctypes.POINTER(ctypes.c_int64)) for k in keep[n:]])
    out = self._empty(out_shape, out_dtype)
    self._call(self._lib.mtfc_broadcast_reduce, _REDUCE[op], n, ptrs, _CODE[xs[0].dtype.name],
               ctypes.c_void_p(out.ptr), _CODE[out_dtype.name], len(out_shape), _i64(out_shape),
               o_arr, len(red_shape), _i64(red_shape), r_arr, self._stream())
    return out

  def reduce(self, name, x, axes):
    axes = sorted(a % len(x.shape) for a in axes)
    kept = [i for i in range(len(x.shape)) if i not in axes]
    return self._broadcast_reduce(
        name, [x], [x.shape[i] for i in kept], [[x.strides[i] for i in kept]],
        [x.shape[i] for i in axes], [[x.strides[i] for i in axes]], x.dtype)

  def argmax(self, x):
    x = self.contiguous(x)
    rows, cols = _volume(x.shape[:-1]), x.shape[-1]
    idx = self._empty(x.shape[:-1], G.int32)
    self._call(self._lib.mtfc_topk_last, ctypes.c_void_p(x.ptr), _CODE[x.dtype.name], rows, cols,
               1, ctypes.c_void_p(0), ctypes.c_void_p(idx.ptr), self._stream())
    return idx

  def top_k(self, x, k):
    x = self.contiguous(x)
    rows, cols = _volume(x.shape[:-1]), x.shape[-1]
    values = self._empty(x.shape[:-1] + (k,), x.dtype)
    idx = self._empty(x.shape[:-1] + (k,), G.int32)
    self._call(self._lib.mtfc_topk_last, ctypes.c_void_p(x.ptr), _CODE[x.dtype.name], rows, cols,
               k, ctypes.c_void_p(values.ptr), ctypes.c_void_p(idx.ptr), self._stream())
    return values, idx

  def gather_last(self, values, indices):
    values, indices = self.contiguous(values), self.contiguous(indices)
    rows, cols, k = _volume(values.shape[:-1]), values.shape[-1], indices.shape[-1]
    out = self._empty(indices.shape, values.dtype)
    self._call(self._lib.mtfc_gather_last, ctypes.c_void_p(values.ptr), _CODE[values.dtype.name],
               ctypes.c_void_p(indices.ptr), rows, cols, k, ctypes.c_void_p(out.ptr),
               self._stream())
    return out

  def one_hot(self, indices, depth, on_value, off_value, dtype):
    indices = self.contiguous(indices)
    out = self._empty(indices.shape + (depth,), dtype)
    self._call(self._lib.mtfc_one_hot, ctypes.c_void_p(indices.ptr), indices.size, depth,
               ctypes.c_float(float(on_value)), ctypes.c_float(float(off_value)),
               ctypes.c_void_p(out.ptr), _CODE[dtype.name], self._stream())
    return out

  # ---------------------------------------------------------------- einsum
  @staticmethod
  def _parse(equation, n):
    lhs, rhs = equation.replace(" ", "").split("->")
    terms = lhs.split(",")
    if len(terms) != n:
      raise ValueError("einsum %s: expected %d operands" % (equation, n))
    return terms, rhs

  def einsum_naive(self, equation, *xs):
    """Broadcast-multiply-reduce: out[o] = sum_r prod_k x_k[o, r]."""
    terms, out_term = self._parse(equation, len(xs))
    if len(xs) > 4:
      head = self.einsum_naive(",".join(terms[:2]) + "->" + _union(terms[:2]), *xs[:2])
      return self.einsum_naive(",".join([_union(terms[:2])] + terms[2:]) + "->" + out_term,
                               head, *xs[2:])
    sizes = {}
    for term, x in zip(terms, xs):
      for letter, s in zip(term, x.shape):
        sizes[letter] = s
    red = [l for l in _union(terms) if l not in out_term]
    stride_of = lambda term, x, l: x.strides[term.index(l)] if l in term else 0
    out_strides = [[stride_of(t, x, l) for l in out_term] for t, x in zip(terms, xs)]
    red_strides = [[stride_of(t, x, l) for l in red] for t, x in zip(terms, xs)]
    return self._broadcast_reduce("SUM", list(xs), [sizes[l] for l in out_term], out_strides,
                                  [sizes[l] for l in red], red_strides, xs[0].dtype)

  def einsum(self, equation, *xs, epilogue=nat.EPILOGUE_NONE, out_dtype=None, out=None,
             gemm_hook=None):
    """Contraction on the GEMM kernels; operand layouts are read in place.

    Dims are classed as batch (in both operands and the output), M (first
    operand and output), N (second operand and output) and K (both operands,
    not the output).  When each class collapses to one stride per tensor the
    named-dim order goes to the kernel as strides; otherwise the operands are
    packed first and the result is unpacked.  `out`, a contiguous array of the
    result's shape, receives the result in place when given.

    `gemm_hook(desc, a_ptr, b_ptr, stored_shape)` is offered the launch when
    the contraction comes down to ONE bf16 -> bf16 GEMM without batch or
    epilogue (desc describes a dense row-major [m, n] output): it may run the
    product itself (e.g. fused with an allreduce) and return the array of
    `stored_shape` that holds the result, or return None to decline.  With a
    hook, the einsum either runs through it or raises HookDeclined before
    anything is launched (a contraction that needs packing, a pre-reduction or
    another kernel never reaches the hook), so the caller can fall back
    without having paid for a product.
    """
    if gemm_hook is not None:
      return self._einsum_impl(equation, xs, epilogue, out_dtype, None, gemm_hook)
    if out is not None:
      res = self._einsum_impl(equation, xs, epilogue, out_dtype, out)
      if res is not out:
        self._copy(res, out)
      return out
    return self._einsum_impl(equation, xs, epilogue, out_dtype, None)

  def _einsum_impl(self, equation, xs, epilogue, out_dtype, out_buf, gemm_hook=None):
    terms, out_term = self._parse(equation, len(xs))
    if gemm_hook is not None and len(xs) != 2:
      raise HookDeclined()
    if len(xs) == 1:
      return self.einsum_naive(equation, *xs)
    if len(xs) > 2:
      later = set("".join(terms[2:]) + out_term)
      mid = "".join(l for l in _union(terms[:2]) if l in later)
      head = self.einsum(",".join(terms[:2]) + "->" + mid, xs[0], xs[1])
      return self.einsum(",".join([mid] + terms[2:]) + "->" + out_term, head, *xs[2:],
                         epilogue=epilogue, out_dtype=out_dtype)
    ta, tb = terms
    a, b = xs
    out_dtype = out_dtype or a.dtype
    # dims that occur in one operand only and not in the output are summed first
    for which, (t, other) in enumerate(((ta, tb), (tb, ta))):
      lone = [l for l in t if l not in other and l not in out_term]
      if lone and gemm_hook is not None:
        raise HookDeclined()
      if lone:
        kept = "".join(l for l in t if l not in lone)
        reduced = self.einsum_naive(t + "->" + kept, a if which == 0 else b)
        if which == 0:
          a, ta = reduced, kept
        else:
          b, tb = reduced, kept
    sizes = {}
    for term, x in ((ta, a), (tb, b)):
      for letter, s in zip(term, x.shape):
        sizes[letter] = s
    batch = [l for l in out_term if l in ta and l in tb]
    m_dims = [l for l in out_term if l in ta and l not in tb]
    n_dims = [l for l in out_term if l in tb and l not in ta]
    k_dims = [l for l in ta if l in tb and l not in out_term]
    if not k_dims or not a.dtype.is_floating:
      if gemm_hook is not None:
        raise HookDeclined()
      return self.einsum_naive(ta + "," + tb + "->" + out_term, a, b)
    sa, sb = dict(zip(ta, a.strides)), dict(zip(tb, b.strides))

    def collapse(dims, strides):
      """(extent, stride) of the dims taken as one axis, or None; a dim the
      tensor lacks has stride 0."""
      dims = [d for d in dims if sizes[d] != 1]
      if not dims:
        return 1, 0
      for hi, lo in zip(dims[:-1], dims[1:]):
        if strides.get(hi, 0) != strides.get(lo, 0) * sizes[lo]:
          return None
      return _volume([sizes[d] for d in dims]), strides.get(dims[-1], 0)

    def plan_for(bt, md, nd):
      p = [collapse(bt, sa), collapse(bt, sb), collapse(md, sa), collapse(nd, sb),
           collapse(k_dims, sa), collapse(k_dims, sb)]
      return None if any(x is None for x in p) else p

    # The output is stored as [batch, M, N] and handed back as a view in the
    # requested dim order, so only the operands' layouts constrain the plan.
    plan = plan_for(batch, m_dims, n_dims)
    if (plan is None and not batch and gemm_hook is None and len(n_dims) > 1
        and _volume([sizes[l] for l in n_dims[1:]]) < self.MIN_GEMM_N
        and 4 * b.size <= a.size and plan_for([], m_dims, []) is not None
        and collapse(k_dims, sa) is not None):
      # Only the second operand's free dims fail to collapse (weights [heads, io, kv]:
      # heads and kv are apart), it is small beside the first, and taking its leading
      # free dim as a batch axis would leave products narrower than the kernel's tile:
      # a copy of it in [K, N] order makes ONE product of full width.  The result is
      # stored [M, N] and handed back as a view in the requested order.
      b = self.contiguous(self.transpose(b, [tb.index(l) for l in k_dims + n_dims]))
      tb = "".join(k_dims + n_dims)
      sb = dict(zip(tb, b.strides))
      plan = plan_for(batch, m_dims, n_dims)
    if plan is None and not batch:
      # a leading free dim that breaks the collapse (weights [heads, io, kv]) can
      # serve as the batch axis: the other operand is simply reused for each
      for cand in ((n_dims[:1], m_dims, n_dims[1:]), (m_dims[:1], m_dims[1:], n_dims)):
        if cand[0] and plan_for(*cand) is not None:
          batch, m_dims, n_dims = cand
          plan = plan_for(batch, m_dims, n_dims)
          break
    store = batch + m_dims + n_dims
    view_perm = [store.index(l) for l in out_term]
    if plan is None and gemm_hook is not None:
      raise HookDeclined()
    if plan is None:
      # pack to [batch, M, K] x [batch, K, N] first
      pa = self.contiguous(self.transpose(a, [ta.index(l) for l in batch + m_dims + k_dims]))
      pb = self.contiguous(self.transpose(b, [tb.index(l) for l in batch + k_dims + n_dims]))
      res = self.einsum("".join(batch + m_dims + k_dims) + "," + "".join(batch + k_dims + n_dims)
                        + "->" + "".join(store), pa, pb, epilogue=epilogue, out_dtype=out_dtype)
      return self.transpose(res, view_perm)
    (nb, a_b), (_, b_b), (m, a_m), (n, b_n), (k, a_k), (_, b_k) = plan
    if gemm_hook is not None and not (
        nb == 1 and epilogue == nat.EPILOGUE_NONE and a.dtype.name == "bfloat16"
        and b.dtype.name == "bfloat16" and out_dtype.name == "bfloat16"):
      raise HookDeclined()
    if (out_buf is not None and view_perm == list(range(len(store))) and out_buf.is_contiguous
        and out_buf.dtype == out_dtype):
      out = out_buf
    else:
      out = self._empty([sizes[l] for l in store], out_dtype)
    c_b, c_m, c_n = m * n, n, 1
    result = out if view_perm == list(range(len(store))) else self.transpose(out, view_perm)
    if (a.dtype.name == "float32" and out_dtype.name == "float32" and a.origin is not None
        and b.origin is not None and k <= self.FP32_TENSOR_CORE_MAX_K and gemm_hook is None):
      # both operands are widened bfloat16 arrays (float32 attention logits of bf16 queries
      # and keys): the bf16 product with fp32 accumulation IS the float32 contraction
      d = nat.GemmDesc()
      d.batch, d.m, d.n, d.k = nb, m, n, k
      d.a_batch, d.a_m, d.a_k = a_b, a_m, a_k
      d.b_batch, d.b_k, d.b_n = b_b, b_k, b_n
      d.c_batch, d.c_m, d.c_n = c_b, c_m, c_n
      d.in_dtype, d.out_dtype = nat.BF16, nat.F32
      d.epilogue, d.force_path = epilogue, 0
      self._call(self._lib.mtfc_gemm, ctypes.byref(d), ctypes.c_void_p(a.origin.ptr),
                 ctypes.c_void_p(b.origin.ptr), ctypes.c_void_p(out.ptr), self._stream())
      return result
    if (a.dtype.name == "float32" and out_dtype.name == "float32" and nb == 1 and k % 4 == 0
        and epilogue == nat.EPILOGUE_NONE and gemm_hook is None
        and (a.origin is not None) != (b.origin is not None)
        and m * n * k >= self.FP32_TENSOR_CORE_MIN_WORK):
      # One operand is a widened bfloat16 array (activations meeting fp32 router weights or
      # their gradients): its values go to the tensor cores as they are, only the other
      # operand is split into three bf16 terms, and the three exact partial products
      # (times the K chunks that keep each accumulation short) are added in fp32.  Half the
      # tensor-core work of the six-term product and no pass over the large operand.
      chunks = -(-k // self.FP32_TENSOR_CORE_MAX_K)
      while chunks <= 8192 and (k % chunks or (k // chunks) % 4):
        chunks += 1
      if chunks <= 8192:
        kk = k // chunks
        a_exact = a.origin is not None
        rows = n if a_exact else m
        s_arr, s_row, s_k = (b, b_n, b_k) if a_exact else (a, a_m, a_k)
        s3 = self._empty([chunks, rows, 6 * kk], G.bfloat16)
        self._call(self._lib.mtfc_split_bf16x3, ctypes.c_void_p(s_arr.ptr), kk * s_k, s_row, s_k,
                   ctypes.c_void_p(s3.ptr), chunks, rows, kk, 1 if a_exact else 0, self._stream())
        part = self._empty([3, chunks, m, n], G.float32)
        exact = (a if a_exact else b).origin
        for term in range(3):      # the first three K blocks of a split row are its three terms
          d = nat.GemmDesc()
          d.batch, d.m, d.n, d.k = chunks, m, n, kk
          if a_exact:
            d.a_batch, d.a_m, d.a_k = kk * a_k, a_m, a_k
            d.b_batch, d.b_k, d.b_n = rows * 6 * kk, 1, 6 * kk
            pa, pb = exact.ptr, s3.ptr + term * kk * 2
          else:
            d.a_batch, d.a_m, d.a_k = rows * 6 * kk, 6 * kk, 1
            d.b_batch, d.b_k, d.b_n = kk * b_k, b_k, b_n
            pa, pb = s3.ptr + term * kk * 2, exact.ptr
          d.c_batch, d.c_m, d.c_n = m * n, n, 1
          d.in_dtype, d.out_dtype = nat.BF16, nat.F32
          d.epilogue, d.force_path = nat.EPILOGUE_NONE, 0
          self._call(self._lib.mtfc_gemm, ctypes.byref(d), ctypes.c_void_p(pa), ctypes.c_void_p(pb),
                     ctypes.c_void_p(part.ptr + term * chunks * m * n * 4), self._stream())
        total = self.reshape(self.reduce("SUM", part, [0, 1]), [sizes[l] for l in store])
        return total if view_perm == list(range(len(store))) else self.transpose(total, view_perm)
    if (a.dtype.name == "float32" and out_dtype.name == "float32" and k % 4 == 0
        and k <= self.FP32_TENSOR_CORE_MAX_K
        and nb * m * n * k >= self.FP32_TENSOR_CORE_MIN_WORK):
      # fp32 on the tensor cores: split both operands into three bf16 terms along
      # K and run one bf16 GEMM over 6K with fp32 accumulation
      na, nbb = (nb if a_b else 1), (nb if b_b else 1)
      a3 = self._empty([na, m, 6 * k], G.bfloat16)
      b3 = self._empty([nbb, n, 6 * k], G.bfloat16)
      self._call(self._lib.mtfc_split_bf16x3, ctypes.c_void_p(a.ptr), a_b, a_m, a_k,
                 ctypes.c_void_p(a3.ptr), na, m, k, 0, self._stream())
      self._call(self._lib.mtfc_split_bf16x3, ctypes.c_void_p(b.ptr), b_b, b_n, b_k,
                 ctypes.c_void_p(b3.ptr), nbb, n, k, 1, self._stream())
      d = nat.GemmDesc()
      d.batch, d.m, d.n, d.k = nb, m, n, 6 * k
      d.a_batch, d.a_m, d.a_k = (m * 6 * k if a_b else 0), 6 * k, 1
      d.b_batch, d.b_k, d.b_n = (n * 6 * k if b_b else 0), 1, 6 * k
      d.c_batch, d.c_m, d.c_n = c_b, c_m, c_n
      d.in_dtype, d.out_dtype = nat.BF16, nat.F32
      d.epilogue, d.force_path = epilogue, 0
      self._call(self._lib.mtfc_gemm, ctypes.byref(d), ctypes.c_void_p(a3.ptr),
                 ctypes.c_void_p(b3.ptr), ctypes.c_void_p(out.ptr), self._stream())
      return result
    if (a.dtype.name == "float32" and out_dtype.name == "float32" and nb == 1
        and k > self.FP32_TENSOR_CORE_MAX_K and epilogue == nat.EPILOGUE_NONE
        and gemm_hook is None and m * n * k >= self.FP32_TENSOR_CORE_MIN_WORK):
      # a long fp32 contraction (a weight gradient summed over all tokens): cut K into
      # chunks short enough for the split-bf16 product, run them as one batched
      # product into fp32 partial sums and add the partial sums in fp32
      chunks = -(-k // self.FP32_TENSOR_CORE_MAX_K)
      while chunks <= 8192 and (k % chunks or (k // chunks) % 4):
        chunks += 1
      if chunks <= 8192:
        kk = k // chunks
        a3 = self._empty([chunks, m, 6 * kk], G.bfloat16)
        b3 = self._empty([chunks, n, 6 * kk], G.bfloat16)
        self._call(self._lib.mtfc_split_bf16x3, ctypes.c_void_p(a.ptr), kk * a_k, a_m, a_k,
                   ctypes.c_void_p(a3.ptr), chunks, m, kk, 0, self._stream())
        self._call(self._lib.mtfc_split_bf16x3, ctypes.c_void_p(b.ptr), kk * b_k, b_n, b_k,
                   ctypes.c_void_p(b3.ptr), chunks, n, kk, 1, self._stream())
        part = self._empty([chunks, m, n], G.float32)
        d = nat.GemmDesc()
        d.batch, d.m, d.n, d.k = chunks, m, n, 6 * kk
        d.a_batch, d.a_m, d.a_k = m * 6 * kk, 6 * kk, 1
        d.b_batch, d.b_k, d.b_n = n * 6 * kk, 1, 6 * kk
        d.c_batch, d.c_m, d.c_n = m * n, n, 1
        d.in_dtype, d.out_dtype = nat.BF16, nat.F32
        d.epilogue, d.force_path = nat.EPILOGUE_NONE, 0
        self._call(self._lib.mtfc_gemm, ctypes.byref(d), ctypes.c_void_p(a3.ptr),
                   ctypes.c_void_p(b3.ptr), ctypes.c_void_p(part.ptr), self._stream())
        total = self.reshape(self.reduce("SUM", part, [0]), [sizes[l] for l in store])
        return total if view_perm == list(range(len(store))) else self.transpose(total, view_perm)
    d = nat.GemmDesc()
    d.batch, d.m, d.n, d.k = nb, m, n, k
    d.a_batch, d.a_m, d.a_k = a_b, a_m, a_k
    d.b_batch, d.b_k, d.b_n = b_b, b_k, b_n
    d.c_batch, d.c_m, d.c_n = c_b, c_m, c_n
    d.in_dtype = _CODE[a.dtype.name]
    d.out_dtype = _CODE[out_dtype.name]
    d.epilogue = epilogue
    d.force_path = 0
    if gemm_hook is not None:
      hooked = gemm_hook(d, a.ptr, b.ptr, [sizes[l] for l in store])
      if hooked is None:
        raise HookDeclined()
      return hooked if view_perm == list(range(len(store))) else self.transpose(hooked, view_perm)
    self._call(self._lib.mtfc_gemm, ctypes.byref(d), ctypes.c_void_p(a.ptr),
               ctypes.c_void_p(b.ptr), ctypes.c_void_p(out.ptr), self._stream())
    return result

  # ---------------------------------------------------------------- attention
  def attention(self, q, k, v, causal):
    """softmax(q.k^T [+ causal bias]).v over [..., heads, length, d] slices.

    bf16 inputs with head size 64 or 128 run on the fused flash-style kernel
    (logits stay in TMEM); anything else is composed from the einsum / softmax
    kernels with the same arithmetic as the op-by-op lowering.
    """
    lead = q.shape[:-3]
    h, lq, d = q.shape[-3:]
    lk = k.shape[-2]

    def as_bhld(x):
      """View as [batch, h, l, d] with one batch stride (packing if necessary)."""
      nb = _volume(lead)
      dims = [i for i, s_ in enumerate(lead) if s_ != 1]
      ok = all(x.strides[a] == x.strides[b] * x.shape[b] for a, b in zip(dims[:-1], dims[1:]))
      if not ok:
        x = self.contiguous(x)
      bstride = x.strides[dims[-1]] if dims else 0
      return DeviceArray(x.buf, (nb,) + tuple(x.shape[-3:]), x.dtype,
                         strides=(bstride,) + tuple(x.strides[-3:]), offset=x.offset)
    if q.dtype.name == "bfloat16":
      qv, kv, vv = as_bhld(q), as_bhld(k), as_bhld(v)
      # stored [..., length, heads, d] so that a following output projection can
      # contract (heads, d) as one contiguous axis; returned as a [..., heads, length, d] view
      nl = len(lead)
      stored = self._empty(tuple(lead) + (lq, h, v.shape[-1]), q.dtype)
      out = self.transpose(stored, list(range(nl)) + [nl + 1, nl, nl + 2])
      ov = as_bhld(out)
      strides = [_i64(t.strides) for t in (qv, kv, vv, ov)]
      if v.shape[-1] == d and self._lib.mtfc_attention_supported(d, *strides) == 1 and all(
          t.ptr % 16 == 0 for t in (qv, kv, vv, ov)):
        self._call(self._lib.mtfc_attention_fwd, ctypes.c_void_p(qv.ptr), ctypes.c_void_p(kv.ptr),
                   ctypes.c_void_p(vv.ptr), ctypes.c_void_p(ov.ptr), qv.shape[0], h, lq, lk, d,
                   *strides, 1 if causal else 0, ctypes.c_float(1.0), self._stream())
        return out
    return self._attention_unfused(q, k, v, causal)

  def _attention_unfused(self, q, k, v, causal):
    lq, lk = q.shape[-2], k.shape[-2]
    nd = len(q.shape)
    letters = "abcdefgh"[:nd - 2]
    qf, kf = self.cast(q, G.float32), self.cast(k, G.float32)
    logits = self.einsum("%sxd,%syd->%sxy" % (letters, letters, letters), qf, kf)
    if causal:
      qpos = self.reshape(self.range(lq, G.float32), [lq, 1])
      kpos = self.reshape(self.range(lk, G.float32), [1, lk])
      bias = self.binary("multiply", self.cast(self.binary("less", qpos, kpos), G.float32), -1e9)
      logits = self.binary("add", logits, bias)
    mx = self.expand_dims(self.reduce("MAX", logits, [nd - 1]), nd - 1)
    shifted = self.binary("sub", logits, mx)
    lse = self.binary("add", self.unary("log", self.expand_dims(
        self.reduce("SUM", self.unary("exp", shifted), [nd - 1]), nd - 1)), mx)
    w = self.cast(self.unary("exp", self.binary("sub", logits, lse)), v.dtype)
    return self.einsum("%sxy,%sye->%sxe" % (letters, letters, letters), w, v)

  # ---------------------------------------------------------------- block rows
  def norm_rows(self, x, scale, bias, epsilon, centered):
    """Layer norm (centered) or RMS norm over the last axis; scale / bias [cols] or None."""
    x = self.contiguous(x)
    cols = x.shape[-1]
    rows = x.size // max(1, cols)
    out = self._empty(x.shape, x.dtype)
    sp = ctypes.c_void_p(self.contiguous(scale).ptr) if scale is not None else ctypes.c_void_p(0)
    bp = ctypes.c_void_p(self.contiguous(bias).ptr) if bias is not None else ctypes.c_void_p(0)
    self._call(self._lib.mtfc_norm_rows, ctypes.c_void_p(x.ptr), sp, bp, ctypes.c_void_p(out.ptr),
               _CODE[x.dtype.name], rows, cols, ctypes.c_float(epsilon), 1 if centered else 0,
               self._stream())
    return out

  def gather_rows(self, table, indices, first_row):
    """out[..., :] = table[indices[...] - first_row, :] (zeros outside the table):
    table [rows, *rest], indices any shape -> indices.shape + rest."""
    table, indices = self.contiguous(table), self.contiguous(indices)
    rest = tuple(table.shape[1:])
    row_bytes = _volume(rest) * table.dtype.itemsize
    out = self._empty(tuple(indices.shape) + rest, table.dtype)
    if row_bytes % 16 != 0:
      raise ValueError("gather_rows: rows of %d bytes are not a multiple of 16" % row_bytes)
    self._call(self._lib.mtfc_gather_rows, ctypes.c_void_p(table.ptr), ctypes.c_void_p(indices.ptr),
               ctypes.c_void_p(out.ptr), indices.size, table.shape[0], first_row, row_bytes,
               self._stream())
    return out

  def xent_stats(self, logits, targets, first_col):
    """Per row of the last axis: (max, sum exp(x - max), logit of the target or 0)."""
    logits, targets = self.contiguous(logits), self.contiguous(targets)
    cols = logits.shape[-1]
    lead = tuple(logits.shape[:-1])
    outs = [self._empty(lead, G.float32) for _ in range(3)]
    self._call(self._lib.mtfc_xent_stats, ctypes.c_void_p(logits.ptr), _CODE[logits.dtype.name],
               ctypes.c_void_p(targets.ptr), _volume(lead), cols, first_col,
               *[ctypes.c_void_p(o.ptr) for o in outs], self._stream())
    return tuple(outs)

  def xent_grad(self, logits, targets, log_z, dloss, z_loss, first_col):
    logits, targets = self.contiguous(logits), self.contiguous(targets)
    log_z, dloss = self.contiguous(log_z), self.contiguous(dloss)
    cols = logits.shape[-1]
    out = self._empty(logits.shape, logits.dtype)
    self._call(self._lib.mtfc_xent_grad, ctypes.c_void_p(logits.ptr), _CODE[logits.dtype.name],
               ctypes.c_void_p(targets.ptr), ctypes.c_void_p(log_z.ptr), ctypes.c_void_p(dloss.ptr),
               ctypes.c_float(z_loss), logits.size // max(1, cols), cols, first_col,
               ctypes.c_void_p(out.ptr), self._stream())
    return out

  # ---------------------------------------------------------------- fused MoE
  def moe_gate_logits(self, x, w):
    """[tokens, parts*experts] fp32 gate logits and `parts`.

    bf16 activations against the fp32 gate kernel run on the tensor cores with
    the kernel split in three bf16 terms; fp32 activations use the FFMA GEMM.
    """
    m, e = w.shape
    tokens = x.size // m
    x2 = self.reshape(x, [tokens, m])
    w = self.contiguous(w)
    if x.dtype.name == "bfloat16":
      w3 = self._empty([m, 3 * e], G.bfloat16)
      self._call(self._lib.mtfc_moe_split_gate_weights, ctypes.c_void_p(w.ptr), m, e,
                 ctypes.c_void_p(w3.ptr), self._stream())
      return self.einsum("tm,me->te", x2, w3, out_dtype=G.float32), 3
    return self.einsum("tm,me->te", self.cast(x2, G.float32), w), 1

  def moe_top2_gating_from_logits(self, logits, parts, lead_shape, group_size, experts, capacity,
                                  policy, threshold, noise, num_groups_total, want_raw=False):
    groups = _volume(lead_shape)
    tok_shape = tuple(lead_shape) + (group_size,)
    logits = self.contiguous(logits)
    i1, i2, p1, p2 = [self._empty(tok_shape, G.int32) for _ in range(4)]
    g1, g2 = self._empty(tok_shape, G.float32), self._empty(tok_shape, G.float32)
    raw = self._empty(tok_shape + (experts,), G.float32) if want_raw else None
    loss_per_group = self._empty([groups], G.float32)
    noise_ptr = ctypes.c_void_p(self.contiguous(noise).ptr) if noise is not None else ctypes.c_void_p(0)
    self._call(self._lib.mtfc_moe_top2_gating, ctypes.c_void_p(logits.ptr), parts, groups,
               group_size, experts, capacity, _POLICY[policy], ctypes.c_float(threshold),
               noise_ptr, ctypes.c_void_p(i1.ptr), ctypes.c_void_p(i2.ptr),
               ctypes.c_void_p(p1.ptr), ctypes.c_void_p(p2.ptr), ctypes.c_void_p(g1.ptr),
               ctypes.c_void_p(g2.ptr), ctypes.c_void_p(raw.ptr if raw is not None else 0),
               ctypes.c_void_p(loss_per_group.ptr), self._stream())
    loss = self.binary("multiply", self.reduce("SUM", loss_per_group, [0]),
                       1.0 / float(num_groups_total))
    result = (i1, i2, p1, p2, g1, g2, loss)
    return result + (raw,) if want_raw else result

  def moe_top2_gating(self, x, w, capacity, policy, threshold, noise, num_groups_total,
                      want_table=False, want_raw=False):
    """Fused `_top_2_gating` on one slice: x [..., S, M], w [M, E].

    Returns (index_1, index_2, position_1, position_2, gate_1, gate_2, loss)
    plus, with `want_table`, the [groups, E, capacity] slot table that
    moe_dispatch reads and, with `want_raw`, the softmax outputs.  bf16
    activations take the single-pass tcgen05 kernel (x is read once); other
    cases form the logits with a GEMM first."""
    m, e = w.shape
    lead, s = tuple(x.shape[:-2]), x.shape[-2]
    if (x.dtype.name == "bfloat16" and x.size > 0 and ((s + 63) // 64) * e <= 8192
        and self._lib.mtfc_moe_gate_fused_supported(m, e) == 1):
      return self._moe_gate_fused(x, w, capacity, policy, threshold, noise, num_groups_total,
                                  want_table, want_raw)
    logits, parts = self.moe_gate_logits(x, w)
    res = self.moe_top2_gating_from_logits(
        logits, parts, lead, s, e, capacity, policy, threshold, noise, num_groups_total,
        want_raw=want_raw)
    if want_table:
      table = self.moe_slot_table(*res[:6], e, capacity, x.dtype.name == "bfloat16")
      res = res[:7] + (table,) + res[7:]
    return res

  def _moe_gate_fused(self, x, w, capacity, policy, threshold, noise, num_groups_total,
                      want_table, want_raw):
    m, e = w.shape
    lead, s = tuple(x.shape[:-2]), x.shape[-2]
    groups = _volume(lead)
    x = self.contiguous(x)
    w = self.contiguous(w)
    ep = int(self._lib.mtfc_moe_gate_padded_experts(e))
    w3t = self._empty([3 * ep, m], G.bfloat16)
    self._call(self._lib.mtfc_moe_gate_prepare, ctypes.c_void_p(w.ptr), m, e,
               ctypes.c_void_p(w3t.ptr), self._stream())
    tok_shape = lead + (s,)
    i1, i2, p1, p2 = [self._empty(tok_shape, G.int32) for _ in range(4)]
    g1, g2 = self._empty(tok_shape, G.float32), self._empty(tok_shape, G.float32)
    raw = self._empty(tok_shape + (e,), G.float32) if want_raw else None
    table = self._empty(lead + (e, capacity), G.int32) if want_table else None
    loss_per_group = self._empty([groups], G.float32)
    loss = self._empty([], G.float32)
    nbytes = int(self._lib.mtfc_moe_gate_scratch_bytes(groups, s, e))
    scratch = self._empty([max(1, nbytes // 4)], G.float32)
    noise_ptr = ctypes.c_void_p(self.contiguous(noise).ptr) if noise is not None else ctypes.c_void_p(0)
    self._call(self._lib.mtfc_moe_gate_top2, ctypes.c_void_p(x.ptr), ctypes.c_void_p(w3t.ptr),
               groups, s, m, e, capacity, _POLICY[policy], ctypes.c_float(threshold), noise_ptr,
               ctypes.c_void_p(i1.ptr), ctypes.c_void_p(i2.ptr), ctypes.c_void_p(p1.ptr),
               ctypes.c_void_p(p2.ptr), ctypes.c_void_p(g1.ptr), ctypes.c_void_p(g2.ptr),
               ctypes.c_void_p(raw.ptr if raw is not None else 0),
               ctypes.c_void_p(loss_per_group.ptr), ctypes.c_void_p(loss.ptr), num_groups_total,
               ctypes.c_void_p(table.ptr if table is not None else 0), 1,
               ctypes.c_void_p(scratch.ptr), nbytes, self._stream())
    res = (i1, i2, p1, p2, g1, g2, loss)
    if want_table:
      res += (table,)
    if want_raw:
      res += (raw,)
    return res

  def moe_slot_table(self, i1, i2, p1, p2, g1, g2, num_experts, capacity, round_bf16):
    """[groups..., E, capacity] int32: token held by each expert slot, -1 if none."""
    lead, s = tuple(i1.shape[:-1]), i1.shape[-1]
    args = [self.contiguous(t) for t in (i1, i2, p1, p2, g1, g2)]
    table = self._empty(lead + (num_experts, capacity), G.int32)
    self._call(self._lib.mtfc_moe_slot_table, *[ctypes.c_void_p(t.ptr) for t in args],
               _volume(lead), s, num_experts, capacity, 1 if round_bf16 else 0,
               ctypes.c_void_p(table.ptr), self._stream())
    return table

  def moe_dispatch(self, x, i1, i2, p1, p2, g1, g2, num_experts, capacity, table=None):
    o, g, s, m = x.shape
    x = self.contiguous(x)
    if table is None:
      table = self.moe_slot_table(i1, i2, p1, p2, g1, g2, num_experts, capacity,
                                  x.dtype.name == "bfloat16")
    table = self.contiguous(table)
    out = self._empty([o, num_experts, g, capacity, m], x.dtype)
    self._call(self._lib.mtfc_moe_dispatch, ctypes.c_void_p(x.ptr), ctypes.c_void_p(table.ptr),
               ctypes.c_void_p(out.ptr), o, g, s, num_experts, capacity, m * x.dtype.itemsize,
               self._stream())
    return out

  def moe_dispatch_weighted(self, x, i1, i2, p1, p2, g1, g2, num_experts, capacity, table=None):
    """Backward of moe_combine w.r.t. the expert outputs: like moe_dispatch, with
    every row scaled by the gate of the choice that filled the slot."""
    o, g, s, m = x.shape
    x = self.contiguous(x)
    if table is None:
      table = self.moe_slot_table(i1, i2, p1, p2, g1, g2, num_experts, capacity,
                                  x.dtype.name == "bfloat16")
    table = self.contiguous(table)
    a1, ap1, ag1, ag2 = [self.contiguous(t) for t in (i1, p1, g1, g2)]
    out = self._empty([o, num_experts, g, capacity, m], x.dtype)
    self._call(self._lib.mtfc_moe_dispatch_weighted, ctypes.c_void_p(x.ptr), _CODE[x.dtype.name],
               ctypes.c_void_p(table.ptr), ctypes.c_void_p(a1.ptr), ctypes.c_void_p(ap1.ptr),
               ctypes.c_void_p(ag1.ptr), ctypes.c_void_p(ag2.ptr), ctypes.c_void_p(out.ptr), o, g, s,
               num_experts, capacity, m, self._stream())
    return out

  def moe_gate_grad(self, logits, i1, i2, g1, g2, dg1, dg2, dloss, num_groups_total, top1_only):
    """d logits of the gating from the gradients of (gate_1, gate_2, loss); any of the three
    may be None.  logits [..., S, E] float32, E <= 64."""
    s, e = logits.shape[-2:]
    groups = _volume(logits.shape[:-2])
    logits = self.contiguous(logits)
    fixed = [self.contiguous(t) for t in (i1, i2, g1, g2)]
    grads = [None if t is None else self.contiguous(t) for t in (dg1, dg2, dloss)]
    out = self._empty(logits.shape, G.float32)
    ptr = lambda t: ctypes.c_void_p(0 if t is None else t.ptr)
    self._call(self._lib.mtfc_moe_gate_grad, ptr(logits), *[ptr(t) for t in fixed],
               *[ptr(t) for t in grads], groups, s, e, num_groups_total, 1 if top1_only else 0,
               ptr(out), self._stream())
    return out

  def moe_combine_gate_grad(self, y, dout, i1, i2, p1, p2, g1, g2):
    """Backward of moe_combine w.r.t. the two gates: per token, the dot product
    of its output gradient with the expert row each kept choice read."""
    o, e, g, c, m = y.shape
    s = i1.shape[-1]
    y, dout = self.contiguous(y), self.contiguous(dout)
    args = [self.contiguous(t) for t in (i1, i2, p1, p2, g1, g2)]
    d1, d2 = self._empty([o, g, s], G.float32), self._empty([o, g, s], G.float32)
    self._call(self._lib.mtfc_moe_combine_gate_grad, ctypes.c_void_p(y.ptr), ctypes.c_void_p(dout.ptr),
               _CODE[y.dtype.name], *[ctypes.c_void_p(t.ptr) for t in args], ctypes.c_void_p(d1.ptr),
               ctypes.c_void_p(d2.ptr), o, g, s, e, c, m, self._stream())
    return d1, d2

  def moe_combine(self, y, i1, i2, p1, p2, g1, g2):
    o, e, g, c, m = y.shape
    s = i1.shape[-1]
    y = self.contiguous(y)
    args = [self.contiguous(t) for t in (i1, i2, p1, p2, g1, g2)]
    out = self._empty([o, g, s, m], y.dtype)
    self._call(self._lib.mtfc_moe_combine, ctypes.c_void_p(y.ptr), _CODE[y.dtype.name],
               *[ctypes.c_void_p(t.ptr) for t in args], ctypes.c_void_p(out.ptr), o, g, s, e, c,
               m, self._stream())
    return out


def _union(terms):
  seen = []
  for t in terms:
    for l in t:
      if l not in seen:
        seen.append(l)
  return "".join(seen)
