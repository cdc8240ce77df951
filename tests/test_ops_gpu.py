"""DeviceOps (libmtfc kernels through the C ABI) against the numpy oracle, op by op."""

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


def _pair(both, value, dtype):
  dev, ora = both
  return dev.from_host(value, dtype), ora.from_host(value, dtype)


def _check(both, got, ref, tol=0.0):
  dev, ora = both
  g, r = dev.to_host(got), ora.to_host(ref)
  assert g.shape == r.shape
  if tol == 0.0:
    np.testing.assert_array_equal(g, r)
  else:
    assert rel_err(g, r) <= tol


UNARY = ["relu", "exp", "log", "negative", "reciprocal", "sqrt", "rsqrt", "square", "tanh",
         "sigmoid", "sign"]


@pytest.mark.parametrize("dtype", [mtf.float32, mtf.bfloat16])
@pytest.mark.parametrize("name", UNARY)
def test_unary(both, name, dtype):
  dev, ora = both
  v = rng(1).standard_normal((7, 33)).astype(np.float32)
  if name in ("log", "sqrt", "rsqrt"):
    v = np.abs(v) + 0.1
  a, b = _pair(both, v, dtype)
  exact = name in ("relu", "negative", "square", "sign")
  _check(both, dev.unary(name, a), ora.unary(name, b), 0.0 if exact else (1e-6 if dtype == mtf.float32 else 8e-3))


def test_cast_round_trip(both):
  dev, ora = both
  v = rng(2).standard_normal((5, 17)).astype(np.float32) * 100
  a, b = _pair(both, v, mtf.float32)
  for dt in (mtf.bfloat16, mtf.int32, mtf.bool_):
    _check(both, dev.cast(a, dt), ora.cast(b, dt))
  _check(both, dev.cast(dev.cast(a, mtf.bfloat16), mtf.float32), ora.cast(ora.cast(b, mtf.bfloat16), mtf.float32))
  i, j = _pair(both, np.arange(-5, 6), mtf.int32)
  _check(both, dev.cast(i, mtf.float32), ora.cast(j, mtf.float32))
  _check(both, dev.cast(i, mtf.bool_), ora.cast(j, mtf.bool_))


BINARY = ["add", "sub", "multiply", "divide", "maximum", "minimum", "less", "greater",
          "less_equal", "greater_equal", "equal", "not_equal"]


@pytest.mark.parametrize("name", BINARY)
def test_binary_broadcast(both, name):
  dev, ora = both
  r = rng(3)
  x = r.standard_normal((4, 1, 6)).astype(np.float32)
  y = r.standard_normal((1, 5, 6)).astype(np.float32)
  for dt in (mtf.float32, mtf.bfloat16):
    a, b = _pair(both, x, dt)
    c, d = _pair(both, y, dt)
    _check(both, dev.binary(name, a, c), ora.binary(name, b, d), 0.0 if dt == mtf.float32 and name != "divide" else 1e-6 if dt == mtf.float32 else 0.0)
    _check(both, dev.binary(name, a, 0.25), ora.binary(name, b, 0.25), 0.0 if name != "divide" else 1e-6)


def test_binary_int_and_views(both):
  dev, ora = both
  x = np.arange(24).reshape(2, 3, 4) - 7
  a, b = _pair(both, x, mtf.int32)
  for name in ("add", "multiply", "floordiv", "mod", "maximum", "less"):
    _check(both, dev.binary(name, a, 3), ora.binary(name, b, 3))
  at, bt = dev.transpose(a, [2, 0, 1]), ora.transpose(b, [2, 0, 1])
  _check(both, dev.binary("add", at, at), ora.binary("add", bt, bt))
  _check(both, dev.contiguous(at), ora.contiguous(bt))
  _check(both, dev.reshape(at, [4, 6]), ora.reshape(bt, [4, 6]))
  _check(both, dev.slice(at, [1, 0, 1], [2, 2, 2]), ora.slice(bt, [1, 0, 1], [2, 2, 2]))
  _check(both, dev.concat([at, at], 1), ora.concat([bt, bt], 1))
  _check(both, dev.expand_dims(at, 1), ora.expand_dims(bt, 1))
  _check(both, dev.broadcast_to(dev.expand_dims(a, 0), [3, 2, 3, 4]), ora.broadcast_to(ora.expand_dims(b, 0), [3, 2, 3, 4]))


@pytest.mark.parametrize("shape,elem", [((3, 5, 8), mtf.bfloat16), ((6, 16, 64), mtf.bfloat16), ((2, 4, 32), mtf.float32)])
def test_strided_copy_paths(both, shape, elem):
  """Scalar and 16-byte-vector paths of the strided copy kernel."""
  dev, ora = both
  v = rng(4).standard_normal(shape).astype(np.float32)
  a, b = _pair(both, v, elem)
  for perm in ([1, 0, 2], [2, 1, 0], [0, 2, 1]):
    _check(both, dev.contiguous(dev.transpose(a, perm)), ora.contiguous(ora.transpose(b, perm)))
  half = list(shape)
  half[1] //= 2 if shape[1] > 1 else 1
  _check(both, dev.contiguous(dev.slice(a, [0, 1, 0], [shape[0], max(1, shape[1] - 1), shape[2]])),
         ora.slice(b, [0, 1, 0], [shape[0], max(1, shape[1] - 1), shape[2]]))


@pytest.mark.parametrize("name", ["SUM", "MAX", "MIN"])
def test_reduce(both, name):
  dev, ora = both
  v = rng(5).standard_normal((6, 70, 9)).astype(np.float32)
  for dt, tol in ((mtf.float32, 1e-6), (mtf.bfloat16, 8e-3)):
    a, b = _pair(both, v, dt)
    for axes in ([1], [0, 2], [2], [0, 1, 2]):
      _check(both, dev.reduce(name, a, axes), ora.reduce(name, b, axes), tol if name == "SUM" else 0.0)
  i, j = _pair(both, np.arange(60).reshape(3, 4, 5), mtf.int32)
  _check(both, dev.reduce(name, i, [1]), ora.reduce(name, j, [1]))


def test_argmax_topk_gather_onehot(both):
  dev, ora = both
  v = rng(6).standard_normal((5, 9, 12)).astype(np.float32)
  v[0, 0, 3] = v[0, 0, 7] = 9.0   # tie -> lowest index
  a, b = _pair(both, v, mtf.float32)
  _check(both, dev.argmax(a), ora.argmax(b))
  gv, gi = dev.top_k(a, 4)
  rv, ri = ora.top_k(b, 4)
  _check(both, gv, rv)
  _check(both, gi, ri)
  _check(both, dev.gather_last(a, gi), ora.gather_last(b, ri))
  idx = np.array([[0, 3, 7], [-1, 8, 2]])
  i, j = _pair(both, idx, mtf.int32)
  for dt in (mtf.float32, mtf.bfloat16, mtf.int32):
    _check(both, dev.one_hot(i, 8, 1.0, 0.0, dt), ora.one_hot(j, 8, 1.0, 0.0, dt))
  _check(both, dev.one_hot(i, 8, -1e9, 0.0, mtf.float32), ora.one_hot(j, 8, -1e9, 0.0, mtf.float32))
  _check(both, dev.fill([3, 4], 2.5, mtf.bfloat16), ora.fill([3, 4], 2.5, mtf.bfloat16))
  _check(both, dev.range(37, mtf.float32), ora.range(37, mtf.float32))
  _check(both, dev.range(37, mtf.int32), ora.range(37, mtf.int32))


EINSUMS = [
    ("ab,bc->ac", [(37, 20), (20, 45)]),
    ("abc,cd->abd", [(3, 10, 16), (16, 24)]),
    ("abcde,bef->abcdf", [(1, 4, 3, 5, 16), (4, 16, 8)]),
    ("abcd,abed->abce", [(2, 3, 9, 8), (2, 3, 7, 8)]),
    ("abcd,abde->abce", [(2, 3, 9, 7), (2, 3, 7, 8)]),
    ("abc,dce->adbe", [(2, 9, 16), (3, 16, 8)]),
    ("abcd,bed->ace", [(2, 3, 9, 8), (3, 16, 8)]),
    ("abcd,abcef->aebfd", [(1, 2, 8, 16), (1, 2, 8, 3, 4)]),
    ("ab,ab->ab", [(5, 6), (5, 6)]),
    ("abc,ab->abc", [(4, 5, 6), (4, 5)]),
    ("abc,abc->a", [(4, 5, 6), (4, 5, 6)]),
    ("ab,bc,cd->ad", [(6, 8), (8, 16), (16, 5)]),
]


@pytest.mark.parametrize("eq,shapes", EINSUMS)
@pytest.mark.parametrize("dtype,tol", [(mtf.float32, 1e-5), (mtf.bfloat16, 2e-2)])
def test_einsum(both, eq, shapes, dtype, tol):
  dev, ora = both
  r = rng(7)
  vals = [r.standard_normal(s).astype(np.float32) for s in shapes]
  da = [dev.from_host(v, dtype) for v in vals]
  oa = [ora.from_host(v, dtype) for v in vals]
  _check(both, dev.einsum(eq, *da), ora.einsum(eq, *oa), tol)
  _check(both, dev.einsum_naive(eq, *da), ora.einsum_naive(eq, *oa), tol)


def test_einsum_tensor_core_shapes(both):
  """bf16 contractions large enough to span several 128x256 tiles and K blocks."""
  dev, ora = both
  r = rng(8)
  for eq, shapes in [("ab,bc->ac", [(300, 256), (256, 520)]),
                     ("abc,cd->abd", [(2, 160, 128), (128, 264)]),
                     ("abcde,bef->abcdf", [(1, 2, 3, 40, 64), (2, 64, 136)])]:
    vals = [r.standard_normal(s).astype(np.float32) for s in shapes]
    da = [dev.from_host(v, mtf.bfloat16) for v in vals]
    oa = [ora.from_host(v, mtf.bfloat16) for v in vals]
    _check(both, dev.einsum(eq, *da), ora.einsum(eq, *oa), 2e-2)
  from mesh_b200 import _native as nat
  nat.device_status()


@pytest.mark.parametrize("eq,shapes", [("ab,bc->ac", [(1024, 1024), (1024, 2048)]),
                                       ("ab,bc->ac", [(4096, 256), (256, 4096)]),
                                       ("abc,cd->abd", [(4, 300, 512), (512, 264)]),
                                       ("bmk,bkn->bmn", [(3, 256, 128), (3, 128, 320)])])
def test_fp32_einsum_on_tensor_cores(both, eq, shapes):
  """float32 contractions large enough for the 3-term bf16 split path must still
  meet the float32 tolerance (1e-5 relative) against a float64 reference."""
  dev, ora = both
  r = rng(9)
  vals = [r.standard_normal(s).astype(np.float32) for s in shapes]
  vals[1] = (vals[1] / np.sqrt(shapes[1][-2])).astype(np.float32)
  got = dev.to_host(dev.einsum(eq, *[dev.from_host(v, mtf.float32) for v in vals]))
  ref = np.einsum(eq, *[v.astype(np.float64) for v in vals])
  assert rel_err(got, ref) < 1e-5
  from mesh_b200 import _native as nat
  nat.device_status()


@pytest.mark.parametrize("eq,shapes,widened", [
    ("tm,me->te", [(4096, 1024), (1024, 32)], 0),        # router logits: activations x fp32 gate kernel
    ("te,tm->me", [(16384, 32), (16384, 1024)], 1),      # its gradient: a contraction over 16384 tokens
    ("te,tm->me", [(65536, 32), (65536, 512)], 1),       # ... and over 65536 (32 K chunks)
    ("ab,bc->ac", [(512, 1024), (1024, 2048)], 0)])
def test_fp32_einsum_with_a_widened_bf16_operand(both, eq, shapes, widened):
  """float32 einsum where one operand is a bfloat16 array cast up (DeviceOps.cast records
  that): the planner feeds the bfloat16 values to the tensor cores as they are and splits
  only the other operand; the result is the float32 contraction to 1e-5."""
  dev, ora = both
  r = rng(33)
  vals = [r.standard_normal(s).astype(np.float32) / np.sqrt(s[0] if i else 1.0) for i, s in enumerate(shapes)]
  arrays = []
  for i, v in enumerate(vals):
    if i == widened:
      narrow = dev.from_host(v, mtf.bfloat16)
      wide = dev.cast(narrow, mtf.float32)
      assert wide.origin is narrow
      vals[i] = dev.to_host(wide).astype(np.float32)       # the values actually multiplied
      arrays.append(wide)
    else:
      arrays.append(dev.from_host(v, mtf.float32))
      assert arrays[-1].origin is None
  got = dev.to_host(dev.einsum(eq, *arrays))
  ref = np.einsum(eq, *[v.astype(np.float64) for v in vals])
  assert rel_err(got, ref) < 1e-5
  # a view of the cast result carries no such record and takes the general path
  if len(shapes[widened]) == 2 and eq == "ab,bc->ac":
    view = dev.transpose(arrays[widened], [1, 0])
    assert view.origin is None


def test_fp32_einsum_of_two_widened_bf16_operands(both):
  """float32 logits of bfloat16 queries and keys (both cast up): one bfloat16 product with
  float32 accumulation, equal to the float32 contraction of the widened values."""
  dev, ora = both
  r = rng(34)
  q = r.standard_normal((2, 4, 256, 64)).astype(np.float32)
  k = r.standard_normal((2, 4, 384, 64)).astype(np.float32)
  wide, exact = [], []
  for v in (q, k):
    w = dev.cast(dev.from_host(v, mtf.bfloat16), mtf.float32)
    assert w.origin is not None
    wide.append(w)
    exact.append(dev.to_host(w).astype(np.float64))
  before = __import__("mesh_b200._native", fromlist=["x"]).launch_count()
  got = dev.to_host(dev.einsum("bhqd,bhkd->bhqk", *wide))
  assert __import__("mesh_b200._native", fromlist=["x"]).launch_count() - before == 1   # no operand split
  assert rel_err(got, np.einsum("bhqd,bhkd->bhqk", *exact)) < 1e-6


@pytest.mark.parametrize("n,shape", [(4, (16, 128)), (3, (8, 96)), (4, (5, 7)), (2, (64, 64))])
@pytest.mark.parametrize("dtype", [mtf.float32, mtf.bfloat16])
def test_in_process_allreduce_follows_the_reference_association(cuda_device, n, shape, dtype):
  """Grouped SUM over slices held by one process: the reference's ring allreduce
  cuts slices of >= 1024 elements in n shards and reduces shard s over the member
  list rotated by s (placement_mesh_impl.py:407-455); same order here, so the sums
  carry the same bits as the oracle's."""
  from mesh_b200.cuda_mesh_impl import CudaMeshImpl
  from oracle.numpy_mesh_impl import NumpyMeshImpl
  from oracle.numpy_ops import Arr, round_to_bf16
  r = rng(33)
  vals = [r.standard_normal(shape).astype(np.float32) for _ in range(n)]
  if dtype == mtf.bfloat16:
    vals = [round_to_bf16(v) for v in vals]
  dev = CudaMeshImpl("all:%d" % n, "", [0] * n)
  ora = NumpyMeshImpl("all:%d" % n, "")
  xd = dev.LaidOutTensor([dev.slice_ops.from_host(v, dtype) for v in vals])
  xo = ora.LaidOutTensor([Arr(v.copy(), dtype) for v in vals])
  for name in ("SUM", "MAX"):
    yd = dev.allreduce(xd, [0], name)
    yo = ora.allreduce(xo, [0], name)
    for a, b in zip(yd.tensor_list, yo.tensor_list):
      np.testing.assert_array_equal(dev.slice_ops.to_host(a), b.a)
