"""Mesh collectives of SlicedMeshImpl (the class CudaMeshImpl derives from)
without a GPU: the in-process group path against the oracle backend, and the
one-process-per-processor path over torch.distributed with the gloo backend
(world sizes 2 and 4), slice by slice against the oracle's slices."""

import os
import socket

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

from mesh_b200 import mtf
from oracle.numpy_mesh_impl import NumpyMeshImpl
from oracle.numpy_ops import Arr
from helpers import NumpySlicedMeshImpl, rel_err, rng

MESHES = [("all:4", "batch:all"), ("rows:2,cols:4", "batch:rows;d:cols"), ("all:2", "x:all")]


def _laid_out(impl, values, dtype=mtf.float32):
  return impl.LaidOutTensor([Arr(v.copy(), dtype) for v in values])


def _same(x, y, exact=True):
  for p, q in zip(x.tensor_list, y.tensor_list):
    assert p.a.shape == q.a.shape
    if exact:
      np.testing.assert_array_equal(p.a, q.a)
    else:
      assert rel_err(p.a, q.a) < 1e-6


@pytest.mark.parametrize("mesh,layout", MESHES)
def test_in_process_collectives_match_oracle(mesh, layout):
  ora, impl = NumpyMeshImpl(mesh, layout), NumpySlicedMeshImpl(mesh, layout)
  r = rng(0)
  vals = [r.standard_normal((4, 8, 6)).astype(np.float32) for _ in range(ora.size)]
  a, b = _laid_out(ora, vals), _laid_out(impl, vals)
  for axis in range(ora.ndims):
    n = ora.shape[axis].size
    for name in ("SUM", "MAX", "MIN"):
      _same(ora.allreduce(a, [axis], name), impl.allreduce(b, [axis], name), exact=(name != "SUM"))
    for ca in range(3):
      _same(ora.allconcat(a, axis, ca), impl.allconcat(b, axis, ca))
      for sa in range(3):
        if vals[0].shape[sa] % n == 0:
          _same(ora.alltoall(a, axis, sa, ca), impl.alltoall(b, axis, sa, ca))
    for offset, wrap in ((1, False), (-1, True), (n, False), (2, True)):
      _same(ora.shift_by_n_processors(a, axis, offset, wrap),
            impl.shift_by_n_processors(b, axis, offset, wrap))
    _same(ora.allsplit(a, axis, 1), impl.allsplit(b, axis, 1))
  every = list(range(ora.ndims))
  _same(ora.allreduce(a, every, "SUM"), impl.allreduce(b, every, "SUM"), exact=False)
  assert impl.allreduce(b, [], "SUM") is b


def test_collective_argument_errors():
  impl = NumpySlicedMeshImpl("all:4", "batch:all")
  x = _laid_out(impl, [np.zeros((6, 3), np.float32)] * 4)
  with pytest.raises(ValueError):
    impl.alltoall(x, 0, 0, 1)          # 6 rows do not split 4 ways
  with pytest.raises(ValueError):
    impl.allreduce(x, [0], "PROD")
  with pytest.raises(ValueError):
    impl.receive(x, 0, [0, 1])         # one source per group member is required


def _free_port():
  s = socket.socket()
  s.bind(("127.0.0.1", 0))
  port = s.getsockname()[1]
  s.close()
  return port


def _worker(rank, world, port, mesh, layout, out_dir):
  os.environ["MASTER_ADDR"] = "127.0.0.1"
  os.environ["MASTER_PORT"] = str(port)
  dist.init_process_group("gloo", rank=rank, world_size=world)
  try:
    ora = NumpyMeshImpl(mesh, layout)
    impl = NumpySlicedMeshImpl(mesh, layout, distributed=True, rank=rank)
    assert impl.local_pnums == [rank]
    r = rng(1)
    vals = [r.standard_normal((4, 8, 6)).astype(np.float32) for _ in range(world)]
    a = _laid_out(ora, vals)
    b = impl.LaidOutTensor([Arr(vals[rank].copy(), mtf.float32)])

    def check(x, y, exact=True):
      p, q = x.tensor_list[rank].a, y.tensor_list[0].a
      assert p.shape == q.shape, (p.shape, q.shape)
      if exact:
        np.testing.assert_array_equal(p, q)
      else:
        assert rel_err(q, p) < 1e-6
    for axis in range(ora.ndims):
      n = ora.shape[axis].size
      for name in ("SUM", "MAX", "MIN"):
        check(ora.allreduce(a, [axis], name), impl.allreduce(b, [axis], name), exact=(name != "SUM"))
        # the same started now and waited for by its first reader
        pending = impl.allreduce_start(b, [axis], name)
        assert list(pending.slice_shape) == list(b.slice_shape)
        check(ora.allreduce(a, [axis], name), pending.to_laid_out_tensor(), exact=(name != "SUM"))
      for ca in range(3):
        check(ora.allconcat(a, axis, ca), impl.allconcat(b, axis, ca))
        for sa in range(3):
          if vals[0].shape[sa] % n == 0:
            check(ora.alltoall(a, axis, sa, ca), impl.alltoall(b, axis, sa, ca))
      for offset, wrap in ((1, False), (-1, True), (2, True)):
        check(ora.shift_by_n_processors(a, axis, offset, wrap),
              impl.shift_by_n_processors(b, axis, offset, wrap))
    check(ora.allreduce(a, list(range(ora.ndims)), "SUM"),
          impl.allreduce(b, list(range(ora.ndims)), "SUM"), exact=False)

    # a whole graph: FFN with the contracted dim split, then export on every rank
    def ffn(backend):
      rr = rng(2)
      g = mtf.Graph()
      m = mtf.Mesh(g, "m")
      x = rr.standard_normal((8, 4, 16)).astype(np.float32)
      wi = rr.standard_normal((16, 32)).astype(np.float32) / 4
      wo = rr.standard_normal((32, 16)).astype(np.float32) / 6
      X = mtf.import_tf_tensor(m, x, "batch:8,length:4,d_model:16")
      WI = mtf.import_tf_tensor(m, wi, "d_model:16,d:32")
      WO = mtf.import_tf_tensor(m, wo, "d:32,d_model:16")
      y = mtf.layers.dense_relu_dense(X, mtf.Dimension("d", 32), wi=WI, wo=WO)
      # and its backward pass: the gradient einsums bring their own allreduces
      grads = mtf.gradients([mtf.reduce_sum(mtf.square(y))], [X, WI, WO])
      low = mtf.Lowering(g, {m: backend})
      return [low.export_to_tf_tensor(t) for t in [y] + grads], low.counter_totals()
    if "d:" in layout:
      got, cg = ffn(impl)
      ref, cr = ffn(ora)
      assert cg == cr
      for a_, b_ in zip(got, ref):
        assert rel_err(a_, b_) < 1e-5
    open(os.path.join(out_dir, "ok%d" % rank), "w").write("ok")
  finally:
    dist.destroy_process_group()


@pytest.mark.parametrize("world,mesh,layout", [(2, "all:2", "d:all"),
                                               (4, "rows:2,cols:2", "batch:rows;d:cols")])
def test_distributed_collectives_over_gloo(tmp_path, world, mesh, layout):
  mp.spawn(_worker, args=(world, _free_port(), mesh, layout, str(tmp_path)), nprocs=world, join=True)
  assert sorted(os.listdir(str(tmp_path))) == ["ok%d" % r for r in range(world)]


def _moe_worker(rank, world, port, out_dir):
  os.environ["MASTER_ADDR"] = "127.0.0.1"
  os.environ["MASTER_PORT"] = str(port)
  dist.init_process_group("gloo", rank=rank, world_size=world)
  try:
    mesh_shape, layout = "all:%d" % world, "batch:all;experts:all"

    def layer(backend):
      r = rng(6)
      g = mtf.Graph()
      m = mtf.Mesh(g, "m")
      b, l, d, f, e = 8, 32, 16, 32, 8
      x = r.standard_normal((b, l, d)).astype(np.float32)
      wg = (r.standard_normal((d, e)) / 4).astype(np.float32)
      wi = (r.standard_normal((e, d, f)) / 4).astype(np.float32)
      wo = (r.standard_normal((e, f, d)) / 6).astype(np.float32)
      X = mtf.import_tf_tensor(m, x, "batch:8,length:32,d_model:16", dtype=mtf.bfloat16)
      WG = mtf.import_tf_tensor(m, wg, "d_model:16,expert_unsplit:8", dtype=mtf.float32)
      WI = mtf.import_tf_tensor(m, wi, "experts:8,d_model:16,d_ff:32", dtype=mtf.bfloat16)
      WO = mtf.import_tf_tensor(m, wo, "experts:8,d_ff:32,d_model:16", dtype=mtf.bfloat16)
      hp = mtf.moe.HParams(moe_group_size=32, moe_second_policy_train="all")
      out, loss = mtf.moe.transformer_moe_layer_v1(
          X, mtf.Dimension("d_model", d), hp, True, mesh_shape, layout, WG, WI, WO)
      low = mtf.Lowering(g, {m: backend})
      return low.export_to_tf_tensor(out), float(low.export_to_tf_tensor(loss)), low.counter_totals()
    got, gl, cg = layer(NumpySlicedMeshImpl(mesh_shape, layout, distributed=True, rank=rank))
    ref, rl, cr = layer(NumpyMeshImpl(mesh_shape, layout))
    np.testing.assert_array_equal(got, ref)
    assert abs(gl - rl) < 1e-7 and cg == cr and cg["alltoall/0/reshape_op"] > 0
    open(os.path.join(out_dir, "ok%d" % rank), "w").write("ok")
  finally:
    dist.destroy_process_group()


def test_moe_layer_with_alltoall_over_gloo(tmp_path):
  mp.spawn(_moe_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
  assert sorted(os.listdir(str(tmp_path))) == ["ok0", "ok1"]


def _moe_v2_worker(rank, world, port, out_dir):
  os.environ["MASTER_ADDR"] = "127.0.0.1"
  os.environ["MASTER_PORT"] = str(port)
  dist.init_process_group("gloo", rank=rank, world_size=world)
  try:
    mesh_shape, layout = "all:%d" % world, "batch:all;expert_x:all"

    def layer(backend):
      r = rng(7)
      g = mtf.Graph()
      m = mtf.Mesh(g, "m")
      b, l, d, f, ex, ey = 4, 16, 8, 12, 2, 2
      imp = lambda a, spec: mtf.import_tf_tensor(m, a.astype(np.float32), spec)
      X = imp(r.standard_normal((b, l, d)), "batch:4,length:16,d_model:8")
      WGO = imp(r.standard_normal((d, ex)), "d_model:8,expert_x_unsplit:2")
      WGI = imp(r.standard_normal((ex, d, ey)), "expert_x:2,d_model:8,expert_y_unsplit:2")
      WI = imp(r.standard_normal((ey, ex, d, f)) / 3, "expert_y:2,expert_x:2,d_model:8,expert_hidden:12")
      WO = imp(r.standard_normal((ey, ex, f, d)) / 3, "expert_y:2,expert_x:2,expert_hidden:12,d_model:8")
      hp = mtf.moe.HParams(moe_num_experts=[ex, ey], moe_group_size=l, moe_second_policy_train="all",
                           moe_min_expert_capacity=2)
      out, loss = mtf.moe.transformer_moe_layer_v2(
          X, mtf.Dimension("d_model", d), hp, True, mesh_shape, layout, WGO, WGI, WI, WO)
      low = mtf.Lowering(g, {m: backend})
      return low.export_to_tf_tensor(out), float(low.export_to_tf_tensor(loss)), low.counter_totals()
    got, gl, cg = layer(NumpySlicedMeshImpl(mesh_shape, layout, distributed=True, rank=rank))
    ref, rl, cr = layer(NumpyMeshImpl(mesh_shape, layout))
    np.testing.assert_array_equal(got, ref)
    assert abs(gl - rl) < 1e-7 and cg == cr
    assert sum(v for k, v in cg.items() if k.startswith("alltoall")) > 0
    open(os.path.join(out_dir, "ok%d" % rank), "w").write("ok")
  finally:
    dist.destroy_process_group()


def test_two_level_moe_layer_over_gloo(tmp_path):
  """transformer_moe_layer_v2 with one process per processor: its layout changes run as
  real alltoalls between the processes and give the in-process oracle's bits."""
  mp.spawn(_moe_v2_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
  assert sorted(os.listdir(str(tmp_path))) == ["ok0", "ok1"]


def _train_worker(rank, world, port, out_dir):
  os.environ["MASTER_ADDR"] = "127.0.0.1"
  os.environ["MASTER_PORT"] = str(port)
  dist.init_process_group("gloo", rank=rank, world_size=world)
  try:
    from test_training_loop import _training_graph
    mesh_shape, layout = "rows:2,cols:2", "batch:rows;experts:rows;heads:cols;vocab:cols"

    def run(backend):
      g, m, loss, variables = _training_graph(mesh_shape, layout)
      losses = []
      for _ in range(3):
        low = mtf.Lowering(g, {m: backend})
        losses.append(float(low.export_to_tf_tensor(loss)))
      low.copy_slices_to_masters()
      return losses, [v.operation.get_master() for v in variables]
    got, got_vars = run(NumpySlicedMeshImpl(mesh_shape, layout, distributed=True, rank=rank))
    ref, ref_vars = run(NumpyMeshImpl(mesh_shape, layout))
    np.testing.assert_allclose(got, ref, rtol=1e-6)
    for a, b in zip(got_vars, ref_vars):
      np.testing.assert_allclose(a, b, rtol=1e-5, atol=1e-7)
    open(os.path.join(out_dir, "ok%d" % rank), "w").write("ok")
  finally:
    dist.destroy_process_group()


def test_training_steps_over_gloo(tmp_path):
  """Three training steps of the small block (MoE, split vocabulary, Adafactor on variables)
  with one process per processor: losses and updated weights equal the in-process oracle's."""
  mp.spawn(_train_worker, args=(4, _free_port(), str(tmp_path)), nprocs=4, join=True)
  assert sorted(os.listdir(str(tmp_path))) == ["ok0", "ok1", "ok2", "ok3"]


def test_move_packs_on_the_source_device():
  """CudaMeshImpl._move with distinct device ordinals in one process: a strided slice
  must be packed by a kernel launched on the device that holds it, and only then
  copied across; no kernel may be given pointers of another device."""
  from mesh_b200.cuda_mesh_impl import CudaMeshImpl

  class FakeBuf(object):
    def __init__(self, device):
      self.device = device
      self.moves = []

    def __getitem__(self, _):
      return self

    def to(self, dev):
      self.moves.append(dev)
      return FakeBuf(dev)

  class FakeSlice(object):
    def __init__(self, device, contiguous):
      self.buf, self.device = FakeBuf(device), device
      self.shape, self.dtype, self.offset, self.size = (4, 4), "f", 0, 16
      self.is_contiguous = contiguous

  class FakeOps(object):
    def __init__(self):
      self.device = "cuda:0"
      self.calls = []

    def contiguous(self, s):
      self.calls.append((self.device, s.device))      # (device the kernel runs on, data's device)
      return FakeSlice(s.device, True)

  impl = object.__new__(CudaMeshImpl)
  impl._devices = ["cuda:0", "cuda:1"]
  impl._ops = FakeOps()
  impl._device_array = lambda buf, shape, dtype: ("array", buf.device, tuple(shape))
  src = FakeSlice("cuda:1", contiguous=False)          # a strided view living on device 1
  moved = impl._move(src, 0)                           # wanted on processor 0's device
  assert impl._ops.calls == [("cuda:1", "cuda:1")]     # packed where the data is
  assert moved == ("array", "cuda:0", (4, 4))
  assert impl._ops.device == "cuda:0"                  # and the ops object ends on the destination
  same = FakeSlice("cuda:0", contiguous=True)
  assert impl._move(same, 0) is same                   # already there: untouched


def _walk_like_the_kernel(slices, plan, itemsize):
  """What mtfc_alltoall_peer stores, replayed over byte arrays: rank `me` copies, for
  every destination, every row of its part from the source offset to the output offset."""
  out_shape, lead, row_bytes, src_part_stride, dst_part_stride = plan
  n = len(slices)
  outs = [np.zeros(int(np.prod(out_shape)) * itemsize, np.uint8) for _ in range(n)]
  for me, s in enumerate(slices):
    src = np.ascontiguousarray(s).view(np.uint8).reshape(-1)
    rows = int(np.prod([d for d, _, _ in lead])) if lead else 1
    for dest in range(n):
      for row in range(rows):
        soff, doff, rest = dest * src_part_stride, me * dst_part_stride, row
        for d, ss, ds in reversed(lead):
          i, rest = rest % d, rest // d
          soff += i * ss
          doff += i * ds
        outs[dest][doff:doff + row_bytes] = src[soff:soff + row_bytes]
  return outs


@pytest.mark.parametrize("shape,n", [((8, 16, 128), 2), ((8, 16, 128), 4), ((2, 8, 4, 6, 64), 2),
                                      ((1, 32, 8, 40, 64), 8), ((16, 64), 4)])
def test_alltoall_peer_plan_moves_every_part_to_its_place(shape, n):
  """The (dims, strides, row) description handed to mtfc_alltoall_peer, replayed in
  numpy for every rank, gives the oracle's alltoall for every (split, concat) pair."""
  from mesh_b200.cuda_mesh_impl import alltoall_peer_plan
  from oracle.numpy_mesh_impl import NumpyMeshImpl
  from oracle.numpy_ops import Arr
  r = rng(77)
  slices = [r.standard_normal(shape).astype(np.float32) for _ in range(n)]
  ora = NumpyMeshImpl("all:%d" % n, "")
  x = ora.LaidOutTensor([Arr(v.copy(), mtf.float32) for v in slices])
  planned = 0
  for split_axis in range(len(shape)):
    if shape[split_axis] % n:
      continue
    for concat_axis in range(len(shape)):
      plan = alltoall_peer_plan(shape, 4, n, split_axis, concat_axis)
      if plan is None:
        continue
      planned += 1
      want = ora.alltoall(x, 0, split_axis, concat_axis).tensor_list
      got = _walk_like_the_kernel(slices, plan, 4)
      assert all(b % 16 == 0 for _, a, c in plan[1] for b in (a, c)) and plan[2] % 16 == 0
      for dest in range(n):
        np.testing.assert_array_equal(got[dest].view(np.float32).reshape(plan[0]), want[dest].a)
  assert planned >= 1


def test_ffn_row_chunks_cover_the_rows_in_multiples_of_256():
  """Chunk boundaries of the row-split FFN schedule at the benchmark's group shapes."""
  from mesh_b200.cuda_mesh_impl import ffn_row_chunks
  cases = {(2, 16384): [0, 12288, 16384],                  # 2x2 mesh: little travels, last chunk a quarter
           (4, 16384): [0, 4096, 8192, 12288, 16384],      # one group of four: equal chunks
           (4, 8192): [0, 4096, 8192],                     # 2x4 mesh
           (2, 32768): [0, 24576, 32768]}
  for (n, mine), want in cases.items():
    assert ffn_row_chunks(n, mine, 1024, 4096 // n, 1024, 4, 4096, 0.74e12) == want
  for n in (2, 4, 8):
    for mine in (256, 512, 2048, 3 * 256, 40 * 256):
      for min_rows in (256, 4096):
        b = ffn_row_chunks(n, mine, 256, 512, 256, 4, min_rows, 0.74e12)
        assert b[0] == 0 and b[-1] == mine and all(x % 256 == 0 for x in b)
        assert all(hi > lo for lo, hi in zip(b[:-1], b[1:]))
  assert ffn_row_chunks(2, 16384, 1024, 2048, 1024, 1, 4096, 0.74e12) == [0, 16384]


def test_a_product_with_one_reader_is_offered_for_deferral():
  """EinsumOperation.lower offers a product that a single operation reads to the backend
  (defer_einsum); the pending product runs when its reader asks for it, the result and the
  lowering's counters are those of the plain lowering, and in a training graph - where the
  hidden activations are read again by the backward pass - the first product is not offered."""
  from oracle.numpy_mesh_impl import NumpyMeshImpl

  class Pending(object):
    def __init__(self, impl, fn, inputs, shape):
      self._impl, self._fn, self._inputs, self._shape, self.runs = impl, fn, inputs, shape, 0

    @property
    def slice_shape(self):
      return list(self._shape)

    def to_laid_out_tensor(self):
      self.runs += 1
      if not hasattr(self, "_value"):
        self._value = self._impl.slicewise(self._fn, *self._inputs)
      return self._value

  class Deferring(NumpyMeshImpl):
    def __init__(self, *a):
      super().__init__(*a)
      self.offered = []

    def defer_einsum(self, fn, inputs, equation, activation):
      shape = self.slicewise(fn, *inputs).slice_shape     # (a real backend knows it without running)
      self.offered.append((equation, activation))
      return Pending(self, fn, inputs, shape)

  def ffn(backend, train):
    r = rng(5)
    g = mtf.Graph()
    m = mtf.Mesh(g, "m")
    x = mtf.import_tf_tensor(m, r.standard_normal((4, 8, 16)).astype(np.float32), "batch:4,length:8,d_model:16")
    wi = mtf.import_tf_tensor(m, r.standard_normal((16, 32)).astype(np.float32), "d_model:16,d_ff:32")
    wo = mtf.import_tf_tensor(m, r.standard_normal((32, 16)).astype(np.float32), "d_ff:32,d_model:16")
    y = mtf.layers.dense_relu_dense(x, mtf.Dimension("d_ff", 32), wi=wi, wo=wo)
    fetch = [y] + (mtf.gradients([y], [wi]) if train else [])
    low = mtf.Lowering(g, {m: backend})
    return [low.export_to_tf_tensor(t) for t in fetch], low.counter_totals()
  plain, counters = ffn(NumpyMeshImpl("all:2", "d_ff:all"), False)
  backend = Deferring("all:2", "d_ff:all")
  got, got_counters = ffn(backend, False)
  assert len(backend.offered) == 1 and backend.offered[0][1] == "relu"
  np.testing.assert_array_equal(got[0], plain[0])
  assert got_counters == counters
  backend = Deferring("all:2", "d_ff:all")
  trained, _ = ffn(backend, True)
  assert all(activation != "relu" for _, activation in backend.offered)
  np.testing.assert_array_equal(trained[0], plain[0])


def test_result_slots_return_when_their_owner_dies():
  """_SlotOwner: the object torch ties to a result's storage gives its slot back to the
  workspace's free list when it is collected (no CUDA involved here)."""
  import gc
  from mesh_b200.cuda_mesh_impl import _AlltoallWorkspace, _SlotOwner
  ws = _AlltoallWorkspace()
  ws.free = [3, 2]
  owner = _SlotOwner(4096, 128, ws, 1)
  assert owner.__cuda_array_interface__["data"] == (4096, False)
  assert owner.__cuda_array_interface__["shape"] == (128,)
  holder = [owner]
  del owner
  gc.collect()
  assert ws.free == [3, 2]
  holder.clear()
  gc.collect()
  assert ws.free == [3, 2, 1]
