"""CudaMeshImpl: a MeshImpl whose slices live on B200 GPUs.

Drop-in for the reference's PlacementMeshImpl
(mesh_tensorflow/placement_mesh_impl.py:31-355) at the MeshImpl operator API:
same constructor contract `(shape, layout, devices)`, same LaidOutTensor duck
type, same methods with the same argument meaning and the same exceptions at
lowering time.  Slice arithmetic runs on libmtfc kernels (DeviceOps); mesh
collectives run

  * in-process, when one process holds every slice (`devices` lists the CUDA
    ordinal of each processor; ordinals may repeat so that n processors share
    one GPU): group members are combined with the same kernels, following the
    reference's grouping (`processor_groups`, ascending processor number);
  * over torch.distributed (NCCL on NVLink / NVSwitch), when the job runs one
    process per GPU: rank r holds processor r's slice only, and each mesh-axis
    set gets its process groups once.  allreduce -> all_reduce, allconcat ->
    all_gather (+ strided-copy kernel when the concat axis is not outermost),
    alltoall -> one kernel that stores into the peers' mapped buffers
    (mtfc_alltoall_peer), or all_to_all_single bracketed by pack / unpack copy
    kernels for small or unaligned slices,
    receive -> batched isend / irecv.

SlicedMeshImpl holds everything that does not depend on where a slice lives;
CudaMeshImpl binds it to DeviceOps and CUDA devices.
"""

from __future__ import annotations

import os

import numpy as np

from mesh_b200 import mtf
from mesh_b200.mtf.layout import pnum_to_processor_coordinates, processor_groups
from mesh_b200.mtf.mesh_impl import convert_args_to_laid_out_tensors


class SlicedMeshImpl(mtf.MeshImpl):
  """MeshImpl machinery over an array library and (optionally) torch.distributed.

  Subclasses provide `_ops_for(pnum)` (array library positioned on the
  processor's device), `_is_slice(x)`, and the torch bridges `_as_torch(x)` /
  `_from_torch(t, shape, dtype, pnum)` used by the distributed collectives.
  """

  allreduce_accepts_donation = True

  def __init__(self, shape, layout, local_pnums, distributed):
    super().__init__(shape, layout)
    self._local_pnums = list(local_pnums)
    self._distributed = distributed
    self._groups = {}
    self.copy_master_to_slice_ops = []

  class LaidOutTensor(object):
    """The slices this process holds, one per local processor
    (placement_mesh_impl.py:39-65)."""

    def __init__(self, tensor_list):
      self._tensor_list = list(tensor_list)

    def __repr__(self):
      return "[" + ",".join(str(t) for t in self._tensor_list) + "]"

    @property
    def tensor_list(self):
      return self._tensor_list

    @classmethod
    def from_tensor_list(cls, tensor_list):
      return cls(tensor_list)

    @property
    def all_slices(self):
      return self._tensor_list

    @property
    def slice_shape(self):
      t = self._tensor_list[0]
      return list(t.shape) if hasattr(t, "shape") else []

    def to_laid_out_tensor(self):
      return self

  class LaidOutVariable(object):
    """Per-processor slices of a variable with copies to and from its master
    (placement_mesh_impl.py:67-157).  The master is a host array; here the
    copies are methods that run at once instead of graph operations.

    `variable` needs `outputs[0]` (shape, dtype), `get_master()` returning the
    host array and `assign_to_master(array)`.
    """

    def __init__(self, variable, mesh_impl):
      self._variable = variable
      self._mesh_impl = mesh_impl
      self._laid_out_tensor = mesh_impl.import_tf_tensor(variable.outputs[0],
                                                         variable.get_master())

    @property
    def laid_out_tensor(self):
      return self._laid_out_tensor

    def assign_to_slices(self, assign_fn, values):
      """Replaces every local slice by assign_fn(variable, old_slice, value)."""
      impl = self._mesh_impl
      new = []
      for pnum, old, value in zip(impl.local_pnums, self._laid_out_tensor.all_slices, values):
        impl._ops_for(pnum)
        new.append(assign_fn(self._variable, old, value))
      self._laid_out_tensor = impl.LaidOutTensor(new)
      return self._laid_out_tensor

    def copy_master_to_slices(self):
      tensor = self._variable.outputs[0]
      fresh = self._mesh_impl.import_tf_tensor(tensor, self._variable.get_master())
      return self.assign_to_slices(lambda var, old, value: value, fresh.all_slices)

    def copy_slices_to_master(self):
      tensor = self._variable.outputs[0]
      self._variable.assign_to_master(
          self._mesh_impl.export_to_tf_tensor(tensor, self._laid_out_tensor), from_slices=self)

  # ------------------------------------------------------------ basics
  @property
  def local_pnums(self):
    return list(self._local_pnums)

  @property
  def is_distributed(self):
    return self._distributed

  def _ops_for(self, pnum):
    raise NotImplementedError

  def _is_slice(self, x):
    raise NotImplementedError

  def _raise_if_a_kernel_gave_up(self):
    """Hook: raises if device code reported a failure since the last check."""

  def slicewise(self, fn, *inputs):
    inputs = convert_args_to_laid_out_tensors(inputs)
    n = len(self._local_pnums)
    cols = [x.tensor_list if isinstance(x, self.LaidOutTensor) else [x] * n for x in inputs]
    ret = []
    for i, pnum in enumerate(self._local_pnums):
      self._ops_for(pnum)
      ret.append(fn(*[col[i] for col in cols]))
    if isinstance(ret[0], tuple):
      return tuple(self.LaidOutTensor(list(t)) for t in zip(*ret))
    return self.LaidOutTensor(ret)

  def laid_out_pnum(self):
    return self.LaidOutTensor(list(self._local_pnums))

  def random(self, shape, tf_fn, kwargs):
    """A random tensor, slice by slice (placement_mesh_impl.py:307-325).

    `tf_fn` is "uniform" (kwargs minval, maxval) or "normal" (mean, stddev), or a
    callable `tf_fn(ops, slice_shape, seed=..., **kwargs)` returning a slice.
    As in the reference, every slice's seed is derived from the operation's seed
    and the slice's offset in the tensor, so processors that hold the same part
    of the tensor draw the same values.  Unlike the reference, whose operation
    seed is Python's unseeded random.random(), the seed here is `kwargs["seed"]`
    (the RandomOperation passes one derived from its name): runs repeat."""
    import hashlib
    kwargs = dict(kwargs)
    op_seed = kwargs.pop("seed", 0)
    dtype = kwargs.pop("dtype", mtf.float32)
    slice_shape = self.slice_shape(shape)

    def my_fn(pnum):
      ops = self._ops_for(pnum)
      text = "%s,%s" % (op_seed, self.slice_begin(shape, pnum))
      seed = int.from_bytes(hashlib.sha256(text.encode()).digest()[:8], "little")
      if callable(tf_fn):
        return tf_fn(ops, slice_shape, seed=seed, dtype=dtype, **kwargs)
      if tf_fn == "uniform":
        return ops.random(slice_shape, "uniform", seed, dtype,
                          float(kwargs.get("minval", 0.0)), float(kwargs.get("maxval", 1.0)))
      if tf_fn == "normal":
        return ops.random(slice_shape, "normal", seed, dtype,
                          float(kwargs.get("mean", 0.0)), float(kwargs.get("stddev", 1.0)))
      raise ValueError("unknown random function %r" % (tf_fn,))
    return self.slicewise(my_fn, self.laid_out_pnum())

  # ------------------------------------------------------------ import/export
  def import_tf_tensor(self, x, tf_x):
    """Host array -> slices; each processor's part is cut on the host and only
    that part is uploaded (ops.py:1249-1269 semantics)."""
    value = tf_x if hasattr(tf_x, "data_ptr") else np.asarray(tf_x)
    layout = self.tensor_layout(x.shape)
    slice_shape = self.slice_shape(x.shape)
    out = []
    for pnum in self._local_pnums:
      ops = self._ops_for(pnum)
      if layout.is_fully_replicated:
        part = value
      else:
        begin = self.slice_begin(x.shape, pnum)
        part = value[tuple(slice(b, b + s) for b, s in zip(begin, slice_shape))]
      out.append(ops.from_host(part, x.dtype))
    return self.LaidOutTensor(out)

  def export_to_tf_tensor(self, x, laid_out_x):
    """Slices -> full host array (combine_slices, ops.py:1271-1305)."""
    laid_out_x = laid_out_x.to_laid_out_tensor()
    host = [self._ops_for(p).to_host(s) for p, s in zip(self._local_pnums, laid_out_x.all_slices)]
    # the copies above waited for the device: a kernel whose bounded wait ran out while
    # producing these values has said so by now, and the values are not handed on
    self._raise_if_a_kernel_gave_up()
    if self._distributed:
      import torch.distributed as dist
      gathered = [None] * self.size
      dist.all_gather_object(gathered, host[0])
      host = gathered
    return _combine_host(self, host, x.shape)

  # ------------------------------------------------------------ collectives
  def allreduce(self, x, mesh_axes, reduction_fn_string, donate=False):
    """Grouped SUM / MAX / MIN (placement_mesh_impl.py:200-212).  Mesh axes of
    size one have single-member groups and are dropped.  `donate=True` says
    the caller holds no other reference to `x`, so its buffers may be reduced
    in place."""
    if reduction_fn_string not in ("SUM", "MAX", "MIN"):
      raise ValueError("unknown reduction %s" % reduction_fn_string)
    mesh_axes = [a for a in mesh_axes if self.shape[a].size > 1]
    if not mesh_axes:
      return x
    x = x.to_laid_out_tensor()
    if self._distributed:
      return self._dist_allreduce(x, mesh_axes, reduction_fn_string, donate)
    name = {"SUM": "add", "MAX": "maximum", "MIN": "minimum"}[reduction_fn_string]

    def chain(ops, local):
      # (x0 + ... + x_lc) + (x_rc + ... + x_{n-1}), as the reference's
      # single-shard chain (placement_mesh_impl.py:378-397)
      n = len(local)
      left_center = n // 2 - 1 if n % 2 == 0 else n // 2
      left = local[0]
      for i in range(1, left_center + 1):
        left = ops.binary(name, left, local[i])
      right = local[n - 1]
      for i in reversed(range(left_center + 1, n - 1)):
        right = ops.binary(name, local[i], right)
      return ops.binary(name, left, right) if n > 1 else left

    def collective(slices, pnums):
      n = len(slices)
      ops = self._ops_for(pnums[0])
      local = [self._move(s, pnums[0]) for s in slices]
      size = 1
      for d in local[0].shape:
        size *= d
      if n > 1 and size >= 1024 and size % n == 0:
        # the reference's sharded ring (placement_mesh_impl.py:407-455): the flat slice
        # is cut in n shards and shard s is reduced over the member list rotated right
        # by s, so the association order differs from shard to shard
        flat = [ops.reshape(t, [size]) for t in local]
        shard = size // n
        parts = []
        for sh in range(n):
          members = [ops.slice(t, [sh * shard], [shard]) for t in flat]
          k = sh % n
          rotated = members[-k:] + members[:-k] if k else members
          parts.append(chain(ops, rotated))
        total = ops.reshape(ops.concat(parts, 0), local[0].shape)
      else:
        total = chain(ops, local)
      return [self._move(total, p) for p in pnums]
    return self._local_groups(x, mesh_axes, collective)

  def allconcat(self, x, mesh_axis, concat_axis):
    x = x.to_laid_out_tensor()
    if self.shape[mesh_axis].size == 1:
      return x
    if self._distributed:
      return self._dist_allconcat(x, mesh_axis, concat_axis)

    def collective(slices, pnums):
      return [self._ops_for(p).concat([self._move(s, p) for s in slices], concat_axis)
              for p in pnums]
    return self._local_groups(x, [mesh_axis], collective)

  def allreduce_start(self, x, mesh_axes, reduction_fn_string):
    """allreduce whose result need not be there yet: one process per GPU starts the
    collective now (on the process group's stream) and hands back an object whose
    to_laid_out_tensor() waits for it, so that what is enqueued before the first reader
    runs beside the exchange; otherwise the same as allreduce."""
    mesh_axes = [a for a in mesh_axes if self.shape[a].size > 1]
    if not self._distributed or not mesh_axes:
      return self.allreduce(x, mesh_axes, reduction_fn_string)
    if reduction_fn_string not in ("SUM", "MAX", "MIN"):
      raise ValueError("unknown reduction %s" % reduction_fn_string)
    import torch.distributed as dist
    x = x.to_laid_out_tensor()
    pg, _ = self._group(mesh_axes)
    op = {"SUM": dist.ReduceOp.SUM, "MAX": dist.ReduceOp.MAX, "MIN": dist.ReduceOp.MIN}[reduction_fn_string]
    s = x.tensor_list[0]
    t = self._as_torch(s).clone()
    work = dist.all_reduce(t, op=op, group=pg, async_op=True)
    return _PendingAllreduce(self, self._from_torch(t, s.shape, s.dtype, self._local_pnums[0]), [work])

  def alltoall(self, x, mesh_axis, split_axis, concat_axis):
    x = x.to_laid_out_tensor()
    n = self.shape[mesh_axis].size
    if n == 1:
      return x
    if x.slice_shape[split_axis] % n != 0:
      raise ValueError("alltoall: axis %d of slice %s is not divisible by %d"
                       % (split_axis, x.slice_shape, n))
    if self._distributed:
      return self._dist_alltoall(x, mesh_axis, split_axis, concat_axis)

    def collective(slices, pnums):
      shape = list(slices[0].shape)
      part = list(shape)
      part[split_axis] = shape[split_axis] // n
      out = []
      for dst, p in enumerate(pnums):
        ops = self._ops_for(p)
        begin = [0] * len(shape)
        begin[split_axis] = dst * part[split_axis]
        pieces = [self._move(self._ops_for(q).contiguous(self._ops_for(q).slice(s, begin, part)), p)
                  for s, q in zip(slices, pnums)]
        self._ops_for(p)
        out.append(ops.concat(pieces, concat_axis))
      return out
    return self._local_groups(x, [mesh_axis], collective)

  def receive(self, x, mesh_axis, source_pcoord):
    x = x.to_laid_out_tensor()
    if len(source_pcoord) != self.shape[mesh_axis].size:
      raise ValueError("source_pcoord must have one entry per processor of the mesh axis")
    if self._distributed:
      return self._dist_receive(x, mesh_axis, source_pcoord)

    def collective(slices, pnums):
      out = []
      for k, p in enumerate(pnums):
        ops = self._ops_for(p)
        src = source_pcoord[k]
        if src is None:
          out.append(ops.fill(slices[0].shape, 0, slices[0].dtype))
        else:
          moved = self._move(slices[src], p)
          out.append(_fresh_copy(ops, moved) if moved is slices[src] else moved)
      return out
    return self._local_groups(x, [mesh_axis], collective)

  # ------------------------------------------------------------ in-process groups
  def _move(self, s, pnum):
    """The slice on processor `pnum`'s device (same object if already there)."""
    return s

  def _local_groups(self, x, mesh_axes, collective):
    ret = [None] * self.size
    for group in processor_groups(self.shape, list(mesh_axes)):
      for pnum, y in zip(group, collective([x.tensor_list[p] for p in group], group)):
        ret[pnum] = y
    return self.LaidOutTensor(ret)

  # ------------------------------------------------------------ distributed
  def _group(self, mesh_axes):
    """Process group of this rank for the given mesh axes, with its member pnums.

    Every rank creates every group of the axis set, in the same order, as
    torch.distributed requires."""
    import torch.distributed as dist
    key = tuple(sorted(mesh_axes))
    if key not in self._groups:
      mine = None
      for members in processor_groups(self.shape, list(key)):
        pg = dist.new_group(ranks=members)
        if self._local_pnums[0] in members:
          mine = (pg, members)
      self._groups[key] = mine
    return self._groups[key]

  def _as_torch(self, s):
    raise NotImplementedError

  def _from_torch(self, t, shape, dtype, pnum):
    raise NotImplementedError

  def _owns_storage(self, s, t):
    """True when the flat tensor `t` made from slice `s` may be overwritten
    without touching memory another slice can see."""
    return False

  def _dist_allreduce(self, x, mesh_axes, name, donate=False):
    import torch.distributed as dist
    pg, _ = self._group(mesh_axes)
    op = {"SUM": dist.ReduceOp.SUM, "MAX": dist.ReduceOp.MAX, "MIN": dist.ReduceOp.MIN}[name]
    pnum = self._local_pnums[0]
    s = x.tensor_list[0]
    t = self._as_torch(s)
    if not (donate and self._owns_storage(s, t)):
      t = t.clone()   # collectives return fresh tensors; the input stays intact
    dist.all_reduce(t, op=op, group=pg)
    return self.LaidOutTensor([self._from_torch(t, s.shape, s.dtype, pnum)])

  def _dist_allconcat(self, x, mesh_axis, concat_axis):
    import torch
    import torch.distributed as dist
    pg, members = self._group([mesh_axis])
    n = len(members)
    pnum = self._local_pnums[0]
    ops = self._ops_for(pnum)
    s = x.tensor_list[0]
    t = self._as_torch(s)
    out = torch.empty(n * t.numel(), dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(out, t, group=pg)
    shape = list(s.shape)
    gathered = self._from_torch(out, [n] + shape, s.dtype, pnum)  # [source, *slice]
    # [source, d0.., d_axis, ..] -> [d0.., source, d_axis, ..] -> merge source into the axis
    perm = list(range(1, concat_axis + 1)) + [0] + list(range(concat_axis + 1, len(shape) + 1))
    merged = list(shape)
    merged[concat_axis] *= n
    return self.LaidOutTensor([ops.reshape(ops.transpose(gathered, perm), merged)])

  def _peer_alltoall(self, s, pg, members, pnum, split_axis, concat_axis):
    """Hook: an alltoall of slice `s` without pack / unpack passes, or None."""
    return None

  def _dist_alltoall(self, x, mesh_axis, split_axis, concat_axis):
    import torch
    import torch.distributed as dist
    pg, members = self._group([mesh_axis])
    n = len(members)
    pnum = self._local_pnums[0]
    ops = self._ops_for(pnum)
    s = x.tensor_list[0]
    fast = self._peer_alltoall(s, pg, members, pnum, split_axis, concat_axis)
    if fast is not None:
      return self.LaidOutTensor([fast])
    shape = list(s.shape)
    part = list(shape)
    part[split_axis] //= n
    # pack: [.., n*part, ..] -> [n(target), .., part, ..]
    split = ops.reshape(s, shape[:split_axis] + [n, part[split_axis]] + shape[split_axis + 1:])
    perm = [split_axis] + [i for i in range(len(shape) + 1) if i != split_axis]
    packed = ops.contiguous(ops.transpose(split, perm))
    t = self._as_torch(packed)
    out = torch.empty_like(t)
    dist.all_to_all_single(out, t, group=pg)
    received = self._from_torch(out, [n] + part, s.dtype, pnum)  # [source, *part]
    perm = list(range(1, concat_axis + 1)) + [0] + list(range(concat_axis + 1, len(part) + 1))
    merged = list(part)
    merged[concat_axis] *= n
    return self.LaidOutTensor([ops.reshape(ops.transpose(received, perm), merged)])

  def _dist_receive(self, x, mesh_axis, source_pcoord):
    import torch
    import torch.distributed as dist
    _, members = self._group([mesh_axis])
    pnum = self._local_pnums[0]
    ops = self._ops_for(pnum)
    me = members.index(pnum)
    s = x.tensor_list[0]
    t = self._as_torch(s)
    p2p = []
    src = source_pcoord[me]
    result = None
    if src is None:
      result = ops.fill(s.shape, 0, s.dtype)
    elif src == me:
      result = _fresh_copy(ops, s)
    else:
      buf = torch.empty_like(t)
      p2p.append(dist.P2POp(dist.irecv, buf, members[src]))
    for k, wanted in enumerate(source_pcoord):
      if wanted == me and k != me:
        p2p.append(dist.P2POp(dist.isend, t, members[k]))
    if p2p:
      for work in dist.batch_isend_irecv(p2p):
        work.wait()
    if result is None:
      result = self._from_torch(buf, s.shape, s.dtype, pnum)
    return self.LaidOutTensor([result])


class _PeerWorkspace(object):
  """Buffers of one fused einsum+allreduce shape (see CudaMeshImpl._peer_workspace)."""
  __slots__ = ("tensors", "handles", "out_tensor", "ctl", "stage_ptrs", "out_ptrs", "flag_ptrs",
               "rank", "nranks", "mc_stage", "mc_out", "exchange")


def ffn_row_chunks(n, mine, k1, fs, m2, max_chunks, min_chunk_rows, link_bytes_per_s):
  """Row boundaries (multiples of 256) of the chunks a rank's `mine` rows are multiplied
  and sent in by the row-split FFN schedule: [0, ..., mine]."""
  travel = (n - 1) * mine * m2 * 2 / link_bytes_per_s
  multiply = 4.0 * mine * k1 * fs * n / 1.4e15
  if max_chunks < 2 or mine < 2 * min_chunk_rows:
    return [0, mine]
  if travel <= multiply / 3:
    last = max(256, (mine // 4) // 256 * 256)
    return [0, mine - last, mine]
  for c in range(max_chunks, 1, -1):
    if mine % (c * 256) == 0 and mine // c >= min_chunk_rows:
      return [mine // c * i for i in range(c + 1)]
  return [0, mine]


def alltoall_peer_plan(shape, itemsize, n, split_axis, concat_axis):
  """How mtfc_alltoall_peer walks a contiguous slice of `shape` whose
  `split_axis` is cut in n parts that are concatenated along `concat_axis`:
  `(out_shape, lead, row_bytes, src_part_stride, dst_part_stride)`, where `lead`
  lists (extent, source byte stride, output byte stride) of the dims of one part
  in front of the row, the row being everything from the later of the two axes
  on (contiguous in the source and in the output).  None when the rows are not
  multiples of 16 bytes, shorter than 256 bytes, or more than four dims lead."""
  shape = [int(d) for d in shape]
  part = list(shape)
  part[split_axis] //= n
  out_shape = list(part)
  out_shape[concat_axis] *= n

  def strides(dims):
    st, run = [], itemsize
    for d in reversed(dims):
      st.append(run)
      run *= d
    return st[::-1]
  sstr, dstr = strides(shape), strides(out_shape)
  ax = max(split_axis, concat_axis)
  row_bytes = itemsize
  for d in part[ax:]:
    row_bytes *= d
  if row_bytes % 16 != 0 or row_bytes < 256:
    return None
  lead = [(part[k], sstr[k], dstr[k]) for k in range(ax) if part[k] != 1]
  if len(lead) > 4:
    return None
  return (out_shape, lead, row_bytes, part[split_axis] * sstr[split_axis],
          part[concat_axis] * dstr[concat_axis])


class _AlltoallWorkspace(object):
  """Buffers of one peer-memory alltoall size (see CudaMeshImpl._alltoall_workspace)."""
  __slots__ = ("tensors", "handles", "out_tensor", "ctl", "out_ptrs", "flag_ptrs", "nbytes", "stride",
               "free", "pinned")


class _SlotOwner(object):
  """One result slot of an alltoall workspace, exposed through the CUDA array
  interface: a torch tensor made from it keeps this object alive for as long as
  its storage (any view included) lives, and the slot goes back to the free list
  when the object dies."""

  def __init__(self, ptr, nbytes, workspace, slot):
    self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                     "strides": None, "version": 2}
    self._workspace, self._slot = workspace, slot

  def __del__(self):
    self._workspace.free.append(self._slot)


class _PipelineWorkspace(object):
  """Buffers, counters and the communication stream of one pipelined
  einsum+allreduce shape (see CudaMeshImpl._einsum_allreduce_pipelined)."""
  __slots__ = ("part", "recv", "out", "flags", "progress", "epochs", "handles", "peer_recv",
               "peer_out", "peer_flag_ptrs", "stream", "rank", "nranks", "chunks", "blocks_per_chunk",
               "part_rows", "tiles_n")


class _DeferredEinsum(object):
  """A product EinsumOperation.lower left pending (CudaMeshImpl.defer_einsum): it runs
  when somebody asks for its slices, unless a contraction + allreduce took it over."""

  def __init__(self, mesh_impl, fn, inputs, slice_shape, activation):
    self._mesh_impl, self._fn = mesh_impl, fn
    self.inputs, self.activation = inputs, activation
    self._slice_shape = [int(d) for d in slice_shape]
    self._value = None

  @property
  def pending(self):
    return self._value is None

  @property
  def slice_shape(self):
    return list(self._slice_shape)

  def to_laid_out_tensor(self):
    if self._value is None:
      self._value = self._mesh_impl.slicewise(self._fn, *self.inputs)
    return self._value


class _FfnWorkspace(object):
  """Buffers of one row-split FFN problem size (see CudaMeshImpl._ffn_workspace)."""
  __slots__ = ("tensors", "handles", "wi_all", "wo_full", "y_recv", "flags", "peer_wi", "peer_wo",
               "peer_y", "peer_flag_ptrs", "h", "epochs", "push", "pull", "lanes", "pull_lanes", "rank")


class _PendingAllreduce(object):
  """Result of einsum_allreduce: the reduced slice once its chunked allreduces
  are waited for (the wait is a stream dependency, not a host block)."""

  def __init__(self, mesh_impl, out, works):
    self._mesh_impl = mesh_impl
    self._out = out
    self._works = works

  @property
  def slice_shape(self):
    return list(self._out.shape)

  def to_laid_out_tensor(self):
    for w in self._works:
      w.wait()
    self._works = []
    return self._mesh_impl.LaidOutTensor([self._out])


def _fresh_copy(ops, s):
  """A new buffer holding `s` (collectives return fresh tensors)."""
  return ops.concat([s], 0) if len(s.shape) else ops.binary("add", s, 0)


def _combine_host(impl, slices, tensor_shape):
  """combine_slices over numpy arrays (mesh_tensorflow/ops.py:1271-1305)."""
  if tensor_shape.ndims == 0:
    return np.asarray(slices[0])
  ret = list(slices)
  ma2ta = impl.tensor_layout(tensor_shape).mesh_axis_to_tensor_axis(impl.ndims)
  for mesh_dim, tensor_axis in zip(impl.shape, ma2ta):
    span = len(ret) // mesh_dim.size
    if tensor_axis is None:
      ret = ret[:span]
    else:
      ret = [np.concatenate([ret[i + span * j] for j in range(mesh_dim.size)], axis=tensor_axis)
             for i in range(span)]
  assert len(ret) == 1
  return ret[0]


class CudaMeshImpl(SlicedMeshImpl):
  """MeshImpl on CUDA devices through libmtfc.

  Args:
    shape: mesh Shape, or "rows:2,cols:4".
    layout: LayoutRules, or "batch:rows;d_ff:cols".
    devices: one CUDA ordinal (or "cuda:N") per processor, length shape.size.
      Ordinals may repeat.  When torch.distributed is initialised with a world
      size equal to the mesh size, the job is one process per processor: this
      process computes processor `rank` on `devices[rank]`.
    distributed: force (True) or forbid (False) that mode; None = detect.
  """

  supports_einsum_epilogue = True

  def __init__(self, shape, layout, devices=None, distributed=None):
    import torch
    from mesh_b200 import _native as nat
    from mesh_b200.device_ops import DeviceArray, DeviceOps
    mesh_shape = mtf.convert_to_shape(shape)
    size = mesh_shape.size
    if distributed is None:
      import torch.distributed as dist
      distributed = (dist.is_available() and dist.is_initialized()
                     and dist.get_world_size() == size and size > 1)
    if devices is None:
      devices = [torch.cuda.current_device()] * size if torch.cuda.is_available() else [0] * size
    if len(devices) != size:
      raise ValueError("devices must have one entry per processor: got %d for mesh size %d"
                       % (len(devices), size))
    if not torch.cuda.is_available():
      raise nat.MtfcError(nat.ERR_CUDA, "CudaMeshImpl needs a CUDA device; none is visible")
    nat.lib()  # fail now, loudly, if the kernels are not built
    self._devices = [torch.device(d if isinstance(d, str) else "cuda:%d" % d) for d in devices]
    if distributed:
      import torch.distributed as dist
      local = [dist.get_rank()]
    else:
      local = list(range(size))
    super().__init__(mesh_shape, layout, local, distributed)
    self._device_array = DeviceArray
    self._ops = DeviceOps(self._devices[local[0]])

  @property
  def devices(self):
    return list(self._devices)

  @property
  def slice_ops(self):
    return self._ops

  def _ops_for(self, pnum):
    dev = self._devices[pnum]
    if self._ops.device != dev:
      self._ops.device = dev
    return self._ops

  def _is_slice(self, x):
    return isinstance(x, self._device_array)

  def _move(self, s, pnum):
    dev = self._devices[pnum]
    if s.device == dev:
      return s
    # pack on the SOURCE device (a strided view is gathered by a kernel that
    # dereferences source-device pointers), then let the copy engine move the
    # packed bytes: torch's cross-device copy enables peer access and orders
    # the copy after the producer's stream
    self._ops.device = s.device
    packed = self._ops.contiguous(s)
    flat = packed.buf[packed.offset:packed.offset + max(1, packed.size)].to(dev)
    self._ops.device = dev
    return self._device_array(flat, s.shape, s.dtype)

  # A host tensor whose slice is replicated over some mesh axes is uploaded in
  # parts: each replica sends 1/k of the slice over its own host link and an
  # allgather over NVLink (an order of magnitude faster than the host link)
  # completes it on every replica.  Slices below this size are uploaded whole.
  SHARED_UPLOAD_MIN_BYTES = 1 << 20

  def _replica_group(self, tensor_shape):
    """(process group, members, my position) over the mesh axes the tensor's
    layout leaves unused, or None when the slice has no other replica."""
    layout = self.tensor_layout(tensor_shape)
    used = set(a for a in layout.tensor_axis_to_mesh_axis if a is not None)
    free = [a for a in range(self.ndims) if a not in used and self.shape[a].size > 1]
    if not free:
      return None
    pg, members = self._group(free)
    return pg, members, members.index(self._local_pnums[0])

  def import_tf_tensor(self, x, tf_x):
    import torch
    if self._distributed and isinstance(tf_x, torch.Tensor):
      shared = self._import_shared(x, tf_x)
      if shared is not None:
        return shared
    return super().import_tf_tensor(x, tf_x)

  def _import_shared(self, x, value):
    import torch
    import torch.distributed as dist
    from mesh_b200.device_ops import _TORCH
    if value.dtype != _TORCH[x.dtype.name]:
      return None
    group = self._replica_group(x.shape)
    if group is None:
      return None
    pg, members, me = group
    k = len(members)
    pnum = self._local_pnums[0]
    slice_shape = self.slice_shape(x.shape)
    begin = self.slice_begin(x.shape, pnum)
    part = value[tuple(slice(b, b + s) for b, s in zip(begin, slice_shape))]
    n = part.numel()
    if not part.is_contiguous() or n % k != 0 or n * part.element_size() < self.SHARED_UPLOAD_MIN_BYTES:
      return None
    ops = self._ops_for(pnum)
    ops._activate()
    flat = part.reshape(-1)
    chunk = n // k
    buf = torch.empty(n, dtype=value.dtype, device=ops.device)
    mine = buf[me * chunk:(me + 1) * chunk]
    mine.copy_(flat[me * chunk:(me + 1) * chunk], non_blocking=True)
    dist.all_gather_into_tensor(buf, mine, group=pg)
    self.last_upload_bytes = chunk * part.element_size()
    return self.LaidOutTensor([self._device_array(buf, slice_shape, x.dtype)])

  def einsum(self, equation, *slices, epilogue=None):
    """Per-slice contraction hook (ops.py:1331-1340) on the GEMM kernels;
    `epilogue="relu"` fuses tf.nn.relu into the store."""
    from mesh_b200 import _native as nat
    code = {None: nat.EPILOGUE_NONE, "relu": nat.EPILOGUE_RELU}[epilogue]
    if self._ops.device != slices[0].device:
      self._ops.device = slices[0].device
    return self._ops.einsum(equation, *slices, epilogue=code)

  # chunks a contraction is cut into when its allreduce is overlapped with it,
  # and the smallest number of output rows per chunk worth a separate launch
  OVERLAP_CHUNKS = 4
  OVERLAP_MIN_ROWS = 2048
  # GEMM and allreduce in one kernel over peer memory (mtfc_gemm_allreduce);
  # falls back to the chunked GEMM + NCCL sequence when the einsum is not a
  # single bf16 GEMM, the result is small, or peer memory cannot be set up.
  # MTFC_FUSED_ALLREDUCE=0 in the environment switches it off.
  FUSED_ALLREDUCE = os.environ.get("MTFC_FUSED_ALLREDUCE", "1") == "1"
  FUSED_MIN_BYTES = 1 << 20
  # above this the exchange dominates and NCCL moves the bytes faster (measured:
  # a 256 MiB attention output projection on 2 GPUs, 4.25 ms fused against 3.86 ms)
  FUSED_MAX_BYTES = 128 << 20
  # largest group the fused kernel is used for (groups of 2 and 4 have run on
  # hardware; MTFC_FUSED_ALLREDUCE_MAX_RANKS=8 opens groups of eight)
  # exchange form of the fused kernel: auto | push | pull | multimem
  FUSED_EXCHANGE = os.environ.get("MTFC_FUSED_EXCHANGE", "auto")
  FUSED_MAX_RANKS = int(os.environ.get("MTFC_FUSED_ALLREDUCE_MAX_RANKS", "4"))

  def einsum_allreduce(self, equation, inputs, mesh_axes):
    """Contraction whose SUM allreduce over `mesh_axes` starts chunk by chunk.

    One process per GPU only.  The output's leading dim must be a free dim of
    the first operand and that operand's leading dim; the contraction then runs
    as OVERLAP_CHUNKS launches over row blocks, and each block's NCCL allreduce
    (asynchronous, on the process group's own stream) overlaps the next block's
    GEMM.  Returns an object with to_laid_out_tensor(), or None when the plain
    einsum-then-allreduce sequence should be used.
    """
    mesh_axes = [a for a in mesh_axes if self.shape[a].size > 1]
    if not self._distributed or not mesh_axes:
      return None
    import torch.distributed as dist
    if isinstance(inputs[0], _DeferredEinsum) and inputs[0].pending:
      resharded = self._ffn_resharded(inputs[0], equation, inputs[1], mesh_axes)
      if resharded is not None:
        return resharded
    inputs = convert_args_to_laid_out_tensors(inputs)
    a, b = inputs[0].tensor_list[0], inputs[1].tensor_list[0]
    lhs, out_term = equation.split("->")
    ta, tb = lhs.split(",")
    lead = out_term[0] if out_term else None
    if (lead is None or ta[0] != lead or lead in tb or not a.dtype.is_floating
        or a.shape[0] % self.OVERLAP_CHUNKS != 0):
      return None
    rows_per_chunk = a.shape[0] // self.OVERLAP_CHUNKS
    other_rows = 1
    for letter, size in zip(ta[1:], a.shape[1:]):
      if letter in out_term:
        other_rows *= size
    if rows_per_chunk * other_rows < self.OVERLAP_MIN_ROWS:
      return None
    pnum = self._local_pnums[0]
    ops = self._ops_for(pnum)
    pg, members = self._group(mesh_axes)
    sizes = dict(zip(ta, a.shape))
    sizes.update(zip(tb, b.shape))
    if self.PIPELINED_ALLREDUCE and 2 <= len(members) <= 8 and a.dtype.name == "bfloat16":
      piped = self._einsum_allreduce_pipelined(ops, equation, a, b, pg, members, pnum)
      if piped is not None:
        return _PendingAllreduce(self, piped, [])
    if (self.FUSED_ALLREDUCE and 2 <= len(members) <= self.FUSED_MAX_RANKS
        and a.dtype.name == "bfloat16"):
      fused = self._einsum_allreduce_fused(ops, equation, a, b, pg, members, pnum)
      if fused is not None:
        return _PendingAllreduce(self, fused, [])
    out = ops._empty([sizes[l] for l in out_term], a.dtype)
    flat = out.buf[out.offset:out.offset + out.size]
    chunk_elems = out.size // self.OVERLAP_CHUNKS
    works = []
    for i in range(self.OVERLAP_CHUNKS):
      a_i = ops.slice(a, [i * rows_per_chunk] + [0] * (len(a.shape) - 1),
                      [rows_per_chunk] + list(a.shape[1:]))
      out_i = ops.slice(out, [i * rows_per_chunk] + [0] * (len(out.shape) - 1),
                        [rows_per_chunk] + list(out.shape[1:]))
      ops.einsum(equation, a_i, b, out=out_i)
      works.append(dist.all_reduce(flat[i * chunk_elems:(i + 1) * chunk_elems],
                                   op=dist.ReduceOp.SUM, group=pg, async_op=True))
    return _PendingAllreduce(self, out, works)

  # ---- x.wi -> activation -> .wo with the hidden dim split over a mesh axis ---------
  # The reference's schedule gives every rank of the axis all rows and 1/n of the hidden
  # dim, and allreduces the [rows, out] partial sums: 2 (n-1)/n of the output crosses
  # every link, and the sums are added in bf16.  When the first product has no other
  # reader, the same result is computed the other way round: every rank takes 1/n of the
  # ROWS and the whole hidden dim (the weight slices, a few MB, are gathered first), so
  # nothing is left to reduce, and the finished row blocks are gathered: (n-1)/n of the
  # output per link, moved by the copy engines chunk by chunk while the next chunk is
  # multiplied.  Inputs and result keep the layouts the graph gave them (rows replicated
  # over the axis).  MTFC_RESHARDED_FFN=0 keeps the reference's schedule.
  RESHARDED_FFN = os.environ.get("MTFC_RESHARDED_FFN", "1") == "1"
  RESHARDED_FFN_MIN_BYTES = 4 << 20
  RESHARDED_FFN_MAX_CHUNKS = 4
  RESHARDED_FFN_LINK_BYTES_PER_S = 0.74e12   # measured peer-copy rate per direction
  RESHARDED_FFN_MIN_CHUNK_ROWS = 4096   # fewer rows leave the second product too few tiles

  def defer_einsum(self, fn, inputs, equation, activation):
    """Hook of EinsumOperation.lower: leaves `[..., k] x [k, f] -> [..., f]` (bf16,
    optional ReLU) pending when one process drives one GPU, so that einsum_allreduce
    may meet it as its operand.  None = compute it now."""
    if not (self._distributed and self.RESHARDED_FFN) or activation not in (None, "relu"):
      return None
    lhs, out_term = equation.split("->")
    ta, tb = lhs.split(",")
    if not (len(tb) == 2 and len(ta) >= 2 and ta[-1] == tb[0] and out_term == ta[:-1] + tb[1]
            and len(set(ta + tb)) == len(ta) + 1):
      return None
    inputs = convert_args_to_laid_out_tensors(inputs)
    a, b = inputs[0].tensor_list[0], inputs[1].tensor_list[0]
    if not (a.dtype.name == "bfloat16" and b.dtype.name == "bfloat16" and a.is_contiguous
            and b.is_contiguous and a.ptr % 16 == 0 and b.ptr % 16 == 0):
      return None
    return _DeferredEinsum(self, fn, inputs, list(a.shape[:-1]) + [b.shape[1]], activation)

  def _ffn_resharded(self, first, equation, wo_input, mesh_axes):
    """`first` (a pending x.wi [+ReLU]) contracted with wo over the hidden dim that is
    split over `mesh_axes`: the row-split schedule described above, or None when it does
    not apply (nothing has been launched then)."""
    import ctypes
    import torch
    from mesh_b200 import _native as nat
    if len(mesh_axes) != 1:
      return None
    lhs, out_term = equation.split("->")
    ta, tb = lhs.split(",")
    if not (len(tb) == 2 and len(ta) >= 2 and ta[-1] == tb[0] and out_term == ta[:-1] + tb[1]
            and len(set(ta + tb)) == len(ta) + 1):
      return None
    pg, members = self._group(mesh_axes)
    n = len(members)
    pnum = self._local_pnums[0]
    x, wi = first.inputs[0].tensor_list[0], first.inputs[1].tensor_list[0]
    wo = convert_args_to_laid_out_tensors([wo_input])[0].tensor_list[0]
    if not (n in (2, 4, 8) and wo.dtype.name == "bfloat16" and wo.is_contiguous and wo.ptr % 16 == 0
            and len(wo.shape) == 2 and wo.shape[0] == wi.shape[1]):
      return None
    k1, fs, m2 = wi.shape[0], wi.shape[1], wo.shape[1]
    rows = x.size // k1
    if rows % (n * 256) != 0 or k1 % 8 != 0 or fs % 8 != 0 or m2 % 8 != 0 or fs < 256 or m2 < 256:
      return None
    if rows * m2 * 2 < self.RESHARDED_FFN_MIN_BYTES:
      return None
    mine = rows // n
    # Row chunks of this rank's share: a chunk's result travels while the next chunk is
    # multiplied, what travels after the last product is exposed, and every chunk costs a
    # chain of dependent stream operations.  With little to move beside the arithmetic
    # (groups of two) two chunks, the last one a quarter; otherwise (a rank pushes n - 1
    # copies of its rows) equal chunks, so that each journey fits behind the next product.
    bounds = ffn_row_chunks(n, mine, k1, fs, m2, self.RESHARDED_FFN_MAX_CHUNKS,
                            self.RESHARDED_FFN_MIN_CHUNK_ROWS, self.RESHARDED_FFN_LINK_BYTES_PER_S)
    chunks = len(bounds) - 1
    ws = self._ffn_workspace(pg, members, pnum, rows, k1, fs, m2, chunks)
    if ws is None:
      return None
    lib = nat.lib()
    me = ws.rank
    others = [r for r in range(n) if r != me]
    f = fs * n
    main = torch.cuda.current_stream()
    ms = ctypes.c_void_p(main.cuda_stream)
    flags, epochs = ws.flags.data_ptr(), ws.epochs.data_ptr()
    wi2d = wi.buf[wi.offset:wi.offset + wi.size].view(k1, fs)
    wo2d = wo.buf[wo.offset:wo.offset + wo.size].view(fs, m2)
    # 1. "whatever read this rank's receive buffer was enqueued before this point": the
    #    peers wait for it only before their first row block travels (on the push stream,
    #    off the critical path).  The weight buffers need no such signal: a rank reads
    #    them for the last time before its last row block leaves, and every rank has
    #    waited for every peer's last block before it returns from the previous call.
    nat.check(lib.mtfc_signal_peers(ws.peer_flag_ptrs, n - 1, 0, ms))
    # 2. the weight slices go to every rank (copy engines).  A rank keeps the hidden dim in
    #    rotated order, its own slice first: block j holds the slice of rank (me + j) mod n
    #    (the sum over the hidden dim does not care), so the product with the own slice can
    #    start at once and hides the journey of the others.
    # (one side stream per peer: copies to different peers run on different copy engines
    # instead of queueing behind each other)
    start = torch.cuda.Event()
    start.record(main)
    for lane, r in zip(ws.lanes, others):
      j = (me - r) % n          # where this rank's slice sits in rank r's buffers
      lane.wait_event(start)
      with torch.cuda.stream(lane):
        ws.peer_wi[r][j].copy_(wi2d, non_blocking=True)
        ws.peer_wo[r][j * fs:(j + 1) * fs].copy_(wo2d, non_blocking=True)
    ws.wo_full[0:fs].copy_(wo2d, non_blocking=True)
    for lane in ws.lanes:
      main.wait_stream(lane)
    # In a group of two the own slice is half of the first product: worth launches of its
    # own ahead of the wait.  In larger groups it is a small product per chunk that costs
    # more in launches than the wait it hides, so one product takes all blocks.
    own_first = n == 2
    if not own_first:
      ws.wi_all[0].copy_(wi2d, non_blocking=True)
    nat.check(lib.mtfc_signal_peers(ws.peer_flag_ptrs, n - 1, 1, ms))
    relu = nat.EPILOGUE_RELU if first.activation == "relu" else nat.EPILOGUE_NONE

    def first_product(c, b_ptr, blocks, first_block):
      """h[chunk c, blocks first_block .. first_block + blocks) = act(x[chunk c] . wi blocks)."""
      r0, r1 = bounds[c], bounds[c + 1]
      d1 = nat.GemmDesc()
      d1.batch, d1.m, d1.n, d1.k = blocks, r1 - r0, fs, k1
      d1.a_batch, d1.a_m, d1.a_k = 0, k1, 1
      d1.b_batch, d1.b_k, d1.b_n = k1 * fs, fs, 1
      d1.c_batch, d1.c_m, d1.c_n = fs, f, 1
      d1.in_dtype = d1.out_dtype = nat.BF16
      d1.epilogue, d1.force_path = relu, 0
      nat.check(lib.mtfc_gemm(ctypes.byref(d1), ctypes.c_void_p(x.ptr + (me * mine + r0) * k1 * 2),
                              ctypes.c_void_p(b_ptr),
                              ctypes.c_void_p(ws.h.data_ptr() + (r0 * f + first_block * fs) * 2), ms))
    if own_first:
      for c in range(chunks):
        first_product(c, wi.ptr, 1, 0)
    nat.check(lib.mtfc_wait_counters(ctypes.c_void_p(flags + 4), 1, n - 1, ctypes.c_void_p(epochs + 4), ms))
    # 3. this rank's rows, chunk by chunk; finished chunks travel while the next is multiplied
    result = torch.empty(rows * m2, dtype=torch.bfloat16, device=ws.h.device)
    res2d = result.view(rows, m2)
    fork = torch.cuda.Event()
    fork.record(main)
    ws.push.wait_event(fork)
    ws.pull.wait_event(fork)
    for c in range(chunks):
      r0, r1 = bounds[c], bounds[c + 1]
      g0, g1 = me * mine + r0, me * mine + r1
      if own_first:
        first_product(c, ws.wi_all.data_ptr() + k1 * fs * 2, n - 1, 1)
      else:
        first_product(c, ws.wi_all.data_ptr(), n, 0)
      d2 = nat.GemmDesc()
      d2.batch, d2.m, d2.n, d2.k = 1, r1 - r0, m2, f
      d2.a_batch, d2.a_m, d2.a_k = 0, f, 1
      d2.b_batch, d2.b_k, d2.b_n = 0, m2, 1
      d2.c_batch, d2.c_m, d2.c_n = (r1 - r0) * m2, m2, 1
      d2.in_dtype = d2.out_dtype = nat.BF16
      d2.epilogue, d2.force_path = nat.EPILOGUE_NONE, 0
      nat.check(lib.mtfc_gemm(ctypes.byref(d2), ctypes.c_void_p(ws.h.data_ptr() + r0 * f * 2),
                              ctypes.c_void_p(ws.wo_full.data_ptr()),
                              ctypes.c_void_p(result.data_ptr() + g0 * m2 * 2), ms))
      done = torch.cuda.Event()
      done.record(main)
      ws.push.wait_event(done)
      with torch.cuda.stream(ws.push):
        if c == 0:
          nat.check(lib.mtfc_wait_counters(ctypes.c_void_p(flags), 1, n - 1, ctypes.c_void_p(epochs),
                                           ctypes.c_void_p(ws.push.cuda_stream)))
      go = torch.cuda.Event()
      go.record(ws.push)
      for lane, r in zip(ws.lanes, others):
        lane.wait_event(go)
        with torch.cuda.stream(lane):
          ws.peer_y[r][g0:g1].copy_(res2d[g0:g1], non_blocking=True)
        ws.push.wait_stream(lane)
      with torch.cuda.stream(ws.push):
        nat.check(lib.mtfc_signal_peers(ws.peer_flag_ptrs, n - 1, 2 + c,
                                        ctypes.c_void_p(ws.push.cuda_stream)))
      with torch.cuda.stream(ws.pull):
        # the peers' chunk c has landed in the receive buffer: into the result it goes
        nat.check(lib.mtfc_wait_counters(ctypes.c_void_p(flags + 4 * (2 + c)), 1, n - 1,
                                         ctypes.c_void_p(epochs + 4 * (2 + c)),
                                         ctypes.c_void_p(ws.pull.cuda_stream)))
      landed = torch.cuda.Event()
      landed.record(ws.pull)
      for lane, r in zip(ws.pull_lanes, others):
        lane.wait_event(landed)
        with torch.cuda.stream(lane):
          res2d[r * mine + r0:r * mine + r1].copy_(ws.y_recv[r * mine + r0:r * mine + r1],
                                                   non_blocking=True)
        ws.pull.wait_stream(lane)
    main.wait_stream(ws.push)
    main.wait_stream(ws.pull)
    out = self._device_array(result, list(x.shape[:-1]) + [m2], x.dtype)
    return self.LaidOutTensor([out])

  def _ffn_workspace(self, pg, members, pnum, rows, k1, fs, m2, chunks):
    """Peer-mapped buffers of the row-split FFN schedule for one problem size: every
    rank's weight slices side by side, the receive buffer for the peers' row blocks,
    the counters; plus the local hidden activations and two side streams."""
    import ctypes
    import torch
    import torch.distributed as dist
    key = (tuple(members), rows, k1, fs, m2, chunks)
    if not hasattr(self, "_ffn_ws"):
      self._ffn_ws = {}
    if key in self._ffn_ws:
      return self._ffn_ws[key]
    ws = None
    try:
      import torch.distributed._symmetric_memory as symm
      dev = torch.device("cuda", torch.cuda.current_device())
      n = len(members)
      me = members.index(pnum)

      def alloc(count, dtype):
        t = symm.empty(count, dtype=dtype, device=dev)
        return t, symm.rendezvous(t, pg)
      wi_t, wi_h = alloc(n * k1 * fs, torch.bfloat16)
      wo_t, wo_h = alloc(n * fs * m2, torch.bfloat16)
      y_t, y_h = alloc(rows * m2, torch.bfloat16)
      flag_t, flag_h = alloc(2 + chunks, torch.int32)
      flag_t.zero_()
      if int(y_h.rank) != me or int(y_h.world_size) != n:
        raise RuntimeError("symmetric-memory rank %d/%d does not match mesh group position %d/%d"
                           % (y_h.rank, y_h.world_size, me, n))
      ws = _FfnWorkspace()
      ws.tensors, ws.handles = (wi_t, wo_t, y_t, flag_t), (wi_h, wo_h, y_h, flag_h)
      ws.wi_all, ws.wo_full = wi_t.view(n, k1, fs), wo_t.view(n * fs, m2)
      ws.y_recv, ws.flags = y_t.view(rows, m2), flag_t
      others = [r for r in range(n) if r != me]
      ws.peer_wi = {r: wi_h.get_buffer(r, (n, k1, fs), torch.bfloat16) for r in others}
      ws.peer_wo = {r: wo_h.get_buffer(r, (n * fs, m2), torch.bfloat16) for r in others}
      ws.peer_y = {r: y_h.get_buffer(r, (rows, m2), torch.bfloat16) for r in others}
      ws.peer_flag_ptrs = (ctypes.c_void_p * len(others))(
          *[ctypes.c_void_p(int(flag_h.buffer_ptrs[r])) for r in others])
      ws.h = torch.empty((rows // n) * fs * n, dtype=torch.bfloat16, device=dev)
      ws.epochs = torch.zeros(2 + chunks, dtype=torch.int32, device=dev)
      ws.push, ws.pull = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
      ws.lanes = [torch.cuda.Stream(device=dev) for _ in others]
      ws.pull_lanes = [torch.cuda.Stream(device=dev) for _ in others]
      ws.rank = me
      torch.cuda.synchronize()
      dist.barrier(group=pg)
    except Exception as e:  # pylint: disable=broad-except
      import warnings
      warnings.warn("peer memory for the row-split FFN schedule unavailable (%r)" % (e,))
      ws = None
    self._ffn_ws[key] = ws
    return ws

  # GEMM on the compute stream, exchange by the copy engines on a second stream
  # (mtfc_gemm_with_progress and friends).  Off by default: the copy engines do overlap
  # the GEMM completely, but each chunk costs two cross-GPU handshakes and about eight
  # dependent stream operations (~60 us measured per chunk at 2 GPUs), which at the
  # benchmark's sizes (64-128 MiB outputs, 0.1-0.2 ms GEMMs) is slower than the
  # single-kernel form; it pays for outputs of several hundred MiB.
  # MTFC_PIPELINED_ALLREDUCE=1 switches it on.
  PIPELINED_ALLREDUCE = os.environ.get("MTFC_PIPELINED_ALLREDUCE", "0") == "1"
  PIPELINE_MIN_BYTES = 4 << 20
  PIPELINE_MAX_CHUNKS = 8

  def _einsum_allreduce_pipelined(self, ops, equation, a, b, pg, members, pnum):
    """The einsum and its SUM allreduce over `members` with the exchange on the copy
    engines, or None when the contraction does not qualify (nothing launched then).

    The product is ONE launch of the CTA-pair GEMM into a local buffer of partial
    sums; it counts finished 256-row blocks.  On a second stream, chunk by chunk of
    row blocks: wait for the chunk's blocks (a small polling kernel), push the part
    of the chunk each other rank owns into that rank's receive buffer (peer copies:
    copy engines, which take nothing from the SMs and overlap the GEMM fully), tell
    the peers, wait for their parts, add the n copies of the own part (fp32
    accumulation, one rounding), push the sum into every rank's output buffer, tell
    the peers.  The chunk's exchange overlaps the multiplication of the later
    chunks; after the last GEMM tile only the last chunk's exchange remains.  Per
    direction and GPU 2 (n-1)/n times the output crosses NVLink, as in a ring
    allreduce.  Every rank receives the same bits (each part is summed once, by its
    owner).  All waits are bounded."""
    import ctypes
    import torch
    from mesh_b200 import _native as nat
    from mesh_b200.device_ops import HookDeclined
    lib = nat.lib()
    n_ranks = len(members)

    def hook(desc, a_ptr, b_ptr, stored_shape):
      m, n = int(desc.m), int(desc.n)
      nbytes = m * n * 2
      if m % 256 != 0 or n % 8 != 0 or nbytes < self.PIPELINE_MIN_BYTES or (m // 256) % n_ranks != 0:
        return None
      ws = self._pipeline_workspace(pg, members, pnum, m, n)
      if ws is None:
        return None
      main = torch.cuda.current_stream()
      comm = ws.stream
      fork = torch.cuda.Event()
      fork.record(main)
      result = torch.empty(m * n, dtype=torch.bfloat16, device=ws.part.device)
      c_desc = nat.GemmDesc()
      ctypes.memmove(ctypes.byref(c_desc), ctypes.byref(desc), ctypes.sizeof(nat.GemmDesc))
      nat.check(lib.mtfc_gemm_with_progress(
          ctypes.byref(c_desc), ctypes.c_void_p(a_ptr), ctypes.c_void_p(b_ptr),
          ctypes.c_void_p(ws.part.data_ptr()), ctypes.c_void_p(ws.progress.data_ptr()),
          ctypes.c_void_p(main.cuda_stream)))
      me, C, bpc, prow = ws.rank, ws.chunks, ws.blocks_per_chunk, ws.part_rows
      others = [r for r in range(n_ranks) if r != me]
      part2d = ws.part.view(m, n)
      out2d = ws.out.view(m, n)
      comm.wait_event(fork)
      with torch.cuda.stream(comm):
        cs = ctypes.c_void_p(comm.cuda_stream)
        flags_ptr, epochs_ptr = ws.flags.data_ptr(), ws.epochs.data_ptr()
        for c in range(C):
          row0 = c * bpc * 256
          nat.check(lib.mtfc_wait_counters(ctypes.c_void_p(ws.progress.data_ptr() + 4 * c * bpc), bpc,
                                           8 * ws.tiles_n, ctypes.c_void_p(epochs_ptr + 4 * (C + 1 + c)), cs))
          for r in others:     # reduce-scatter: my partial of rank r's part goes to rank r
            ws.peer_recv[r][me, c].copy_(part2d[row0 + r * prow:row0 + (r + 1) * prow], non_blocking=True)
          nat.check(lib.mtfc_signal_peers(ws.peer_flag_ptrs, len(others), c, cs))
          nat.check(lib.mtfc_wait_counters(ctypes.c_void_p(flags_ptr + 4 * c), 1, n_ranks - 1,
                                           ctypes.c_void_p(epochs_ptr + 4 * c), cs))
          mine = slice(row0 + me * prow, row0 + (me + 1) * prow)
          srcs = (ctypes.c_void_p * n_ranks)(*[
              ctypes.c_void_p(part2d[mine].data_ptr() if r == me else ws.recv[r, c].data_ptr())
              for r in range(n_ranks)])
          nat.check(lib.mtfc_add_n_bf16(srcs, n_ranks, ctypes.c_void_p(out2d[mine].data_ptr()),
                                        prow * n, cs))
          for r in others:     # allgather: my sum goes to every rank's output
            ws.peer_out[r][mine].copy_(out2d[mine], non_blocking=True)
          nat.check(lib.mtfc_signal_peers(ws.peer_flag_ptrs, len(others), C + c, cs))
        nat.check(lib.mtfc_wait_counters(ctypes.c_void_p(flags_ptr + 4 * C), C, n_ranks - 1,
                                         ctypes.c_void_p(epochs_ptr + 4 * C), cs))
        # the buffers serve the next contraction of this shape: hand back a copy
        result.copy_(ws.out, non_blocking=True)
      main.wait_stream(comm)
      return self._device_array(result, stored_shape, a.dtype)
    try:
      return ops.einsum(equation, a, b, gemm_hook=hook)
    except HookDeclined:
      return None

  def _pipeline_workspace(self, pg, members, pnum, m, n):
    """Receive / output / counter buffers (peer-mapped) and the local partial-sum
    buffer for an [m, n] bf16 GEMM allreduced over `members`; created collectively on
    first use.  None when symmetric memory is unavailable."""
    import ctypes
    import torch
    import torch.distributed as dist
    key = (tuple(members), m, n)
    if not hasattr(self, "_pipe_ws"):
      self._pipe_ws = {}
    if key in self._pipe_ws:
      return self._pipe_ws[key]
    ws = None
    try:
      import torch.distributed._symmetric_memory as symm
      dev = torch.device("cuda", torch.cuda.current_device())
      n_ranks = len(members)
      me = members.index(pnum)
      num_rb = m // 256
      per_rank = num_rb // n_ranks
      chunks = max(c for c in range(1, self.PIPELINE_MAX_CHUNKS + 1) if per_rank % c == 0)
      bpc = num_rb // chunks
      prow = bpc * 256 // n_ranks

      def alloc(count, dtype):
        t = symm.empty(count, dtype=dtype, device=dev)
        return t, symm.rendezvous(t, pg)
      recv_t, recv_h = alloc(m * n, torch.bfloat16)       # [source rank, chunk, part rows, n]
      out_t, out_h = alloc(m * n, torch.bfloat16)
      flag_t, flag_h = alloc(2 * chunks, torch.int32)
      flag_t.zero_()
      if int(recv_h.rank) != me or int(recv_h.world_size) != n_ranks:
        raise RuntimeError("symmetric-memory rank %d/%d does not match mesh group position %d/%d"
                           % (recv_h.rank, recv_h.world_size, me, n_ranks))
      ws = _PipelineWorkspace()
      ws.part = torch.empty(m * n, dtype=torch.bfloat16, device=dev)
      ws.recv = recv_t.view(n_ranks, chunks, prow, n)
      ws.out = out_t
      ws.flags = flag_t
      ws.progress = torch.zeros(num_rb, dtype=torch.int32, device=dev)
      ws.epochs = torch.zeros(2 * chunks + 2, dtype=torch.int32, device=dev)
      ws.handles = (recv_h, out_h, flag_h)
      ws.peer_recv = {r: recv_h.get_buffer(r, (n_ranks, chunks, prow, n), torch.bfloat16)
                      for r in range(n_ranks) if r != me}
      ws.peer_out = {r: out_h.get_buffer(r, (m, n), torch.bfloat16) for r in range(n_ranks) if r != me}
      peers = [int(flag_h.buffer_ptrs[r]) for r in range(n_ranks) if r != me]
      ws.peer_flag_ptrs = (ctypes.c_void_p * len(peers))(*[ctypes.c_void_p(p) for p in peers])
      ws.stream = torch.cuda.Stream(device=dev)
      ws.rank, ws.nranks = me, n_ranks
      ws.chunks, ws.blocks_per_chunk, ws.part_rows = chunks, bpc, prow
      ws.tiles_n = (n + 255) // 256
      torch.cuda.synchronize()
      dist.barrier(group=pg)
    except Exception as e:  # pylint: disable=broad-except
      import warnings
      warnings.warn("peer memory for the pipelined einsum+allreduce unavailable (%r)" % (e,))
      ws = None
    self._pipe_ws[key] = ws
    return ws

  def _einsum_allreduce_fused(self, ops, equation, a, b, pg, members, pnum):
    """The einsum and its allreduce over `members` as one kernel launch per
    rank, or None when the contraction is not a single bf16 GEMM (then nothing
    has been launched)."""
    import ctypes
    import torch
    from mesh_b200 import _native as nat
    lib = nat.lib()

    def hook(desc, a_ptr, b_ptr, stored_shape):
      nbytes = int(desc.m) * int(desc.n) * 2
      if desc.n % 8 != 0 or nbytes < self.FUSED_MIN_BYTES or nbytes > self.FUSED_MAX_BYTES:
        return None
      ws = self._peer_workspace(pg, members, pnum, int(desc.m), int(desc.n))
      if ws is None:
        return None
      nat.check(lib.mtfc_gemm_allreduce_ex(
          ctypes.byref(desc), ctypes.c_void_p(a_ptr), ctypes.c_void_p(b_ptr), ws.stage_ptrs,
          ws.out_ptrs, ws.flag_ptrs, ctypes.c_void_p(ws.ctl.data_ptr()), ws.rank, ws.nranks,
          ws.exchange, ctypes.c_void_p(ws.mc_stage), ctypes.c_void_p(ws.mc_out),
          ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
      # the workspace is reused by the next contraction of this size: hand back a copy
      flat = ws.out_tensor[:nbytes].view(torch.bfloat16).clone()
      return self._device_array(flat, stored_shape, a.dtype)

    from mesh_b200.device_ops import HookDeclined
    try:
      return ops.einsum(equation, a, b, gemm_hook=hook)
    except HookDeclined:
      return None

  # The alltoall as one kernel over peer-mapped memory (mtfc_alltoall_peer): every rank
  # stores its parts straight into the peers' output buffers in the concatenated
  # layout.  MTFC_PEER_ALLTOALL=0 selects the library alltoall with its pack and unpack
  # passes, which also serves slices under 64 KiB, rows that are not multiples of 16
  # bytes, and processes without peer mappings.
  PEER_ALLTOALL = os.environ.get("MTFC_PEER_ALLTOALL", "1") == "1"
  PEER_ALLTOALL_MIN_BYTES = 64 * 1024

  # Result slots per alltoall size beside the shared one (slot 0): a result lives in a slot
  # of its own for as long as any tensor made from it does, so nothing has to be copied
  # out; with every slot taken, slot 0 is used and its contents are copied.
  PEER_ALLTOALL_SLOTS = 6
  PEER_ALLTOALL_POOL_BYTES = 1 << 30

  def _alltoall_workspace(self, pg, members, pnum, nbytes):
    """Peer-mapped result slots for alltoalls of `nbytes` plus the flag array, per
    group and size (created collectively on first use).  None when symmetric
    memory is unavailable."""
    import ctypes
    import torch
    import torch.distributed as dist
    from mesh_b200 import _native as nat
    key = (tuple(members), nbytes)
    if not hasattr(self, "_a2a_ws"):
      self._a2a_ws = {}
    if key in self._a2a_ws:
      return self._a2a_ws[key]
    ws = None
    try:
      import torch.distributed._symmetric_memory as symm
      dev = torch.device("cuda", torch.cuda.current_device())
      stride = (nbytes + 255) // 256 * 256
      slots = 1 + max(0, min(self.PEER_ALLTOALL_SLOTS, self.PEER_ALLTOALL_POOL_BYTES // stride - 1))
      out_t = symm.empty(slots * stride, dtype=torch.uint8, device=dev)
      out_h = symm.rendezvous(out_t, pg)
      flag_t = symm.empty(int(nat.lib().mtfc_alltoall_peer_flag_bytes()), dtype=torch.uint8, device=dev)
      flag_h = symm.rendezvous(flag_t, pg)
      flag_t.zero_()
      ctl = torch.zeros(2, dtype=torch.int32, device=dev)
      torch.cuda.synchronize()
      dist.barrier(group=pg)
      if int(out_h.rank) != members.index(pnum) or int(out_h.world_size) != len(members):
        raise RuntimeError("symmetric-memory rank %d/%d does not match mesh group position"
                           % (out_h.rank, out_h.world_size))

      def ptr_array(handle):
        ptrs = list(handle.buffer_ptrs)
        return (ctypes.c_void_p * len(ptrs))(*[ctypes.c_void_p(int(p)) for p in ptrs])
      ws = _AlltoallWorkspace()
      ws.tensors, ws.handles = (out_t, flag_t), (out_h, flag_h)
      ws.out_tensor, ws.ctl = out_t, ctl
      ws.out_ptrs, ws.flag_ptrs = ptr_array(out_h), ptr_array(flag_h)
      ws.nbytes, ws.stride = nbytes, stride
      ws.free = list(range(slots - 1, 0, -1))     # slot 0 is the shared one
      ws.pinned = []
    except Exception as e:  # pylint: disable=broad-except
      import warnings
      warnings.warn("peer memory for the alltoall unavailable (%r); using NCCL" % (e,))
      ws = None
    self._a2a_ws[key] = ws
    return ws

  def _peer_alltoall(self, s, pg, members, pnum, split_axis, concat_axis):
    """The peer-memory alltoall of slice `s`, or None when it does not apply."""
    import ctypes
    import torch
    from mesh_b200 import _native as nat
    from mesh_b200.device_ops import _TORCH
    n = len(members)
    nbytes = s.size * s.dtype.itemsize
    if not self.PEER_ALLTOALL or n > 8 or nbytes < self.PEER_ALLTOALL_MIN_BYTES:
      return None
    plan = alltoall_peer_plan(s.shape, s.dtype.itemsize, n, split_axis, concat_axis)
    if plan is None:
      return None
    out_shape, lead, row_bytes, src_part_stride, dst_part_stride = plan
    ws = self._alltoall_workspace(pg, members, pnum, nbytes)
    if ws is None:
      return None
    ops = self._ops_for(pnum)
    src = ops.contiguous(s)
    slot = ws.free.pop() if ws.free else 0
    i64s = lambda vals: (ctypes.c_int64 * max(1, len(vals)))(*vals)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    nat.check(nat.lib().mtfc_alltoall_peer(
        ctypes.c_void_p(src.ptr), ws.out_ptrs, ws.flag_ptrs, n, members.index(pnum), len(lead),
        i64s([d for d, _, _ in lead]), i64s([a for _, a, _ in lead]), i64s([b for _, _, b in lead]),
        row_bytes, src_part_stride, dst_part_stride, slot, ws.stride,
        ctypes.c_void_p(ws.ctl.data_ptr()), stream))
    if slot == 0:
      # every slot is taken: the shared one serves, and its contents are handed back as a copy
      shared = ws.out_tensor[:nbytes].view(_TORCH[s.dtype.name])
      return _fresh_copy(ops, self._device_array(shared, out_shape, s.dtype))
    # The result stays where the peers stored it.  The slot returns to the free list when
    # the last tensor over this memory is gone; a slot taken while a CUDA graph is being
    # recorded belongs to the graph until release_graphs().
    owner = _SlotOwner(ws.out_tensor.data_ptr() + slot * ws.stride, nbytes, ws, slot)
    if getattr(self, "_capturing", False):
      ws.pinned.append(owner)
    flat = torch.as_tensor(owner, device=ws.out_tensor.device).view(_TORCH[s.dtype.name])
    return self._device_array(flat, out_shape, s.dtype)

  def _peer_workspace(self, pg, members, pnum, m, n):
    """Peer-mapped staging / output / flag buffers for an [m, n] bf16 GEMM that
    is allreduced over `members` (created collectively on first use: every rank
    of the group reaches this point for the same contraction).  None when
    symmetric memory is unavailable."""
    import ctypes
    import torch
    import torch.distributed as dist
    from mesh_b200 import _native as nat
    key = (tuple(members), m, n)
    if not hasattr(self, "_peer_ws"):
      self._peer_ws = {}
    if key in self._peer_ws:
      return self._peer_ws[key]
    ws = None
    try:
      import torch.distributed._symmetric_memory as symm
      dev = torch.device("cuda", torch.cuda.current_device())
      lib = nat.lib()
      nbytes = m * n * 2

      def alloc(size):
        t = symm.empty(size, dtype=torch.uint8, device=dev)
        return t, symm.rendezvous(t, pg)
      part_t, part_h = alloc(int(lib.mtfc_gemm_allreduce_stage_bytes(m, n, len(members))))
      out_t, out_h = alloc(nbytes)
      flag_t, flag_h = alloc(int(lib.mtfc_gemm_allreduce_flag_bytes()))
      flag_t.zero_()
      ctl = torch.zeros(4, dtype=torch.int32, device=dev)
      torch.cuda.synchronize()
      dist.barrier(group=pg)

      def ptr_array(handle):
        ptrs = list(handle.buffer_ptrs)
        return (ctypes.c_void_p * len(ptrs))(*[ctypes.c_void_p(int(p)) for p in ptrs])
      ws = _PeerWorkspace()
      ws.tensors = (part_t, out_t, flag_t)
      ws.handles = (part_h, out_h, flag_h)
      ws.out_tensor = out_t
      ws.ctl = ctl
      ws.stage_ptrs, ws.out_ptrs, ws.flag_ptrs = ptr_array(part_h), ptr_array(out_h), ptr_array(flag_h)
      ws.rank, ws.nranks = members.index(pnum), len(members)
      # How the partial products travel (see mtfc_gemm_allreduce_ex).  "auto" is the
      # form that measured fastest: remote epilogue stores ("push").  At 2 GPUs with a
      # 128 MiB output: push 0.43 ms, pull 0.50, multimem 0.58 for a 0.20 ms GEMM (the
      # switch-reduced form moves (1 + 1/n) x the output per direction, which only
      # undercuts push's 2 (n-1)/n from four ranks up).
      ws.mc_stage = ws.mc_out = 0
      mc_s, mc_o = int(part_h.multicast_ptr or 0), int(out_h.multicast_ptr or 0)
      form = self.FUSED_EXCHANGE
      if form == "auto":
        form = "push"
      if form == "multimem" and not (mc_s and mc_o):
        form = "pull"
      if form == "multimem":
        ws.mc_stage, ws.mc_out = mc_s, mc_o
      ws.exchange = {"push": nat.EXCHANGE_PUSH, "pull": nat.EXCHANGE_PULL,
                     "multimem": nat.EXCHANGE_MULTIMEM}[form]
      if int(part_h.rank) != ws.rank or int(part_h.world_size) != ws.nranks:
        raise RuntimeError("symmetric-memory rank %d/%d does not match mesh group position %d/%d"
                           % (part_h.rank, part_h.world_size, ws.rank, ws.nranks))
    except Exception as e:  # pylint: disable=broad-except
      import warnings
      warnings.warn("peer memory for the fused einsum+allreduce unavailable (%r); using NCCL" % (e,))
      ws = None
    self._peer_ws[key] = ws
    return ws

  def _as_torch(self, s):
    packed = self._ops.contiguous(s)
    return packed.buf[packed.offset:packed.offset + max(1, packed.size)]

  def _from_torch(self, t, shape, dtype, pnum):
    return self._device_array(t, shape, dtype)

  def _owns_storage(self, s, t):
    # a slice that spans its whole buffer shares it with no other view
    return s.offset == 0 and s.is_contiguous and s.buf.numel() == max(1, s.size) \
        and t.data_ptr() == s.buf.data_ptr()

  def export_to_host_tensors(self, laid_out_x, out=None, tensor=None):
    """Copies this process's slices to host torch tensors in their own dtype.

    `out`, a list of (pinned) CPU tensors, one per local slice, makes the
    copies asynchronous on the current stream; call synchronize() before
    reading them.  The cheap sibling of export_to_tf_tensor for callers that
    consume slices rather than the assembled full tensor.

    With `tensor` (the mtf.Tensor the slices belong to) in a one-process-per-GPU
    job, a slice that other processes hold replicas of is downloaded in parts:
    replica j of k copies only elements [j*n/k, (j+1)*n/k) of the flattened
    slice into the same region of its `out` buffer, so every byte of the tensor
    crosses a host link once.  Returns, in that case, [(out, begin, end)]."""
    laid_out_x = laid_out_x.to_laid_out_tensor()
    if tensor is not None and self._distributed and out is not None:
      group = self._replica_group(tensor.shape)
      s = laid_out_x.all_slices[0]
      if group is not None and s.size % len(group[1]) == 0:
        _, members, me = group
        ops = self._ops_for(self._local_pnums[0])
        ops._activate()
        packed = ops.contiguous(s)
        chunk = s.size // len(members)
        src = packed.buf[packed.offset + me * chunk:packed.offset + (me + 1) * chunk]
        out[0].reshape(-1)[me * chunk:(me + 1) * chunk].copy_(src, non_blocking=True)
        return [(out[0], me * chunk, (me + 1) * chunk)]
    result = []
    for i, (pnum, s) in enumerate(zip(self._local_pnums, laid_out_x.all_slices)):
      ops = self._ops_for(pnum)
      result.append(ops.to_host_tensor(s, None if out is None else out[i]))
    return result

  def capture(self, fn, warmup=2):
    """Records `fn` (e.g. a whole `mtf.Lowering` of a graph) into a CUDA graph.

    The lowering of a Mesh TensorFlow graph is a fixed sequence of kernel
    launches, copies and collectives; replaying it as one CUDA graph removes
    the per-operation host work from every later step.  `fn` runs `warmup`
    times eagerly (first-use set-up must not happen during capture), then once
    under capture.  Returns `(result, replay)`: `result` is what the captured
    run of `fn` returned — its slices are rewritten in place by every
    `replay()`.  `fn` must not synchronise with the host (no export).
    """
    import torch
    dev = self._devices[self._local_pnums[0]]
    with torch.cuda.device(dev):
      for _ in range(max(1, warmup)):
        fn()
      torch.cuda.synchronize()
      graph = torch.cuda.CUDAGraph()
      self._capturing = True
      try:
        with torch.cuda.graph(graph):
          result = fn()
      finally:
        self._capturing = False
      torch.cuda.synchronize()
    if not hasattr(self, "_graphs"):
      self._graphs = []
    self._graphs.append(graph)
    return result, graph.replay

  def release_graphs(self):
    """Destroys every CUDA graph recorded through capture().  A recorded graph
    that contains NCCL kernels holds a reference on their communicator, and the
    communicator's teardown waits for those references: release the graphs
    (after synchronising) before destroying the process group."""
    import torch
    torch.cuda.synchronize()
    for graph in getattr(self, "_graphs", []):
      graph.reset()
    self._graphs = []
    for ws in getattr(self, "_a2a_ws", {}).values():
      if ws is not None:
        ws.pinned = []

  def _raise_if_a_kernel_gave_up(self):
    self.synchronize()

  def synchronize(self):
    """Waits for all enqueued work and raises if a kernel reported a timeout."""
    import torch
    from mesh_b200 import _native as nat
    try:
      for dev in sorted(set(self._devices[p] for p in self._local_pnums), key=str):
        with torch.cuda.device(dev):
          nat.device_status()
    except nat.MtfcError:
      # a fused einsum+allreduce whose wait ran out leaves its flags and epoch
      # counters out of step with the other ranks: never reuse those buffers
      self._peer_ws = {}
      self._pipe_ws = {}
      self._ffn_ws = {}
      self._a2a_ws = {}
      raise
