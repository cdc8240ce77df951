"""NumpyMeshImpl: the reference's PlacementMeshImpl, restated over numpy slices.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

One numpy slice per processor in a Python list, exactly the shape of
mesh_tensorflow/placement_mesh_impl.py:31-355.  Collectives follow the
reference's data movement and, for allreduce, its order of floating-point
additions (allreduce_ring_single_shard 358-404, the per-shard rotation of
allreduce_ring 407-455).  allconcat / alltoall / receive only copy, so they
are written as their specification (alltoall_pointtwise 490-510).
"""

from __future__ import annotations

import numpy as np

from mesh_b200 import mtf
from mesh_b200.mtf.mesh_impl import convert_args_to_laid_out_tensors
from oracle.numpy_ops import Arr, NumpyOps, _finish


class NumpyMeshImpl(mtf.MeshImpl):
  """CPU mesh backend with PlacementMeshImpl semantics."""

  def __init__(self, shape, layout, devices=None, fast=False):
    super().__init__(shape, layout)
    self._devices = list(devices) if devices is not None else [""] * self.size
    if len(self._devices) != self.size:
      raise ValueError("devices must have one entry per processor")
    self._ops = NumpyOps(fast=fast)

  class LaidOutTensor(object):
    """One slice per processor (placement_mesh_impl.py:39-65)."""

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
      return list(t.shape) if isinstance(t, Arr) else []

    def to_laid_out_tensor(self):
      return self

  class LaidOutVariable(object):
    """Slices of a variable and the copies to / from its host master
    (placement_mesh_impl.py:67-157)."""

    def __init__(self, variable, mesh_impl):
      self._variable, self._mesh_impl = variable, mesh_impl
      self._laid_out_tensor = mesh_impl.import_tf_tensor(variable.outputs[0],
                                                         variable.get_master())

    @property
    def laid_out_tensor(self):
      return self._laid_out_tensor

    def assign_to_slices(self, assign_fn, values):
      self._laid_out_tensor = self._mesh_impl.LaidOutTensor(
          [assign_fn(self._variable, old, v)
           for old, v in zip(self._laid_out_tensor.all_slices, values)])
      return self._laid_out_tensor

    def copy_master_to_slices(self):
      fresh = self._mesh_impl.import_tf_tensor(self._variable.outputs[0],
                                               self._variable.get_master())
      return self.assign_to_slices(lambda var, old, value: value, fresh.all_slices)

    def copy_slices_to_master(self):
      self._variable.assign_to_master(self._mesh_impl.export_to_tf_tensor(
          self._variable.outputs[0], self._laid_out_tensor), from_slices=self)

  @property
  def slice_ops(self):
    return self._ops

  @property
  def devices(self):
    return self._devices

  def slicewise(self, fn, *inputs):
    inputs = convert_args_to_laid_out_tensors(inputs)
    per_input = [x.tensor_list if isinstance(x, self.LaidOutTensor) else [x] * self.size
                 for x in inputs]
    ret = [fn(*[col[p] for col in per_input]) for p in range(self.size)]
    if isinstance(ret[0], tuple):
      return tuple(self.LaidOutTensor(list(t)) for t in zip(*ret))
    return self.LaidOutTensor(ret)

  def laid_out_pnum(self):
    return self.LaidOutTensor(list(range(self.size)))

  def random(self, shape, tf_fn, kwargs):
    """placement_mesh_impl.py:307-325: one draw per slice, seeded from the
    operation's seed and the slice's offset so that replicas agree."""
    import hashlib
    kwargs = dict(kwargs)
    op_seed = kwargs.pop("seed", 0)
    dtype = kwargs.pop("dtype", mtf.float32)
    slice_shape = self.slice_shape(shape)
    ops = self._ops

    def my_fn(pnum):
      text = "%s,%s" % (op_seed, self.slice_begin(shape, pnum))
      seed = int.from_bytes(hashlib.sha256(text.encode()).digest()[:8], "little")
      if callable(tf_fn):
        return tf_fn(ops, slice_shape, seed=seed, dtype=dtype, **kwargs)
      if tf_fn == "uniform":
        return ops.random(slice_shape, "uniform", seed, dtype,
                          float(kwargs.get("minval", 0.0)), float(kwargs.get("maxval", 1.0)))
      return ops.random(slice_shape, "normal", seed, dtype,
                        float(kwargs.get("mean", 0.0)), float(kwargs.get("stddev", 1.0)))
    return self.slicewise(my_fn, self.laid_out_pnum())

  def import_tf_tensor(self, x, tf_x):
    full = self._ops.from_host(tf_x, x.dtype)
    return self.LaidOutTensor(self.make_slices(full, x.shape))

  def export_to_tf_tensor(self, x, laid_out_x):
    return self._ops.to_host(self.combine_slices(laid_out_x.all_slices, x.shape))

  # ------------------------------------------------------------ collectives
  def _collective_with_groups(self, x, mesh_axes, collective):
    if not mesh_axes:
      return x
    x = x.to_laid_out_tensor()
    if len(mesh_axes) == self.ndims:
      return self.LaidOutTensor(collective(x.tensor_list))
    ret = [None] * self.size
    for group in mtf.processor_groups(self.shape, mesh_axes):
      for pnum, y in zip(group, collective([x.tensor_list[p] for p in group])):
        ret[pnum] = y
    return self.LaidOutTensor(ret)

  def allreduce(self, x, mesh_axes, reduction_fn_string):
    return self._collective_with_groups(
        x, mesh_axes, lambda xs: allreduce_ring(xs, reduction_fn_string))

  def allconcat(self, x, mesh_axis, concat_axis):
    return self._collective_with_groups(
        x, [mesh_axis],
        lambda xs: [Arr(np.concatenate([t.a for t in xs], axis=concat_axis), xs[0].dtype)
                    for _ in xs])

  def alltoall(self, x, mesh_axis, split_axis, concat_axis):
    def collective(xs):
      n = len(xs)
      parts = [np.split(t.a, n, axis=split_axis) for t in xs]  # [source][target]
      return [Arr(np.concatenate([parts[src][dst] for src in range(n)], axis=concat_axis),
                  xs[0].dtype) for dst in range(n)]
    return self._collective_with_groups(x, [mesh_axis], collective)

  def receive(self, x, mesh_axis, source_pcoord):
    def collective(xs):
      return [Arr(np.zeros_like(xs[0].a), xs[0].dtype) if src is None
              else Arr(xs[src].a.copy(), xs[0].dtype) for src in source_pcoord]
    return self._collective_with_groups(x, [mesh_axis], collective)


def _reduce2(name, a, b, dtype):
  """tf.add / tf.maximum / tf.minimum on two slices (ops.py:5687-5695)."""
  if name == "SUM":
    r = a + b
  elif name == "MAX":
    r = np.maximum(a, b)
  elif name == "MIN":
    r = np.minimum(a, b)
  else:
    raise ValueError("unknown reduction %s" % name)
  return _finish(r, dtype).a


def allreduce_single_shard(arrays, name, dtype):
  """(x0 + ... + x_lc) + (x_rc + ... + x_{n-1}) with the left sum built
  left-to-right and the right sum right-to-left (placement_mesh_impl.py:378-397)."""
  n = len(arrays)
  if n == 1:
    return arrays[0]
  left_center = n // 2 - 1 if n % 2 == 0 else n // 2
  left = arrays[0]
  for i in range(1, left_center + 1):
    left = _reduce2(name, left, arrays[i], dtype)
  right = arrays[n - 1]
  for i in reversed(range(left_center + 1, n - 1)):
    right = _reduce2(name, arrays[i], right, dtype)
  return _reduce2(name, left, right, dtype)


def allreduce_ring(xs, name):
  """Sharded variant: shard s is reduced over the list rotated right by s
  when the slice has >= 1024 elements divisible by n (placement_mesh_impl.py:407-455)."""
  n = len(xs)
  if n == 1:
    return xs
  dtype = xs[0].dtype
  shape = xs[0].a.shape
  size = int(np.prod(shape)) if shape else 1
  if size < 1024 or size % n != 0:
    total = allreduce_single_shard([t.a for t in xs], name, dtype)
    return [Arr(total.copy(), dtype) for _ in xs]
  shards = [np.split(t.a.reshape(-1), n) for t in xs]  # [device][shard]
  reduced = []
  for s in range(n):
    column = [shards[d][s] for d in range(n)]
    k = s % n
    rotated = column[-k:] + column[:-k] if k else column
    reduced.append(allreduce_single_shard(rotated, name, dtype))
  total = np.concatenate(reduced).reshape(shape)
  return [Arr(total.copy(), dtype) for _ in xs]
