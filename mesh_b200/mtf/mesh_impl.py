"""MeshImpl: the operator API that Lowering drives, plus its layout algebra.

Restates the abstract backend of mesh_tensorflow/ops.py:867-1340.  A backend
holds, for every processor it owns, one slice of each laid-out tensor and
provides

  * `slice_ops`: the array library its slices are computed with (the role
    TensorFlow's `tf.*` plays in the reference), and
  * the collectives allreduce / allconcat / alltoall / receive.

Everything else (slice shapes and offsets, allsplit, shift_by_n_processors,
processor coordinates, broadcast, make_slices / combine_slices) is derived
here, in the same terms as the reference so that the same graphs lower to the
same sequence of backend calls.

A backend may own all processors of the mesh (one process drives every slice,
as PlacementMeshImpl does) or a subset (one process per GPU); `local_pnums`
lists the processors whose slices live in this process, in ascending order.
"""

from __future__ import annotations

from mesh_b200.mtf.layout import (convert_to_layout_rules,
                                  pnum_to_processor_coordinates)
from mesh_b200.mtf.shapes import Shape, convert_to_shape, list_product


class LazyAllreduceSum(object):
  """A laid-out tensor whose SUM allreduce has not been run yet.

  Adding two compatible lazies first and reducing once halves the traffic
  (mesh_tensorflow/ops.py:1343-1382).
  """

  def __init__(self, mesh_impl, laid_out_input, mesh_axes, add_counter_fn=None):
    self.mesh_impl = mesh_impl
    self.laid_out_input = laid_out_input
    self.mesh_axes = mesh_axes
    self.add_counter_fn = add_counter_fn
    self._reduced = None

  def to_laid_out_tensor(self):
    if self._reduced is None:
      # the unreduced input is reachable only through this object: a backend
      # that can reduce in place is told so
      if getattr(self.mesh_impl, "allreduce_accepts_donation", False):
        self._reduced = self.mesh_impl.allreduce(self.laid_out_input, self.mesh_axes, "SUM",
                                                 donate=True)
      else:
        self._reduced = self.mesh_impl.allreduce(self.laid_out_input, self.mesh_axes, "SUM")
      self.laid_out_input = None
      if self.add_counter_fn:
        self.add_counter_fn()
    return self._reduced

  @property
  def slice_shape(self):
    if self._reduced is not None:
      return self._reduced.slice_shape
    return self.laid_out_input.slice_shape


class LazyLaidOutTensor(object):
  """A LaidOutTensor made by a function when it is first needed
  (mesh_tensorflow/ops.py:3941-3958): `to_laid_out_tensor_fn()` runs on every
  to_laid_out_tensor() call.  Importing one (import_laid_out_tensor) makes the
  function run once per lowering, which is how a step's input is uploaded
  from host memory at the time the step is lowered."""

  def __init__(self, to_laid_out_tensor_fn, slice_shape):
    self._to_laid_out_tensor_fn = to_laid_out_tensor_fn
    self._slice_shape = list(slice_shape)

  def to_laid_out_tensor(self):
    return self._to_laid_out_tensor_fn()

  @property
  def slice_shape(self):
    return self._slice_shape


def compatible_lazy_allreduce_sums(xs):
  if not xs or not all(isinstance(x, LazyAllreduceSum) for x in xs):
    return False
  first = xs[0]
  if any(x.laid_out_input is None for x in xs):
    return False   # already reduced (and its input given up): use the reduced value
  return all(y.mesh_impl is first.mesh_impl and y.mesh_axes == first.mesh_axes
             for y in xs[1:])


def convert_args_to_laid_out_tensors(xs):
  return [x.to_laid_out_tensor() if hasattr(x, "to_laid_out_tensor") else x for x in xs]


class MeshImpl(object):
  """Base class of mesh backends (mesh_tensorflow/ops.py:867-1340)."""

  def __init__(self, shape, layout_rules):
    self._shape = convert_to_shape(shape)
    self._layout_rules = convert_to_layout_rules(layout_rules)

  # ------------------------------------------------------------ properties
  @property
  def shape(self):
    return self._shape

  @property
  def ndims(self):
    return len(self._shape)

  @property
  def layout_rules(self):
    return self._layout_rules

  @property
  def size(self):
    return self._shape.size

  @property
  def supports_control_dependencies(self):
    return True

  @property
  def local_pnums(self):
    """Processor numbers whose slices this process holds (default: all)."""
    return list(range(self.size))

  @property
  def slice_ops(self):
    """The array library slices are computed with."""
    raise NotImplementedError("slice_ops not implemented")

  # ------------------------------------------------------------ layout algebra
  def tensor_dimension_to_mesh_axis(self, tensor_dimension):
    return self._layout_rules.tensor_dimension_to_mesh_axis(tensor_dimension, self._shape)

  def tensor_layout(self, arg):
    if not isinstance(arg, Shape):
      arg = arg.shape
    return self._layout_rules.tensor_layout(arg, self._shape)

  def mesh_axis_to_cumprod(self, tensor_shape):
    """Per mesh axis: product of the tensor dims before the dim split over it."""
    ma2ta = self.tensor_layout(tensor_shape).mesh_axis_to_tensor_axis(self.ndims)
    cumprod = tensor_shape.cumprod
    return [None if ta is None else cumprod[ta] for ta in ma2ta]

  def slice_shape(self, tensor_shape):
    layout = self.tensor_layout(tensor_shape)
    out = []
    for dim, mesh_axis in zip(tensor_shape, layout.tensor_axis_to_mesh_axis):
      if mesh_axis is None:
        out.append(dim.size)
        continue
      parts = self._shape[mesh_axis].size
      if dim.size % parts != 0:
        raise ValueError(
            "Tensor dimension size not divisible by mesh dimension size:"
            " tensor_shape=%s tensor_layout=%s" % (tensor_shape, layout))
      out.append(dim.size // parts)
    return out

  def slice_begin(self, tensor_shape, pnum):
    layout = self.tensor_layout(tensor_shape)
    coord = pnum_to_processor_coordinates(self._shape, pnum)
    out = []
    for size, mesh_axis in zip(tensor_shape.to_integer_list, layout.tensor_axis_to_mesh_axis):
      if mesh_axis is None:
        out.append(0)
      else:
        out.append(size // self._shape[mesh_axis].size * coord[mesh_axis])
    return out

  def slice_size(self, tensor_shape):
    return list_product(self.slice_shape(tensor_shape))

  def laid_out_size(self, tensor_shape):
    return self.slice_size(tensor_shape) * self.size

  # ------------------------------------------------------------ backend hooks
  def slicewise(self, fn, *inputs):
    raise NotImplementedError("Slicewise not implemented")

  def allreduce(self, x, mesh_axes, reduction_fn_string):
    raise NotImplementedError("Allreduce not implemented")

  def allconcat(self, x, mesh_axis, concat_axis):
    raise NotImplementedError("Allconcat not implemented")

  def alltoall(self, x, mesh_axis, split_axis, concat_axis):
    raise NotImplementedError("Alltoall not implemented")

  def receive(self, x, mesh_axis, source_pcoord):
    raise NotImplementedError("Receive not implemented")

  def laid_out_pnum(self):
    raise NotImplementedError("laid_out_pnum not implemented")

  def export_to_tf_tensor(self, x, laid_out_x):
    raise NotImplementedError("export_to_tf_tensor not implemented")

  def import_tf_tensor(self, x, tf_x):
    raise NotImplementedError("Import not implemented")

  def einsum(self, equation, *slices):
    """Per-slice contraction hook (mesh_tensorflow/ops.py:1331-1340)."""
    return self.slice_ops.einsum(equation, *slices)

  def Print(self, x, data, message, **kwargs):  # pylint: disable=invalid-name
    del data, message, kwargs
    return x

  # ------------------------------------------------------------ derived ops
  def slicewise_delay_allreduce(self, fn, *inputs):
    """Stays lazy when every input is a compatible LazyAllreduceSum."""
    if compatible_lazy_allreduce_sums(inputs):
      return LazyAllreduceSum(
          self, self.slicewise(fn, *[x.laid_out_input for x in inputs]),
          inputs[0].mesh_axes, add_counter_fn=inputs[0].add_counter_fn)
    return self.slicewise(fn, *inputs)

  def allsplit(self, x, mesh_axis, split_axis, which=None):
    """Keeps this processor's 1/n of each slice; no communication."""
    if which is None:
      which = self.laid_out_pcoord(mesh_axis)
    parts = self._shape[mesh_axis].size
    ops = self.slice_ops

    def keep_own_part(xs, part):
      shape = list(ops.shape(xs))
      begin = [0] * len(shape)
      size = list(shape)
      size[split_axis] = shape[split_axis] // parts
      begin[split_axis] = size[split_axis] * int(part)
      return ops.slice(xs, begin, size)
    return self.slicewise(keep_own_part, x, which)

  def shift_by_n_processors(self, x, mesh_axis, offset, wrap):
    """Each processor receives the slice of the one `offset` places before it."""
    n = self._shape[mesh_axis].size
    source_pcoord = []
    for i in range(n):
      c = i - offset
      if c != c % n:
        c = c % n if wrap else None
      source_pcoord.append(c)
    return self.receive(x, mesh_axis, source_pcoord)

  def laid_out_pcoord(self, mesh_axis):
    divisor = list_product(self._shape.to_integer_list[mesh_axis + 1:])
    modulus = self._shape[mesh_axis].size
    return self.slicewise(lambda pnum: (int(pnum) // divisor) % modulus, self.laid_out_pnum())

  def laid_out_slice_num(self, tensor_shape):
    """An integer per processor, equal exactly for processors with equal slices."""
    ret = self.slicewise(lambda pnum: 0, self.laid_out_pnum())
    for mesh_axis in self.tensor_layout(tensor_shape).tensor_axis_to_mesh_axis:
      if mesh_axis is not None:
        size = self._shape[mesh_axis].size
        ret = self.slicewise(lambda acc, pc, size=size: acc * size + pc,
                             ret, self.laid_out_pcoord(mesh_axis))
    return ret

  def broadcast_impl(self, old_slices, old_shape, new_shape):
    new_slice_shape = self.slice_shape(new_shape)
    ops = self.slice_ops

    def widen(xs):
      return ops.broadcast_to(expand_dims_to(ops, xs, old_shape, new_shape), new_slice_shape)
    return self.slicewise(widen, old_slices)

  def make_slices(self, full_tensor, tensor_shape):
    """One slice of `full_tensor` per local processor (ops.py:1249-1269)."""
    layout = self.tensor_layout(tensor_shape)
    slice_shape = self.slice_shape(tensor_shape)
    ops = self.slice_ops
    out = []
    for pnum in self.local_pnums:
      if layout.is_fully_replicated:
        out.append(full_tensor)
      else:
        out.append(ops.slice(full_tensor, self.slice_begin(tensor_shape, pnum), slice_shape))
    return out

  def combine_slices(self, slices, tensor_shape, device=None):
    """Reassembles the full tensor from all `self.size` slices (ops.py:1271-1305).

    Mesh axes are folded first to last; a mesh axis no tensor dim is split over
    keeps the first replica.
    """
    del device
    if tensor_shape.ndims == 0:
      return slices[0]
    ops = self.slice_ops
    ret = list(slices)
    ma2ta = self.tensor_layout(tensor_shape).mesh_axis_to_tensor_axis(self.ndims)
    for mesh_dim, tensor_axis in zip(self._shape, ma2ta):
      span = len(ret) // mesh_dim.size
      if tensor_axis is None:
        ret = ret[:span]
      else:
        ret = [ops.concat([ret[i + span * j] for j in range(mesh_dim.size)], tensor_axis)
               for i in range(span)]
    assert len(ret) == 1
    return ret[0]


def expand_dims_to(ops, x, input_shape, output_shape):
  """Transposes/unsqueezes a slice of `input_shape` so it broadcasts against
  slices of `output_shape` (mesh_tensorflow/ops.py:5322-5343)."""
  for d in input_shape.dims:
    if d not in output_shape.dims:
      raise ValueError("dimension %s of %s is not in %s" % (d, input_shape, output_shape))
  if input_shape == output_shape or input_shape.ndims == 0:
    return x
  perm = [input_shape.dims.index(d) for d in output_shape.dims if d in input_shape.dims]
  x = ops.transpose(x, perm)
  for axis, d in enumerate(output_shape.dims):
    if d not in input_shape.dims:
      x = ops.expand_dims(x, axis)
  return x
