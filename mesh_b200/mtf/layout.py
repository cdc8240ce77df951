"""Layout rules: which tensor dimension is split over which mesh dimension.

Restates LayoutRules / TensorLayout (mesh_tensorflow/ops.py:225-378) and the
processor-number arithmetic (ops.py:5407-5486).  Processor numbers are
row-major over the mesh dimensions: the last mesh dimension varies fastest.
"""

from __future__ import annotations

from mesh_b200.mtf.shapes import Shape, parse_pairs


class TensorLayout(object):
  """Injective partial map tensor axis -> mesh axis (None = not split)."""

  def __init__(self, tensor_axis_to_mesh_axis):
    self._t2m = tuple(tensor_axis_to_mesh_axis)

  def __eq__(self, other):
    return self._t2m == other._t2m

  def __ne__(self, other):
    return self._t2m != other._t2m

  def __repr__(self):
    return "TensorLayout%s" % (self._t2m,)

  def __len__(self):
    return len(self._t2m)

  def __getitem__(self, key):
    return self._t2m[key]

  def __iter__(self):
    return iter(self._t2m)

  @property
  def tensor_axis_to_mesh_axis(self):
    return self._t2m

  @property
  def is_fully_replicated(self):
    return all(a is None for a in self._t2m)

  def mesh_axis_to_tensor_axis(self, mesh_ndims):
    return tuple(self._t2m.index(ma) if ma in self._t2m else None
                 for ma in range(mesh_ndims))


class LayoutRules(object):
  """A set of (tensor dimension name, mesh dimension name) pairs."""

  def __init__(self, pairs):
    self._pairs = set((str(a), str(b)) for a, b in pairs)

  def __repr__(self):
    return "LayoutRules%s" % (sorted(self._pairs),)

  @property
  def pairs(self):
    return set(self._pairs)

  def tensor_dimension_to_mesh_axis(self, tensor_dimension, mesh_shape):
    hits = [i for i, md in enumerate(mesh_shape)
            if (tensor_dimension.name, md.name) in self._pairs]
    if len(hits) > 1:
      raise ValueError(
          "Tensor dimension maps to multiple mesh dimensions"
          " tensor_dimension=%s mesh_shape=%s layout=%s"
          % (tensor_dimension, mesh_shape, sorted(self._pairs)))
    return hits[0] if hits else None

  def tensor_layout(self, tensor_shape, mesh_shape):
    axes = [self.tensor_dimension_to_mesh_axis(d, mesh_shape) for d in tensor_shape]
    used = [a for a in axes if a is not None]
    if len(used) != len(set(used)):
      raise ValueError(
          "Two Tensor Dimensions may not map to the same Mesh Dimension:"
          " layout=%s tensor_shape=%s mesh_shape=%s " % (self, tensor_shape, mesh_shape))
    return TensorLayout(axes)

  def mesh_dimension_name_to_tensor_dimension_names(self, mesh_dimension_name):
    return [t for t, m in self._pairs if m == mesh_dimension_name]


def convert_to_layout_rules(x):
  """Accepts LayoutRules, "batch:rows;d_ff:cols" or an iterable of pairs."""
  if isinstance(x, LayoutRules):
    return x
  if isinstance(x, str):
    x = parse_pairs(x)
  if isinstance(x, dict):
    x = list(x.items())
  return LayoutRules(x)


def _sizes(mesh_shape):
  if isinstance(mesh_shape, Shape):
    return mesh_shape.to_integer_list
  if not isinstance(mesh_shape, list):
    raise ValueError("mesh_shape must be a Shape or a list of integers")
  return mesh_shape


def pnum_to_processor_coordinates(mesh_shape, pnum):
  coords = []
  for size in reversed(_sizes(mesh_shape)):
    coords.append(pnum % size)
    pnum //= size
  return coords[::-1]


def processor_coordinates_to_pnum(mesh_shape, coord):
  pnum = 0
  for c, size in zip(coord, _sizes(mesh_shape)):
    pnum = pnum * size + c
  return pnum


def pnum_to_group(mesh_shape, group_dims, pnum):
  """Index of the group of processors that differ from `pnum` only in group_dims."""
  sizes = _sizes(mesh_shape)
  coord = pnum_to_processor_coordinates(sizes, pnum)
  keep = [i for i in range(len(sizes)) if i not in group_dims]
  return processor_coordinates_to_pnum([sizes[i] for i in keep], [coord[i] for i in keep])


def processor_groups(mesh_shape, group_dims):
  """Groups in ascending group number, members in ascending processor number."""
  sizes = _sizes(mesh_shape)
  total = 1
  for s in sizes:
    total *= s
  groups = {}
  for pnum in range(total):
    groups.setdefault(pnum_to_group(sizes, group_dims, pnum), []).append(pnum)
  return [groups[g] for g in sorted(groups)]


def tensor_dim_to_mesh_dim_size(layout, mesh_shape, tensor_dim):
  """Size of the mesh dimension `tensor_dim` is split over, or 1 (ops.py:5872-5886)."""
  from mesh_b200.mtf.shapes import convert_to_shape
  layout_rules = convert_to_layout_rules(layout)
  mesh_shape = convert_to_shape(mesh_shape)
  axis = layout_rules.tensor_dimension_to_mesh_axis(tensor_dim, mesh_shape)
  return 1 if axis is None else mesh_shape.dims[axis].size
