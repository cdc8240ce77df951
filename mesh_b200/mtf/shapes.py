"""Named dimensions and shapes of the mesh-tensor language.

Restates Dimension / Shape of mesh_tensorflow/ops.py:41-223 (same attribute
names and the same conversions from strings and lists), without TensorFlow.
"""

from __future__ import annotations

import collections
import functools
import operator
import re


def list_product(xs):
  return functools.reduce(operator.mul, xs, 1)


class Dimension(collections.namedtuple("Dimension", ["name", "size"])):
  """A named tensor or mesh dimension (mesh_tensorflow/ops.py:41-47)."""
  __slots__ = ()

  def __new__(cls, name, size):
    if not isinstance(name, str):
      raise ValueError("Dimension name must be a string, got %r" % (name,))
    return super().__new__(cls, name, int(size))


def convert_to_dimension(d):
  """Accepts a Dimension, a (name, size) pair or None (ops.py:50-67)."""
  if d is None:
    return None
  if isinstance(d, Dimension):
    return d
  name, size = d
  if isinstance(name, str) and isinstance(size, int):
    return Dimension(name, size)
  raise ValueError("could not convert %r to a Dimension" % (d,))


def parse_pairs(text, seconds_to_int=False):
  """Parses "a:b c:d", "a:b,c:d", "a:b;c:d" or "a:b.c:d" (ops.py:5612-5639)."""
  pairs = []
  for token in re.split(r"[,.; ]", text):
    if not token:
      continue
    first, second = token.split(":")
    pairs.append((first, int(second) if seconds_to_int else second))
  return pairs


class Shape(object):
  """An ordered list of Dimensions with unique names (ops.py:70-223)."""

  def __init__(self, dims):
    self._dims = [convert_to_dimension(d) for d in tuple(dims)]
    names = [d.name for d in self._dims]
    if len(set(names)) != len(names):
      raise ValueError("Shape must not have repeated dimension names: %s" % (names,))

  # ---- container protocol
  def __repr__(self):
    return "Shape[%s]" % ", ".join("%s=%d" % (d.name, d.size) for d in self._dims)

  to_string = property(__repr__)

  def __eq__(self, other):
    return isinstance(other, Shape) and self._dims == other._dims

  def __ne__(self, other):
    return not self == other

  def __hash__(self):
    return hash(tuple(self._dims))

  def __len__(self):
    return len(self._dims)

  def __getitem__(self, key):
    return self._dims[key]

  def __iter__(self):
    return iter(self._dims)

  def __add__(self, other):
    if isinstance(other, Shape):
      other = other.dims
    if isinstance(other, Dimension):
      other = [other]
    return Shape(self.dims + list(other))

  def __sub__(self, other):
    if other is None:
      return self
    if isinstance(other, Shape):
      other = other.dims
    if isinstance(other, Dimension):
      if other not in self._dims:
        raise ValueError("cannot subtract %s: not in %s" % (other, self))
      other = [other]
    return Shape([d for d in self._dims if d not in other])

  # ---- properties
  @property
  def dims(self):
    return list(self._dims)

  @property
  def ndims(self):
    return len(self._dims)

  @property
  def to_integer_list(self):
    return [d.size for d in self._dims]

  @property
  def size(self):
    return list_product(self.to_integer_list)

  @property
  def dimension_names(self):
    return [d.name for d in self._dims]

  @property
  def cumprod(self):
    """Exclusive running product of the sizes: cumprod[i] = prod(size[:i])."""
    out, acc = [], 1
    for d in self._dims:
      out.append(acc)
      acc *= d.size
    return out

  def cumprod_to_tensor_axis(self, cumprod):
    """Largest axis whose exclusive running product equals `cumprod`, or None."""
    mine = self.cumprod
    for axis in range(len(mine) - 1, -1, -1):
      if mine[axis] == cumprod:
        return axis
    return None

  def rename_dimension(self, old_name, new_name):
    if old_name not in self.dimension_names:
      raise ValueError("Shape %s has no dimension named %s" % (self, old_name))
    return Shape([Dimension(new_name, d.size) if d.name == old_name else d
                  for d in self._dims])

  def resize_dimension(self, name, new_size):
    if name not in self.dimension_names:
      raise ValueError("Shape %s has no dimension named %s" % (self, name))
    return Shape([Dimension(name, new_size) if d.name == name else d
                  for d in self._dims])

  def get_dim_by_name(self, name):
    for d in self._dims:
      if d.name == name:
        return d
    raise ValueError("Dimension %s not found in %s" % (name, self))


def convert_to_shape(x):
  """Accepts a Shape, a list of Dimensions/pairs, or "name:size,..." (ops.py:226-243)."""
  if x is None:
    return None
  if isinstance(x, Shape):
    return x
  if isinstance(x, str):
    x = parse_pairs(x, seconds_to_int=True)
  return Shape(x)


def shape_union(shapes):
  """Dimensions of all shapes in first-appearance order (ops.py:5374-5383)."""
  seen = []
  for s in shapes:
    for d in s.dims:
      if d not in seen:
        seen.append(d)
  return Shape(seen)
