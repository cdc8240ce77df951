"""Graph, Mesh, Tensor, Operation and Lowering of the mesh-tensor language.

Restates the graph containers and the lowering driver of
mesh_tensorflow/ops.py (Graph 381-440, Lowering 676-838, Tensor 1423-1640,
Operation 1523-1648).  Lowering walks the operations in construction order
and each Operation.lower() speaks only the MeshImpl operator API, so any
backend with that API can be handed to `Lowering(graph, {mesh: impl})`.
"""

from __future__ import annotations

import collections

from mesh_b200.mtf.shapes import convert_to_shape


class DType(collections.namedtuple("DType", ["name", "is_floating", "is_integer", "itemsize"])):
  __slots__ = ()

  def __repr__(self):
    return "mtf.%s" % self.name

  @property
  def is_bool(self):
    return self.name == "bool"


float32 = DType("float32", True, False, 4)
bfloat16 = DType("bfloat16", True, False, 2)
int32 = DType("int32", False, True, 4)
bool_ = DType("bool", False, False, 4)


class Graph(object):
  """An ordered list of operations (mesh_tensorflow/ops.py:381-440)."""

  def __init__(self):
    self._operations = []
    self._names = collections.Counter()

  @property
  def operations(self):
    return self._operations

  def unique_name(self, name):
    self._names[name] += 1
    n = self._names[name]
    return name if n == 1 else "%s_%d" % (name, n - 1)

  @property
  def to_string(self):
    return "\n".join(op.to_string for op in self._operations)


class Mesh(object):
  """A placeholder for a mesh; its shape and layout come from the MeshImpl."""

  def __init__(self, graph, name, variable_placer=None):
    del variable_placer
    self._graph = graph
    self._name = name

  @property
  def graph(self):
    return self._graph

  @property
  def name(self):
    return self._name


class Tensor(object):
  """A distributed tensor with a named Shape, produced by an Operation."""

  def __init__(self, operation, shape, dtype, name=None, index=0):
    self._operation = operation
    self._shape = convert_to_shape(shape)
    if not isinstance(dtype, DType):
      raise ValueError("dtype must be an mtf DType, got %r" % (dtype,))
    self._dtype = dtype
    self._name = name or "%s:%d" % (operation.name, index)

  @property
  def shape(self):
    return self._shape

  @property
  def size(self):
    return self._shape.size

  @property
  def mesh(self):
    return self._operation.mesh

  @property
  def graph(self):
    return self._operation.graph

  @property
  def operation(self):
    return self._operation

  @property
  def dtype(self):
    return self._dtype

  @property
  def name(self):
    return self._name

  def __repr__(self):
    return "Tensor[%s, %s, %s]" % (self._name, self._shape, self._dtype)

  to_string = property(__repr__)

  # Operators are bound by mesh_b200.mtf.ops at import time.


class Operation(object):
  """A node of the graph; subclasses implement lower()."""

  def __init__(self, inputs, mesh=None, name=None):
    if mesh is None:
      if not inputs:
        raise ValueError("mesh must be given for operations without inputs")
      mesh = inputs[0].mesh
    self._inputs = list(inputs)
    self._outputs = []
    self._mesh = mesh
    self._name = mesh.graph.unique_name(name or type(self).__name__)
    mesh.graph.operations.append(self)

  @property
  def graph(self):
    return self._mesh.graph

  @property
  def mesh(self):
    return self._mesh

  @property
  def name(self):
    return self._name

  @property
  def inputs(self):
    return list(self._inputs)

  @property
  def outputs(self):
    return list(self._outputs)

  @property
  def to_string(self):
    return "%s[Inputs=(%s) Outputs=(%s)]" % (
        type(self).__name__, ", ".join(x.to_string for x in self._inputs),
        ", ".join(x.to_string for x in self._outputs))

  @property
  def has_gradient(self):
    """Whether gradients() differentiates through this operation
    (mesh_tensorflow/ops.py:1569-1573): by default when every output is
    floating point; operations without a gradient() override it."""
    return all(t.dtype.is_floating for t in self._outputs)

  def gradient(self, grad_ys):
    """Gradients with respect to the inputs, one per input (None where there is
    none), given the gradients of the outputs (None where none flows in)."""
    raise NotImplementedError("Gradient not implemented for %s" % type(self).__name__)

  def lower(self, lowering):
    raise NotImplementedError("Lower not implemented")


class Lowering(object):
  """Runs every operation of a graph on the given mesh backends.

  `tensors` maps each graph Tensor to a LaidOutTensor or a lazy wrapper with
  `to_laid_out_tensor()`; counters record the laid-out sizes of outputs,
  einsums and collectives exactly as the reference does (ops.py:792-798).
  """

  def __init__(self, graph, mesh_to_impl, autostack=True, log_file=None):
    del autostack, log_file
    self.mesh_to_impl = mesh_to_impl
    self.graph = graph
    self._counters = []
    self._consumers = None
    self.tensors = {}
    self.operations = {}
    self.variables = {}
    for op in graph.operations:
      op.lower(self)
      for out in op.outputs:
        self.add_counter("output/%s" % type(op).__name__, self.laid_out_size(out))
        self.add_counter("output_unique/%s" % type(op).__name__, out.size)

  def mesh_impl(self, m):
    if not isinstance(m, Mesh):
      m = m.mesh
    return self.mesh_to_impl[m]

  def consumers(self, tensor):
    """How many operation inputs of the graph read `tensor`."""
    if self._consumers is None:
      self._consumers = collections.Counter(t for op in self.graph.operations for t in op.inputs)
    return self._consumers[tensor]

  def export_to_tf_tensor(self, x):
    """The full tensor on the host (a numpy array; bfloat16 widened to float32)."""
    impl = self.mesh_impl(x)
    return impl.export_to_tf_tensor(x, self.tensors[x].to_laid_out_tensor())

  export = export_to_tf_tensor

  def copy_slices_to_masters(self, variables=None):
    """Device slices -> host masters for every lowered variable (or the given
    ones), mesh_tensorflow/ops.py:730-737."""
    for var, laid_out_variable in self.variables.items():
      if variables is None or var in variables:
        laid_out_variable.copy_slices_to_master()

  def copy_masters_to_slices(self, variables=None):
    """Host masters -> device slices (mesh_tensorflow/ops.py:739-745)."""
    for var, laid_out_variable in self.variables.items():
      if variables is None or var in variables:
        laid_out_variable.copy_master_to_slices()

  def lowered_operation(self, op):
    return self.operations[op]

  def add_counter(self, key, value):
    assert isinstance(value, int)
    self._counters.append((key, value))

  @property
  def counters(self):
    return self._counters

  def counter_totals(self):
    totals = collections.OrderedDict()
    for k, v in self._counters:
      totals[k] = totals.get(k, 0) + v
    return totals

  def laid_out_size(self, tensor):
    return self.mesh_impl(tensor).laid_out_size(tensor.shape)

  def set_tensor_lowering(self, tensor, laid_out_tensor):
    self.verify_slice_shapes(tensor, laid_out_tensor)
    self.tensors[tensor] = laid_out_tensor

  def verify_slice_shapes(self, tensor, laid_out_tensor):
    correct = self.mesh_impl(tensor).slice_shape(tensor.shape)
    actual = list(laid_out_tensor.slice_shape)
    if actual != correct:
      raise ValueError(
          "Wrong slice shape: correct_shape = %s actual shape = %s" % (correct, actual))
