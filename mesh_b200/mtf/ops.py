"""Operations of the mesh-tensor language and their lowerings.

Each Operation.lower() below issues the same MeshImpl calls, in the same
order, as its counterpart in mesh_tensorflow/ops.py; the per-slice work is
expressed against `mesh_impl.slice_ops` (the array library of the backend)
where the reference closes over `tf.*`.  Only the operations the dense FFN,
top-2 mixture-of-experts and attention layers are built from are present.
"""

from __future__ import annotations

import functools

import numpy as np

from mesh_b200.mtf import graph as G
from mesh_b200.mtf.graph import Operation, Tensor
from mesh_b200.mtf.mesh_impl import LazyAllreduceSum, LazyLaidOutTensor, expand_dims_to
from mesh_b200.mtf.shapes import (Dimension, Shape, convert_to_dimension, list_product,
                                  convert_to_shape, shape_union)


# --------------------------------------------------------------------- import
class ImportOperation(Operation):
  """Brings a host array into the graph (mesh_tensorflow/ops.py:3854-3890)."""

  def __init__(self, mesh, value, shape, dtype, name=None):
    super().__init__([], mesh=mesh, name=name or "import")
    self._value = value
    self._outputs = [Tensor(self, shape, dtype)]
    self._uploaded = {}

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    # A numpy array is a constant of the graph: it is laid out once per backend
    # and later lowerings of the same graph reuse the slices (which also keeps
    # host copies out of a lowering that is being recorded as a CUDA graph).
    # Torch host tensors are live inputs and are copied on every lowering.
    constant = isinstance(self._value, np.ndarray)
    laid_out = self._uploaded.get(id(impl)) if constant else None
    if laid_out is None:
      laid_out = impl.import_tf_tensor(self.outputs[0], self._value)
      if constant:
        self._uploaded[id(impl)] = laid_out
    lowering.set_tensor_lowering(self.outputs[0], laid_out)


_NP_TO_DTYPE = {"float32": G.float32, "float64": G.float32, "int32": G.int32,
                "int64": G.int32, "bool": G.bool_, "bfloat16": G.bfloat16}


def import_tf_tensor(mesh, tf_tensor, shape=None, name=None, dtype=None):
  """Imports a host array (numpy, a torch CPU tensor, or anything np.asarray
  accepts) as a Tensor.

  `dtype` selects the on-device type; values are rounded to it on import
  (mtf.bfloat16 rounds float32 data to nearest-even).
  """
  value = tf_tensor if hasattr(tf_tensor, "data_ptr") else np.asarray(tf_tensor)
  if shape is None:
    shape = Shape([])
    if tuple(value.shape) != ():
      raise ValueError("shape must be given for a non-scalar import")
  shape = convert_to_shape(shape)
  if list(value.shape) != shape.to_integer_list:
    raise ValueError("Incompatible shape: array %s vs %s" % (value.shape, shape))
  if dtype is None:
    dtype = _NP_TO_DTYPE.get(getattr(value.dtype, "name", str(value.dtype).replace("torch.", "")))
    if dtype is None:
      raise ValueError("cannot infer an mtf dtype from %s" % value.dtype)
  return ImportOperation(mesh, value, shape, dtype, name=name).outputs[0]


import_tensor = import_tf_tensor


class ImportLaidOutTensorOperation(Operation):
  """Brings slices that already live on the mesh into the graph
  (mesh_tensorflow/ops.py:3893-3938)."""

  def __init__(self, mesh, laid_out_tensor, shape, dtype, name=None):
    super().__init__([], mesh=mesh, name=name or "import")
    self._laid_out_tensor = laid_out_tensor
    self._outputs = [Tensor(self, shape, dtype)]

  def lower(self, lowering):
    value = self._laid_out_tensor
    if isinstance(value, LazyLaidOutTensor):
      value = value.to_laid_out_tensor()   # once per lowering, not once per consumer
    lowering.set_tensor_lowering(self.outputs[0], value)


def import_laid_out_tensor(mesh, laid_out_tensor, shape, dtype, name=None):
  """Imports a LaidOutTensor (one slice per processor, already on the devices);
  lowering checks its slice shape against the layout."""
  return ImportLaidOutTensorOperation(
      mesh, laid_out_tensor, convert_to_shape(shape), dtype, name=name).outputs[0]


class Variable(Operation):
  """A tensor with a host-resident master copy (mesh_tensorflow/ops.py:3961-4070).

  Lowering lays the master out through `mesh_impl.LaidOutVariable` and records
  it in `lowering.variables`.  The laid-out slices are kept per backend between
  lowerings, so a training loop that lowers the same graph once per step keeps
  its weights and optimizer slots on the devices: the master is uploaded again
  only after the host changed it (assign_to_master, a restored checkpoint), and
  slices travel back only on request (Assign(copy_to_master=True),
  Lowering.copy_slices_to_masters)."""

  def __init__(self, mesh, name, shape, dtype, initial_value, trainable=True):
    super().__init__([], mesh=mesh, name=name)
    shape = convert_to_shape(shape)
    value = np.asarray(initial_value)
    if list(value.shape) != shape.to_integer_list:
      raise ValueError("initial value %s does not match %s" % (value.shape, shape))
    self._master = value
    self._master_version = 0
    self._laid_out = {}      # id(backend) -> (LaidOutVariable, master version it holds)
    self._trainable = trainable
    self._outputs = [Tensor(self, shape, dtype)]
    if not hasattr(mesh.graph, "all_variables"):
      mesh.graph.all_variables = []
    mesh.graph.all_variables.append(self)

  @property
  def trainable(self):
    return self._trainable

  def get_master(self):
    return self._master

  def assign_to_master(self, value, from_slices=None):
    """New master value; `from_slices` names the LaidOutVariable the value was
    read from, whose slices therefore stay current."""
    self._master = np.asarray(value)
    self._master_version += 1
    for key, (lv, _) in list(self._laid_out.items()):
      if lv is from_slices:
        self._laid_out[key] = (lv, self._master_version)

  @property
  def value(self):
    return self.outputs[0]

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    held = self._laid_out.get(id(impl))
    if held is None:
      laid_out_variable = impl.LaidOutVariable(self, impl)
    else:
      laid_out_variable, version = held
      if version != self._master_version:
        laid_out_variable.copy_master_to_slices()
    self._laid_out[id(impl)] = (laid_out_variable, self._master_version)
    lowering.variables[self] = laid_out_variable
    lowering.set_tensor_lowering(self.outputs[0], laid_out_variable.laid_out_tensor)


class Assign(Operation):
  """Replaces the slices of variables by new values (mesh_tensorflow/ops.py:4090-4148).
  Lowering it after the variables' own operations updates their laid-out
  slices in place of the imported ones; `copy_to_master=True` also writes the
  assembled result back to each variable's master copy."""

  def __init__(self, variables, new_values, copy_to_master=True, name=None):
    super().__init__(list(new_values), variables[0].mesh, name=name or "assign")
    for var, val in zip(variables, new_values):
      if var.outputs[0].shape != val.shape:
        raise ValueError("shape mismatch in assign: %s vs %s" % (var.outputs[0].shape, val.shape))
    self._variables = list(variables)
    self._copy_to_master = copy_to_master
    self._outputs = []

  @property
  def has_gradient(self):
    return False

  def lower(self, lowering):
    for var, val in zip(self._variables, self.inputs):
      if var not in lowering.variables:
        raise ValueError("variable %s is assigned before it is lowered" % var.name)
      impl = lowering.mesh_impl(var)
      ops = impl.slice_ops
      dtype = var.outputs[0].dtype
      new = lowering.tensors[val].to_laid_out_tensor()
      laid_out_variable = lowering.variables[var]
      laid_out_variable.assign_to_slices(
          lambda v, old, value: ops.cast(value, dtype), new.all_slices)
      if self._copy_to_master:
        laid_out_variable.copy_slices_to_master()


def assign(variable, new_value, copy_to_master=True):
  """variable <- new_value; `variable` is a Variable or its tensor."""
  var = variable.operation if isinstance(variable, Tensor) else variable
  if not isinstance(var, Variable):
    raise ValueError("assign needs a Variable, got %s" % (var,))
  return Assign([var], [new_value], copy_to_master=copy_to_master)


def assign_add(variable, value, copy_to_master=True):
  var = variable.operation if isinstance(variable, Tensor) else variable
  return assign(var, var.outputs[0] + cast(value, var.outputs[0].dtype), copy_to_master=copy_to_master)


def assign_sub(variable, value, copy_to_master=True):
  var = variable.operation if isinstance(variable, Tensor) else variable
  return assign(var, var.outputs[0] - cast(value, var.outputs[0].dtype), copy_to_master=copy_to_master)


def get_variable(mesh, name, shape, dtype=G.float32, initial_value=None, trainable=True):
  """Creates a Variable and returns its tensor; `.operation` is the Variable."""
  shape = convert_to_shape(shape)
  if initial_value is None:
    initial_value = np.zeros(shape.to_integer_list, dtype=np.float32)
  return Variable(mesh, name, shape, dtype, initial_value, trainable=trainable).outputs[0]


def save_checkpoint(path, variables, lowering=None):
  """Writes the masters of `variables` (Variable operations or their tensors) to
  `path` as a numpy .npz archive keyed by variable name.  With `lowering`, the
  device slices are copied to the masters first, as the reference's checkpoint
  listener does before every save (mesh_tensorflow/ops.py:5740-5757).  The
  reference's files are TensorFlow checkpoints; that container needs TensorFlow
  and is not written here."""
  ops_ = [v.operation if isinstance(v, Tensor) else v for v in variables]
  if lowering is not None:
    lowering.copy_slices_to_masters(ops_)
  arrays = {v.name: np.asarray(v.get_master()) for v in ops_}
  with open(path, "wb") as f:
    np.savez(f, **arrays)


def restore_checkpoint(path, variables):
  """Reads masters back from a save_checkpoint archive; the next lowering lays
  them out again (the reference's restore hook, ops.py:5760-5779)."""
  ops_ = [v.operation if isinstance(v, Tensor) else v for v in variables]
  with np.load(path) as data:
    for v in ops_:
      if v.name not in data:
        raise KeyError("checkpoint %s has no variable %s" % (path, v.name))
      value = data[v.name]
      if list(value.shape) != v.outputs[0].shape.to_integer_list:
        raise ValueError("checkpoint value of %s has shape %s, expected %s"
                         % (v.name, value.shape, v.outputs[0].shape))
      v.assign_to_master(value)


def constant(mesh, value, shape=None, dtype=G.float32):
  """A tensor filled with `value` (mesh_tensorflow/ops.py:4337-4378)."""
  shape = convert_to_shape(shape) if shape is not None else Shape([])
  return ConstantOperation(mesh, value, shape, dtype).outputs[0]


class ConstantOperation(Operation):

  def __init__(self, mesh, value, shape, dtype, name=None):
    super().__init__([], mesh=mesh, name=name or "constant")
    self._value = value
    self._outputs = [Tensor(self, shape, dtype)]

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    slice_shape = impl.slice_shape(self.outputs[0].shape)
    ops = impl.slice_ops
    dtype = self.outputs[0].dtype
    value = self._value
    lowering.set_tensor_lowering(
        self.outputs[0],
        impl.slicewise(lambda pnum: ops.fill(slice_shape, value, dtype), impl.laid_out_pnum()))


def zeros(mesh, shape, dtype=G.float32):
  return constant(mesh, 0, shape=convert_to_shape(shape), dtype=dtype)


def zeros_like(t):
  return zeros(t.mesh, t.shape, dtype=t.dtype)


def mtf_range(mesh, dim, dtype, name=None):
  """[0, dim.size) along `dim`, imported like any host tensor (ops.py:5544-5584)."""
  dim = convert_to_dimension(dim)
  np_dtype = np.int32 if dtype.is_integer else np.float32
  op = ImportOperation(mesh, np.arange(dim.size, dtype=np_dtype), Shape([dim]), dtype,
                       name=name or "range")
  op.is_plain_range = True
  return op.outputs[0]


# ------------------------------------------------------------------ slicewise
class SlicewiseOperation(Operation):
  """Applies a per-slice function to same-shaped inputs (ops.py:1651-1723)."""

  def __init__(self, slice_fn, inputs, output_shape, output_dtype, splittable_dims,
               name=None, grad_function=None):
    super().__init__(inputs, name=name or "slicewise")
    self._slice_fn = slice_fn
    self._grad_function = grad_function
    self._outputs = [Tensor(self, output_shape, output_dtype)]
    self._splittable_dims = [convert_to_dimension(d).name if not isinstance(d, str) else d
                             for d in splittable_dims]

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    for t in self.inputs + self.outputs:
      layout = impl.tensor_layout(t)
      for d, mesh_axis in zip(t.shape.dims, layout.tensor_axis_to_mesh_axis):
        if mesh_axis is not None and d.name not in self._splittable_dims:
          raise ValueError("dimension %s is not declared as splittable" % (d,))
    ops = impl.slice_ops
    fn = self._slice_fn
    value = impl.slicewise(lambda *xs: fn(ops, *xs),
                           *[lowering.tensors[x] for x in self.inputs])
    lowering.set_tensor_lowering(self.outputs[0], value)

  @property
  def has_gradient(self):
    return self._grad_function is not None and super().has_gradient

  def gradient(self, grad_ys):
    """`grad_function(op, dy)` returns one gradient per input
    (mesh_tensorflow/ops.py:1686-1693)."""
    return self._grad_function(self, grad_ys[0])


def cwise(slice_fn, xs, output_dtype=None, name=None, grad_function=None):
  """Component-wise op on same-shaped tensors; `slice_fn(ops, *slices)`."""
  return SlicewiseOperation(slice_fn, xs, xs[0].shape, output_dtype or xs[0].dtype,
                            splittable_dims=xs[0].shape.dims, name=name or "cwise",
                            grad_function=grad_function).outputs[0]


def _mask_times(dy, x, comparison):
  """dy where x > 0, else 0, in one pass over the two tensors (what
  tf.nn.relu's gradient computes)."""
  assert comparison == "greater"
  return cwise(lambda ops, g, v: ops.binary("select_positive", g, v), [dy, x], name="relu_grad")


# d/dx of each differentiable unary op, from x = op.inputs[0], y = op.outputs[0]
# and dy (mesh_tensorflow/ops.py:1724-1962 give the same formulas through
# tf.gradients of the slice function).
_UNARY_GRADS = {
    "identity": lambda op, dy: [dy],
    "relu": lambda op, dy: [_mask_times(dy, op.inputs[0], "greater")],
    "exp": lambda op, dy: [dy * op.outputs[0]],
    "log": lambda op, dy: [dy / op.inputs[0]],
    "negative": lambda op, dy: [negative(dy)],
    "reciprocal": lambda op, dy: [negative(dy * square(op.outputs[0]))],
    "sqrt": lambda op, dy: [dy * 0.5 / op.outputs[0]],
    "rsqrt": lambda op, dy: [dy * -0.5 * op.outputs[0] * square(op.outputs[0])],
    "square": lambda op, dy: [dy * op.inputs[0] * 2.0],
    "tanh": lambda op, dy: [dy * (1.0 - square(op.outputs[0]))],
    "sigmoid": lambda op, dy: [dy * op.outputs[0] * (1.0 - op.outputs[0])],
}


def _unary(name):
  def api(x, name=name):
    return cwise(lambda ops, xs: ops.unary(name, xs), [x], name=name,
                 grad_function=_UNARY_GRADS.get(name))
  api.__name__ = name
  return api


relu = _unary("relu")
exp = _unary("exp")
log = _unary("log")
negative = _unary("negative")
reciprocal = _unary("reciprocal")
sqrt = _unary("sqrt")
rsqrt = _unary("rsqrt")
square = _unary("square")
tanh = _unary("tanh")
sigmoid = _unary("sigmoid")
sign = _unary("sign")
logical_not = _unary("logical_not")
identity = _unary("identity")


def stop_gradient(x, name="stop_gradient"):
  """Identity that gradients() does not cross (mesh_tensorflow/ops.py:1973-1986)."""
  return cwise(lambda ops, xs: ops.unary("identity", xs), [x], name=name)


def cast(x, dtype, name="cast"):
  if dtype == x.dtype:
    return x
  back = x.dtype
  return cwise(lambda ops, xs: ops.cast(xs, dtype), [x], output_dtype=dtype, name=name,
               grad_function=(lambda op, dy: [cast(dy, back)]) if back.is_floating else None)


def to_float(x, name="to_float"):
  return cast(x, G.float32, name=name)


def to_bfloat16(x, name="to_bfloat16"):
  return cast(x, G.bfloat16, name=name)


def to_int32(x, name="to_int32"):
  return cast(x, G.int32, name=name)


class ScalarMultiplyOperation(Operation):

  def __init__(self, x, scalar, name=None):
    super().__init__([x], name=name or "scalar_mul")
    self._outputs = [Tensor(self, x.shape, x.dtype)]
    self._scalar = scalar

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    ops, c = impl.slice_ops, self._scalar
    lowering.set_tensor_lowering(
        self.outputs[0],
        impl.slicewise(lambda xs: ops.binary("multiply", xs, c), lowering.tensors[self.inputs[0]]))

  def gradient(self, grad_ys):
    return [grad_ys[0] * self._scalar]


class ScalarAddOperation(Operation):

  def __init__(self, x, scalar, name=None):
    super().__init__([x], name=name or "scalar_add")
    self._outputs = [Tensor(self, x.shape, x.dtype)]
    self._scalar = scalar

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    ops, c = impl.slice_ops, self._scalar
    lowering.set_tensor_lowering(
        self.outputs[0],
        impl.slicewise(lambda xs: ops.binary("add", xs, c), lowering.tensors[self.inputs[0]]))

  def gradient(self, grad_ys):
    return [grad_ys[0]]


# --------------------------------------------------------------------- binary
def is_subsequence(short, long):
  it = iter(long)
  return all(d in it for d in short)


def _infer_binary_broadcast_shape(shape1, shape2, given_output_shape=None):
  shape1, shape2 = convert_to_shape(shape1), convert_to_shape(shape2)
  given_output_shape = convert_to_shape(given_output_shape)
  if given_output_shape is not None:
    return given_output_shape
  if is_subsequence(shape1.dims, shape2.dims):
    return shape2
  if is_subsequence(shape2.dims, shape1.dims):
    return shape1
  return Shape(shape1.dims + [d for d in shape2.dims if d not in shape1.dims])


def binary_arguments_to_tensors(x1, x2):
  t1, t2 = isinstance(x1, Tensor), isinstance(x2, Tensor)
  if not t1 and not t2:
    raise ValueError("at least one of x1 and x2 must be an mtf Tensor")
  if t1 and t2:
    return x1, x2
  if t1:
    return x1, import_tf_tensor(x1.mesh, np.asarray(x2), Shape([]), dtype=x1.dtype)
  return import_tf_tensor(x2.mesh, np.asarray(x1), Shape([]), dtype=x2.dtype), x2


class BinaryOpWithBroadcasting(Operation):
  """Binary op with named-dim broadcasting (mesh_tensorflow/ops.py:2044-2084)."""

  def __init__(self, op_name, x1, x2, output_shape, output_dtype, name=None):
    super().__init__([x1, x2], name=name or op_name)
    if x1.dtype != x2.dtype:
      raise ValueError("Dtypes must be equal- got %s and %s" % (x1.dtype, x2.dtype))
    self._outputs = [Tensor(self, output_shape, output_dtype)]
    self._op_name = op_name

  def lower(self, lowering):
    x1, x2 = self.inputs
    out = self.outputs[0]
    lx1, lx2 = lowering.tensors[x1], lowering.tensors[x2]
    impl = lowering.mesh_impl(self)
    ops = impl.slice_ops
    if x1.shape != out.shape:
      lx1 = impl.slicewise(lambda xs: expand_dims_to(ops, xs, x1.shape, out.shape), lx1)
    if x2.shape != out.shape:
      lx2 = impl.slicewise(lambda xs: expand_dims_to(ops, xs, x2.shape, out.shape), lx2)
    op_name = self._op_name
    fn = lambda a, b: ops.binary(op_name, a, b)
    if op_name == "add":
      y = impl.slicewise_delay_allreduce(fn, lx1, lx2)
    else:
      y = impl.slicewise(fn, lx1, lx2)
    lowering.set_tensor_lowering(out, y)

  @property
  def has_gradient(self):
    return self._op_name in _BINARY_GRADS and super().has_gradient

  def gradient(self, grad_ys):
    """Per-operand gradients, summed over the dims an operand was broadcast
    along (mesh_tensorflow/ops.py:2086-2199)."""
    x1, x2 = self.inputs
    g1, g2 = _BINARY_GRADS[self._op_name](x1, x2, self.outputs[0], grad_ys[0])
    return [None if g is None else reduce_sum(g, output_shape=x.shape)
            for g, x in ((g1, x1), (g2, x2))]


def binary_op_with_broadcasting(op_name, x1, x2, output_shape=None, output_dtype=None):
  x1, x2 = binary_arguments_to_tensors(x1, x2)
  output_shape = _infer_binary_broadcast_shape(x1.shape, x2.shape, output_shape)
  return BinaryOpWithBroadcasting(op_name, x1, x2, output_shape,
                                  output_dtype or x1.dtype).outputs[0]


def _select_grad(comparison):
  """Gradients of maximum / minimum: dy goes to the operand that was selected
  (ties to the first)."""
  def fn(x1, x2, y, dy):
    del y
    first = cast(binary_op_with_broadcasting(comparison, x1, x2, output_dtype=G.bool_), dy.dtype)
    return dy * first, dy * (1.0 - first)
  return fn


_BINARY_GRADS = {
    "add": lambda x1, x2, y, dy: (dy, dy),
    "sub": lambda x1, x2, y, dy: (dy, negative(dy)),
    "multiply": lambda x1, x2, y, dy: (dy * x2, dy * x1),
    "divide": lambda x1, x2, y, dy: (dy / x2, negative(dy * y / x2)),
    "maximum": _select_grad("greater_equal"),
    "minimum": _select_grad("less_equal"),
}


def _compare(op_name):
  def api(x1, x2, output_shape=None):
    return binary_op_with_broadcasting(op_name, x1, x2, output_shape=output_shape,
                                       output_dtype=G.bool_)
  api.__name__ = op_name
  return api


less = _compare("less")
greater = _compare("greater")
less_equal = _compare("less_equal")
greater_equal = _compare("greater_equal")
equal = _compare("equal")
not_equal = _compare("not_equal")
logical_and = _compare("logical_and")
logical_or = _compare("logical_or")


def maximum(x1, x2, output_shape=None):
  return binary_op_with_broadcasting("maximum", x1, x2, output_shape=output_shape)


def minimum(x1, x2, output_shape=None):
  return binary_op_with_broadcasting("minimum", x1, x2, output_shape=output_shape)


def add(x1, x2, output_shape=None, name=None):
  output_shape = convert_to_shape(output_shape)
  if not isinstance(x2, Tensor):
    return ScalarAddOperation(x1, x2).outputs[0]
  x1, x2 = binary_arguments_to_tensors(x1, x2)
  return BinaryOpWithBroadcasting(
      "add", x1, x2, _infer_binary_broadcast_shape(x1.shape, x2.shape, output_shape),
      x1.dtype, name=name or "add").outputs[0]


def add_n(xs):
  return functools.reduce(add, xs) if xs else 0


def sub(x1, x2, output_shape=None, name=None):
  output_shape = convert_to_shape(output_shape)
  if not isinstance(x2, Tensor):
    return ScalarAddOperation(x1, -x2).outputs[0]
  x1, x2 = binary_arguments_to_tensors(x1, x2)
  return add(x1, negative(x2), output_shape=output_shape)


def multiply(x1, x2, output_shape=None, name=None):
  """A product is an einsum whose output keeps every dim (ops.py:5135-5153)."""
  if not isinstance(x2, Tensor):
    return ScalarMultiplyOperation(x1, x2).outputs[0]
  x1, x2 = binary_arguments_to_tensors(x1, x2)
  return einsum([x1, x2],
                output_shape=_infer_binary_broadcast_shape(x1.shape, x2.shape, output_shape))


def divide(x1, x2, output_shape=None, name=None):
  """x1 * reciprocal(x2) (mesh_tensorflow/ops.py:5156-5172)."""
  output_shape = convert_to_shape(output_shape)
  if not isinstance(x2, Tensor):
    return ScalarMultiplyOperation(x1, 1.0 / x2).outputs[0]
  x1, x2 = binary_arguments_to_tensors(x1, x2)
  return multiply(x1, reciprocal(x2), output_shape=output_shape)


# ------------------------------------------------------------ reduce / einsum
def _reduce_helper(ops, input_shape, output_shape, input_tensor_layout, reduction="SUM"):
  """Per-slice reduction fn and the mesh axes it leaves unreduced (ops.py:2267-2299)."""
  reduce_axes = [i for i, d in enumerate(input_shape.dims) if d not in output_shape.dims]
  kept = [d for d in input_shape.dims if d in output_shape.dims]
  perm = [kept.index(d) for d in output_shape.dims]

  def reduce_slice_fn(xs):
    ret = xs
    if reduce_axes:
      ret = ops.reduce(reduction, xs, reduce_axes)
    if perm != list(range(len(perm))):
      ret = ops.transpose(ret, perm)
    return ret
  reduced_mesh_axes = [input_tensor_layout[i] for i in reduce_axes
                       if input_tensor_layout[i] is not None]
  return reduce_slice_fn, reduced_mesh_axes


class ReduceOperation(Operation):
  """Output dims are a subset of input dims, in any order (ops.py:2302-2338)."""

  def __init__(self, x, output_shape, reduction, name=None):
    super().__init__([x], name=name or "reduce")
    self._outputs = [Tensor(self, output_shape, x.dtype)]
    self._reduction = reduction

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    x, out = self.inputs[0], self.outputs[0]
    fn, reduced_mesh_axes = _reduce_helper(
        impl.slice_ops, x.shape, out.shape, impl.tensor_layout(x), self._reduction)
    y = impl.slicewise(fn, lowering.tensors[x])
    if reduced_mesh_axes:
      def add_counter_fn():
        lowering.add_counter("allreduce/%s/reduce_op" % reduced_mesh_axes,
                             lowering.laid_out_size(out))
      if self._reduction == "SUM":
        y = LazyAllreduceSum(impl, y, reduced_mesh_axes, add_counter_fn=add_counter_fn)
      else:
        y = impl.allreduce(y, reduced_mesh_axes, self._reduction)
        add_counter_fn()
    lowering.set_tensor_lowering(out, y)

  def gradient(self, grad_ys):
    """SUM: dy broadcast back; MAX / MIN: dy to the positions that hold the
    extremum (mesh_tensorflow/ops.py:2340-2362 and 2388-2400)."""
    x, y, dy = self.inputs[0], self.outputs[0], grad_ys[0]
    if self._reduction == "SUM":
      return [broadcast(dy, x.shape)]
    if self._reduction in ("MAX", "MIN"):
      hit = cast(binary_op_with_broadcasting("equal", x, y, output_shape=x.shape,
                                             output_dtype=G.bool_), x.dtype)
      return [multiply(dy, hit, output_shape=x.shape)]
    raise NotImplementedError("gradient of reduction %s" % self._reduction)


def _reduction_output_shape(x, output_shape, reduced_dim):
  if output_shape is None:
    if reduced_dim is None:
      return Shape([])
    if reduced_dim not in x.shape.dims:
      raise ValueError("reduced_dim=%s not in x.shape.dims=%s" % (reduced_dim, x.shape))
    return x.shape - reduced_dim
  if reduced_dim is not None:
    raise ValueError("do not specify both reduced_dim and output_shape")
  return output_shape


def _reduce_api(reduction):
  def api(x, disable_positional_args=None, output_shape=None, reduced_dim=None, name=None):
    assert disable_positional_args is None
    output_shape = _reduction_output_shape(
        x, convert_to_shape(output_shape), convert_to_dimension(reduced_dim))
    if output_shape == x.shape:
      return x
    return ReduceOperation(x, output_shape, reduction, name=name).outputs[0]
  return api


reduce_sum = _reduce_api("SUM")
reduce_max = _reduce_api("MAX")
reduce_min = _reduce_api("MIN")


def reduce_mean(x, disable_positional_args=None, output_shape=None, reduced_dim=None,
                name=None):
  """reduce_sum scaled by the size ratio (mesh_tensorflow/ops.py:4778-4808)."""
  assert disable_positional_args is None
  output_shape = _reduction_output_shape(
      x, convert_to_shape(output_shape), convert_to_dimension(reduced_dim))
  if output_shape == x.shape:
    return x
  return reduce_sum(x, output_shape=output_shape) * (output_shape.size / x.shape.size)


def _einsum_equation(input_shapes, output_shape):
  """Letters in first-appearance order over inputs then output (ops.py:5346-5371)."""
  letters = {}
  parts = []
  for shape in list(input_shapes) + [output_shape]:
    term = []
    for d in shape.dims:
      if d not in letters:
        letters[d] = chr(ord("a") + len(letters))
      term.append(letters[d])
    parts.append("".join(term))
  return ",".join(parts[:-1]) + "->" + parts[-1]


def _einsum_helper(input_shapes, output_shape, mesh_impl, floating, activation=None):
  """Per-slice einsum fn and the mesh axes of split contracted dims (ops.py:2784-2823).

  When some operand or the output already spans every dimension, the product
  is formed by broadcast-multiply-reduce (`einsum_naive`); otherwise, for
  floating types, by the backend's contraction hook `mesh_impl.einsum`.
  `activation` ("relu") is applied to the slice result; a backend that
  declares `supports_einsum_epilogue` gets it as the hook's `epilogue`
  argument and fuses it into the contraction.
  """
  ops = mesh_impl.slice_ops
  union = shape_union(input_shapes)
  full_shapes = [s for s in list(input_shapes) + [output_shape] if s.ndims == union.ndims]
  full_shape = full_shapes[0] if full_shapes else union
  layout = mesh_impl.tensor_layout(full_shape)
  reduce_axes = [i for i, d in enumerate(full_shape.dims) if d not in output_shape.dims]
  reduced_mesh_axes = [layout[i] for i in reduce_axes if layout[i] is not None]
  equation = _einsum_equation(input_shapes, output_shape)
  fuse = activation is not None and not reduced_mesh_axes
  uses_hook = not (full_shapes or not floating)
  if full_shapes or not floating:
    if fuse:
      fn = lambda *slices: ops.unary(activation, ops.einsum_naive(equation, *slices))
    else:
      fn = lambda *slices: ops.einsum_naive(equation, *slices)
  elif fuse and getattr(mesh_impl, "supports_einsum_epilogue", False):
    fn = lambda *slices: mesh_impl.einsum(equation, *slices, epilogue=activation)
  elif fuse:
    fn = lambda *slices: ops.unary(activation, mesh_impl.einsum(equation, *slices))
  else:
    fn = lambda *slices: mesh_impl.einsum(equation, *slices)
  return fn, reduced_mesh_axes, equation, uses_hook


class EinsumOperation(Operation):
  """Einstein summation over named dims (mesh_tensorflow/ops.py:2826-2880)."""

  def __init__(self, inputs, output_shape, name=None, activation=None):
    super().__init__(inputs, name=name or "einsum")
    self._activation = activation
    if not inputs:
      raise ValueError("Einsum needs at least one input")
    for x in inputs:
      if x.dtype != inputs[0].dtype:
        raise ValueError("Input dtypes must be equal got %s" % ([y.dtype for y in inputs],))
    self._outputs = [Tensor(self, output_shape, inputs[0].dtype)]

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    xs = self.inputs
    in_dims = set(sum([x.shape.dims for x in xs], []))
    output_shape = self.outputs[0].shape
    intersection = Shape([d for d in output_shape.dims if d in in_dims])
    fn, reduced_mesh_axes, equation, uses_hook = _einsum_helper(
        [x.shape for x in xs], intersection, impl, xs[0].dtype.is_floating, self._activation)

    def add_counter_fn():
      lowering.add_counter("allreduce/%s/einsum_op" % reduced_mesh_axes,
                           impl.laid_out_size(intersection))
    overlapped = None
    if reduced_mesh_axes and uses_hook and len(xs) == 2 and hasattr(impl, "einsum_allreduce"):
      # a backend may run the contraction in chunks and start each chunk's
      # allreduce while the next chunk is still being computed; it returns None
      # when it prefers the plain sequence
      overlapped = impl.einsum_allreduce(
          equation, [lowering.tensors[x] for x in xs], reduced_mesh_axes)
    if overlapped is not None:
      y = overlapped
      add_counter_fn()
      if self._activation is not None:
        ops, act = impl.slice_ops, self._activation
        y = impl.slicewise(lambda t: ops.unary(act, t), y)
    else:
      y = None
      if (not reduced_mesh_axes and uses_hook and len(xs) == 2 and intersection == output_shape
          and hasattr(impl, "defer_einsum") and lowering.consumers(self.outputs[0]) == 1):
        # a product with a single reader may be left pending: a backend that sees it arrive
        # as the operand of a contraction + allreduce can then schedule both together
        # (anything else that touches it makes it run as usual); None = run it now
        y = impl.defer_einsum(fn, [lowering.tensors[x] for x in xs], equation, self._activation)
      if y is None:
        y = impl.slicewise(fn, *[lowering.tensors[x] for x in xs])
    if reduced_mesh_axes and overlapped is None:
      y = LazyAllreduceSum(impl, y, reduced_mesh_axes, add_counter_fn=add_counter_fn)
      if self._activation is not None:
        # the activation has to see the reduced sum
        ops, act = impl.slice_ops, self._activation
        y = impl.slicewise(lambda t: ops.unary(act, t), y)
    if intersection != output_shape:
      y = impl.broadcast_impl(y, intersection, output_shape)
    lowering.set_tensor_lowering(self.outputs[0], y)
    computation_shape = Shape(sorted(in_dims))
    lowering.add_counter("einsum", impl.laid_out_size(computation_shape))
    lowering.add_counter("einsum_unique", computation_shape.size)

  def gradient(self, grad_ys):
    """d/dx_i = einsum(dy, the other inputs) onto x_i's shape
    (mesh_tensorflow/ops.py:2846-2854); a fused activation is undone first."""
    dy = grad_ys[0]
    if self._activation == "relu":
      dy = _mask_times(dy, self.outputs[0], "greater")
    elif self._activation is not None:
      raise NotImplementedError("gradient through fused activation %s" % self._activation)
    xs = self.inputs
    return [einsum([dy] + [xs[j] for j in range(len(xs)) if j != i], output_shape=xs[i].shape)
            for i in range(len(xs))]


def einsum(xs, output_shape=None, reduced_dims=None, name=None, activation=None):
  """Einstein summation; exactly one of output_shape / reduced_dims may be given
  (mesh_tensorflow/ops.py:4656-4726).  `activation="relu"` applies the ReLU of
  a following mtf.relu inside the same operation."""
  output_shape = convert_to_shape(output_shape)
  union = shape_union([x.shape for x in xs])
  if output_shape is None:
    reduced = [convert_to_dimension(d) for d in (reduced_dims or [])]
    output_shape = Shape([d for d in union.dims if d not in reduced])
  elif reduced_dims is not None:
    computed = [d for d in union.dims if d not in output_shape.dims]
    if set(computed) != set(convert_to_dimension(d) for d in reduced_dims):
      raise ValueError("reduced_dims and output_shape disagree")
  return EinsumOperation(xs, output_shape, name=name, activation=activation).outputs[0]


def matmul(a, b, output_shape=None, reduced_dims=None, name=None):
  return einsum([a, b], output_shape=output_shape, reduced_dims=reduced_dims, name=name)


class BroadcastOperation(Operation):
  """Adds dimensions (mesh_tensorflow/ops.py:2201-2225)."""

  def __init__(self, x, output_shape, name=None):
    super().__init__([x], name=name or "broadcast")
    self._outputs = [Tensor(self, output_shape, x.dtype)]

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    x, out = self.inputs[0], self.outputs[0]
    lowering.set_tensor_lowering(
        out, impl.broadcast_impl(lowering.tensors[x], x.shape, out.shape))

  def gradient(self, grad_ys):
    return [reduce_sum(grad_ys[0], output_shape=self.inputs[0].shape)]


def broadcast(x, new_shape):
  new_shape = convert_to_shape(new_shape)
  if x.shape == new_shape:
    return x
  return BroadcastOperation(x, new_shape).outputs[0]


# -------------------------------------------------------------------- reshape
class ReshapeOperation(Operation):
  """Reshape with the layout change it implies (mesh_tensorflow/ops.py:4477-4584).

  Per mesh axis, the product of the tensor dims preceding the dim split over
  it is compared between old and new shape: newly split -> allsplit (before
  the local reshape when that boundary exists in the old shape, after it
  otherwise), no longer split -> allconcat, split differently -> alltoall.
  """

  def __init__(self, x, new_shape, name=None):
    super().__init__([x], name=name or "reshape")
    self._outputs = [Tensor(self, new_shape, x.dtype)]

  def gradient(self, grad_ys):
    return [reshape(grad_ys[0], self.inputs[0].shape)]

  def lower(self, lowering):
    old_shape = self.inputs[0].shape
    new_shape = self.outputs[0].shape
    impl = lowering.mesh_impl(self)
    slices = lowering.tensors[self.inputs[0]]
    old_cp = impl.mesh_axis_to_cumprod(old_shape)
    new_cp = impl.mesh_axis_to_cumprod(new_shape)
    to_split, to_concat, to_exchange = [], [], []
    for mesh_axis, (old, new) in enumerate(zip(old_cp, new_cp)):
      if new == old:
        continue
      if old is None:
        to_split.append(mesh_axis)
      elif new is None:
        to_concat.append(mesh_axis)
      else:
        to_exchange.append(mesh_axis)

    laid_out_size = impl.laid_out_size(old_shape)
    split_after_reshape = []
    for mesh_axis in to_split:
      tensor_axis = old_shape.cumprod_to_tensor_axis(new_cp[mesh_axis])
      if tensor_axis is None:
        split_after_reshape.append(
            (mesh_axis, new_shape.cumprod_to_tensor_axis(new_cp[mesh_axis])))
      else:
        slices = impl.allsplit(slices, mesh_axis, tensor_axis)
        laid_out_size //= impl.shape[mesh_axis].size
    for mesh_axis in to_exchange:
      split_axis = old_shape.cumprod_to_tensor_axis(new_cp[mesh_axis])
      if split_axis is None:
        raise NotImplementedError(
            "Try first reshaping to insert a new tf dimension,"
            " then changing layout. input_shape=%s output_shape=%s" % (old_shape, new_shape))
      concat_axis = old_shape.cumprod_to_tensor_axis(old_cp[mesh_axis])
      assert concat_axis is not None
      slices = impl.alltoall(slices, mesh_axis, split_axis, concat_axis)
      lowering.add_counter("alltoall/%s/reshape_op" % mesh_axis, laid_out_size)
    for mesh_axis in to_concat:
      tensor_axis = old_shape.cumprod_to_tensor_axis(old_cp[mesh_axis])
      assert tensor_axis is not None
      slices = impl.allconcat(slices, mesh_axis, tensor_axis)
      laid_out_size *= impl.shape[mesh_axis].size
      lowering.add_counter("allconcat/%s/reshape_op" % mesh_axis, laid_out_size)

    new_slice_shape = impl.slice_shape(new_shape)
    for mesh_axis, tensor_axis in split_after_reshape:
      new_slice_shape[tensor_axis] *= impl.shape[mesh_axis].size
    ops = impl.slice_ops
    slices = impl.slicewise_delay_allreduce(lambda xs: ops.reshape(xs, new_slice_shape), slices)
    for mesh_axis, tensor_axis in split_after_reshape:
      slices = impl.allsplit(slices, mesh_axis, tensor_axis)
    lowering.set_tensor_lowering(self.outputs[0], slices)


def reshape(x, new_shape, name="reshape"):
  new_shape = convert_to_shape(new_shape)
  if x.shape.size != new_shape.size:
    raise ValueError("reshape: sizes differ: %s vs %s" % (x.shape, new_shape))
  if x.shape == new_shape:
    return x
  return ReshapeOperation(x, new_shape, name=name).outputs[0]


def rename_dimension(x, old_name, new_name):
  return reshape(x, x.shape.rename_dimension(old_name, new_name))


def replace_dimensions(tensor_or_shape, old_dim_or_dims, new_dim_or_dims):
  """Replaces a run of consecutive dims of a Tensor (by reshape) or of a Shape
  by another run (ops.py:4609-4653)."""
  if isinstance(tensor_or_shape, Tensor):
    return reshape(tensor_or_shape, replace_dimensions(
        tensor_or_shape.shape, old_dim_or_dims, new_dim_or_dims))
  if not isinstance(tensor_or_shape, Shape):
    raise ValueError("tensor_or_shape must be a Tensor or Shape got %s" % (tensor_or_shape,))
  old = [old_dim_or_dims] if isinstance(old_dim_or_dims, Dimension) else list(old_dim_or_dims)
  new = [new_dim_or_dims] if isinstance(new_dim_or_dims, Dimension) else list(new_dim_or_dims)
  dims = tensor_or_shape.dims
  if not old or not new or old[0] not in dims:
    raise ValueError("old_dim_or_dims must be a subsequence of the input's dimensions"
                     " old_dim_or_dims=%s input's dimensions=%s" % (old, dims))
  start = dims.index(old[0])
  if dims[start:start + len(old)] != old:
    raise ValueError("old_dim_or_dims must be a subsequence of the input's dimensions"
                     " old_dim_or_dims=%s input's dimensions=%s" % (old, dims))
  return Shape(dims[:start] + new + dims[start + len(old):])


# ------------------------------------------------------------ top-k / one-hot
class TopKOperation(Operation):
  """Top-k values and indices along one dim (mesh_tensorflow/ops.py:4895-4961)."""

  def __init__(self, x, reduced_dim, k_dim, name=None):
    super().__init__([x], name=name or "top_k")
    if reduced_dim not in x.shape.dims:
      raise ValueError("reduced dim %s must be in x.shape %s" % (reduced_dim, x.shape))
    if k_dim.size > reduced_dim.size:
      raise ValueError("k_dim.size must be <= reduced_dim.size: %s vs %s" % (k_dim, reduced_dim))
    output_shape = x.shape - reduced_dim + k_dim
    self._outputs = [Tensor(self, output_shape, x.dtype, index=0),
                     Tensor(self, output_shape, G.int32, index=1)]
    self._reduced_dim = reduced_dim
    self._k_dim = k_dim

  @property
  def has_gradient(self):
    return self.outputs[0].dtype.is_floating

  def gradient(self, grad_ys):
    """The values' gradient scattered back through one-hot indices; the indices
    carry none (mesh_tensorflow/ops.py:4916-4920)."""
    dy = grad_ys[0]
    if dy is None:
      return [None]
    x = self.inputs[0]
    hot = one_hot(self.outputs[1], self._reduced_dim, dtype=x.dtype)
    return [einsum([dy, hot], output_shape=x.shape)]

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    ops = impl.slice_ops
    x = self.inputs[0]
    ndims = x.shape.ndims
    reduced_axis = x.shape.dims.index(self._reduced_dim)
    reduced_mesh_axis = impl.tensor_dimension_to_mesh_axis(self._reduced_dim)
    if reduced_mesh_axis is not None:
      per_shard = self._reduced_dim.size // impl.shape[reduced_mesh_axis].size
    else:
      per_shard = self._reduced_dim.size
    k = self._k_dim.size

    def slicewise_top_k(t):
      t = ops.transpose(t, [i for i in range(ndims) if i != reduced_axis] + [reduced_axis])
      if k == 1:
        return (ops.expand_dims(ops.reduce("MAX", t, [ndims - 1]), ndims - 1),
                ops.expand_dims(ops.argmax(t), ndims - 1))
      return ops.top_k(t, min(k, per_shard))
    values, indices = impl.slicewise(slicewise_top_k, lowering.tensors[x])
    if reduced_mesh_axis is not None:
      indices = impl.slicewise(
          lambda idx, pcoord: ops.binary("add", idx, int(pcoord) * per_shard),
          indices, impl.laid_out_pcoord(reduced_mesh_axis))
      values = impl.allconcat(values, reduced_mesh_axis, ndims - 1)
      indices = impl.allconcat(indices, reduced_mesh_axis, ndims - 1)

      def global_top_k(vals, global_indices):
        vals, local = ops.top_k(vals, k)
        return vals, ops.gather_last(global_indices, local)
      values, indices = impl.slicewise(global_top_k, values, indices)
    lowering.set_tensor_lowering(self.outputs[0], values)
    lowering.set_tensor_lowering(self.outputs[1], indices)


def top_k(x, reduced_dim, k_dim, name=None):
  """Values and int32 indices, k_dim appended last; k in 2..4 runs as repeated
  top_1 with the winner pushed down by -1e9 (mesh_tensorflow/ops.py:4964-5015)."""
  reduced_dim = convert_to_dimension(reduced_dim)
  k_dim = convert_to_dimension(k_dim)
  if 1 < k_dim.size < 5:
    values, indices = [], []
    for i in range(k_dim.size):
      v, idx = top_1(x, reduced_dim)
      values.append(v)
      indices.append(idx)
      if i + 1 < k_dim.size:
        x = x + one_hot(idx, reduced_dim, on_value=-1e9, dtype=x.dtype)
    return stack(values, k_dim.name, -1), stack(indices, k_dim.name, -1)
  op = TopKOperation(x, reduced_dim, k_dim, name=name)
  return op.outputs[0], op.outputs[1]


def top_1(x, reduced_dim, name=None):
  """Max and argmax along `reduced_dim` (mesh_tensorflow/ops.py:5018-5033)."""
  reduced_dim = convert_to_dimension(reduced_dim)
  one = Dimension("_one", 1)
  op = TopKOperation(x, reduced_dim, one, name=name)
  values, indices = op.outputs
  return reshape(values, values.shape - one), reshape(indices, indices.shape - one)


def argmax(x, reduced_dim, name=None):
  return top_1(x, convert_to_dimension(reduced_dim), name=name)[1]


def sample_with_temperature(logits, dim, temperature=1.0, name=None):
  """An index along `dim` per position, drawn with probability proportional to
  exp(logits / temperature) by the Gumbel trick (ops.py:5050-5086): temperature 0 is
  the argmax, 1 samples from softmax(logits).  The uniform draws stay inside (0, 1) so
  that -log(-log(u)) is finite; the arithmetic is float32."""
  dim = convert_to_dimension(dim)
  if temperature != 0.0:
    logits = cast(logits, G.float32)
    u = random_uniform(logits.mesh, logits.shape, minval=1e-9, maxval=1.0, dtype=G.float32)
    logits = logits + (-log(-log(u))) * temperature
  return argmax(logits, dim, name=name)


class StackOperation(Operation):
  """Stacks same-shaped tensors along a new unsplit dim (ops.py:2592-2630)."""

  def __init__(self, xs, dim_name, axis, name=None):
    super().__init__(xs, name=name or "stack")
    self._axis = axis
    dims = xs[0].shape.dims
    self._outputs = [Tensor(self, Shape(dims[:axis] + [Dimension(dim_name, len(xs))] + dims[axis:]),
                            xs[0].dtype)]

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    if impl.tensor_dimension_to_mesh_axis(self.outputs[0].shape.dims[self._axis]) is not None:
      raise ValueError("can't stack along a split axis")
    ops, axis = impl.slice_ops, self._axis
    fn = lambda *xs: ops.concat([ops.expand_dims(x, axis) for x in xs], axis)
    lowering.set_tensor_lowering(
        self.outputs[0], impl.slicewise(fn, *[lowering.tensors[x] for x in self.inputs]))

  def gradient(self, grad_ys):
    """Each input receives its own layer of dy (mesh_tensorflow/ops.py:2616-2618)."""
    return [UnstackOperation(grad_ys[0], self._axis, i).outputs[0]
            for i in range(len(self.inputs))]


class UnstackOperation(Operation):
  """Layer `index` of an unsplit dim, the dim dropped (one output of
  mesh_tensorflow/ops.py:2633-2670)."""

  def __init__(self, x, axis, index, name=None):
    super().__init__([x], name=name or "unstack")
    self._axis, self._index = axis, index
    dims = x.shape.dims
    self._outputs = [Tensor(self, Shape(dims[:axis] + dims[axis + 1:]), x.dtype)]

  def gradient(self, grad_ys):
    dim = self.inputs[0].shape.dims[self._axis]
    layers = [grad_ys[0] if i == self._index else zeros_like(grad_ys[0]) for i in range(dim.size)]
    return [stack(layers, dim.name, self._axis)]

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    if impl.tensor_dimension_to_mesh_axis(self.inputs[0].shape.dims[self._axis]) is not None:
      raise ValueError("can't unstack along a split axis")
    ops, axis, index = impl.slice_ops, self._axis, self._index

    def fn(xs):
      shape = list(ops.shape(xs))
      begin = [0] * len(shape)
      begin[axis] = index
      size = list(shape)
      size[axis] = 1
      return ops.reshape(ops.slice(xs, begin, size), shape[:axis] + shape[axis + 1:])
    lowering.set_tensor_lowering(self.outputs[0], impl.slicewise(fn, lowering.tensors[self.inputs[0]]))


def stack(xs, dim_name, axis=0, name=None):
  if axis < 0:
    axis = xs[0].shape.ndims + 1 + axis
  return StackOperation(xs, dim_name, axis, name).outputs[0]


class OneHotOperation(Operation):
  """One-hot along a new last dim (mesh_tensorflow/ops.py:3810-3851).

  An index outside [0, depth) gives an all-`off` row; when the new dim is
  split, each processor subtracts the offset of its slice first.
  """

  def __init__(self, indices, output_dim, on_value, off_value, dtype, name=None):
    super().__init__([indices], name=name or "one_hot")
    if not indices.dtype.is_integer:
      raise ValueError("indices requires an integer dtype got %s" % (indices,))
    self._output_dim = output_dim
    self._on, self._off, self._dtype = on_value, off_value, dtype
    self._outputs = [Tensor(self, Shape(indices.shape.dims + [output_dim]), dtype)]

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    ops = impl.slice_ops
    depth = impl.slice_shape(self.outputs[0].shape)[-1]
    mesh_axis = impl.tensor_dimension_to_mesh_axis(self._output_dim)
    if mesh_axis is None:
      offset = 0
    else:
      offset = impl.slicewise(lambda pc: int(pc) * depth, impl.laid_out_pcoord(mesh_axis))
    on, off, dtype = self._on, self._off, self._dtype

    def fn(idx, off_set):
      if off_set:
        idx = ops.binary("add", idx, -int(off_set))
      return ops.one_hot(idx, depth, on, off, dtype)
    lowering.set_tensor_lowering(
        self.outputs[0], impl.slicewise(fn, lowering.tensors[self.inputs[0]], offset))


def one_hot(indices, output_dim, on_value=1.0, off_value=0.0, dtype=G.float32, name=None):
  return OneHotOperation(indices, convert_to_dimension(output_dim), on_value, off_value, dtype,
                         name=name).outputs[0]


class GatherOperation(Operation):
  """weights[indices] along `dim`, the leading dim of `weights`, as a row gather.

  The reference forms this product as einsum(one_hot(indices, dim), weights)
  (ops.py:5231-5251); the values are the same, row copies being exact.  When
  `dim` is split over a mesh axis each processor gathers the rows it holds and
  leaves zeros for the others, and the slices are summed lazily over that axis,
  exactly what the one-hot einsum's contraction of a split dim does.
  """

  def __init__(self, weights, indices, dim, name=None):
    super().__init__([weights, indices], name=name or "gather")
    self._dim = dim
    self._outputs = [Tensor(self, Shape(indices.shape.dims + weights.shape.dims[1:]), weights.dtype)]

  def gradient(self, grad_ys):
    """The one-hot einsum's own gradient: d(weights) = one_hot(indices)^T . dy."""
    weights, indices = self.inputs
    hot = one_hot(indices, self._dim, dtype=weights.dtype)
    return [einsum([hot, grad_ys[0]], output_shape=weights.shape), None]

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    ops = impl.slice_ops
    weights, indices = self.inputs
    mesh_axis = impl.tensor_dimension_to_mesh_axis(self._dim)
    rows_here = impl.slice_shape(weights.shape)[0]
    row_bytes = list_product(impl.slice_shape(weights.shape)[1:]) * weights.dtype.itemsize

    def fn(w, idx, pcoord):
      first = int(pcoord) * rows_here
      if row_bytes % 16 == 0 and row_bytes > 0:
        return ops.gather_rows(w, idx, first)
      # rows too short for the vector kernel: the reference's own form, on slices
      local = idx if first == 0 else ops.binary("sub", idx, first)
      hot = ops.one_hot(local, rows_here, 1.0, 0.0, w.dtype)     # out of range: all off
      nd = len(ops.shape(idx))
      lead = "abcdefgh"[:nd]
      rest = "ijklmnop"[:len(ops.shape(w)) - 1]
      return ops.einsum("%sz,z%s->%s%s" % (lead, rest, lead, rest), hot, w)
    pcoord = impl.laid_out_pcoord(mesh_axis) if mesh_axis is not None else 0
    y = impl.slicewise(fn, lowering.tensors[weights], lowering.tensors[indices], pcoord)
    if mesh_axis is not None:
      y = LazyAllreduceSum(impl, y, [mesh_axis])
    lowering.set_tensor_lowering(self.outputs[0], y)


def gather(weights, indices, dim, output_shape=None):
  """weights indexed along `dim` by integer `indices` (ops.py:5231-5251).

  The common case - `dim` leading in `weights`, no dim shared between `indices`
  and the rest of `weights`, default output order - is a row gather
  (GatherOperation); anything else is the reference's one-hot einsum."""
  dim = convert_to_dimension(dim)
  output_shape = convert_to_shape(output_shape)
  if not isinstance(indices, Tensor):
    indices = constant(weights.mesh, indices, dtype=G.int32)
  if weights.dtype.is_bool:
    return cast(gather(to_float(weights), indices, dim, output_shape), G.bool_)
  rest = weights.shape.dims[1:]
  natural = Shape(indices.shape.dims + rest)
  if (weights.shape.ndims >= 2 and weights.shape.dims[0] == dim and indices.shape.ndims >= 1
      and not set(indices.shape.dims) & set(weights.shape.dims)
      and (output_shape is None or output_shape == natural)):
    return GatherOperation(weights, indices, dim).outputs[0]
  return einsum([one_hot(indices, dim, dtype=weights.dtype), weights],
                reduced_dims=[dim], output_shape=output_shape)


def nth_largest_element(x, n, reduced_dim, name=None):
  """n-th largest (zero-indexed) along `reduced_dim` (ops.py:6589-6605)."""
  reduced_dim = convert_to_dimension(reduced_dim)
  k_dim = Dimension("_top_k_", n + 1)
  values, _ = top_k(x, reduced_dim=reduced_dim, k_dim=k_dim, name=name)
  return gather(values, n, k_dim)


def nth_smallest_element(x, n, reduced_dim, name=None):
  return -nth_largest_element(-x, n, reduced_dim, name=name)


# ------------------------------------------------------------ cumsum / softmax
def cumsum(x, dim, exclusive=False):
  """Cumulative sum as a product with a 0/1 triangular matrix (ops.py:2761-2781)."""
  dim = convert_to_dimension(dim)
  tmp = Dimension("tmp_dim_cumsum", dim.size)
  new_shape = x.shape.rename_dimension(dim.name, tmp.name)
  comparator = less if exclusive else less_equal
  m = cast(comparator(mtf_range(x.mesh, dim, dtype=G.float32),
                      mtf_range(x.mesh, tmp, dtype=G.float32)), x.dtype)
  return reshape(einsum([x, m], output_shape=new_shape), x.shape)


def reduce_logsumexp(x, reduced_dim, extra_logit=None, name=None):
  """log(sum(exp(x))) with the max subtracted first (ops.py:5493-5520)."""
  reduced_dim = convert_to_dimension(reduced_dim)
  reduced_shape = x.shape - reduced_dim
  max_logit = reduce_max(stop_gradient(x), output_shape=reduced_shape)
  if extra_logit is not None:
    max_logit = maximum(max_logit, extra_logit)
  x = x - max_logit
  sum_exp = reduce_sum(exp(x), output_shape=reduced_shape)
  if extra_logit is not None:
    sum_exp = sum_exp + exp(extra_logit - max_logit)
  return log(sum_exp) + max_logit


def log_softmax(x, reduced_dim, extra_logit=None, name=None):
  return x - reduce_logsumexp(x, reduced_dim, extra_logit=extra_logit, name=name)


def softmax(x, reduced_dim, extra_logit=None, name=None):
  """exp(x - logsumexp(x)) (mesh_tensorflow/ops.py:5539-5541)."""
  return exp(log_softmax(x, reduced_dim, extra_logit=extra_logit))


# ----------------------------------------------------------------------- shift
class ShiftOperation(Operation):
  """Shifts along a dim, zero-filled or wrapped (mesh_tensorflow/ops.py:3569-3661).

  When the dim is split, whole slices move between neighbouring processors
  through MeshImpl.shift_by_n_processors.
  """

  def __init__(self, x, offset, dim, wrap, name=None):
    super().__init__([x], name=name or "shift")
    self._dim = dim
    self._axis = x.shape.dims.index(dim)
    self._offset = offset
    self._wrap = wrap
    self._outputs = [Tensor(self, x.shape, x.dtype)]

  def gradient(self, grad_ys):
    """The opposite shift (mesh_tensorflow/ops.py:3594-3596)."""
    return [shift(grad_ys[0], -self._offset, self._dim, self._wrap)]

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    ops = impl.slice_ops
    mesh_axis = impl.tensor_dimension_to_mesh_axis(self._dim)
    inputs = lowering.tensors[self.inputs[0]]
    ndims = self.inputs[0].shape.ndims
    axis, wrap = self._axis, self._wrap
    if mesh_axis is None:
      off = self._offset
      n = self._dim.size

      def local_shift(xs):
        return _shift_slice(ops, xs, axis, off, n, wrap, ndims)
      lowering.set_tensor_lowering(self.outputs[0], impl.slicewise(local_shift, inputs))
      return
    mesh_size = impl.shape[mesh_axis].size
    partial = self._dim.size // mesh_size
    inputs = inputs.to_laid_out_tensor()
    src_a = self._offset // partial          # whole slices to move
    rem = self._offset - src_a * partial     # 0 <= rem < partial
    from_a = impl.shift_by_n_processors(inputs, mesh_axis, src_a, wrap)
    if rem == 0:
      lowering.set_tensor_lowering(self.outputs[0], from_a)
      return
    from_b = impl.shift_by_n_processors(inputs, mesh_axis, src_a + 1, wrap)

    def stitch(a, b):
      shape = list(ops.shape(a))
      head_size = list(shape)
      head_size[axis] = rem
      tail_size = list(shape)
      tail_size[axis] = partial - rem
      begin_b = [0] * ndims
      begin_b[axis] = partial - rem
      return ops.concat([ops.slice(b, begin_b, head_size),
                         ops.slice(a, [0] * ndims, tail_size)], axis)
    lowering.set_tensor_lowering(self.outputs[0], impl.slicewise(stitch, from_a, from_b))


def _shift_slice(ops, xs, axis, offset, n, wrap, ndims):
  shape = list(ops.shape(xs))
  offset = offset % n if wrap else offset
  if offset == 0:
    return xs
  if abs(offset) >= n:
    return ops.fill(shape, 0, ops.dtype(xs))
  keep = list(shape)
  keep[axis] = n - abs(offset)
  lost = list(shape)
  lost[axis] = abs(offset)
  begin_keep = [0] * ndims
  begin_lost = [0] * ndims
  if offset > 0:
    begin_lost[axis] = n - offset
    kept = ops.slice(xs, begin_keep, keep)
    pad = ops.slice(xs, begin_lost, lost) if wrap else ops.fill(lost, 0, ops.dtype(xs))
    return ops.concat([pad, kept], axis)
  begin_keep[axis] = -offset
  kept = ops.slice(xs, begin_keep, keep)
  pad = ops.slice(xs, begin_lost, lost) if wrap else ops.fill(lost, 0, ops.dtype(xs))
  return ops.concat([kept, pad], axis)


def shift(x, offset, dim, wrap, name=None):
  return ShiftOperation(x, offset, convert_to_dimension(dim), wrap, name=name).outputs[0]


# --------------------------------------------------------- operator overloads
def _floordiv(x1, x2):
  return binary_op_with_broadcasting("floordiv", x1, x2)


def _mod(x1, x2):
  return binary_op_with_broadcasting("mod", x1, x2)


Tensor.__add__ = lambda self, other: add(self, other)
Tensor.__radd__ = lambda self, other: add(self, other)
Tensor.__sub__ = lambda self, other: sub(self, other)
Tensor.__rsub__ = lambda self, other: sub(other, self)
Tensor.__mul__ = lambda self, other: multiply(self, other)
Tensor.__rmul__ = lambda self, other: multiply(self, other)
Tensor.__neg__ = lambda self: negative(self)
Tensor.__truediv__ = lambda self, other: divide(self, other)
Tensor.__rtruediv__ = lambda self, other: divide(other, self)
Tensor.__floordiv__ = lambda self, other: _floordiv(self, other)
Tensor.__mod__ = lambda self, other: _mod(self, other)


# ------------------------------------------------------------------ gradients
def gradients(ys, xs, grad_ys=None, operations=None):
  """Symbolic d(sum ys)/d(xs): walks the operations backwards, asks each for
  its input gradients and sums what arrives at a tensor
  (mesh_tensorflow/ops.py:6493-6586).  Returns one tensor (or None) per x."""
  if not ys:
    return [None] * len(xs)
  graph = ys[0].graph
  operations = list(graph.operations if operations is None else operations)
  if not grad_ys:
    grad_ys = [constant(y.mesh, 1.0, y.shape, y.dtype) for y in ys]
  # tensors that depend on some x through differentiable operations
  downstream = set(xs)
  for op in operations:
    if op.has_gradient and set(op.inputs) & downstream:
      downstream |= set(op.outputs)
  tensor_to_gradient = dict(zip(ys, grad_ys))
  for op in reversed(operations):
    grad_outputs = [tensor_to_gradient.get(out) for out in op.outputs]
    if (not op.has_gradient or all(g is None for g in grad_outputs)
        or not set(op.inputs) & downstream):
      continue
    for inp, grad in zip(op.inputs, op.gradient(grad_outputs)):
      if inp in downstream and grad is not None:
        if inp in tensor_to_gradient:
          tensor_to_gradient[inp] = add(tensor_to_gradient[inp], grad)
        else:
          tensor_to_gradient[inp] = grad
  return [tensor_to_gradient.get(x) for x in xs]


def gradients_by_recompute(inputs, build_fn, grad_ys):
  """Gradients of a fused operation through an equivalent chain of ordinary
  operations: `build_fn(*inputs)` adds that chain to the graph and returns its
  outputs, which are differentiated against `grad_ys` (None entries are left
  out).  The chain is only ever lowered if the gradient is; it recomputes the
  forward values it needs (the approach of mesh_tensorflow/ops.py:6607-6720,
  recompute_grad).  Returns one gradient (or None) per input."""
  graph = inputs[0].graph
  start = len(graph.operations)
  ys = list(build_fn(*inputs))
  pairs = [(y, g) for y, g in zip(ys, grad_ys) if g is not None]
  if not pairs:
    return [None] * len(inputs)
  chain = graph.operations[start:]
  return gradients([y for y, _ in pairs], list(inputs), grad_ys=[g for _, g in pairs],
                   operations=chain)


class RecomputeGradOperation(Operation):
  """y = fn(*inputs) whose gradient re-runs fn instead of keeping what the
  forward pass computed inside it (mesh_tensorflow/ops.py:6607-6720)."""

  def __init__(self, fn, explicit_inputs, name=None):
    forward = fn(*explicit_inputs)
    self._single = isinstance(forward, Tensor)
    self._forward = [forward] if self._single else list(forward)
    super().__init__(list(explicit_inputs), name=name or "recompute_grad")
    self._fn = fn
    self._outputs = [Tensor(self, y.shape, y.dtype, index=i) for i, y in enumerate(self._forward)]

  def lower(self, lowering):
    for out, y in zip(self.outputs, self._forward):
      lowering.set_tensor_lowering(out, lowering.tensors[y])

  def gradient(self, grad_ys):
    def chain(*xs):
      ys = self._fn(*xs)
      return [ys] if isinstance(ys, Tensor) else list(ys)
    return gradients_by_recompute(self.inputs, chain, grad_ys)


def recompute_grad(fn, explicit_inputs):
  op = RecomputeGradOperation(fn, explicit_inputs)
  return op.outputs[0] if op._single else op.outputs


def anonymous_shape(shape):
  shape = convert_to_shape(shape)
  return Shape([Dimension("_anonymous_%i" % i, d.size) for i, d in enumerate(shape.dims)])


def anonymize(x):
  return reshape(x, anonymous_shape(x.shape))


def import_fully_replicated(mesh, tf_tensor, shape, name=None, dtype=None):
  """Imports under anonymous dim names (so that no layout rule applies and the
  whole array is uploaded everywhere), then reshapes to `shape`, which slices
  locally (mesh_tensorflow/ops.py:3935-3938)."""
  shape = convert_to_shape(shape)
  return reshape(import_tf_tensor(mesh, tf_tensor, anonymous_shape(shape), name, dtype=dtype), shape)


class RandomOperation(Operation):
  """A tensor of random values (mesh_tensorflow/ops.py:5782-5799); `tf_fn` is
  "uniform" or "normal" (what tf.random.uniform / tf.random.normal are to the
  reference).  The operation's seed defaults to a hash of its name, so the same
  graph draws the same numbers in every lowering on every backend."""

  def __init__(self, mesh, shape, tf_fn, **kwargs):
    super().__init__([], mesh=mesh, name=kwargs.pop("name", None) or "random")
    self._tf_fn = tf_fn
    if kwargs.get("seed") is None:
      import zlib
      kwargs["seed"] = zlib.crc32(self.name.encode())
    self._kwargs = kwargs
    self._outputs = [Tensor(self, shape, kwargs.get("dtype", G.float32))]

  @property
  def has_gradient(self):
    return False

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    lowering.set_tensor_lowering(
        self.outputs[0], impl.random(self.outputs[0].shape, self._tf_fn, self._kwargs))


def random_uniform(mesh, shape, **kwargs):
  """Uniform in [minval, maxval) (ops.py:5802-5814)."""
  return RandomOperation(mesh, convert_to_shape(shape), "uniform", **kwargs).outputs[0]


def random_normal(mesh, shape, **kwargs):
  """Normal with `mean` and `stddev` (ops.py:5817-5829)."""
  return RandomOperation(mesh, convert_to_shape(shape), "normal", **kwargs).outputs[0]


def dropout(x, is_training, keep_prob=None, rate=None, noise_shape=None, name=None):
  """Zeroes elements with probability 1 - keep_prob and scales the rest by
  1 / keep_prob for floating types (ops.py:5832-5871)."""
  if (keep_prob is None) == (rate is None):
    raise ValueError("exactly one of keep_prob and rate should be set")
  if keep_prob is None:
    keep_prob = 1.0 - rate
  noise_shape = convert_to_shape(noise_shape)
  if noise_shape is None:
    noise_shape = x.shape
  if keep_prob == 1.0 or not is_training:
    return x
  noise = cast(less(random_uniform(x.mesh, noise_shape, name=name,
                                   dtype=(x.dtype if x.dtype.is_floating else G.float32)),
                    keep_prob), x.dtype)
  if x.dtype.is_floating:
    noise = noise / keep_prob
  return x * noise


def serialize_training_step(features, model_fn, batch_dim, num_splits, variables):
  """Splits the training batch into `num_splits` microbatches run one after the
  other, with gradients and outputs accumulated (mesh_tensorflow/ops.py:6493-6586).

  features: dict of Tensors, each with `batch_dim`; model_fn: feature dict ->
  output dict containing "loss"; variables: the tensors to differentiate with
  respect to (the reference takes graph.trainable_variables).  Returns
  (grads, outputs): gradients summed over the microbatches, and outputs summed
  (no batch dim) or re-assembled to the full batch (batch dim).

  The reference runs the microbatches in an mtf.while_loop whose accumulators
  may stay un-reduced; here the loop is unrolled in the graph, which has the
  same effect: a gradient whose einsum contracts a mesh-split dim is a lazy
  allreduce, sums of such lazies stay lazy (ops.py:1343-1382, 2079-2081), and
  the one allreduce per variable runs after the last microbatch.  Microbatch m
  holds the examples m, m + num_splits, ... as the reference's reshape to
  [batch / num_splits, microbatch] implies.
  """
  if batch_dim.size % num_splits != 0:
    raise ValueError("num_splits=%d must divide %s" % (num_splits, batch_dim))
  microbatch_dim = Dimension("microbatch", num_splits)
  smaller_batch_dim = Dimension(batch_dim.name, batch_dim.size // num_splits)

  def select(t, microbatch_num):
    return gather(replace_dimensions(t, batch_dim, [smaller_batch_dim, microbatch_dim]),
                  microbatch_num, microbatch_dim)
  combined_grads, combined_outputs = None, {}
  for m in range(num_splits):
    outputs = model_fn({k: select(v, m) for k, v in features.items()})
    grads = gradients([outputs["loss"]], list(variables))
    if None in grads:
      raise ValueError("Found variable(s) with None gradient; check for variables "
                       "disconnected from the loss")
    for k, t in outputs.items():
      if smaller_batch_dim in t.shape.dims:
        # pad the microbatch's rows into the full batch; summing completes the concatenation
        t = einsum([t, one_hot(constant(t.mesh, m, dtype=G.int32), microbatch_dim, dtype=t.dtype)],
                   output_shape=replace_dimensions(t.shape, smaller_batch_dim,
                                                   [smaller_batch_dim, microbatch_dim]))
        t = replace_dimensions(t, [smaller_batch_dim, microbatch_dim], batch_dim)
      combined_outputs[k] = t if k not in combined_outputs or m == 0 else add(combined_outputs[k], t)
    combined_grads = grads if combined_grads is None else [add(a, b) for a, b in zip(combined_grads, grads)]
  return combined_grads, combined_outputs


# ------------------------------------------------- concat / split / slice / pad
def _resized(shape, dim_name, size):
  return Shape([Dimension(d.name, size) if d.name == dim_name else d for d in shape.dims])


def _dim_axis(x, dim_name, what):
  names = [d.name for d in x.shape.dims]
  if dim_name not in names:
    raise ValueError("%s: %s has no dimension named %s" % (what, x.shape, dim_name))
  return names.index(dim_name)


def _not_split(lowering, op, dim_name, what):
  if lowering.mesh_impl(op).tensor_dimension_to_mesh_axis(Dimension(dim_name, 0)) is not None:
    raise ValueError("can't %s along split axis" % what)


class ConcatOperation(Operation):
  """tf.concat along a named dim (mesh_tensorflow/ops.py:2537-2583)."""

  def __init__(self, xs, concat_dim_name, name=None):
    super().__init__(xs, name=name or "concat")
    self._concat_dim_name = concat_dim_name
    self._axis = _dim_axis(xs[0], concat_dim_name, "concat")
    if not all(_resized(x.shape, concat_dim_name, 0) == _resized(xs[0].shape, concat_dim_name, 0)
               for x in xs):
      raise ValueError("shapes are not compatible %s" % (xs,))
    self._input_sizes = [x.shape.dims[self._axis].size for x in xs]
    self._outputs = [Tensor(self, _resized(xs[0].shape, concat_dim_name, sum(self._input_sizes)),
                            xs[0].dtype)]

  def gradient(self, grad_ys):
    return split(grad_ys[0], self.outputs[0].shape.dims[self._axis], self._input_sizes)

  def lower(self, lowering):
    _not_split(lowering, self, self._concat_dim_name, "concat")
    impl = lowering.mesh_impl(self)
    ops, axis = impl.slice_ops, self._axis
    lowering.set_tensor_lowering(
        self.outputs[0],
        impl.slicewise(lambda *args: ops.concat(list(args), axis),
                       *[lowering.tensors[x] for x in self.inputs]))


def concat(xs, concat_dim_name, name=None):
  """Concatenates along the dim named `concat_dim_name`, which must not be split."""
  return ConcatOperation(xs, concat_dim_name, name).outputs[0]


class SplitOperation(Operation):
  """tf.split along a dim into given sizes (mesh_tensorflow/ops.py:2586-2648)."""

  def __init__(self, x, split_dim, num_or_size_splits, name=None):
    super().__init__([x], name=name or "split")
    self._split_dim = split_dim
    self._axis = x.shape.dims.index(split_dim)
    if isinstance(num_or_size_splits, list):
      self._output_sizes = list(num_or_size_splits)
      if sum(self._output_sizes) != split_dim.size:
        raise ValueError("Sizes do not add up %s %s" % (num_or_size_splits, split_dim))
    else:
      if split_dim.size % num_or_size_splits != 0:
        raise ValueError("num_splits does not divide %s" % (split_dim,))
      self._output_sizes = [split_dim.size // num_or_size_splits] * num_or_size_splits
    self._outputs = [Tensor(self, _resized(x.shape, split_dim.name, size), x.dtype, index=i)
                     for i, size in enumerate(self._output_sizes)]

  def gradient(self, grad_ys):
    grad_ys = [g if g is not None else zeros_like(o) for g, o in zip(grad_ys, self.outputs)]
    return [concat(grad_ys, self._split_dim.name)]

  def lower(self, lowering):
    _not_split(lowering, self, self._split_dim.name, "split")
    impl = lowering.mesh_impl(self)
    ops, axis = impl.slice_ops, self._axis
    sizes = self._output_sizes

    def fn(xs):
      shape = list(ops.shape(xs))
      out, at = [], 0
      for size in sizes:
        begin = [0] * len(shape)
        begin[axis] = at
        extent = list(shape)
        extent[axis] = size
        out.append(ops.contiguous(ops.slice(xs, begin, extent)))
        at += size
      return tuple(out)
    values = impl.slicewise(fn, lowering.tensors[self.inputs[0]])
    for out, value in zip(self.outputs, values):
      lowering.set_tensor_lowering(out, value)


def split(x, split_dim, num_or_size_splits, name=None):
  return SplitOperation(x, split_dim, num_or_size_splits, name=name).outputs


class SliceOperation(Operation):
  """tf.slice along one dim (mesh_tensorflow/ops.py:2758... mtf_slice 2723-2758)."""

  def __init__(self, x, begin, size, slice_dim_name, name=None):
    super().__init__([x], name=name or "slice")
    self._axis = _dim_axis(x, slice_dim_name, "slice")
    dim = x.shape.dims[self._axis]
    if begin < 0 or size < 0 or begin + size > dim.size:
      raise ValueError("slice [%d, %d) is outside %s" % (begin, begin + size, dim))
    self._begin, self._size, self._slice_dim_name = begin, size, slice_dim_name
    self._outputs = [Tensor(self, _resized(x.shape, slice_dim_name, size), x.dtype)]

  def gradient(self, grad_ys):
    total = self.inputs[0].shape.dims[self._axis].size
    return [pad(grad_ys[0], [self._begin, total - self._size - self._begin], self._slice_dim_name)]

  def lower(self, lowering):
    _not_split(lowering, self, self._slice_dim_name, "slice")
    impl = lowering.mesh_impl(self)
    ops, axis, b, n = impl.slice_ops, self._axis, self._begin, self._size

    def fn(xs):
      shape = list(ops.shape(xs))
      begin = [0] * len(shape)
      begin[axis] = b
      shape[axis] = n
      return ops.contiguous(ops.slice(xs, begin, shape))
    lowering.set_tensor_lowering(self.outputs[0], impl.slicewise(fn, lowering.tensors[self.inputs[0]]))


def mtf_slice(x, begin, size, slice_dim_name, name=None):
  """x[..., begin:begin+size, ...] along the named dim (must not be split)."""
  return SliceOperation(x, begin, size, slice_dim_name, name=name).outputs[0]


class PadOperation(Operation):
  """tf.pad with zeros along one dim (mesh_tensorflow/ops.py:2651-2720)."""

  def __init__(self, x, paddings, pad_dim_name, name=None):
    super().__init__([x], name=name or "pad")
    if len(paddings) != 2 or min(paddings) < 0:
      raise ValueError("paddings must be [before, after], got %s" % (paddings,))
    self._axis = _dim_axis(x, pad_dim_name, "pad")
    self._paddings, self._pad_dim_name = list(paddings), pad_dim_name
    size = x.shape.dims[self._axis].size + sum(paddings)
    self._outputs = [Tensor(self, _resized(x.shape, pad_dim_name, size), x.dtype)]

  def gradient(self, grad_ys):
    size = self.inputs[0].shape.dims[self._axis].size
    return [mtf_slice(grad_ys[0], self._paddings[0], size, self._pad_dim_name)]

  def lower(self, lowering):
    _not_split(lowering, self, self._pad_dim_name, "pad")
    impl = lowering.mesh_impl(self)
    ops, axis, (before, after) = impl.slice_ops, self._axis, self._paddings

    def fn(xs):
      shape = list(ops.shape(xs))
      parts = []
      for n in (before, None, after):
        if n is None:
          parts.append(xs)
        elif n > 0:
          z = list(shape)
          z[axis] = n
          parts.append(ops.fill(z, 0, ops.dtype(xs)))
      return ops.concat(parts, axis) if len(parts) > 1 else xs
    lowering.set_tensor_lowering(self.outputs[0], impl.slicewise(fn, lowering.tensors[self.inputs[0]]))


def pad(x, paddings, dim_name, name=None):
  """Zero padding [before, after] along the named dim (must not be split)."""
  return PadOperation(x, paddings, dim_name, name=name).outputs[0]


def halo_exchange(x, blocks_dim, block_size_dim, halo_size, wrap=False):
  """Each block concatenated with the margins of its neighbours along `blocks_dim`
  (mesh_tensorflow/ops.py:6381-6418): `block_size_dim` grows by 2 * halo_size.  With
  `blocks_dim` split over a mesh axis the shifts are collective permutes between
  neighbouring processors (MeshImpl.receive)."""
  if halo_size == 0:
    return x
  block_size = block_size_dim.size
  partial_size = halo_size % block_size
  num_complete_blocks = halo_size // block_size
  parts = [x]
  for i in range(1, num_complete_blocks + 1):
    parts = [shift(x, i, blocks_dim, wrap)] + parts + [shift(x, -i, blocks_dim, wrap)]
  if partial_size > 0:
    left_margin = mtf_slice(x, 0, partial_size, block_size_dim.name)
    right_margin = mtf_slice(x, block_size - partial_size, partial_size, block_size_dim.name)
    parts = ([shift(right_margin, num_complete_blocks + 1, blocks_dim, wrap)] + parts
             + [shift(left_margin, -(num_complete_blocks + 1), blocks_dim, wrap)])
  return concat(parts, block_size_dim.name)


def left_halo_exchange(x, blocks_dim, block_size_dim, halo_size, wrap=False):
  """As halo_exchange, margins from the left neighbours only (ops.py:6421-6452)."""
  if halo_size == 0:
    return x
  block_size = block_size_dim.size
  partial_size = halo_size % block_size
  num_complete_blocks = halo_size // block_size
  parts = [x]
  for i in range(1, num_complete_blocks + 1):
    parts = [shift(x, i, blocks_dim, wrap)] + parts
  if partial_size > 0:
    right_margin = mtf_slice(x, block_size - partial_size, partial_size, block_size_dim.name)
    parts = [shift(right_margin, num_complete_blocks + 1, blocks_dim, wrap)] + parts
  return concat(parts, block_size_dim.name)

