"""Layer builders on the mesh-tensor language: dense, FFN, attention.

Graph construction only — every product goes through mtf.einsum and hence
through the MeshImpl under the lowering.  Follows mesh_tensorflow/layers.py
(dense 129-208, dense_product 256-295, dense_relu_dense 1148-1181,
dot_product_attention 1614-1652, multihead_attention 1655-1723, masks
1839-1850).  Weights are ordinary tensors (imported arrays): the reference's
variable machinery is outside this package's scope, so where the reference
creates a variable these builders take the tensor from the caller or draw it
from a seeded generator with the reference's initializer scale.
"""

from __future__ import annotations

import functools

import numpy as np

from mesh_b200.mtf import graph as G
from mesh_b200.mtf import ops as mtf
from mesh_b200.mtf.shapes import Dimension, Shape


class WeightSource(object):
  """Seeded normal initialisers standing in for variable creation."""

  def __init__(self, seed=0):
    self._rng = np.random.Generator(np.random.PCG64(seed))

  def normal(self, mesh, shape, stddev, dtype, name=None):
    shape = Shape(shape)
    value = (self._rng.standard_normal(shape.to_integer_list, dtype=np.float32)
             * np.float32(stddev))
    return mtf.import_tf_tensor(mesh, value, shape, dtype=dtype, name=name)


def get_dense_kernel_weights(x, new_dims, reduced_dims, expert_dims, weights,
                             name=None, variable_dtype=None):
  """Kernel of shape expert_dims + reduced_dims + new_dims, cast to x.dtype.

  Variance-scaling init: stddev = fan_in ** -0.5 over the reduced dims
  (mesh_tensorflow/layers.py:211-253, 298-340).
  """
  w_shape = Shape(list(expert_dims) + list(reduced_dims) + list(new_dims))
  fan_in = Shape(reduced_dims).size
  w = weights.normal(x.mesh, w_shape, fan_in ** -0.5, variable_dtype or x.dtype,
                     name=(name or "dense") + "/kernel")
  return mtf.cast(w, x.dtype)


def dense(x, new_dims, reduced_dims=None, expert_dims=None, use_bias=True, activation=None,
          kernel_weights=None, bias=None, weights=None, variable_dtype=None, name=None):
  """y = activation(einsum(x, w) [+ b]) (mesh_tensorflow/layers.py:129-208)."""
  if not isinstance(new_dims, list):
    new_dims = [new_dims]
  expert_dims = list(expert_dims or [])
  if reduced_dims is None:
    reduced_dims = x.shape.dims[-1:]
  reduced_dims = list(reduced_dims)
  # A reduced dim that reappears among the new dims is renamed in the input so
  # the kernel can carry both.
  for i, d in enumerate(reduced_dims):
    if d in new_dims:
      tmp = "_" + d.name
      reduced_dims[i] = Dimension(tmp, d.size)
      x = mtf.rename_dimension(x, d.name, tmp)
  output_shape = Shape([d for d in x.shape.dims if d not in reduced_dims] + new_dims)
  if kernel_weights is None:
    if weights is None:
      raise ValueError("dense() needs kernel_weights or a WeightSource")
    kernel_weights = get_dense_kernel_weights(
        x, new_dims, reduced_dims, expert_dims, weights, name=name,
        variable_dtype=variable_dtype)
  # ReLU straight after the product rides in the einsum (a GEMM epilogue on
  # backends that support it) instead of a separate pass over the output.
  fused_relu = activation is mtf.relu and not use_bias
  y = mtf.einsum([x, kernel_weights], output_shape, activation="relu" if fused_relu else None)
  if fused_relu:
    return y
  if use_bias:
    if bias is None:
      bias = mtf.zeros(x.mesh, Shape(expert_dims + new_dims), dtype=x.dtype)
    y = y + bias
  if activation is not None:
    y = activation(y)
  return y


def dense_product(x, reduced_dims, new_dims, activation_functions=None, name="dense_product",
                  kernel_weights=None, **kwargs):
  """Component-wise product of dense layers (mesh_tensorflow/layers.py:256-295)."""
  if not isinstance(activation_functions, list):
    activation_functions = [activation_functions]
  n = len(activation_functions)
  if kernel_weights is not None and not isinstance(kernel_weights, list):
    kernel_weights = [kernel_weights]
  factors = []
  for i, activation in enumerate(activation_functions):
    if activation == "linear":
      activation = None
    elif isinstance(activation, str):
      activation = getattr(mtf, activation)
    factors.append(dense(
        x, reduced_dims=reduced_dims, new_dims=new_dims, activation=activation,
        name="%s_%d" % (name, i) if n > 1 else name,
        kernel_weights=kernel_weights[i] if kernel_weights else None, **kwargs))
  return functools.reduce(mtf.multiply, factors)


def dense_relu_dense(x, hidden_channels, is_training=False, dropout=0.0, weights=None,
                     wi=None, wo=None, name=None):
  """ReLU hidden layer then linear projection back to the input channels
  (mesh_tensorflow/layers.py:1148-1181); dropout 0 only."""
  del is_training
  if dropout != 0.0:
    raise NotImplementedError("dropout is outside the lowered forward path")
  io_channels = x.shape.dims[-1]
  h = dense(x, hidden_channels, use_bias=False, activation=mtf.relu, kernel_weights=wi,
            weights=weights, name="wi")
  return dense(h, io_channels, use_bias=False, activation=None, kernel_weights=wo,
               weights=weights, name="wo")


# ------------------------------------------------------- norms, embedding, loss
class NormOperation(mtf.Operation):
  """Layer norm (`centered`) or RMS norm over `dim` as one operation.

  When `dim` is the last dim of x and not split over the mesh, a slice's rows
  are normalised by one kernel (fp32 statistics, one rounding at the store);
  otherwise the statistics are formed with slice reductions and an allreduce
  over the mesh axis `dim` is split over, in the reference's order of
  operations (layers.py:968-979, transformer/transformer.py:516)."""

  def __init__(self, x, scale, bias, dim, epsilon, centered, name=None):
    inputs = [x] + [t for t in (scale, bias) if t is not None]
    super().__init__(inputs, name=name or ("layer_norm" if centered else "rms_norm"))
    self._dim, self._epsilon, self._centered = dim, epsilon, centered
    self._has_scale, self._has_bias = scale is not None, bias is not None
    self._outputs = [mtf.Tensor(self, x.shape, x.dtype)]

  def _unpack(self, tensors):
    it = iter(tensors[1:])
    return tensors[0], (next(it) if self._has_scale else None), (next(it) if self._has_bias else None)

  def gradient(self, grad_ys):
    dim, eps, centered = self._dim, self._epsilon, self._centered

    def chain(*tensors):
      x, scale, bias = self._unpack(list(tensors))
      return [_norm_chain(x, dim, eps, centered, scale, bias)]
    return mtf.gradients_by_recompute(self.inputs, chain, grad_ys)

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    ops = impl.slice_ops
    x = self.inputs[0]
    dim, eps, centered = self._dim, self._epsilon, self._centered
    axis = x.shape.dims.index(dim)
    mesh_axis = impl.tensor_dimension_to_mesh_axis(dim)
    lowered = [lowering.tensors[t] for t in self.inputs]
    has_scale, has_bias = self._has_scale, self._has_bias

    def split_args(args):
      it = iter(args[1:])
      return args[0], (next(it) if has_scale else None), (next(it) if has_bias else None)
    if mesh_axis is None and axis == x.shape.ndims - 1:
      def fn(*args):
        xs, sc, bi = split_args(args)
        return ops.norm_rows(xs, sc, bi, eps, centered)
      lowering.set_tensor_lowering(self.outputs[0], impl.slicewise(fn, *lowered))
      return
    # general layout: partial sums per slice, completed over the mesh axis
    nd = x.shape.ndims
    inv = 1.0 / float(dim.size)

    def mean_over_dim(values):
      part = impl.slicewise(lambda v: ops.expand_dims(ops.reduce("SUM", v, [axis]), axis), values)
      if mesh_axis is not None:
        part = impl.allreduce(part, [mesh_axis], "SUM")
      return impl.slicewise(lambda v: ops.binary("multiply", v, inv), part)
    xs = lowered[0]
    if centered:
      mean = mean_over_dim(xs)
      xs = impl.slicewise(lambda v, m: ops.binary("sub", v, m), xs, mean)
    var = mean_over_dim(impl.slicewise(lambda v: ops.unary("square", v), xs))

    def finish(v, variance, *rest):
      _, sc, bi = split_args((None,) + rest)
      out = ops.binary("multiply", v, ops.unary("rsqrt", ops.binary("add", variance, eps)))
      shape = [1] * nd
      if sc is not None:
        shape[axis] = ops.shape(sc)[0]
        out = ops.binary("multiply", out, ops.reshape(sc, shape))
      if bi is not None:
        shape[axis] = ops.shape(bi)[0]
        out = ops.binary("add", out, ops.reshape(bi, shape))
      return out
    lowering.set_tensor_lowering(self.outputs[0], impl.slicewise(finish, xs, var, *lowered[1:]))


def _norm_chain(x, dim, epsilon, centered, scale, bias):
  """The reference's op chains (layers.py:968-979; transformer.py:516)."""
  reduced_shape = x.shape - dim
  if centered:
    mean = mtf.reduce_mean(x, output_shape=reduced_shape)
    variance = mtf.reduce_mean(mtf.square(x - mean), output_shape=reduced_shape)
    y = (x - mean) * mtf.rsqrt(variance + epsilon)
  else:
    variance = mtf.reduce_mean(mtf.square(x), output_shape=reduced_shape)
    y = x * mtf.rsqrt(variance + epsilon)
  if scale is not None:
    y = y * scale
  if bias is not None:
    y = y + bias
  return y


def layer_norm(x, dim, epsilon=1e-6, scale=None, bias=None, fused=True, name="layer_norm"):
  """Layer normalisation over `dim` (mesh_tensorflow/layers.py:950-979): scale and
  bias are tensors of shape [dim] (the reference creates them as variables
  initialised to ones / zeros; None leaves the factor / offset out).  fused=False
  builds the reference's op chain instead of the single operation."""
  if not fused:
    return _norm_chain(x, dim, epsilon, True, scale, bias)
  return NormOperation(x, scale, bias, dim, epsilon, True, name=name).outputs[0]


def rms_norm(x, dim, epsilon=1e-6, scale=None, fused=True, name="rms_norm"):
  """x * rsqrt(mean(x^2) + epsilon) * scale (transformer/transformer.py:493-516)."""
  if not fused:
    return _norm_chain(x, dim, epsilon, False, scale, None)
  return NormOperation(x, scale, None, dim, epsilon, False, name=name).outputs[0]


def embedding_weights(mesh, vocab_dim, output_dim, dtype, weights, ensemble_dim=None, name="embedding"):
  """[ensemble dims,] vocab x output table ~ N(0, 1) (mesh_tensorflow/layers.py:2049-2066)."""
  ensemble = [] if not ensemble_dim else (ensemble_dim if isinstance(ensemble_dim, list) else [ensemble_dim])
  return weights.normal(mesh, Shape(ensemble + [vocab_dim, output_dim]), 1.0, dtype, name=name)


def embedding(indices, vocab_dim, output_dim, dtype, weights=None, table=None, name="embedding"):
  """Embedding lookup (mesh_tensorflow/layers.py:2069-2073): a row gather of the
  [vocab, output] table; `table` passes an existing one."""
  if table is None:
    table = embedding_weights(indices.mesh, vocab_dim, output_dim, dtype, weights, name=name)
  return mtf.gather(table, indices, vocab_dim)


class SoftmaxCrossEntropyOperation(mtf.Operation):
  """Per-example softmax loss with hard targets as one pass over the logits.

  Outputs: loss [logits.shape - vocab_dim] in the logits' dtype, and log_z in
  float32 (kept for the backward pass).  Each slice of a mesh-split vocabulary
  yields its row max, its sum of exp(x - max) and the target's logit if it holds
  the target column; an allreduce MAX and two allreduce SUMs over the vocabulary's
  mesh axis complete them - the collectives the reference's reduce_logsumexp
  and reduce_sum(log_softmax * one_hot) perform (layers.py:1109-1116,
  ops.py:5493-5520) on tensors a vocabulary-size smaller."""

  def __init__(self, logits, targets, vocab_dim, z_loss, name=None):
    super().__init__([logits, targets], name=name or "softmax_cross_entropy")
    self._vocab_dim, self._z_loss = vocab_dim, z_loss
    out_shape = logits.shape - vocab_dim
    self._outputs = [mtf.Tensor(self, out_shape, logits.dtype, index=0),
                     mtf.Tensor(self, out_shape, G.float32, index=1)]

  def gradient(self, grad_ys):
    logits, targets = self.inputs
    if grad_ys[0] is None:
      return [None, None]
    dlogits = SoftmaxCrossEntropyGradOperation(
        logits, targets, self.outputs[1], mtf.cast(grad_ys[0], G.float32), self._vocab_dim,
        self._z_loss).outputs[0]
    return [dlogits, None]

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    ops = impl.slice_ops
    logits, targets = self.inputs
    vocab, z = self._vocab_dim, self._z_loss
    axis = logits.shape.dims.index(vocab)
    nd = logits.shape.ndims
    mesh_axis = impl.tensor_dimension_to_mesh_axis(vocab)
    cols_here = impl.slice_shape(logits.shape)[axis]
    # targets' dims in the order the logits have them (minus the vocabulary)
    t_perm = [targets.shape.dims.index(d) for d in logits.shape.dims if d != vocab]

    def stats(x, t, pcoord):
      if axis != nd - 1:
        x = ops.transpose(x, [i for i in range(nd) if i != axis] + [axis])
      if t_perm != list(range(len(t_perm))):
        t = ops.transpose(t, t_perm)
      return ops.xent_stats(x, t, int(pcoord) * cols_here)
    pcoord = impl.laid_out_pcoord(mesh_axis) if mesh_axis is not None else 0
    m, s, picked = impl.slicewise(stats, lowering.tensors[logits], lowering.tensors[targets], pcoord)
    if mesh_axis is not None:
      gmax = impl.allreduce(m, [mesh_axis], "MAX")
      s = impl.slicewise(lambda sv, mv, gv: ops.binary("multiply", sv, ops.unary("exp", ops.binary("sub", mv, gv))),
                         s, m, gmax)
      s = impl.allreduce(s, [mesh_axis], "SUM")
      picked = impl.allreduce(picked, [mesh_axis], "SUM")
      m = gmax
    log_z = impl.slicewise(lambda sv, mv: ops.binary("add", ops.unary("log", sv), mv), s, m)

    def loss_fn(lz, pk):
      out = ops.binary("sub", lz, pk)
      if z != 0:
        out = ops.binary("add", out, ops.binary("multiply", ops.unary("square", lz), z))
      return ops.cast(out, logits.dtype)
    lowering.set_tensor_lowering(self.outputs[0], impl.slicewise(loss_fn, log_z, picked))
    lowering.set_tensor_lowering(self.outputs[1], log_z)


class SoftmaxCrossEntropyGradOperation(mtf.Operation):
  """dlogits = dloss * ((1 + 2 z_loss log_z) softmax(logits) - one_hot(targets))."""

  def __init__(self, logits, targets, log_z, dloss, vocab_dim, z_loss, name=None):
    super().__init__([logits, targets, log_z, dloss], name=name or "softmax_cross_entropy_grad")
    self._vocab_dim, self._z_loss = vocab_dim, z_loss
    self._outputs = [mtf.Tensor(self, logits.shape, logits.dtype)]

  @property
  def has_gradient(self):
    return False

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    ops = impl.slice_ops
    logits = self.inputs[0]
    vocab, z = self._vocab_dim, self._z_loss
    axis = logits.shape.dims.index(vocab)
    nd = logits.shape.ndims
    if axis != nd - 1:
      raise NotImplementedError("cross-entropy gradient needs the vocabulary as the last dim of the logits")
    mesh_axis = impl.tensor_dimension_to_mesh_axis(vocab)
    cols_here = impl.slice_shape(logits.shape)[axis]
    pcoord = impl.laid_out_pcoord(mesh_axis) if mesh_axis is not None else 0
    fn = lambda x, t, lz, dl, pc: ops.xent_grad(x, t, lz, dl, z, int(pc) * cols_here)
    lowering.set_tensor_lowering(
        self.outputs[0], impl.slicewise(fn, *[lowering.tensors[t] for t in self.inputs], pcoord))


def softmax_cross_entropy_with_logits(logits, targets, vocab_dim, z_loss=0.0, fused=True):
  """Per-example softmax loss (mesh_tensorflow/layers.py:1062-1117); hard targets
  (integer dtype) take the single-pass operation unless fused=False, soft
  targets the reference's op chain."""
  if targets.dtype.is_integer:
    if set(targets.shape.dims) != set(logits.shape.dims).difference([vocab_dim]):
      raise ValueError(
          "softmax_cross_entropy_with_logits with hard targets "
          "dims in targets=%s should be dims in logits=%s other than "
          "vocab_dim=%s" % (targets, logits, vocab_dim))
    if fused and vocab_dim in logits.shape.dims:
      return SoftmaxCrossEntropyOperation(logits, targets, vocab_dim, z_loss).outputs[0]
    targets = mtf.one_hot(targets, vocab_dim, dtype=logits.dtype)
  elif set(targets.shape.dims) != set(logits.shape.dims):
    raise ValueError(
        "softmax_cross_entropy_with_logits with soft targets "
        "dims in targets=%s should be dims in logits=%s" % (targets, logits))
  if vocab_dim not in logits.shape.dims:
    raise ValueError("vocab_dim must be in logits.shape.dims")
  log_z = mtf.reduce_logsumexp(logits, vocab_dim)
  log_softmax = logits - log_z
  loss = mtf.negative(mtf.reduce_sum(log_softmax * targets, reduced_dim=vocab_dim))
  if z_loss != 0:
    loss += z_loss * mtf.square(log_z)
  return loss


def multiplicative_jitter(x, epsilon=1e-2):
  """x times uniform noise in [1 - epsilon, 1 + epsilon) (mesh_tensorflow/layers.py:1936-1952)."""
  if epsilon == 0:
    return x
  return x * mtf.random_uniform(x.mesh, x.shape, minval=1.0 - epsilon, maxval=1.0 + epsilon,
                                dtype=x.dtype)


def rename_length_to_memory_length(x, length_name="length", memory_length_name="memory_length"):
  return mtf.rename_dimension(x, length_name, memory_length_name)


def attention_mask_autoregressive(query_pos, dtype=G.float32):
  """-1e9 where a query would look right of itself (mesh_tensorflow/layers.py:1839-1850).

  When `query_pos` is the plain range over the length dim the returned tensor is
  tagged as the causal mask, which lets dot_product_attention use the fused
  kernel's built-in masking instead of adding this tensor to the logits.
  """
  memory_pos = rename_length_to_memory_length(query_pos)
  mask = mtf.cast(mtf.less(query_pos, memory_pos), dtype) * -1e9
  if getattr(query_pos.operation, "is_plain_range", False):
    mask.causal_hint = True
  return mask


class FusedAttentionOperation(mtf.Operation):
  """softmax(q.k + causal bias).v as one operation per slice.

  q [..., length_q, d_k], k [..., length_kv, d_k], v [..., length_kv, d_v] with the
  same leading dims (typically batch, heads).  Leading dims may be split over
  the mesh freely; the two length dims and the depth dims must not be, because
  the softmax statistics are slice-local.
  """

  def __init__(self, q, k, v, causal, name=None):
    super().__init__([q, k, v], name=name or "fused_attention")
    self._causal = causal
    self._outputs = [mtf.Tensor(self, Shape(q.shape.dims[:-1] + [v.shape.dims[-1]]), v.dtype)]

  def gradient(self, grad_ys):
    """Backward pass through the op-by-op chain (einsum, fp32 softmax, einsum),
    which recomputes the attention weights: the fused kernel keeps no logits.
    The chain materialises [..., length_q, length_kv] fp32 tensors."""
    causal = self._causal

    def chain(q, k, v):
      mask = None
      if causal:
        q_pos = mtf.mtf_range(q.mesh, q.shape.dims[-2], G.float32)
        k_pos = mtf.mtf_range(q.mesh, k.shape.dims[-2], G.float32)
        mask = mtf.cast(mtf.less(q_pos, k_pos), G.float32) * -1e9
      return [dot_product_attention(q, k, v, mask, fused=False)]
    return mtf.gradients_by_recompute(self.inputs, chain, grad_ys)

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    q, k, v = self.inputs
    for d in (q.shape.dims[-2], q.shape.dims[-1], k.shape.dims[-2], v.shape.dims[-1]):
      if impl.tensor_dimension_to_mesh_axis(d) is not None:
        raise ValueError("fused attention needs %s unsplit; pass fused=False to "
                         "dot_product_attention for this layout" % (d,))
    ops, causal = impl.slice_ops, self._causal
    lowering.set_tensor_lowering(
        self.outputs[0],
        impl.slicewise(lambda a, b, c: ops.attention(a, b, c, causal),
                       *[lowering.tensors[t] for t in self.inputs]))


def multihead_attention_params(mesh, heads, io_channels, kv_channels, weights, dtype):
  """wq, wk, wv, wo of shape [heads, io_channels, kv_channels]
  (mesh_tensorflow/layers.py:1564-1611; the 1/sqrt(d) scale lives in wq, wk)."""
  qk_stddev = (io_channels.size ** -0.5) * (kv_channels.size ** -0.25)
  v_stddev = io_channels.size ** -0.5
  o_stddev = (io_channels.size * heads.size) ** -0.5
  shape = Shape([heads, io_channels, kv_channels])
  return [weights.normal(mesh, shape, s, dtype, name=n)
          for n, s in zip("qkvo", [qk_stddev, qk_stddev, v_stddev, o_stddev])]


def dot_product_attention(q, k, v, mask, is_training=False, dropout=0.0, extra_logit=None,
                          float32_logits=True, fused=None):
  """softmax(q.k + mask).v (mesh_tensorflow/layers.py:1614-1652).

  With float32_logits the logits and softmax are computed in float32 and the
  weights cast back to v.dtype, as transformer/attention.py:71-88 does.
  `fused` selects the single-operation form (FusedAttentionOperation); the
  default fuses bfloat16 attention whose mask is absent or the causal mask.
  """
  del is_training
  if dropout != 0.0:
    raise NotImplementedError("dropout is outside the lowered forward path")
  fusable = (extra_logit is None and float32_logits
             and (mask is None or getattr(mask, "causal_hint", False)))
  if fused is None:
    fused = fusable and q.dtype == G.bfloat16
  if fused:
    if not fusable:
      raise ValueError("fused attention supports no mask or the causal mask only")
    return FusedAttentionOperation(q, k, v, causal=mask is not None).outputs[0]
  length_kv = k.shape.dims[-2]
  logits_shape = Shape(q.shape.dims[:-1] + [length_kv])
  if float32_logits:
    q, k = mtf.cast(q, G.float32), mtf.cast(k, G.float32)
  logits = mtf.einsum([q, k], logits_shape)
  if mask is not None:
    logits = logits + mtf.cast(mask, logits.dtype)
  w = mtf.softmax(logits, length_kv, extra_logit=extra_logit)
  w = mtf.cast(w, v.dtype)
  outputs_shape = Shape(q.shape.dims[:-1] + [v.shape.dims[-1]])
  return mtf.einsum([w, v], outputs_shape)


def local_attention_1d(q, k, v, length_dim, key_dim, value_dim, fully_autoregressive=True,
                       length_dim_num_splits=1, radius=128, sequence_id=1,
                       write_priority=None, read_priority=None):
  """Attention to a neighbourhood of each position
  (mesh_tensorflow/transformer/attention.py:724-827).

  Query position p sees memory positions in (p - radius, p] when
  `fully_autoregressive`, else in (p - radius, p + radius]; positions of another
  `sequence_id` and, if priorities are given, positions with
  write_priority > read_priority[p] are hidden as well.  The length is cut into
  blocks (the largest divisor of the per-processor length that is at most
  max(radius, 128)); a block of queries attends to its own block of memory extended
  by the margins of its neighbours (halo exchange: collective permutes between
  neighbouring processors when the length is split over a mesh axis), so the logits
  are [.., blocks, block, block + margins] instead of [.., length, length].
  `v=None` uses the keys as values.  Returns q's shape with key_dim -> value_dim."""
  length_per_split = length_dim.size // length_dim_num_splits
  block_length = max(radius, 128)
  while length_per_split % block_length != 0:
    block_length -= 1
  query_block = Dimension("query_block_length", block_length)
  memory_block = Dimension("memory_block_length", block_length)
  # the blocks dim takes the length dim's name, so the layout splits it the same way
  num_blocks = Dimension(length_dim.name, length_dim.size // block_length)
  exchange = mtf.left_halo_exchange if fully_autoregressive else mtf.halo_exchange

  def as_queries(x):
    return mtf.replace_dimensions(x, length_dim, [num_blocks, query_block])

  def as_memory(x):
    x = mtf.replace_dimensions(x, length_dim, [num_blocks, memory_block])
    return exchange(x, num_blocks, memory_block, radius)
  mesh = q.mesh
  q = as_queries(q)
  k = as_memory(k)
  v = as_memory(v) if v is not None else k
  if sequence_id is None:
    sequence_id = 1
  if not isinstance(sequence_id, mtf.Tensor) or length_dim not in sequence_id.shape.dims:
    # margins that reach past the ends arrive as zeros: sequence 0, which nobody belongs to
    sequence_id = mtf.zeros(mesh, Shape([length_dim]), dtype=G.int32) + sequence_id
  position = mtf.mtf_range(mesh, length_dim, G.int32)
  relative = as_memory(position) - as_queries(position)
  visible = mtf.equal(as_queries(sequence_id), as_memory(sequence_id))
  visible = mtf.logical_and(visible, mtf.greater(relative, -radius))
  visible = mtf.logical_and(visible, mtf.less_equal(relative, 0 if fully_autoregressive else radius))
  if read_priority is not None:
    visible = mtf.logical_and(
        visible, mtf.greater_equal(as_queries(read_priority), as_memory(write_priority)))
  bias = mtf.cast(mtf.logical_not(visible), G.float32) * -1e9
  padded_memory = Dimension("memory_block_length",
                            (1 if fully_autoregressive else 2) * radius + block_length)
  # logits and softmax in float32, weights back in v's type (attention.py:71-88)
  logits = mtf.einsum([mtf.cast(q, G.float32), mtf.cast(k, G.float32)],
                      reduced_dims=[key_dim]) + bias
  weights = mtf.cast(mtf.softmax(logits, padded_memory), v.dtype)
  out_dims = [d for d in q.shape.dims if d != key_dim] + [value_dim]
  o = mtf.einsum([weights, v], output_shape=Shape(out_dims))
  return mtf.replace_dimensions(o, [num_blocks, query_block], length_dim)


def multihead_attention(query_antecedent, memory_antecedent, mask, kv_channels, heads,
                        is_training=False, dropout=0.0, weights=None, params=None,
                        float32_logits=True, fused=None, name="multihead_attention"):
  """Projections, attention and output projection (mesh_tensorflow/layers.py:1655-1723).

  The output projection contracts (heads, kv_channels); with `heads` split
  over a mesh axis its result is a LazyAllreduceSum over that axis.
  """
  del name
  batch_dims = query_antecedent.shape.dims[:-2]
  query_length, io_channels = query_antecedent.shape.dims[-2:]
  if params is None:
    params = multihead_attention_params(
        query_antecedent.mesh, heads, io_channels, kv_channels, weights,
        query_antecedent.dtype)
  wq, wk, wv, wo = params
  if memory_antecedent is None:
    memory_antecedent = rename_length_to_memory_length(query_antecedent, query_length.name)
  memory_length, memory_channels = memory_antecedent.shape.dims[-2:]
  if memory_antecedent.shape.dims[:-2] != batch_dims:
    raise ValueError("memory batch must equal query batch")
  if memory_channels != io_channels:
    raise ValueError("memory channels must equal query channels")
  q = mtf.einsum([query_antecedent, wq], Shape(batch_dims + [heads, query_length, kv_channels]))
  k = mtf.einsum([memory_antecedent, wk], Shape(batch_dims + [heads, memory_length, kv_channels]))
  v = mtf.einsum([memory_antecedent, wv], Shape(batch_dims + [heads, memory_length, kv_channels]))
  o = dot_product_attention(q, k, v, mask, is_training, dropout, float32_logits=float32_logits,
                            fused=fused)
  return mtf.einsum([o, wo], Shape(batch_dims + [query_length, io_channels]))
