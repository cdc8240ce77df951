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
