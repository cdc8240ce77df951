"""Top-2 mixture-of-experts layer on the mesh-tensor language.

Follows mesh_tensorflow/transformer/moe.py: `transformer_moe_layer_v1`
(191-525), `_top_2_gating` (1312-1513), `_split_into_groups` (1549-1582) and
`HParams` (1585-1596).  Two graph forms compute the same layer:

  * unfused: the reference's own op chain — softmax, two top_1, triangular
    cumsum, dense [G,S,E,C] combine/dispatch tensors and two dense einsums;
  * fused (default): three operations whose per-slice work is one kernel each
    — gating (logits, softmax, top-2, capacity positions), dispatch (row
    gather into expert slots) and combine (gated row scatter-add) — with the
    same reshapes, and therefore the same alltoalls, in between.

Both forms return (output, loss * moe_loss_coef).
"""

from __future__ import annotations

from mesh_b200.mtf import graph as G
from mesh_b200.mtf import layers
from mesh_b200.mtf import ops as mtf
from mesh_b200.mtf.graph import Operation, Tensor
from mesh_b200.mtf.layout import tensor_dim_to_mesh_dim_size
from mesh_b200.mtf.mesh_impl import LazyAllreduceSum
from mesh_b200.mtf.shapes import Dimension, Shape


class HParams(object):
  """Attribute bag with the reference's MoE hyper-parameter names (moe.py:36-89)."""

  def __init__(self, **kwargs):
    self.moe_gating = "top_2"
    self.moe_num_experts = 16
    self.moe_loss_coef = 1e-2
    self.moe_hidden_size = 4096
    self.moe_group_size = 1024
    self.moe_capacity_factor_train = 1.25
    self.moe_capacity_factor_eval = 2.0
    self.moe_capacity_factor_second_level = 1.0
    self.moe_use_second_place_loss = False
    self.moe_second_policy_train = "random"
    self.moe_second_policy_eval = "random"
    self.moe_second_threshold_train = 0.2
    self.moe_second_threshold_eval = 0.2
    self.moe_dropout_rate = 0.0
    self.moe_min_expert_capacity = 4
    self.moe_switch_policy_train = "argmax"
    self.moe_switch_policy_eval = "argmax"
    self.moe_switch_dropout = 0.1
    self.moe_switch_jitter = 1e-2
    self.moe_switch_temperature = 1.0
    self.moe_z_loss = None
    self.moe_ntlb_top_k = 4
    self.moe_use_fused_kernels = True
    for k, v in kwargs.items():
      if not hasattr(self, k):
        raise ValueError("unknown hyper-parameter %s" % k)
      setattr(self, k, v)


def _split_into_groups(n, max_group_size, mesh_dim_size):
  """Largest group_size <= max_group_size with num_groups a multiple of the
  mesh dimension (moe.py:1549-1582)."""
  if n % mesh_dim_size != 0:
    raise ValueError("n=%d is not a multiple of mesh_dim_size=%d" % (n, mesh_dim_size))
  num_groups = max(1, n // max_group_size)
  while num_groups % mesh_dim_size != 0 or n % num_groups != 0:
    num_groups += 1
  return num_groups, n // num_groups


def expert_capacity(group_size, num_experts, capacity_factor, min_capacity):
  """Slots per expert and group (moe.py:368-371)."""
  return max(min(group_size, int((group_size * capacity_factor) / num_experts)), min_capacity)


def _second_policy(hparams, train):
  if train:
    return hparams.moe_second_policy_train, hparams.moe_second_threshold_train
  return hparams.moe_second_policy_eval, hparams.moe_second_threshold_eval


# ------------------------------------------------------------ unfused gating
def _top_2_gating(inputs, experts_dim, expert_capacity_dim, hparams, train, gate_weights,
                  second_noise=None, importance=None):
  """The reference's op chain (moe.py:1380-1513); returns dispatch, combine, loss.

  `importance` [..., group] (1.0, 0.5 or 0.0 per position) is how the two-level
  layer tells its inner routers what a position is: only positions of importance 1
  take part as first choices (and in the loss), positions of importance 0 (empty
  slots of the outer level) are not routed at all.  The gate kernel may carry
  leading expert dims (one router per outer expert)."""
  group_size_dim = inputs.shape.dims[-2]
  gate_inputs = mtf.to_float(inputs)
  raw_gates = layers.dense(gate_inputs, experts_dim, use_bias=False,
                           kernel_weights=gate_weights, name="gate")
  raw_gates = mtf.softmax(raw_gates, experts_dim)
  capacity_f = float(expert_capacity_dim.size)

  gate_1, index_1 = mtf.top_1(raw_gates, experts_dim)
  mask_1 = mtf.one_hot(index_1, experts_dim, dtype=raw_gates.dtype)
  density_1_proxy = raw_gates
  if importance is not None:
    full = mtf.to_float(mtf.equal(importance, 1.0))
    mask_1 *= full
    gate_1 *= full
    density_1_proxy *= full
  gates_without_top_1 = raw_gates * (1.0 - mask_1)
  gate_2, index_2 = mtf.top_1(gates_without_top_1, experts_dim)
  mask_2 = mtf.one_hot(index_2, experts_dim, dtype=raw_gates.dtype)
  if importance is not None:
    mask_2 *= mtf.to_float(mtf.greater(importance, 0.0))

  denom = gate_1 + gate_2 + 1e-9
  gate_1 /= denom
  gate_2 /= denom

  density_1 = mtf.reduce_mean(mask_1, reduced_dim=group_size_dim)
  density_1_proxy = mtf.reduce_mean(density_1_proxy, reduced_dim=group_size_dim)
  loss = (mtf.reduce_mean(density_1_proxy * density_1)
          * float(experts_dim.size * experts_dim.size))
  if hparams.moe_use_second_place_loss:
    # the same product for the second choices, with the gates renormalised after the
    # top one is taken out as the smooth stand-in, at half weight (moe.py:1428-1440)
    density_2 = mtf.reduce_mean(mask_2, reduced_dim=group_size_dim)
    normalized = gates_without_top_1 / (
        mtf.reduce_sum(gates_without_top_1, reduced_dim=experts_dim) + 1e-9)
    density_2_proxy = mtf.reduce_mean(normalized, reduced_dim=group_size_dim)
    loss += (mtf.reduce_mean(density_2_proxy * density_2)
             * float(experts_dim.size * experts_dim.size)) * 0.5

  policy, threshold = _second_policy(hparams, train)
  if policy == "all":
    pass
  elif policy == "none":
    mask_2 = mtf.zeros_like(mask_2)
  elif policy == "threshold":
    mask_2 *= mtf.to_float(mtf.greater(gate_2, threshold))
  elif policy == "random":
    if second_noise is None:
      raise ValueError("policy 'random' needs the uniform noise tensor as an input")
    mask_2 *= mtf.to_float(mtf.less(second_noise, gate_2 / max(threshold, 1e-9)))
  else:
    raise ValueError("Unknown policy %s" % policy)

  position_in_expert_1 = mtf.cumsum(mask_1, group_size_dim, exclusive=True) * mask_1
  mask_1 *= mtf.to_float(mtf.less(position_in_expert_1, capacity_f))
  mask_1_count = mtf.reduce_sum(mask_1, reduced_dim=group_size_dim)
  mask_1_flat = mtf.reduce_sum(mask_1, reduced_dim=experts_dim)
  position_in_expert_1 = mtf.reduce_sum(position_in_expert_1, reduced_dim=experts_dim)
  gate_1 *= mask_1_flat

  position_in_expert_2 = mtf.cumsum(mask_2, group_size_dim, exclusive=True) + mask_1_count
  position_in_expert_2 *= mask_2
  mask_2 *= mtf.to_float(mtf.less(position_in_expert_2, capacity_f))
  mask_2_flat = mtf.reduce_sum(mask_2, reduced_dim=experts_dim)
  gate_2 *= mask_2_flat
  position_in_expert_2 = mtf.reduce_sum(position_in_expert_2, reduced_dim=experts_dim)

  combine_tensor = (
      gate_1 * mask_1_flat
      * mtf.one_hot(index_1, experts_dim)
      * mtf.one_hot(mtf.to_int32(position_in_expert_1), expert_capacity_dim) +
      gate_2 * mask_2_flat
      * mtf.one_hot(index_2, experts_dim)
      * mtf.one_hot(mtf.to_int32(position_in_expert_2), expert_capacity_dim))
  combine_tensor = mtf.cast(combine_tensor, inputs.dtype)
  loss = mtf.cast(loss, inputs.dtype)
  dispatch_tensor = mtf.cast(mtf.cast(combine_tensor, G.bool_), combine_tensor.dtype)
  aux = dict(index_1=index_1, index_2=index_2,
             position_1=mtf.to_int32(position_in_expert_1),
             position_2=mtf.to_int32(position_in_expert_2),
             gate_1=gate_1, gate_2=gate_2, raw_gates=raw_gates)
  return dispatch_tensor, combine_tensor, loss, aux


def _switch_gating(inputs, experts_dim, expert_capacity_dim, hparams, train, gate_weights,
                   importance=None):
  """Top-1 ("Switch") routing as the reference's op chain (moe.py:1184-1309):
  softmax, top_1 with the raw gate kept as it is, first-come positions within the
  expert's capacity, the same load-balancing loss as top-2 gating plus the
  optional router z-loss.  Policies argmax, input_jitter, input_dropout and sample (the
  expert drawn from the router's distribution at hparams.moe_switch_temperature).
  `importance` [..., group]: positions that are not 1.0 (padding) are not routed."""
  policy = hparams.moe_switch_policy_train if train else hparams.moe_switch_policy_eval
  group_size_dim = inputs.shape.dims[-2]
  gate_inputs = mtf.to_float(inputs)
  if policy == "input_dropout":
    gate_inputs = mtf.dropout(gate_inputs, is_training=train, keep_prob=1.0 - hparams.moe_switch_dropout)
  elif train and policy == "input_jitter":
    gate_inputs = layers.multiplicative_jitter(gate_inputs, hparams.moe_switch_jitter)
  elif policy not in ("argmax", "input_jitter", "sample"):
    raise ValueError("Unknown Switch gating policy %s" % policy)
  gate_logits = layers.dense(gate_inputs, experts_dim, use_bias=False, kernel_weights=gate_weights,
                             name="switch_gating")
  raw_gates = mtf.softmax(gate_logits, experts_dim)
  if policy == "sample":
    # the expert is drawn from the router's distribution; the gate is its probability
    expert_index = mtf.sample_with_temperature(gate_logits, experts_dim,
                                               temperature=hparams.moe_switch_temperature)
    expert_gate = mtf.reduce_sum(
        raw_gates * mtf.one_hot(expert_index, experts_dim, dtype=raw_gates.dtype), reduced_dim=experts_dim)
  else:
    expert_gate, expert_index = mtf.top_1(raw_gates, experts_dim)
  expert_mask = mtf.one_hot(expert_index, experts_dim, dtype=raw_gates.dtype)
  density_1 = mtf.reduce_mean(expert_mask, reduced_dim=group_size_dim)
  density_1_proxy = mtf.reduce_mean(raw_gates, reduced_dim=group_size_dim)
  if importance is not None:
    # padding takes no slot, carries no gate and does not count in the loss's proxy
    real = mtf.to_float(mtf.equal(importance, 1.0))
    expert_mask *= real
    expert_gate *= real
    density_1_proxy *= real
  loss = mtf.reduce_mean(density_1_proxy * density_1) * float(experts_dim.size * experts_dim.size)
  if train and hparams.moe_z_loss is not None:
    log_z = mtf.reduce_logsumexp(gate_logits, experts_dim)
    loss += mtf.reduce_mean(mtf.square(log_z)) * hparams.moe_z_loss
  position_in_expert = mtf.cumsum(expert_mask, group_size_dim, exclusive=True) * expert_mask
  expert_mask *= mtf.to_float(mtf.less(position_in_expert, float(expert_capacity_dim.size)))
  expert_mask_flat = mtf.reduce_sum(expert_mask, reduced_dim=experts_dim)
  position_flat = mtf.reduce_sum(position_in_expert, reduced_dim=experts_dim)
  expert_gate *= expert_mask_flat
  combine_tensor = (expert_gate * expert_mask_flat
                    * mtf.one_hot(expert_index, experts_dim, dtype=raw_gates.dtype)
                    * mtf.one_hot(mtf.to_int32(position_flat), expert_capacity_dim, dtype=raw_gates.dtype))
  combine_tensor = mtf.cast(combine_tensor, inputs.dtype)
  loss = mtf.cast(loss, inputs.dtype)
  dispatch_tensor = mtf.cast(mtf.cast(combine_tensor, G.bool_), combine_tensor.dtype)
  aux = dict(index_1=expert_index, position_1=mtf.to_int32(position_flat), gate_1=expert_gate,
             raw_gates=raw_gates)
  return dispatch_tensor, combine_tensor, loss, aux


# ------------------------------------------------- further top-1 style routers
def _router_gates(inputs, experts_dim, hparams, train, gate_weights, name, reduced_dim=None,
                  perturb_in_float=True, allow_dropout=True, logit_bias=None):
  """What the Switch-family routers share up to the softmax: exploration noise on the
  router's input (policies input_jitter / input_dropout), the gate dense layer, the
  softmax over `reduced_dim` (the experts unless stated).  Returns (gate_logits, raw_gates)."""
  policy = hparams.moe_switch_policy_train if train else hparams.moe_switch_policy_eval
  if policy not in ("argmax", "input_jitter", "input_dropout"):
    raise ValueError("Unknown Switch gating policy %s" % policy)
  gate_inputs = mtf.to_float(inputs) if perturb_in_float else inputs
  if policy == "input_dropout" and allow_dropout:
    gate_inputs = mtf.dropout(gate_inputs, is_training=train, keep_prob=1.0 - hparams.moe_switch_dropout)
  elif train and policy == "input_jitter":
    gate_inputs = layers.multiplicative_jitter(gate_inputs, hparams.moe_switch_jitter)
  gate_logits = layers.dense(gate_inputs, experts_dim, use_bias=False, kernel_weights=gate_weights,
                             name=name)
  if logit_bias is not None:
    gate_logits += logit_bias
  raw_gates = mtf.softmax(gate_logits, reduced_dim or experts_dim)
  return gate_logits, mtf.to_float(raw_gates)


def _balance_loss(raw_gates, expert_mask, group_size_dim, experts_dim, real=None):
  """mean over (group, expert) of [fraction of tokens choosing e] x [mean gate of e],
  times E^2 (the loss of moe.py:1420-1424, shared by the top-1 routers).  `real`
  (1.0 for positions that are not padding) meets the already averaged gates, as in
  the reference (moe.py:858-866): a group's term is scaled by its share of real
  positions."""
  density = mtf.reduce_mean(expert_mask, reduced_dim=group_size_dim)
  density_proxy = mtf.reduce_mean(raw_gates, reduced_dim=group_size_dim)
  if real is not None:
    density_proxy *= real
  return mtf.reduce_mean(density_proxy * density) * float(experts_dim.size * experts_dim.size)


def _finish_router(combine_tensor, dispatch_source, loss, inputs):
  combine_tensor = mtf.cast(combine_tensor, inputs.dtype)
  source = combine_tensor if dispatch_source is None else dispatch_source
  dispatch_tensor = mtf.cast(mtf.cast(source, G.bool_), combine_tensor.dtype)
  return dispatch_tensor, combine_tensor, mtf.cast(loss, inputs.dtype)


def _ntlb_gating(inputs, experts_dim, expert_capacity_dim, hparams, train, gate_weights,
                 importance=None):
  """"No token left behind" routing (moe.py:804-940): every token ranks its
  hparams.moe_ntlb_top_k best experts; round i offers the still unrouted tokens
  their i-th choice, first come first served within what is left of each
  expert's capacity.  A token routed in round i carries its i-th gate."""
  outer_batch_dim, batch_dim, group_size_dim = inputs.shape.dims[:3]
  _, raw_gates = _router_gates(inputs, experts_dim, hparams, train, gate_weights, "ntlb_gating",
                               perturb_in_float=False, allow_dropout=False)
  k_dim = Dimension("k", hparams.moe_ntlb_top_k)
  expert_gate, expert_index = mtf.top_k(raw_gates, reduced_dim=experts_dim, k_dim=k_dim)
  expert_mask = mtf.one_hot(expert_index, experts_dim)
  real = None if importance is None else mtf.to_float(mtf.equal(importance, 1.0))
  density_mask = expert_mask          # the loss's choice fractions are taken before the mask
  if real is not None:
    expert_mask *= real
    expert_gate *= real
  loss = _balance_loss(raw_gates, density_mask, group_size_dim, experts_dim, real)
  masks = mtf.split(expert_mask, k_dim, k_dim.size)
  gates = mtf.split(expert_gate, k_dim, k_dim.size)
  indices = mtf.split(expert_index, k_dim, k_dim.size)
  mesh = inputs.mesh
  token_shape = Shape([outer_batch_dim, batch_dim, group_size_dim])
  combine_tensor = mtf.constant(mesh, 0, Shape([outer_batch_dim, batch_dim, experts_dim, expert_capacity_dim]))
  taken = mtf.constant(mesh, 0, Shape([outer_batch_dim, batch_dim, experts_dim]))
  unrouted = mtf.constant(mesh, 1.0, token_shape)
  capacity = float(expert_capacity_dim.size)
  for mask_i, gate_i, index_i in zip(masks, gates, indices):
    mask_i = mtf.reshape(mask_i, Shape(token_shape.dims + [experts_dim])) * unrouted
    gate_i = mtf.reshape(gate_i, token_shape)
    index_i = mtf.reshape(index_i, token_shape)
    # arrival number of each candidate at its expert, counting what earlier rounds placed
    arrival = taken + mtf.cumsum(mask_i, group_size_dim)
    placed = mask_i * mtf.to_float(mtf.less_equal(arrival, capacity))
    taken += mtf.reduce_sum(placed, reduced_dim=group_size_dim)
    placed_flat = mtf.reduce_sum(placed, reduced_dim=experts_dim)
    unrouted -= placed_flat
    combine_tensor += (gate_i * placed_flat * mtf.one_hot(index_i, experts_dim)
                       * mtf.one_hot(mtf.to_int32(arrival - 1), expert_capacity_dim))
  return _finish_router(combine_tensor, None, loss, inputs)


def _switch_max_gating(inputs, experts_dim, expert_capacity_dim, hparams, train, gate_weights,
                       importance=None):
  """Top-1 routing in which an expert over capacity keeps its highest-gate
  tokens instead of the first ones (moe.py:943-1054): top-`capacity` over the
  group of (mask x gate) per expert."""
  group_size_dim = inputs.shape.dims[-2]
  _, raw_gates = _router_gates(inputs, experts_dim, hparams, train, gate_weights, "switch_max_gating")
  expert_gate, expert_index = mtf.top_1(raw_gates, experts_dim)
  expert_mask = mtf.one_hot(expert_index, experts_dim, dtype=raw_gates.dtype)
  real = None if importance is None else mtf.to_float(mtf.equal(importance, 1.0))
  density_mask = expert_mask
  if real is not None:
    expert_mask *= real
    expert_gate *= real
  loss = _balance_loss(raw_gates, density_mask, group_size_dim, experts_dim, real)
  kept_gate, kept_token = mtf.top_k(expert_mask * expert_gate, reduced_dim=group_size_dim,
                                    k_dim=expert_capacity_dim)
  combine_tensor = mtf.one_hot(kept_token, group_size_dim, dtype=raw_gates.dtype) * kept_gate
  return _finish_router(combine_tensor, None, loss, inputs)


def _expert_selection_gating(inputs, experts_dim, group_size_dim, expert_capacity_dim, hparams, train,
                             gate_weights, normalize_by_num_experts_routed=True, importance=None):
  """Experts choose tokens (moe.py:1057-1173): the softmax runs over the GROUP, every
  expert takes its `capacity` most probable tokens, and a token's contributions are
  divided by the number of experts that took it.  The loss pushes the mean (over
  experts) token probability towards uniform."""
  # padding gets -1e9 on its logits: the softmax runs over the positions of the group
  _, raw_gates = _router_gates(inputs, experts_dim, hparams, train, gate_weights,
                               "expert_selection_gating", reduced_dim=group_size_dim,
                               logit_bias=None if importance is None else
                               mtf.to_float(mtf.equal(importance, 0.0)) * -1e9)
  token_prob, token_index = mtf.top_k(raw_gates, reduced_dim=group_size_dim, k_dim=expert_capacity_dim)
  dispatch_tensor = mtf.one_hot(token_index, group_size_dim, dtype=raw_gates.dtype)
  combine_tensor = dispatch_tensor * token_prob
  if normalize_by_num_experts_routed:
    times_taken = mtf.reduce_sum(
        dispatch_tensor, output_shape=Shape(dispatch_tensor.shape.dims[:2] + [group_size_dim]))
    combine_tensor /= mtf.maximum(times_taken, 1.0)
  mean_prob = mtf.reduce_mean(raw_gates, reduced_dim=experts_dim)
  if importance is None:
    real_positions = float(group_size_dim.size)      # no padding mask: every position counts
  else:
    mean_prob *= mtf.to_float(mtf.equal(importance, 1.0))
    real_positions = mtf.to_float(mtf.reduce_sum(importance, reduced_dim=group_size_dim))
  loss = mtf.reduce_mean(mean_prob * mean_prob * real_positions) * float(group_size_dim.size)
  return _finish_router(combine_tensor, dispatch_tensor, loss, inputs)


# -------------------------------------------------------------- fused gating
class Top2GatingOperation(Operation):
  """Fused `_top_2_gating`: one kernel per slice instead of ~60 operations.

  inputs [O,G,S,M] and gate weights [M,E] -> per token: expert indices,
  slot positions (position >= capacity means dropped), gates after capacity
  and bf16 rounding semantics, and the per-slice sum over groups of the
  load-balancing loss.  Groups are independent, so any split of O or G over
  the mesh is slice-local; the loss is a LazyAllreduceSum over the mesh axes
  those dims are split over.
  """

  def __init__(self, inputs, gate_weights, experts_dim, capacity, policy, threshold,
               second_noise=None, name=None):
    xs = [inputs, gate_weights] + ([second_noise] if second_noise is not None else [])
    super().__init__(xs, name=name or "top_2_gating")
    token_shape = Shape(inputs.shape.dims[:-1])
    self._experts_dim = experts_dim
    self._capacity = capacity
    self._policy = policy
    self._threshold = threshold
    # output 7: the (expert, slot) -> token table of every group, which the
    # gating kernel has at hand and the dispatch would otherwise rebuild
    table_shape = Shape(inputs.shape.dims[:-2] + [experts_dim, Dimension("expert_capacity", capacity)])
    self._outputs = (
        [Tensor(self, token_shape, G.int32, index=i) for i in range(4)] +
        [Tensor(self, token_shape, G.float32, index=4), Tensor(self, token_shape, G.float32, index=5),
         Tensor(self, Shape([]), G.float32, index=6), Tensor(self, table_shape, G.int32, index=7)])

  # False differentiates the restated op chain instead of using MoeGateGradOperation
  fused_gradient = True

  @property
  def has_gradient(self):
    return True   # through the two gates and the loss; indices and positions carry none

  def gradient(self, grad_ys):
    """d(gate_1, gate_2, loss) / d(inputs, gate_weights): the routing decisions
    (indices, capacity masks) are constants, as in the reference, whose top_1
    gradient is a one-hot scatter (ops.py:4916-4920) and whose masks come out of
    comparisons; what remains is softmax -> picked gates -> renormalisation and
    the loss's mean-gate factor (moe.py:1384-1424, 1485-1494), rebuilt here from
    ordinary operations and differentiated."""
    x, w = self.inputs[0], self.inputs[1]
    i1, i2, _, _, g1_out, g2_out, _, _ = self.outputs
    experts_dim = self._experts_dim
    group_size_dim = x.shape.dims[-2]
    if experts_dim.size <= MoeGateGradOperation.MAX_EXPERTS and self.fused_gradient:
      # the same derivative as one operation between two einsums: logits again,
      # d logits from the kernel, then d inputs = d logits . W^T and d W = inputs^T . d logits
      xf = mtf.to_float(x)
      logits = layers.dense(xf, experts_dim, use_bias=False, kernel_weights=w, name="gate_grad")
      dlogits = MoeGateGradOperation(
          logits, i1, i2, g1_out, g2_out, grad_ys[4], grad_ys[5], grad_ys[6],
          num_groups_total=Shape(x.shape.dims[:-2]).size,
          top1_only=self._policy == "switch").outputs[0]
      dx = mtf.einsum([dlogits, w], output_shape=x.shape)
      dw = mtf.einsum([xf, dlogits], output_shape=w.shape)
      if dx.dtype != x.dtype:
        dx = mtf.cast(dx, x.dtype)
      return [dx, dw] + [None] * (len(self.inputs) - 2)

    def chain(x_, w_):
      raw = layers.dense(mtf.to_float(x_), experts_dim, use_bias=False, kernel_weights=w_,
                         name="gate_grad")
      raw = mtf.softmax(raw, experts_dim)
      m1 = mtf.one_hot(i1, experts_dim, dtype=raw.dtype)
      m2 = mtf.one_hot(i2, experts_dim, dtype=raw.dtype)
      g1 = mtf.reduce_sum(raw * m1, reduced_dim=experts_dim)
      g2 = mtf.reduce_sum(raw * m2, reduced_dim=experts_dim)
      keep1 = mtf.to_float(mtf.not_equal(g1_out, 0.0))
      keep2 = mtf.to_float(mtf.not_equal(g2_out, 0.0))
      density_1 = mtf.reduce_mean(m1, reduced_dim=group_size_dim)
      proxy = mtf.reduce_mean(raw, reduced_dim=group_size_dim)
      loss = mtf.reduce_mean(proxy * density_1) * float(experts_dim.size * experts_dim.size)
      if self._policy == "switch":        # top-1 routing keeps the raw gate
        return [g1 * keep1, g2 * 0.0, loss]
      denom = g1 + g2 + 1e-9
      return [g1 / denom * keep1, g2 / denom * keep2, loss]
    dx, dw = mtf.gradients_by_recompute([x, w], chain, [grad_ys[4], grad_ys[5], grad_ys[6]])
    if dx is not None and dx.dtype != x.dtype:
      dx = mtf.cast(dx, x.dtype)
    return [dx, dw] + [None] * (len(self.inputs) - 2)

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    ops = impl.slice_ops
    x, w = self.inputs[0], self.inputs[1]
    for d in (x.shape.dims[-2], x.shape.dims[-1], self._experts_dim):
      if impl.tensor_dimension_to_mesh_axis(d) is not None:
        raise ValueError("fused gating needs %s unsplit" % (d,))
    capacity, policy, threshold = self._capacity, self._policy, self._threshold
    num_groups_total = Shape(x.shape.dims[:-2]).size

    def fn(xs, ws, *noise):
      return ops.moe_top2_gating(xs, ws, capacity, policy, threshold,
                                 noise[0] if noise else None, num_groups_total, want_table=True)
    results = impl.slicewise(fn, *[lowering.tensors[t] for t in self.inputs])
    for out, value in zip(self.outputs[:6], results[:6]):
      lowering.set_tensor_lowering(out, value)
    lowering.set_tensor_lowering(self.outputs[7], results[7])
    layout = impl.tensor_layout(Shape(x.shape.dims[:-2]))
    mesh_axes = [a for a in layout.tensor_axis_to_mesh_axis if a is not None]
    loss = results[6]
    if mesh_axes and hasattr(impl, "allreduce_start"):
      # the sum over the other processors' groups starts now and is waited for by the
      # loss's first reader (the layer puts it after the combine), not here
      loss = impl.allreduce_start(loss, mesh_axes, "SUM")
    elif mesh_axes:
      loss = LazyAllreduceSum(impl, loss, mesh_axes)
    lowering.set_tensor_lowering(self.outputs[6], loss)


class MoeGateGradOperation(Operation):
  """d logits [.., S, E] of the gating from the gradients of gate_1, gate_2 [.., S] and
  of the loss (scalar), any of which may be missing: softmax backward of the picked and
  renormalised gates and of the loss's mean-gate factor, with the routing decisions as
  constants - what differentiating the op chain of moe.py:1384-1424, 1485-1494 gives,
  as one operation."""

  MAX_EXPERTS = 64

  def __init__(self, logits, i1, i2, g1_out, g2_out, dg1, dg2, dloss, num_groups_total, top1_only,
               name=None):
    self._present = [t is not None for t in (dg1, dg2, dloss)]
    super().__init__([logits, i1, i2, g1_out, g2_out] + [t for t in (dg1, dg2, dloss) if t is not None],
                     name=name or "moe_gate_grad")
    self._num_groups_total, self._top1_only = num_groups_total, top1_only
    self._outputs = [Tensor(self, logits.shape, G.float32)]

  @property
  def has_gradient(self):
    return False

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    logits = self.inputs[0]
    if impl.tensor_dimension_to_mesh_axis(logits.shape.dims[-1]) is not None or (
        impl.tensor_dimension_to_mesh_axis(logits.shape.dims[-2]) is not None):
      raise ValueError("the gating gradient needs the group and expert dims unsplit")
    ops = impl.slice_ops
    present, total, top1 = self._present, self._num_groups_total, self._top1_only

    def fn(z, a1, a2, g1, g2, *grads):
      it = iter(grads)
      dg1, dg2, dloss = [next(it) if p else None for p in present]
      return ops.moe_gate_grad(z, a1, a2, g1, g2, dg1, dg2, dloss, total, top1)
    lowering.set_tensor_lowering(
        self.outputs[0], impl.slicewise(fn, *[lowering.tensors[t] for t in self.inputs]))


class MoeDispatchOperation(Operation):
  """expert_inputs[O,E,G,C,M]: row gather replacing the dispatch einsum
  `inputs[O,G,S,M] x dispatch[O,G,S,E,C]` (moe.py:443-447)."""

  def __init__(self, inputs, routing, experts_dim, capacity_dim, slot_table=None, name=None):
    extra = [slot_table] if slot_table is not None else []
    super().__init__([inputs] + list(routing) + extra, name=name or "moe_dispatch")
    o, g, _, m = inputs.shape.dims
    self._num_experts = experts_dim.size
    self._capacity = capacity_dim.size
    self._outputs = [Tensor(self, Shape([o, experts_dim, g, capacity_dim, m]), inputs.dtype)]

  def gradient(self, grad_ys):
    """dx[g, s] = the sum of the gradient rows of the slots the token was copied
    to: a combine with unit gates.  The dispatch tensor itself comes from a cast
    to bool (moe.py:1510-1511), so nothing flows to the gates from here."""
    x = self.inputs[0]
    i1, i2, p1, p2, g1, g2 = self.inputs[1:7]
    # 1.0 where the gate, rounded to the activation type, is non-zero
    unit = lambda g: mtf.cast(mtf.cast(mtf.cast(g, x.dtype), G.bool_), G.float32)
    dx = MoeCombineOperation(grad_ys[0], [i1, i2, p1, p2, unit(g1), unit(g2)],
                             x.shape.dims[2]).outputs[0]
    return [dx] + [None] * (len(self.inputs) - 1)

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    ops = impl.slice_ops
    e, c = self._num_experts, self._capacity
    fn = lambda xs, i1, i2, p1, p2, g1, g2, *table: ops.moe_dispatch(
        xs, i1, i2, p1, p2, g1, g2, e, c, *table)
    lowering.set_tensor_lowering(
        self.outputs[0], impl.slicewise(fn, *[lowering.tensors[t] for t in self.inputs]))


class MoeCombineOperation(Operation):
  """output[O,G,S,M]: gated two-row gather replacing the combine einsum
  `expert_output[O,E,G,C,M] x combine[O,G,S,E,C]` (moe.py:509-510)."""

  def __init__(self, expert_output, routing, group_size_dim, name=None):
    super().__init__([expert_output] + list(routing), name=name or "moe_combine")
    o, _, g, _, m = expert_output.shape.dims
    self._outputs = [Tensor(self, Shape([o, g, group_size_dim, m]), expert_output.dtype)]

  def gradient(self, grad_ys):
    """Both transposes of the combine einsum: the expert-output gradient is a
    gate-weighted dispatch of dout, the gate gradients are per-token row dots."""
    y = self.inputs[0]
    routing = self.inputs[1:7]
    dy = MoeDispatchWeightedOperation(grad_ys[0], routing, y.shape.dims[1], y.shape.dims[3]).outputs[0]
    dg1, dg2 = MoeCombineGateGradOperation(y, grad_ys[0], routing).outputs
    return [dy, None, None, None, None, dg1, dg2]

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    ops = impl.slice_ops
    fn = lambda ys, i1, i2, p1, p2, g1, g2: ops.moe_combine(ys, i1, i2, p1, p2, g1, g2)
    lowering.set_tensor_lowering(
        self.outputs[0], impl.slicewise(fn, *[lowering.tensors[t] for t in self.inputs]))


class MoeDispatchWeightedOperation(Operation):
  """d(expert_output)[O,E,G,C,M] of MoeCombineOperation: slot (e, c) receives
  gate * dout[token in the slot] (the combine einsum's transpose, ops.py:2846-2854)."""

  def __init__(self, dout, routing, experts_dim, capacity_dim, name=None):
    super().__init__([dout] + list(routing), name=name or "moe_dispatch_weighted")
    o, g, _, m = dout.shape.dims
    self._num_experts = experts_dim.size
    self._capacity = capacity_dim.size
    self._outputs = [Tensor(self, Shape([o, experts_dim, g, capacity_dim, m]), dout.dtype)]

  @property
  def has_gradient(self):
    return False

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    ops = impl.slice_ops
    e, c = self._num_experts, self._capacity
    fn = lambda xs, i1, i2, p1, p2, g1, g2: ops.moe_dispatch_weighted(xs, i1, i2, p1, p2, g1, g2, e, c)
    lowering.set_tensor_lowering(
        self.outputs[0], impl.slicewise(fn, *[lowering.tensors[t] for t in self.inputs]))


class MoeCombineGateGradOperation(Operation):
  """d(gate_1), d(gate_2) [O,G,S] of MoeCombineOperation: <dout[s], y[i_k, p_k]>."""

  def __init__(self, expert_output, dout, routing, name=None):
    super().__init__([expert_output, dout] + list(routing), name=name or "moe_combine_gate_grad")
    token_shape = Shape(dout.shape.dims[:-1])
    self._outputs = [Tensor(self, token_shape, G.float32, index=0),
                     Tensor(self, token_shape, G.float32, index=1)]

  @property
  def has_gradient(self):
    return False

  def lower(self, lowering):
    impl = lowering.mesh_impl(self)
    ops = impl.slice_ops
    fn = lambda ys, d, i1, i2, p1, p2, g1, g2: ops.moe_combine_gate_grad(ys, d, i1, i2, p1, p2, g1, g2)
    d1, d2 = impl.slicewise(fn, *[lowering.tensors[t] for t in self.inputs])
    lowering.set_tensor_lowering(self.outputs[0], d1)
    lowering.set_tensor_lowering(self.outputs[1], d2)


# ------------------------------------------------------------------ the layer
def transformer_moe_layer_v1(inputs, output_dim, hparams, train, mesh_shape, layout,
                             gate_weights, wi, wo, second_noise=None, activation=mtf.relu,
                             return_aux=False, nonpadding=None):
  """Top-2 MoE feed-forward layer (moe.py:191-525).

  inputs: [<batch dims>, length, d_model]; gate_weights [d_model, experts_unsplit];
  wi [experts, d_model, hidden]; wo [experts, hidden, output_dim].  `mesh_shape`
  and `layout` are needed at graph-construction time to choose the number of
  groups, exactly as in the reference.
  """
  orig_inputs = inputs
  hidden_dim = wi.shape.dims[-1]
  experts_dim = wi.shape.dims[0]
  batch_and_length_dims, input_dim = orig_inputs.shape.dims[:-1], orig_inputs.shape.dims[-1]
  if orig_inputs.shape.dims[0].name == "outer_batch":
    outer_batch_dim, orig_batch_dim = orig_inputs.shape.dims[:2]
  else:
    outer_batch_dim, orig_batch_dim = Dimension("outer_batch", 1), orig_inputs.shape.dims[0]
  n = Shape(batch_and_length_dims).size // outer_batch_dim.size
  mesh_dim_size = tensor_dim_to_mesh_dim_size(layout, mesh_shape, orig_batch_dim)
  num_groups, group_size = _split_into_groups(n, hparams.moe_group_size, mesh_dim_size)
  group_size_dim = Dimension("group", group_size)
  num_groups_dim = Dimension(orig_batch_dim.name, num_groups)
  moe_input_dims = [outer_batch_dim, num_groups_dim, group_size_dim, input_dim]
  inputs = mtf.reshape(inputs, moe_input_dims)

  cf = hparams.moe_capacity_factor_train if train else hparams.moe_capacity_factor_eval
  capacity = expert_capacity(group_size, experts_dim.size, cf, hparams.moe_min_expert_capacity)
  capacity_dim = Dimension("expert_capacity", capacity)
  experts_dim_unsplit = Dimension("expert_unsplit", experts_dim.size)
  batch_dim_unsplit = Dimension("batch_unsplit", num_groups_dim.size)
  routers = ("top_2", "switch", "ntlb", "switch_max", "expert_selection")
  if hparams.moe_gating not in routers:
    raise ValueError("unknown hparams.moe_gating=%s" % hparams.moe_gating)
  if gate_weights.shape.dims[-1].name != experts_dim_unsplit.name:
    gate_weights = mtf.reshape(gate_weights, Shape([gate_weights.shape.dims[0], experts_dim_unsplit]))
  if second_noise is not None:
    second_noise = mtf.reshape(second_noise, moe_input_dims[:-1])
  elif hparams.moe_gating == "top_2" and _second_policy(hparams, train)[0] == "random":
    # the uniform draw of moe.py:1461-1465, one value per token
    second_noise = mtf.random_uniform(inputs.mesh, Shape(moe_input_dims[:-1]), dtype=G.float32)

  if nonpadding is not None:
    # ones for real positions, zeros for padding ([<batch dims>, length]): padding is not routed
    nonpadding = mtf.zeros(inputs.mesh, Shape(batch_and_length_dims), dtype=inputs.dtype) + nonpadding
    nonpadding = mtf.reshape(nonpadding, Shape(moe_input_dims[:-1]))
  aux = {}
  fused = (hparams.moe_use_fused_kernels and hparams.moe_gating in ("top_2", "switch")
           and nonpadding is None)
  switch = hparams.moe_gating == "switch"
  if switch:
    # the single-pass kernel serves plain argmax routing; perturbed gate inputs and the
    # router z-loss (which needs the logits) take the op chain
    switch_policy = hparams.moe_switch_policy_train if train else hparams.moe_switch_policy_eval
    plain = switch_policy == "argmax" or (switch_policy == "input_jitter" and not train)
    fused = fused and plain and not (train and hparams.moe_z_loss is not None)
  if fused and hparams.moe_use_second_place_loss:
    raise ValueError("moe_use_second_place_loss is not available with the fused kernels")
  if fused:
    policy, threshold = ("switch", 0.0) if switch else _second_policy(hparams, train)
    gating = Top2GatingOperation(inputs, gate_weights, experts_dim_unsplit, capacity, policy,
                                 threshold, second_noise=second_noise)
    i1, i2, p1, p2, g1, g2, loss_sum, slot_table = gating.outputs
    routing = [i1, i2, p1, p2, g1, g2]
    loss = None     # read at the end of the layer: its allreduce runs beside everything between
    aux = dict(index_1=i1, index_2=i2, position_1=p1, position_2=p2, gate_1=g1, gate_2=g2)
    expert_inputs = MoeDispatchOperation(inputs, routing, experts_dim_unsplit, capacity_dim,
                                         slot_table=slot_table).outputs[0]
  else:
    if hparams.moe_gating == "ntlb":
      dispatch_tensor, combine_tensor, loss = _ntlb_gating(
          inputs, experts_dim_unsplit, capacity_dim, hparams, train, gate_weights, importance=nonpadding)
    elif hparams.moe_gating == "switch_max":
      dispatch_tensor, combine_tensor, loss = _switch_max_gating(
          inputs, experts_dim_unsplit, capacity_dim, hparams, train, gate_weights, importance=nonpadding)
    elif hparams.moe_gating == "expert_selection":
      dispatch_tensor, combine_tensor, loss = _expert_selection_gating(
          inputs, experts_dim_unsplit, group_size_dim, capacity_dim, hparams, train, gate_weights,
          importance=nonpadding)
    elif switch:
      dispatch_tensor, combine_tensor, loss, aux = _switch_gating(
          inputs, experts_dim_unsplit, capacity_dim, hparams, train, gate_weights,
          importance=nonpadding)
    else:
      dispatch_tensor, combine_tensor, loss, aux = _top_2_gating(
          inputs, experts_dim_unsplit, capacity_dim, hparams, train, gate_weights,
          second_noise=second_noise, importance=nonpadding)
    aux = dict(aux, combine_tensor=combine_tensor, dispatch_tensor=dispatch_tensor)
    expert_inputs = mtf.einsum(
        [inputs, dispatch_tensor],
        Shape([outer_batch_dim, experts_dim_unsplit, num_groups_dim, capacity_dim, input_dim]))

  d_model_split_dim = Dimension("d_model_split", input_dim.size)
  expert_inputs = mtf.reshape(expert_inputs, Shape(
      [outer_batch_dim, experts_dim, batch_dim_unsplit, capacity_dim, d_model_split_dim]))
  # split over batch -> split over experts (an alltoall when both are split)
  expert_inputs = mtf.reshape(expert_inputs, Shape(
      [outer_batch_dim, experts_dim, batch_dim_unsplit, capacity_dim, input_dim]))

  h = layers.dense_product(expert_inputs, reduced_dims=expert_inputs.shape.dims[-1:],
                           new_dims=[hidden_dim], expert_dims=[experts_dim],
                           activation_functions=activation, use_bias=False,
                           kernel_weights=wi, name="wi")
  expert_output = layers.dense(h, output_dim, expert_dims=[experts_dim], use_bias=False,
                               reduced_dims=h.shape.dims[-1:], kernel_weights=wo, name="wo")
  expert_output = mtf.reshape(expert_output, Shape(
      [outer_batch_dim, experts_dim_unsplit, num_groups_dim, capacity_dim, d_model_split_dim]))
  # split over experts -> split over batch (the return alltoall)
  expert_output = mtf.reshape(expert_output, Shape(
      [outer_batch_dim, experts_dim_unsplit, num_groups_dim, capacity_dim, output_dim]))
  moe_output_dims = moe_input_dims[:-1] + [output_dim]
  if fused:
    output = MoeCombineOperation(expert_output, routing, group_size_dim).outputs[0]
  else:
    output = mtf.einsum([expert_output, combine_tensor], Shape(moe_output_dims))
  output = mtf.reshape(output, batch_and_length_dims + [output_dim])
  if loss is None:
    loss = mtf.cast(loss_sum, inputs.dtype)
  loss = loss * hparams.moe_loss_coef
  if return_aux:
    return output, loss, aux
  return output, loss


def transformer_moe_layer_v2(inputs, output_dim, hparams, train, mesh_shape, layout,
                             gate_weights_outer, gate_weights_inner, wi, wo, activation=mtf.relu,
                             nonpadding=None):
  """Two-level top-2 MoE feed-forward layer (moe.py:528-801).

  hparams.moe_num_experts = [x, y]: an outer router sends every position to up to two of
  x expert groups; inside each group an inner router (one per group) sends the positions
  that arrived to up to two of the group's y experts.  A slot of the outer level counts
  fully in the inner routing if a first choice filled it, half if a second choice did,
  and not at all if it stayed empty (the `importance` of `_top_2_gating`).

  inputs [outer_batch?, batch, length, d_model]; gate_weights_outer [d_model,
  expert_x_unsplit]; gate_weights_inner [expert_x, d_model, expert_y_unsplit];
  wi [expert_y, expert_x, d_model, hidden]; wo [expert_y, expert_x, hidden, output_dim].
  Four layout changes (alltoalls when the dims are split): groups -> expert_x,
  inner groups -> expert_y, and back.  `nonpadding` [<batch dims>, length] (ones for
  real positions, zeros for padding) keeps padding out of the outer routing.
  Returns (output, loss * moe_loss_coef).
  """
  if hparams.moe_gating != "top_2":
    raise ValueError("unknown hparams.moe_gating=%s" % hparams.moe_gating)
  if not isinstance(hparams.moe_num_experts, (list, tuple)) or len(hparams.moe_num_experts) != 2:
    raise ValueError("the two-level layer needs moe_num_experts = [x, y]")
  if nonpadding is not None:
    nonpadding = mtf.zeros(inputs.mesh, Shape(inputs.shape.dims[:-1]), dtype=inputs.dtype) + nonpadding
  insert_outer_batch_dim = inputs.shape.ndims == 3
  if insert_outer_batch_dim:
    inputs = mtf.reshape(inputs, Shape([Dimension("outer_batch", 1)] + inputs.shape.dims))
    if nonpadding is not None:
      nonpadding = mtf.reshape(nonpadding, Shape(inputs.shape.dims[:-1]))
  a0, b1, l, m = inputs.shape.dims
  x1 = Dimension("expert_x", hparams.moe_num_experts[0])
  y0 = Dimension("expert_y", hparams.moe_num_experts[1])
  x = Dimension("expert_x_unsplit", x1.size)
  y = Dimension("expert_y_unsplit", y0.size)
  n = output_dim

  # outer level: groups of the (batch, length) positions
  num_groups, group_size = _split_into_groups(
      b1.size * l.size, hparams.moe_group_size, tensor_dim_to_mesh_dim_size(layout, mesh_shape, b1))
  g1 = Dimension(b1.name, num_groups)
  g = Dimension(b1.name + "_unsplit", num_groups)
  s = Dimension("group_size_x", group_size)
  cf = hparams.moe_capacity_factor_train if train else hparams.moe_capacity_factor_eval
  c = Dimension("expert_capacity_x",
                expert_capacity(s.size, x.size, cf, hparams.moe_min_expert_capacity))
  # inner level: groups of the slots an expert group received
  num_groups, group_size = _split_into_groups(
      a0.size * g.size * c.size, hparams.moe_group_size,
      tensor_dim_to_mesh_dim_size(layout, mesh_shape, a0))
  t = Dimension("group_size_y", group_size)
  h0 = Dimension(a0.name, num_groups)
  h = Dimension(a0.name + "_unsplit", num_groups)
  d = Dimension("expert_capacity_y",
                expert_capacity(t.size, y.size, hparams.moe_capacity_factor_second_level,
                                hparams.moe_min_expert_capacity))

  def noise_for(shape):
    if _second_policy(hparams, train)[0] != "random":
      return None
    return mtf.random_uniform(inputs.mesh, shape, dtype=G.float32)

  inputs = mtf.reshape(inputs, Shape([a0, g1, s, m]))
  if nonpadding is not None:
    nonpadding = mtf.reshape(nonpadding, Shape([a0, g1, s]))
  dispatch_x, combine_x, loss_outer, _ = _top_2_gating(
      inputs, x, c, hparams, train, gate_weights_outer, second_noise=noise_for(Shape([a0, g1, s])),
      importance=nonpadding)
  # expert groups first: that is the dim the layout change splits
  expert_inputs_x = mtf.einsum([inputs, dispatch_x], Shape([x, a0, g1, c, m]))
  weight_in_slot = mtf.reduce_sum(combine_x, output_shape=Shape([x, a0, g1, c]))
  importance = 0.5 * (mtf.to_float(mtf.greater(weight_in_slot, 0.5))
                      + mtf.to_float(mtf.greater(weight_in_slot, 0.0)))
  expert_inputs_x = mtf.reshape(expert_inputs_x, Shape([x1, a0, g, c, m]))     # groups -> expert_x
  importance = mtf.reshape(importance, Shape([x1, a0, g, c]))

  inputs_y = mtf.reshape(expert_inputs_x, Shape([x1, h0, t, m]))
  importance = mtf.reshape(importance, Shape([x1, h0, t]))
  dispatch_y, combine_y, loss_inner, _ = _top_2_gating(
      inputs_y, y, d, hparams, train, gate_weights_inner, importance=importance,
      second_noise=noise_for(Shape([x1, h0, t])))
  expert_inputs_y = mtf.einsum([inputs_y, dispatch_y], Shape([y, x1, h0, d, m]))
  expert_inputs_y = mtf.reshape(expert_inputs_y, Shape([y0, x1, h, d, m]))     # inner groups -> expert_y

  hidden_dim = wi.shape.dims[-1]
  hidden = layers.dense(expert_inputs_y, hidden_dim, expert_dims=[y0, x1],
                        reduced_dims=expert_inputs_y.shape.dims[-1:], activation=activation,
                        use_bias=False, kernel_weights=wi, name="wi")
  expert_output = layers.dense(hidden, n, expert_dims=[y0, x1], reduced_dims=hidden.shape.dims[-1:],
                               use_bias=False, kernel_weights=wo, name="wo")

  # and back, level by level
  expert_output = mtf.reshape(expert_output, Shape([y, x1, h0, d, n]))         # expert_y -> inner groups
  output_y = mtf.einsum([expert_output, combine_y], Shape([x1, h0, t, n]))
  output = mtf.reshape(output_y, Shape([x1, a0, g, c, n]))
  expert_output_x = mtf.reshape(output, Shape([x, a0, g1, c, n]))              # expert_x -> groups
  output_x = mtf.einsum([expert_output_x, combine_x], Shape([a0, g1, s, n]))
  output = mtf.reshape(output_x, Shape([a0, b1, l, n]))
  if insert_outer_batch_dim:
    output = mtf.reshape(output, Shape([b1, l, n]))
  return output, (loss_outer + loss_inner) * hparams.moe_loss_coef
