"""Optimizers as graph operations: SGD and Adafactor.

Follows mesh_tensorflow/optimize.py (Optimizer 38-66, SgdOptimizer 69-93,
AdafactorOptimizer 207-390): `apply_grads` adds, for every (gradient,
variable) pair, the operations that update the variable and its slots, built
from ordinary mtf operations, so the update runs slice by slice on whatever
backend lowers the graph and the slots live there as variables.  Learning
rate and decay rate are numbers fixed when the graph is built (the reference
derives its defaults from TensorFlow's global step); `adafactor_decay_rate_pow`
and `adafactor_learning_rate` give the reference's default schedules for a
given step.
"""

from __future__ import annotations

import numpy as np

from mesh_b200.mtf import graph as G
from mesh_b200.mtf import ops as mtf
from mesh_b200.mtf.shapes import Shape


def reduce_rms(x, **kwargs):
  """sqrt(mean(x^2)) (optimize.py:30-31)."""
  return mtf.sqrt(mtf.reduce_mean(mtf.square(x), **kwargs))


def adafactor_decay_rate_pow(step, exponent=0.8):
  """1 - (step + 1)^-exponent (optimize.py:411-420)."""
  return 1.0 - float(step + 1.0) ** -exponent


def adafactor_decay_rate_adam(step, beta2):
  """Adam-style bias-corrected second-moment decay (optimize.py:393-408)."""
  t = float(step) + 1.0
  return beta2 * (1.0 - beta2 ** (t - 1.0)) / (1.0 - beta2 ** t)


def adafactor_learning_rate(step, multiply_by_parameter_scale=True):
  """min(rsqrt(step + 1), 0.01), times 0.05 without parameter scaling (optimize.py:381-388)."""
  rate = min((float(step) + 1.0) ** -0.5, 0.01)
  return rate if multiply_by_parameter_scale else rate * 0.05


class Optimizer(object):
  """Base class (optimize.py:38-66)."""

  def apply_grads(self, grads, variables):
    ops = []
    for grad, var in zip(grads, variables):
      ops.extend(self.apply_grad(grad, var))
    return ops

  def apply_grad(self, grad, var):
    raise NotImplementedError


def _variable_op(var):
  return var.operation if isinstance(var, G.Tensor) else var


class SgdOptimizer(Optimizer):
  """var -= learning_rate * grad (optimize.py:69-93)."""

  def __init__(self, learning_rate, copy_to_master=False):
    self._lr = learning_rate
    self._copy = copy_to_master

  def apply_grad(self, grad, var):
    if grad is None:
      return []
    var = _variable_op(var)
    return [mtf.assign_sub(var, grad * self._lr, copy_to_master=self._copy)]


class AdafactorOptimizer(Optimizer):
  """Adafactor (optimize.py:207-390): second moments factored into row and
  column means for variables with two dims of at least `min_dim_size_to_factor`,
  update clipping by root-mean-square, and steps proportional to the scale
  of the parameters."""

  def __init__(self, multiply_by_parameter_scale=True, learning_rate=None, decay_rate=None,
               beta1=0.0, clipping_threshold=1.0, factored=True, epsilon1=1e-30, epsilon2=1e-3,
               min_dim_size_to_factor=128, stacked_dim_names=None,
               exclude_from_parameter_scale=None, step=0, copy_to_master=False):
    self._multiply_by_parameter_scale = multiply_by_parameter_scale
    if learning_rate is None:
      learning_rate = adafactor_learning_rate(step, multiply_by_parameter_scale)
    self._learning_rate = learning_rate
    if decay_rate is None:
      decay_rate = adafactor_decay_rate_pow(step)
    self._decay_rate = decay_rate
    self._beta1 = beta1
    self._clipping_threshold = clipping_threshold
    self._factored = factored
    self._epsilon1 = epsilon1
    self._epsilon2 = epsilon2
    self._min_dim_size_to_factor = min_dim_size_to_factor
    self._stacked_dim_names = stacked_dim_names or []
    self._exclude_from_parameter_scale = exclude_from_parameter_scale or []
    self._copy = copy_to_master

  def _factored_dims(self, shape):
    """The two largest dims if both reach min_dim_size_to_factor, else None (optimize.py:270-292)."""
    if not self._factored:
      return None
    dims = [d for d in shape.dims if d.name not in self._stacked_dim_names]
    if len(dims) < 2:
      return None
    sorted_dims = sorted(dims, key=lambda d: -d.size)
    if sorted_dims[1].size < self._min_dim_size_to_factor:
      return None
    return sorted_dims[:2]

  def _parameter_scale(self, value):
    output_shape = Shape([d for d in value.shape.dims if d.name in self._stacked_dim_names])
    return mtf.maximum(reduce_rms(value, output_shape=output_shape), self._epsilon2)

  def _slot(self, var, suffix, shape):
    return mtf.get_variable(var.mesh, var.name + suffix, shape, dtype=G.float32,
                            initial_value=np.zeros(shape.to_integer_list, np.float32),
                            trainable=False).operation

  def apply_grad(self, grad, var):
    if grad is None:
      return []
    var = _variable_op(var)
    value = var.outputs[0]
    grad = mtf.to_float(grad)
    factored_dims = self._factored_dims(value.shape)
    if factored_dims:
      d0, d1 = factored_dims
      vr_shape, vc_shape = value.shape - d0, value.shape - d1
      vr, vc = self._slot(var, "_slot_vr", vr_shape), self._slot(var, "_slot_vc", vc_shape)
    else:
      v = self._slot(var, "_slot_v", value.shape)
    if self._beta1:
      m = self._slot(var, "_slot_m", value.shape)
    grad_squared = mtf.square(grad) + self._epsilon1
    decay_rate = self._decay_rate
    old_val = mtf.to_float(value)
    if self._multiply_by_parameter_scale and not any(
        s in var.name for s in self._exclude_from_parameter_scale):
      update_scale = self._parameter_scale(old_val) * self._learning_rate
    else:
      update_scale = self._learning_rate
    mixing_rate = 1.0 - decay_rate
    updates = []
    if factored_dims:
      grad_squared_row_mean = mtf.reduce_mean(grad_squared, output_shape=vr_shape)
      grad_squared_col_mean = mtf.reduce_mean(grad_squared, output_shape=vc_shape)
      new_vr = vr.outputs[0] * decay_rate + grad_squared_row_mean * mixing_rate
      new_vc = vc.outputs[0] * decay_rate + grad_squared_col_mean * mixing_rate
      updates.append(mtf.assign(vr, new_vr, copy_to_master=self._copy))
      updates.append(mtf.assign(vc, new_vc, copy_to_master=self._copy))
      long_term_mean = mtf.reduce_mean(new_vr, reduced_dim=d1)
      r_factor = mtf.rsqrt(new_vr / long_term_mean)
      c_factor = mtf.rsqrt(new_vc)
      x = grad * r_factor * c_factor
    else:
      new_v = v.outputs[0] * decay_rate + grad_squared * mixing_rate
      updates.append(mtf.assign(v, new_v, copy_to_master=self._copy))
      x = grad * mtf.rsqrt(new_v)
    if self._clipping_threshold is not None:
      clipping_denom = mtf.maximum(reduce_rms(x) / self._clipping_threshold, 1.0)
      x = x / clipping_denom
    subtrahend = x * update_scale
    if self._beta1:
      new_m = m.outputs[0] * self._beta1 + subtrahend * (1.0 - self._beta1)
      subtrahend = new_m
      updates.append(mtf.assign(m, new_m, copy_to_master=self._copy))
    # subtract in place of assigning var - subtrahend computed elsewhere: the slice
    # value is rounded once per step, which matters for bfloat16 variables
    updates.append(mtf.assign_sub(var, subtrahend, copy_to_master=self._copy))
    return updates
