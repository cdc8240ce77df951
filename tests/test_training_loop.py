"""A small language-model block trained for a few steps on the oracle backend: token
embedding (row gather), layer norm, causal multi-head attention, residual, the top-2 MoE
layer (fused gating / dispatch / combine operations and their backward operations), a
vocabulary-split softmax cross-entropy, Adafactor on variables that stay on the backend.
The whole path the boundary serves, forward and backward, on one processor and on a 2x2
mesh; the two must agree, the loss must fall, and a checkpoint must resume the run."""

import os

import numpy as np
import pytest

from mesh_b200 import mtf
from oracle.numpy_mesh_impl import NumpyMeshImpl
from helpers import rng

BATCH, LENGTH, D_MODEL, VOCAB, HEADS, D_KV, EXPERTS, D_FF = 4, 16, 16, 32, 2, 8, 4, 24


def _model(seed=3):
  """Graph of one training step; returns (graph, mesh, loss, variables)."""
  r = rng(seed)
  g = mtf.Graph()
  m = mtf.Mesh(g, "m")
  tokens = r.integers(0, VOCAB, size=(BATCH, LENGTH)).astype(np.int32)
  targets = np.roll(tokens, -1, axis=1)
  ids = mtf.import_tf_tensor(m, tokens, "batch:%d,length:%d" % (BATCH, LENGTH), dtype=mtf.int32)
  labels = mtf.import_tf_tensor(m, targets, "batch:%d,length:%d" % (BATCH, LENGTH), dtype=mtf.int32)
  var = lambda name, spec, scale: mtf.get_variable(
      m, name, spec, initial_value=(r.standard_normal(mtf.convert_to_shape(spec).to_integer_list)
                                    * scale).astype(np.float32))
  table = var("embedding", "vocab:%d,d_model:%d" % (VOCAB, D_MODEL), 1.0)
  wq, wk, wv, wo = [var("w" + n, "heads:%d,d_model:%d,d_kv:%d" % (HEADS, D_MODEL, D_KV), D_MODEL ** -0.5)
                    for n in "qkvo"]
  gate = var("gate", "d_model:%d,expert_unsplit:%d" % (D_MODEL, EXPERTS), D_MODEL ** -0.5)
  wi = var("wi", "experts:%d,d_model:%d,d_ff:%d" % (EXPERTS, D_MODEL, D_FF), D_MODEL ** -0.5)
  wo2 = var("wo2", "experts:%d,d_ff:%d,d_model:%d" % (EXPERTS, D_FF, D_MODEL), D_FF ** -0.5)
  softmax_w = var("softmax", "d_model:%d,vocab:%d" % (D_MODEL, VOCAB), D_MODEL ** -0.5)
  variables = [table, wq, wk, wv, wo, gate, wi, wo2, softmax_w]

  length, d_model, vocab = (mtf.Dimension(n, s) for n, s in
                            (("length", LENGTH), ("d_model", D_MODEL), ("vocab", VOCAB)))
  x = mtf.layers.embedding(ids, vocab, d_model, mtf.float32, table=table)
  h = mtf.layers.layer_norm(x, d_model)
  pos = mtf.mtf_range(m, length, mtf.float32)
  mask = mtf.layers.attention_mask_autoregressive(pos)
  x = x + mtf.layers.multihead_attention(h, None, mask, mtf.Dimension("d_kv", D_KV),
                                         mtf.Dimension("heads", HEADS), params=[wq, wk, wv, wo])
  hparams = mtf.moe.HParams(moe_group_size=LENGTH, moe_second_policy_train="all",
                            moe_capacity_factor_train=2.0)
  return g, m, x, hparams, gate, wi, wo2, softmax_w, labels, vocab, d_model, variables


def _training_graph(mesh_shape, layout):
  g, m, x, hparams, gate, wi, wo2, softmax_w, labels, vocab, d_model, variables = _model()
  y, aux_loss = mtf.moe.transformer_moe_layer_v1(
      mtf.layers.rms_norm(x, d_model), d_model, hparams, True, mesh_shape, layout, gate, wi, wo2)
  x = x + y
  logits = mtf.einsum([x, softmax_w], reduced_dims=[d_model])
  xent = mtf.layers.softmax_cross_entropy_with_logits(logits, labels, vocab)
  loss = mtf.reduce_mean(xent) + aux_loss
  grads = mtf.gradients([loss], variables)
  assert all(gr is not None for gr in grads)
  mtf.optimize.AdafactorOptimizer(learning_rate=0.05, min_dim_size_to_factor=8).apply_grads(grads, variables)
  return g, m, loss, variables


def _train(mesh_shape, layout, steps):
  g, m, loss, variables = _training_graph(mesh_shape, layout)
  impl = NumpyMeshImpl(mesh_shape, layout)
  losses = []
  for _ in range(steps):
    low = mtf.Lowering(g, {m: impl})
    losses.append(float(low.export_to_tf_tensor(loss)))
  return losses, low, variables, g, m, impl, loss


def test_block_trains_and_agrees_across_meshes():
  one, *_ = _train("all:1", "", 6)
  split, *_ = _train("rows:2,cols:2", "batch:rows;experts:rows;heads:cols;vocab:cols", 6)
  assert one[-1] < one[0] - 0.05, one
  np.testing.assert_allclose(split, one, rtol=2e-4)


def test_checkpoint_resumes_the_run(tmp_path):
  mesh_shape, layout = "rows:2,cols:2", "batch:rows;experts:rows;heads:cols;vocab:cols"
  straight, *_ = _train(mesh_shape, layout, 5)
  losses, low, variables, g, m, impl, loss = _train(mesh_shape, layout, 3)
  path = os.path.join(str(tmp_path), "block.npz")
  everything = list(g.all_variables)                    # weights and optimizer slots
  mtf.save_checkpoint(path, everything, lowering=low)
  # a fresh process: same graph, masters from the file
  g2, m2, loss2, _ = _training_graph(mesh_shape, layout)
  mtf.restore_checkpoint(path, list(g2.all_variables))
  impl2 = NumpyMeshImpl(mesh_shape, layout)
  resumed = [float(mtf.Lowering(g2, {m2: impl2}).export_to_tf_tensor(loss2)) for _ in range(2)]
  np.testing.assert_allclose(losses + resumed, straight, rtol=2e-5)
