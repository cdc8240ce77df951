"""The timed CPU arm: the reference's lowering of the benchmark layers on host cores.

TEST / MEASUREMENT INFRASTRUCTURE ONLY (see oracle/__init__.py).

The reference cannot be installed here (TensorFlow is absent), so what is timed
is its restatement: the same graphs lowered on NumpyMeshImpl — list-of-slices
PlacementMeshImpl semantics — with float32 contractions on all host threads.
"""

from __future__ import annotations

import os
import time

import numpy as np

from mesh_b200 import mtf
from oracle.numpy_mesh_impl import NumpyMeshImpl


def host_threads():
  import torch
  n = os.cpu_count() or 1
  torch.set_num_threads(n)
  return n


def ffn_inputs(batch, length, d_model, d_ff, seed):
  """Seeded synthetic inputs of the dense_relu_dense configuration:
  x ~ N(0,1), wi ~ N(0, 1/d_model), wo ~ N(0, 1/d_ff), float32 on the host."""
  r = np.random.Generator(np.random.PCG64(seed))
  x = r.standard_normal((batch, length, d_model), dtype=np.float32)
  wi = r.standard_normal((d_model, d_ff), dtype=np.float32) * np.float32(d_model ** -0.5)
  wo = r.standard_normal((d_ff, d_model), dtype=np.float32) * np.float32(d_ff ** -0.5)
  return x, wi, wo


def build_ffn_graph(x, wi, wo, dtype):
  g = mtf.Graph()
  mesh = mtf.Mesh(g, "mesh")
  b, l, d = x.shape
  f = wi.shape[1]
  X = mtf.import_tf_tensor(mesh, x, "batch:%d,length:%d,d_model:%d" % (b, l, d), dtype=dtype)
  WI = mtf.import_tf_tensor(mesh, wi, "d_model:%d,d_ff:%d" % (d, f), dtype=dtype)
  WO = mtf.import_tf_tensor(mesh, wo, "d_ff:%d,d_model:%d" % (f, d), dtype=dtype)
  y = mtf.layers.dense_relu_dense(X, mtf.Dimension("d_ff", f), wi=WI, wo=WO)
  return g, mesh, y


def ffn_flops(batch, length, d_model, d_ff):
  return 2.0 * batch * length * d_model * d_ff * 2.0


def time_ffn(batch, length, d_model, d_ff, mesh_shape, layout, steps, warmup, seed=1235):
  """Seconds per lowering of the FFN graph on the CPU backend (median of `steps`)."""
  x, wi, wo = ffn_inputs(batch, length, d_model, d_ff, seed)
  g, mesh, y = build_ffn_graph(x, wi, wo, mtf.bfloat16)
  impl = NumpyMeshImpl(mesh_shape, layout, fast=True)
  times = []
  for i in range(warmup + steps):
    t0 = time.perf_counter()
    low = mtf.Lowering(g, {mesh: impl})
    low.tensors[y].to_laid_out_tensor()
    dt = time.perf_counter() - t0
    if i >= warmup:
      times.append(dt)
  return float(np.median(times)), times


def time_moe(x, wg, wi, wo, group_size, steps, warmup):
  """Seconds per lowering (median of `steps`) of the reference's own op chain
  for the top-2 MoE layer on the CPU backend: softmax, two top_1, triangular
  cumsum, dense [G,S,E,C] dispatch / combine tensors and their dense einsums
  (what transformer_moe_layer_v1, transformer/moe.py:191-525, costs the
  reference).  x [groups, length, d_model]; wi [E, d_model, d_ff]; wo [E, d_ff, d_model]."""
  b, l, m = x.shape
  e, _, h = wi.shape
  g = mtf.Graph()
  mesh = mtf.Mesh(g, "mesh")
  X = mtf.import_tf_tensor(mesh, x, "batch:%d,length:%d,d_model:%d" % (b, l, m), dtype=mtf.bfloat16)
  WG = mtf.import_tf_tensor(mesh, wg, "d_model:%d,expert_unsplit:%d" % (m, e), dtype=mtf.float32)
  WI = mtf.import_tf_tensor(mesh, wi, "experts:%d,d_model:%d,d_ff:%d" % (e, m, h), dtype=mtf.bfloat16)
  WO = mtf.import_tf_tensor(mesh, wo, "experts:%d,d_ff:%d,d_model:%d" % (e, h, m), dtype=mtf.bfloat16)
  hp = mtf.moe.HParams(moe_group_size=group_size, moe_second_policy_train="all",
                       moe_use_fused_kernels=False)
  out, _ = mtf.moe.transformer_moe_layer_v1(X, mtf.Dimension("d_model", m), hp, True, "", "", WG, WI, WO)
  impl = NumpyMeshImpl("", "", fast=True)
  times = []
  for i in range(warmup + steps):
    t0 = time.perf_counter()
    mtf.Lowering(g, {mesh: impl}).tensors[out].to_laid_out_tensor()
    dt = time.perf_counter() - t0
    if i >= warmup:
      times.append(dt)
  return float(np.median(times)), times
