"""Per-configuration measurements beside bench.py's headline line.

  python -m mesh_b200.bench_configs --config moe|einsum_fp32|attention|collectives|ffn_train [--gpus N]

Each configuration prints JSON lines (one per measured quantity) with the
algorithmic bytes or flops it was divided by, so roofline fractions can be
checked by hand.  Inputs are seeded synthetic tensors of the configuration's
shapes.  Timing: CUDA events on the launching stream, warm-up first, inputs
larger than L2 or an L2 flush (a 256 MiB fill) between iterations.
Multi-GPU configurations are launched with torch.distributed.run, one process
per GPU, and report the maximum over ranks.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import numpy as np
import torch

from mesh_b200 import _native as nat
from mesh_b200 import mtf
from mesh_b200.cuda_mesh_impl import CudaMeshImpl


def _peaks():
  root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
  path = os.path.join(root, "MEASURED_PEAKS.json")
  if os.path.exists(path):
    p = json.load(open(path))
    return {"hbm_gbs": p["hbm_gbs"], "tflops": p["bf16_tflops_sustained"], "source": "measured"}
  return {"hbm_gbs": 6650.0, "tflops": 1400.0, "source": "fallback"}


class _Flusher(object):
  """Evicts L2 by writing a buffer larger than it (through the library's fill kernel)."""

  def __init__(self, ops):
    self._ops = ops
    self._n = 64 * 1024 * 1024

  def __call__(self):
    self._ops.fill([self._n], 0.0, mtf.float32)


def _time(fn, iters=10, warmup=3, flush=None):
  for _ in range(warmup):
    fn()
  torch.cuda.synchronize()
  times = []
  for _ in range(iters):
    if flush is not None:
      flush()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    times.append(e0.elapsed_time(e1))
  return statistics.median(times)


def _leave(dist_module=None):
  """Ends a multi-rank run: barrier, flush, exit.  Recorded CUDA graphs holding
  NCCL kernels make the process-group destructor wait forever, so the ranks
  leave without tearing NCCL down once nothing is in flight."""
  import torch.distributed as dist
  dist.barrier()
  torch.cuda.synchronize()
  sys.stdout.flush()
  sys.stderr.flush()
  os._exit(0)


def _emit(**kw):
  print(json.dumps(kw), flush=True)


def config_moe(args):
  """Top-2 MoE layer: 65536 tokens in groups of 1024, d_model 1024, 32 experts,
  d_ff 4096, capacity factor 1.25 (capacity 40), bf16, policy "all"."""
  peaks = _peaks()
  n = args.gpus
  rank = int(os.environ.get("RANK", "0"))
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local_rank)
  if n > 1:
    import torch.distributed as dist
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
  B, L, M, E, H = 64, 1024, 1024, 32, 4096
  mesh_shape, layout = "all:%d" % n, "batch:all;experts:all"
  impl = CudaMeshImpl(mesh_shape, layout, list(range(n)) if n > 1 else [local_rank], distributed=n > 1)
  ops = impl.slice_ops
  r = np.random.Generator(np.random.PCG64(1236))
  b_loc, e_loc = B // n, E // n
  x = torch.from_numpy(r.standard_normal((b_loc, L, M), dtype=np.float32)).to(torch.bfloat16)
  wg = r.standard_normal((M, E), dtype=np.float32) * np.float32(M ** -0.5)
  wi = torch.from_numpy(r.standard_normal((e_loc, M, H), dtype=np.float32) * np.float32(M ** -0.5)).to(torch.bfloat16)
  wo = torch.from_numpy(r.standard_normal((e_loc, H, M), dtype=np.float32) * np.float32(H ** -0.5)).to(torch.bfloat16)
  lx = impl.LaidOutTensor([ops.from_host(x, mtf.bfloat16)])
  lwg = impl.LaidOutTensor([ops.from_host(wg, mtf.float32)])
  lwi = impl.LaidOutTensor([ops.from_host(wi, mtf.bfloat16)])
  lwo = impl.LaidOutTensor([ops.from_host(wo, mtf.bfloat16)])

  g = mtf.Graph()
  mesh = mtf.Mesh(g, "mesh")
  X = mtf.import_laid_out_tensor(mesh, lx, "batch:%d,length:%d,d_model:%d" % (B, L, M), mtf.bfloat16)
  WG = mtf.import_laid_out_tensor(mesh, lwg, "d_model:%d,expert_unsplit:%d" % (M, E), mtf.float32)
  WI = mtf.import_laid_out_tensor(mesh, lwi, "experts:%d,d_model:%d,d_ff:%d" % (E, M, H), mtf.bfloat16)
  WO = mtf.import_laid_out_tensor(mesh, lwo, "experts:%d,d_ff:%d,d_model:%d" % (E, H, M), mtf.bfloat16)
  hp = mtf.moe.HParams(moe_group_size=1024, moe_second_policy_train="all")
  out, loss = mtf.moe.transformer_moe_layer_v1(
      X, mtf.Dimension("d_model", M), hp, True, mesh_shape, layout, WG, WI, WO)

  def step():
    low = mtf.Lowering(g, {mesh: impl})
    return low.tensors[out].to_laid_out_tensor()

  before = nat.launch_count()
  step()
  launches = nat.launch_count() - before
  impl.synchronize()
  run = step
  if not args.eager:
    _, run = impl.capture(step)
  ms = _time(run, iters=args.iters, warmup=3)
  if n > 1:
    import torch.distributed as dist
    t = torch.tensor([ms], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
  tokens = B * L
  expert_flops = 2.0 * (E * (B * L // 1024) * 40) * M * H * 2.0
  if rank == 0:
    _emit(config="moe", quantity="layer", n_gpus=n, tokens=tokens, ms=ms,
          tokens_per_s=tokens / (ms * 1e-3), expert_tflops=expert_flops / (ms * 1e-3) / 1e12,
          libmtfc_launches_per_step=launches,
          stepping="eager" if args.eager else "cuda-graph replay")

  # per-kernel times on this rank's slice (groups are independent)
  xs = ops.reshape(lx.tensor_list[0], [1, b_loc * L // 1024, 1024, M])
  G, S, C = xs.shape[1], 1024, 40
  flush = _Flusher(ops)
  w = lwg.tensor_list[0]
  logits, parts = ops.moe_gate_logits(xs, w)
  t_logits = _time(lambda: ops.moe_gate_logits(xs, w), flush=flush)
  routing = ops.moe_top2_gating_from_logits(logits, parts, xs.shape[:2], S, E, C, "all", 0.2, None, G)
  t_gate = _time(lambda: ops.moe_top2_gating_from_logits(logits, parts, xs.shape[:2], S, E, C, "all",
                                                         0.2, None, G), flush=flush)
  i1, i2, p1, p2, g1, g2, _ = routing
  disp = ops.moe_dispatch(xs, i1, i2, p1, p2, g1, g2, E, C)
  t_disp = _time(lambda: ops.moe_dispatch(xs, i1, i2, p1, p2, g1, g2, E, C), flush=flush)
  t_comb = _time(lambda: ops.moe_combine(disp, i1, i2, p1, p2, g1, g2), flush=flush)
  tok = G * S
  kept = float(np.mean(ops.to_host(g1) != 0) + np.mean(ops.to_host(g2) != 0))
  rows = [
      ("gate_logits (tcgen05 GEMM, N=3E)", t_logits, tok * (2 * M + 4 * 3 * E)),
      ("top2_gating", t_gate, tok * (4 * 3 * E + 24)),
      ("dispatch (slot_table + rows)", t_disp, tok * (kept * 2 * M + (E * C / S) * 2 * M + 24)),
      ("combine", t_comb, tok * (kept * 2 * M + 2 * M + 24)),
  ]
  if rank == 0:
    for name, t, nbytes in rows:
      gbs = nbytes / (t * 1e-3) / 1e9
      _emit(config="moe", quantity=name, n_gpus=n, tokens_on_rank=tok, ms=t, algorithmic_bytes=nbytes,
            gb_per_s=gbs, frac_of_hbm_peak=gbs / peaks["hbm_gbs"], peak_gbs=peaks["hbm_gbs"],
            peak_source=peaks["source"], kept_choices_per_token=kept)
  if n > 1:
    _leave(dist_module=None)


def config_ffn_train(args):
  """Forward and backward of the dense FFN (x[64,1024,1024], wi[1024,4096],
  wo[4096,1024], bf16) on one GPU: y, then dx, dwi, dwo from a given dy through
  mtf.gradients - three GEMM pairs with permuted operand roles and the ReLU
  mask, lowered onto the same kernels and replayed as a CUDA graph."""
  peaks = _peaks()
  torch.cuda.set_device(0)
  impl = CudaMeshImpl("all:1", "", [0])
  ops = impl.slice_ops
  b, l, d, f = 64, 1024, 1024, 4096
  r = np.random.Generator(np.random.PCG64(1238))

  def laid(shape, scale):
    t = torch.from_numpy(r.standard_normal(shape, dtype=np.float32) * np.float32(scale)).to(torch.bfloat16)
    return impl.LaidOutTensor([ops.from_host(t, mtf.bfloat16)])
  lx, ldy = laid((b, l, d), 1.0), laid((b, l, d), 1.0)
  lwi, lwo = laid((d, f), d ** -0.5), laid((f, d), f ** -0.5)
  g = mtf.Graph()
  mesh = mtf.Mesh(g, "mesh")
  act = "batch:%d,length:%d,d_model:%d" % (b, l, d)
  X = mtf.import_laid_out_tensor(mesh, lx, act, mtf.bfloat16)
  DY = mtf.import_laid_out_tensor(mesh, ldy, act, mtf.bfloat16)
  WI = mtf.import_laid_out_tensor(mesh, lwi, "d_model:%d,d_ff:%d" % (d, f), mtf.bfloat16)
  WO = mtf.import_laid_out_tensor(mesh, lwo, "d_ff:%d,d_model:%d" % (f, d), mtf.bfloat16)
  y = mtf.layers.dense_relu_dense(X, mtf.Dimension("d_ff", f), wi=WI, wo=WO)
  grads = mtf.gradients([y], [X, WI, WO], grad_ys=[DY])

  def step():
    low = mtf.Lowering(g, {mesh: impl})
    return [low.tensors[t].to_laid_out_tensor() for t in [y] + grads]
  before = nat.launch_count()
  step()
  launches = nat.launch_count() - before
  impl.synchronize()
  run = step
  if not args.eager:
    _, run = impl.capture(step)
  ms = _time(run, iters=args.iters, warmup=3)
  flops = 3 * 2.0 * 2.0 * b * l * d * f     # forward + two gradient GEMMs per forward GEMM
  _emit(config="ffn_train", quantity="dense_relu_dense forward + backward (dx, dwi, dwo)", ms=ms,
        tflops=flops / (ms * 1e-3) / 1e12, frac_of_peak=flops / (ms * 1e-3) / 1e12 / peaks["tflops"],
        peak_tflops=peaks["tflops"], peak_source=peaks["source"], libmtfc_launches_per_step=launches,
        stepping="eager" if args.eager else "cuda-graph replay")


def config_einsum_fp32(args):
  """x[4096,1024] . w[1024,4096] in fp32 (one GPU: the whole problem)."""
  torch.cuda.set_device(0)
  impl = CudaMeshImpl("all:1", "", [0])
  ops = impl.slice_ops
  r = np.random.Generator(np.random.PCG64(1234))
  x = ops.from_host(r.standard_normal((4096, 1024), dtype=np.float32), mtf.float32)
  w = ops.from_host(r.standard_normal((1024, 4096), dtype=np.float32) / 32, mtf.float32)
  ms = _time(lambda: ops.einsum("ab,bc->ac", x, w), flush=_Flusher(ops))
  _emit(config="einsum_fp32", quantity="x[4096,1024].w[1024,4096]", ms=ms,
        tflops=2.0 * 4096 * 1024 * 4096 / (ms * 1e-3) / 1e12, kernel="split_bf16x3 x2 + einsum_gemm_tcgen05 over 6K")


def config_attention(args):
  """Multi-head attention: x[batch,2048,4096] bf16, 32 heads of 128, causal;
  q/k/v projections, fused attention kernel, output projection; inputs and
  weights resident, the lowering replayed as a CUDA graph.  With --gpus N the
  heads are split over a 1-D mesh (layout heads:all): every rank holds the whole
  x, its own heads' weights, and the output projection ends in an allreduce."""
  peaks = _peaks()
  n = args.gpus
  rank = int(os.environ.get("RANK", "0"))
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local_rank)
  if n > 1:
    import torch.distributed as dist
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
  mesh_shape, layout = "all:%d" % n, ("heads:all" if n > 1 else "")
  impl = CudaMeshImpl(mesh_shape, layout, list(range(n)) if n > 1 else [local_rank], distributed=n > 1)
  ops = impl.slice_ops
  b, l, d, h, kv = args.attention_batch, 2048, 4096, 32, 128
  h_loc = h // n
  r = np.random.Generator(np.random.PCG64(1237))
  x = torch.from_numpy(r.standard_normal((b, l, d), dtype=np.float32)).to(torch.bfloat16)
  lx = impl.LaidOutTensor([ops.from_host(x, mtf.bfloat16)])
  stds = [d ** -0.5 * kv ** -0.25] * 2 + [d ** -0.5, (d * h) ** -0.5]
  lws = []
  for sd in stds:
    w = r.standard_normal((h, d, kv), dtype=np.float32) * np.float32(sd)
    w = w[rank * h_loc:(rank + 1) * h_loc]
    lws.append(impl.LaidOutTensor([ops.from_host(torch.from_numpy(np.ascontiguousarray(w)).to(torch.bfloat16),
                                                 mtf.bfloat16)]))
  g = mtf.Graph()
  mesh = mtf.Mesh(g, "mesh")
  X = mtf.import_laid_out_tensor(mesh, lx, "batch:%d,length:%d,d_model:%d" % (b, l, d), mtf.bfloat16)
  heads, kvd = mtf.Dimension("heads", h), mtf.Dimension("d_kv", kv)
  params = [mtf.import_laid_out_tensor(mesh, w, "heads:%d,d_model:%d,d_kv:%d" % (h, d, kv), mtf.bfloat16)
            for w in lws]
  pos = mtf.mtf_range(mesh, X.shape.dims[1], mtf.float32)
  mask = mtf.layers.attention_mask_autoregressive(pos)
  y = mtf.layers.multihead_attention(X, None, mask, kvd, heads, params=params)

  def step():
    return mtf.Lowering(g, {mesh: impl}).tensors[y].to_laid_out_tensor()
  before = nat.launch_count()
  step()
  launches = nat.launch_count() - before
  impl.synchronize()
  run = step
  if not args.eager:
    _, run = impl.capture(step)
  ms = _time(run, iters=args.iters, warmup=3)
  if n > 1:
    t = torch.tensor([ms], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
  proj = 4 * 2.0 * b * l * d * h * kv
  attn_full = 2 * 2.0 * b * h * l * l * kv
  if rank == 0:
    _emit(config="attention", quantity="multihead_attention layer (fused kernel)", n_gpus=n, batch=b, ms=ms,
          tflops_full=(proj + attn_full) / (ms * 1e-3) / 1e12,
          tflops_causal_work=(proj + attn_full / 2 * (1 + 128.0 / l)) / (ms * 1e-3) / 1e12,
          allreduce_bytes_per_gpu=(b * l * d * 2 if n > 1 else 0),
          libmtfc_launches_per_step=launches, peak_tflops=peaks["tflops"], peak_source=peaks["source"],
          stepping="eager" if args.eager else "cuda-graph replay")
  if n > 1:
    _leave(dist_module=None)
  # the fused kernel alone on q, k, v [batch, heads, length, d_kv]
  q, k, v = [ops.from_host(torch.from_numpy(
      r.standard_normal((b, h, l, kv), dtype=np.float32) * np.float32(0.3)).to(torch.bfloat16), mtf.bfloat16)
             for _ in range(3)]
  for causal in (True, False):
    t = _time(lambda: ops.attention(q, k, v, causal), iters=args.iters, warmup=3)
    work = attn_full * ((0.5 * (1 + 128.0 / l)) if causal else 1.0)
    _emit(config="attention", quantity="attn_fwd_tcgen05 alone", causal=causal, batch=b, ms=t,
          tflops_executed=work / (t * 1e-3) / 1e12,
          frac_of_peak=work / (t * 1e-3) / 1e12 / peaks["tflops"])


def config_collectives(args):
  """allreduce / allconcat / alltoall bus bandwidth on a 1-D mesh of --gpus GPUs."""
  import torch.distributed as dist
  n = args.gpus
  rank = int(os.environ.get("RANK", "0"))
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local_rank)
  dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
  impl = CudaMeshImpl("all:%d" % n, "", list(range(n)), distributed=True)
  ops = impl.slice_ops
  for dtype in (mtf.bfloat16, mtf.float32):
    for k in range(0, 11):
      nbytes = 1024 * 4 ** k
      if nbytes > args.max_bytes:
        break
      elems = nbytes // dtype.itemsize
      xs = impl.LaidOutTensor([ops.fill([n, elems // n], 0.5, dtype)])
      for name, fn, factor in (
          ("allreduce", lambda: impl.allreduce(xs, [0], "SUM"), 2.0 * (n - 1) / n),
          ("allconcat", lambda: impl.allconcat(xs, 0, 0), float(n - 1)),
          ("alltoall", lambda: impl.alltoall(xs, 0, 0, 0), (n - 1) / n)):
        ms = _time(fn, iters=5, warmup=2)
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        if rank == 0:
          _emit(config="collectives", op=name, dtype=dtype.name, n_gpus=n, slice_bytes=nbytes,
                ms=ms, bus_gb_per_s=nbytes * factor / (ms * 1e-3) / 1e9)
  _leave(dist_module=dist)


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--config", required=True, choices=["moe", "einsum_fp32", "attention", "collectives", "ffn_train"])
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--iters", type=int, default=10)
  ap.add_argument("--eager", action="store_true")
  ap.add_argument("--attention-batch", type=int, default=2)
  ap.add_argument("--max-bytes", type=int, default=1 << 30)
  args = ap.parse_args()
  if not torch.cuda.is_available():
    sys.exit("needs a CUDA device")
  {"moe": config_moe, "einsum_fp32": config_einsum_fp32, "attention": config_attention,
   "ffn_train": config_ffn_train,
   "collectives": config_collectives}[args.config](args)


if __name__ == "__main__":
  main()
