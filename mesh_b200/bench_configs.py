"""Per-configuration measurements beside bench.py's headline number.

  python -m mesh_b200.bench_configs --config moe|moe_train|einsum_fp32|attention|collectives|ffn_train [--gpus N]

`measure_moe`, `measure_attention` and `measure_einsum_fp32` return records
(dicts) that bench.py places in its JSON line; the command line above prints
the same records one JSON line each.  Every record states the algorithmic
bytes or flops it was divided by, so roofline fractions can be checked by
hand.  Inputs are seeded synthetic tensors of the configuration's shapes.
Timing: CUDA events on the launching stream, warm-up first, inputs larger than
L2 or an L2 flush (a 256 MiB fill) between iterations.  Multi-GPU
configurations run one process per GPU under torch.distributed.run and report
the maximum over ranks.
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

MOE_SEED = 1236       # 1234 + configuration index
ATTENTION_SEED = 1237


def peaks():
  root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
  path = os.path.join(root, "MEASURED_PEAKS.json")
  if os.path.exists(path):
    p = json.load(open(path))
    return {"hbm_gbs": p["hbm_gbs"], "tflops": p["bf16_tflops_sustained"],
            "tflops_burst": p["bf16_tflops"], "source": "measured"}
  return {"hbm_gbs": 6650.0, "tflops": 1400.0, "tflops_burst": 1590.0, "source": "fallback"}


class Flusher(object):
  """Evicts L2 by writing a buffer larger than it (through the library's fill kernel)."""

  def __init__(self, ops):
    self._ops = ops
    self._n = 64 * 1024 * 1024

  def __call__(self):
    self._ops.fill([self._n], 0.0, mtf.float32)


def time_fn(fn, iters=10, warmup=3, flush=None):
  """Median CUDA-event time of fn() in ms, each iteration timed on its own."""
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


def time_steps(step, steps, warmup, n_ranks, join=None):
  """ms per step of `steps` back-to-back calls, bracketed by barrier +
  synchronize, maximum over ranks; also the libmtfc launches in the region."""
  import torch.distributed as dist

  def barrier():
    if n_ranks > 1:
      dist.barrier()
    torch.cuda.synchronize()
  for _ in range(warmup):
    step()
  if join is not None:
    join()
  barrier()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  launches0 = nat.launch_count()
  e0.record()
  for _ in range(steps):
    step()
  if join is not None:
    join()
  e1.record()
  barrier()
  ms = e0.elapsed_time(e1)
  launches = nat.launch_count() - launches0
  if n_ranks > 1:
    t = torch.tensor([ms], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
  return ms / steps, launches


def _max_over_ranks(value, n_ranks):
  if n_ranks <= 1:
    return value
  import torch.distributed as dist
  t = torch.tensor([value], device="cuda", dtype=torch.float64)
  dist.all_reduce(t, op=dist.ReduceOp.MAX)
  return float(t.item())


def barrier_all():
  import torch.distributed as dist
  if dist.is_available() and dist.is_initialized():
    dist.barrier()
  torch.cuda.synchronize()


def leave():
  """Ends a multi-rank run: barrier, flush, exit without tearing NCCL down."""
  import torch.distributed as dist
  dist.barrier()
  torch.cuda.synchronize()
  sys.stdout.flush()
  sys.stderr.flush()
  os._exit(0)


def _emit(**kw):
  print(json.dumps(kw), flush=True)


def _normal(seed_words, shape, scale=1.0):
  r = np.random.Generator(np.random.PCG64(seed_words))
  a = r.standard_normal(shape, dtype=np.float32)
  if scale != 1.0:
    a *= np.float32(scale)
  return a


# ------------------------------------------------------------------------ MoE
MOE = dict(B=64, L=1024, M=1024, E=32, H=4096, S=1024, C=40)


def moe_inputs(rows=None, experts=None):
  """Seeded inputs of the top-2 MoE configuration: x ~ N(0,1) [64,1024,1024],
  gate kernel fp32 ~ N(0,1/1024) [1024,32], expert kernels ~ N(0,1/fan_in).
  Every batch row and every expert has its own generator stream, so a rank
  (or a checker) can draw just the rows / experts it needs."""
  c = MOE
  rows = range(c["B"]) if rows is None else rows
  experts = range(c["E"]) if experts is None else experts
  x = np.stack([_normal([MOE_SEED, 0, b], (c["L"], c["M"])) for b in rows]) if len(rows) else None
  wg = _normal([MOE_SEED, 1], (c["M"], c["E"]), c["M"] ** -0.5)
  wi = [_normal([MOE_SEED, 2, e], (c["M"], c["H"]), c["M"] ** -0.5) for e in experts]
  wo = [_normal([MOE_SEED, 3, e], (c["H"], c["M"]), c["H"] ** -0.5) for e in experts]
  return x, wg, wi, wo


def _bf16_f64(a):
  return torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16).to(torch.float64).numpy()


def moe_parity(x_rows, wg, routing_host, out_rows, group, n_tokens=4):
  """Checks one group of the device result against the per-group specification
  restated here in numpy (float64 logits, float32 softmax as exp(l - lse),
  lowest-index ties, index-order positions), and `n_tokens` output rows against
  float64 expert FFNs.  Returns a dict for the bench line; tokens whose gate
  margins are under 1e-5 make the group incomparable (reported, not failed)."""
  c = MOE
  S, E, C = c["S"], c["E"], c["C"]
  xb = _bf16_f64(x_rows)                                   # [S, M] of this group
  logits = (xb @ wg.astype(np.float64)).astype(np.float32)
  mx = logits.max(-1, keepdims=True)
  lse = np.log(np.exp(logits - mx, dtype=np.float32).sum(-1, keepdims=True, dtype=np.float32)) + mx
  raw = np.exp(logits - lse, dtype=np.float32)
  top = np.sort(raw, -1)[:, ::-1]
  safe = bool(np.all((top[:, 0] - top[:, 1] > 1e-5) & (top[:, 1] - top[:, 2] > 1e-5)))
  i1 = raw.argmax(-1)
  g1 = raw[np.arange(S), i1]
  raw2 = raw.copy()
  raw2[np.arange(S), i1] = 0
  i2 = raw2.argmax(-1)
  g2 = raw2[np.arange(S), i2]
  recip = np.float32(1.0) / ((g1 + g2) + np.float32(1e-9))
  g1, g2 = g1 * recip, g2 * recip
  p1, p2 = np.zeros(S, np.int64), np.zeros(S, np.int64)
  seen = np.zeros(E, np.int64)
  for s in range(S):
    p1[s] = seen[i1[s]]
    seen[i1[s]] += 1
  cnt1 = np.minimum(seen, C)
  seen2 = np.zeros(E, np.int64)
  for s in range(S):
    p2[s] = seen2[i2[s]] + cnt1[i2[s]]
    seen2[i2[s]] += 1
  got = [np.asarray(t).reshape(-1, S)[group] for t in routing_host]
  exact = all(np.array_equal(a, b) for a, b in zip(got[:4], (i1, i2, p1, p2)))
  keep = np.array_equal(got[4] != 0, p1 < C) and np.array_equal(got[5] != 0, p2 < C)
  rec = {"group_checked": int(group), "margins_ok": safe,
         "indices_positions_exact": bool(exact), "keep_masks_exact": bool(keep)}
  # output rows: w1 * FFN_{i1}(x) + w2 * FFN_{i2}(x) with bf16 roundings where the layer has them
  worst, scale = 0.0, 1e-30
  pick = np.random.Generator(np.random.PCG64([MOE_SEED, 9, group]))
  w1b = _bf16_f64(np.where(p1 < C, g1, 0).astype(np.float32))
  w2b = _bf16_f64(np.where(p2 < C, g2, 0).astype(np.float32))
  for s in pick.choice(S, n_tokens, replace=False):
    acc = np.zeros(c["M"])
    for e, w in ((i1[s], w1b[s]), (i2[s], w2b[s])):
      if w != 0:
        _, _, wi, wo = moe_inputs(rows=[], experts=[int(e)])
        h = _bf16_f64(np.maximum(xb[s] @ _bf16_f64(wi[0]), 0).astype(np.float32))
        acc += w * _bf16_f64((h @ _bf16_f64(wo[0])).astype(np.float32))
    worst = max(worst, float(np.max(np.abs(out_rows[s] - acc))))
    scale = max(scale, float(np.max(np.abs(acc))))
  rec.update(rows=int(n_tokens), rel_err=worst / scale)
  return rec


def measure_moe(n, rank, local_rank, steps, warmup, eager=False, kernel_iters=10, check=True):
  """Top-2 MoE layer (transformer_moe_layer_v1 semantics): 65536 tokens in 64
  groups of 1024, d_model 1024, 32 experts, d_ff 4096, capacity factor 1.25
  (capacity 40), bf16, policy "all"; mesh all:n with batch:all;experts:all
  (groups and experts split n ways, two alltoalls per layer)."""
  c = MOE
  B, L, M, E, H, S, C = (c[k] for k in "BLMEHSC")
  pk = peaks()
  mesh_shape, layout = "all:%d" % n, "batch:all;experts:all"
  impl = CudaMeshImpl(mesh_shape, layout, list(range(n)) if n > 1 else [local_rank], distributed=n > 1)
  ops = impl.slice_ops
  b_loc, e_loc = B // n, E // n
  my_rows = list(range(rank * b_loc, (rank + 1) * b_loc))
  x, wg, wi, wo = moe_inputs(rows=my_rows, experts=range(rank * e_loc, (rank + 1) * e_loc))
  to_bf16 = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16)
  x_host = to_bf16(x).pin_memory()
  lx = impl.LaidOutTensor([ops.from_host(x_host, mtf.bfloat16)])
  lwg = impl.LaidOutTensor([ops.from_host(wg, mtf.float32)])
  lwi = impl.LaidOutTensor([ops.from_host(to_bf16(np.stack(wi)), mtf.bfloat16)])
  lwo = impl.LaidOutTensor([ops.from_host(to_bf16(np.stack(wo)), mtf.bfloat16)])
  del wi, wo
  out_hosts = [torch.empty((b_loc, L, M), dtype=torch.bfloat16).pin_memory() for _ in range(2)]

  def build(x_source):
    g = mtf.Graph()
    mesh = mtf.Mesh(g, "mesh")
    X = x_source(mesh)
    WG = mtf.import_laid_out_tensor(mesh, lwg, "d_model:%d,expert_unsplit:%d" % (M, E), mtf.float32)
    WI = mtf.import_laid_out_tensor(mesh, lwi, "experts:%d,d_model:%d,d_ff:%d" % (E, M, H), mtf.bfloat16)
    WO = mtf.import_laid_out_tensor(mesh, lwo, "experts:%d,d_ff:%d,d_model:%d" % (E, H, M), mtf.bfloat16)
    hp = mtf.moe.HParams(moe_group_size=S, moe_second_policy_train="all")
    out, loss, aux = mtf.moe.transformer_moe_layer_v1(
        X, mtf.Dimension("d_model", M), hp, True, mesh_shape, layout, WG, WI, WO, return_aux=True)
    return g, mesh, out, aux
  x_shape = "batch:%d,length:%d,d_model:%d" % (B, L, M)
  g_dev, mesh_dev, out_dev, aux_dev = build(lambda m: mtf.import_laid_out_tensor(m, lx, x_shape, mtf.bfloat16))

  names = ["index_1", "index_2", "position_1", "position_2", "gate_1", "gate_2"]

  def step_device():
    low = mtf.Lowering(g_dev, {mesh_dev: impl})
    return (low.tensors[out_dev].to_laid_out_tensor(),
            [low.tensors[aux_dev[k]].to_laid_out_tensor() for k in names])

  # end to end: this rank's rows come from pinned host memory every step and the
  # output rows go back to pinned host memory
  def make_step_e2e(slot):
    def x_source(m):
      fresh = lambda: impl.LaidOutTensor([ops.from_host(x_host, mtf.bfloat16)])
      return mtf.import_laid_out_tensor(m, mtf.LazyLaidOutTensor(fresh, [b_loc, L, M]), x_shape,
                                        mtf.bfloat16)
    g_e, mesh_e, out_e, _ = build(x_source)

    def step():
      low = mtf.Lowering(g_e, {mesh_e: impl})
      impl.export_to_host_tensors(low.tensors[out_e].to_laid_out_tensor(), out=[out_hosts[slot]])
    return step

  before = nat.launch_count()
  step_device()
  launches_per_step = nat.launch_count() - before
  impl.synchronize()
  run_device, result = step_device, None
  run_e2e, join_e2e = make_step_e2e(0), None
  pipelined = False
  if not eager:
    result, run_device = impl.capture(step_device)
    if n == 1:
      # one GPU, no collectives in the step: two recorded copies of the step (own device
      # buffers, own pinned output) alternate on two streams, so one step's upload
      # overlaps the other's compute and download
      replays = [impl.capture(make_step_e2e(slot))[1] for slot in range(2)]
      streams = [torch.cuda.Stream() for _ in range(2)]
      turn = [0]
      pipelined = True

      def run_e2e():
        k = turn[0] & 1
        turn[0] += 1
        streams[k].wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(streams[k]):
          replays[k]()

      def join_e2e():
        for st in streams:
          torch.cuda.current_stream().wait_stream(st)
    else:
      _, run_e2e = impl.capture(run_e2e)
  ms, _ = time_steps(run_device, steps, warmup, n)
  impl.synchronize()
  ms_e2e, _ = time_steps(run_e2e, steps, max(3, warmup // 2), n, join=join_e2e)
  impl.synchronize()
  tokens = B * L
  expert_flops = 2.0 * (E * (tokens // S) * C) * M * H * 2.0
  rec = {
      "workload": "top-2 MoE layer: 65536 tokens (64 groups x 1024), d_model 1024, 32 experts, "
                  "d_ff 4096, capacity 40, bf16, second-expert policy all",
      "mesh": mesh_shape, "layout": layout, "n_gpus": n,
      "tokens_per_s": tokens / (ms * 1e-3), "ms_per_step": ms,
      "expert_tflops": expert_flops / (ms * 1e-3) / 1e12,
      "expert_flops_per_step": expert_flops,
      "gpu_launches": launches_per_step * steps,
      "stepping": "eager lowering" if eager else "CUDA-graph replay of the lowering",
      "e2e": {"tokens_per_s": tokens / (ms_e2e * 1e-3), "ms_per_step": ms_e2e,
              "h2d_bytes_per_step": x_host.numel() * 2 * n, "d2h_bytes_per_step": x_host.numel() * 2 * n,
              "overlap": "two recorded steps alternate on two streams" if pipelined else "one stream"},
  }

  # per-kernel times on this rank's groups (groups are independent), L2 flushed
  xs = ops.reshape(lx.tensor_list[0], [1, b_loc * L // S, S, M])
  G = xs.shape[1]
  flush = Flusher(ops)
  w = lwg.tensor_list[0]
  # each op is recorded as a CUDA graph and the replay is timed, so that the gaps
  # the host leaves between the launches of one op do not count as kernel time
  def flush_then(fn):
    def both():
      flush()
      return fn()
    return both
  _, flush_replay = impl.capture(flush_then(lambda: None), warmup=1)
  t_flush = time_fn(flush_replay, iters=kernel_iters)

  def graph_time(fn):
    """Device time of fn's kernels behind an L2 flush: a recorded [flush, fn] sequence
    minus the recorded flush alone, so neither host launch gaps nor the replay's own
    start-up are counted as kernel time."""
    _, replay = impl.capture(flush_then(fn), warmup=1)
    return max(time_fn(replay, iters=kernel_iters) - t_flush, 1e-6)
  routing = ops.moe_top2_gating(xs, w, C, "all", 0.2, None, G, want_table=True)
  t_gate = graph_time(lambda: ops.moe_top2_gating(xs, w, C, "all", 0.2, None, G, want_table=True))
  i1, i2, p1, p2, g1, g2, _, table = routing
  disp = ops.moe_dispatch(xs, i1, i2, p1, p2, g1, g2, E, C, table)
  t_disp = graph_time(lambda: ops.moe_dispatch(xs, i1, i2, p1, p2, g1, g2, E, C, table))
  t_comb = graph_time(lambda: ops.moe_combine(disp, i1, i2, p1, p2, g1, g2))
  del disp
  tok = G * S
  slots = E * C / S   # expert-buffer rows per token: 1.25
  per_token = [   # algorithmic HBM bytes per token
      ("gating: gate logits + softmax + top-2 + positions (gate_top2_fused, top2_positions)",
       t_gate, 2 * M + 16),
      ("dispatch (dispatch_rows)", t_disp, 2 * M + slots * 2 * M),
      ("combine (combine_rows)", t_comb, slots * 2 * M + 2 * M),
  ]
  roofs = []
  for name, t, bpt in per_token:
    t = _max_over_ranks(t, n)
    gbs = tok * bpt / (t * 1e-3) / 1e9
    roofs.append({"kernel": name, "bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s",
                  "frac": gbs / pk["hbm_gbs"], "launch_ms": t, "bytes_per_token": bpt,
                  "tokens_per_launch": tok, "peak_source": pk["source"] + " copy bandwidth"})
  total_t = sum(r["launch_ms"] for r in roofs)
  total_b = sum(r["bytes_per_token"] for r in roofs)
  rec["roofline"] = roofs
  rec["routing_path"] = {"bytes_per_token": total_b, "ms": total_t,
                         "achieved": tok * total_b / (total_t * 1e-3) / 1e9, "unit": "GB/s",
                         "frac": tok * total_b / (total_t * 1e-3) / 1e9 / pk["hbm_gbs"],
                         "timing": "each operation recorded behind an L2 flush and replayed; the replay of "
                                   "the flush alone (%.4f ms) is subtracted" % t_flush}
  if check:
    out_lt, routing_lt = result if result is not None else step_device()
    impl.synchronize()
    routing_host = [ops.to_host(t.tensor_list[0]) for t in routing_lt]
    out_host = impl.export_to_host_tensors(out_lt)[0].float().numpy().reshape(-1, S, M)
    impl.synchronize()
    group = 0
    rec["parity"] = moe_parity(x[group], wg, routing_host, out_host[group].astype(np.float64), group)
    e2e_host = out_hosts[0].float().numpy().reshape(-1, S, M)
    rec["parity"]["e2e_output_equals_device_output"] = bool(np.array_equal(e2e_host, out_host))
  impl.release_graphs()
  return rec


# ------------------------------------------------------------------ attention
def measure_attention(n, rank, local_rank, steps, warmup, batch=16, eager=False, kernel_alone=True):
  """Multi-head attention: x[batch,2048,4096] bf16, 32 heads of 128, causal;
  q/k/v projections, fused attention kernel, output projection.  With n > 1 the
  heads are split over a 1-D mesh (layout heads:all): every rank holds the whole
  x and its own heads' weights, and the output projection ends in an allreduce."""
  pk = peaks()
  mesh_shape, layout = "all:%d" % n, ("heads:all" if n > 1 else "")
  impl = CudaMeshImpl(mesh_shape, layout, list(range(n)) if n > 1 else [local_rank], distributed=n > 1)
  ops = impl.slice_ops
  b, l, d, h, kv = batch, 2048, 4096, 32, 128
  h_loc = h // n
  x = torch.from_numpy(_normal([ATTENTION_SEED, 0], (b, l, d))).to(torch.bfloat16)
  lx = impl.LaidOutTensor([ops.from_host(x, mtf.bfloat16)])
  del x
  stds = [d ** -0.5 * kv ** -0.25] * 2 + [d ** -0.5, (d * h) ** -0.5]
  lws = []
  for i, sd in enumerate(stds):
    w = np.stack([_normal([ATTENTION_SEED, 1 + i, hh], (d, kv), sd)
                  for hh in range(rank * h_loc, (rank + 1) * h_loc)])
    lws.append(impl.LaidOutTensor([ops.from_host(torch.from_numpy(w).to(torch.bfloat16), mtf.bfloat16)]))
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
  if not eager:
    _, run = impl.capture(step)
  ms, _ = time_steps(run, steps, warmup, n)
  impl.synchronize()
  proj = 4 * 2.0 * b * l * d * h * kv
  attn_full = 2 * 2.0 * b * h * l * l * kv
  rec = {"workload": "multihead attention x[%d,2048,4096] bf16, 32 heads x 128, causal" % b,
         "mesh": mesh_shape, "layout": layout, "n_gpus": n, "ms_per_step": ms,
         "tflops_full": (proj + attn_full) / (ms * 1e-3) / 1e12,
         "tflops_causal_work": (proj + attn_full / 2 * (1 + 128.0 / l)) / (ms * 1e-3) / 1e12,
         "flops_full": proj + attn_full,
         "allreduce_bytes_per_gpu": (b * l * d * 2 if n > 1 else 0),
         "gpu_launches": launches * steps, "peak_tflops": pk["tflops"], "peak_source": pk["source"],
         "stepping": "eager lowering" if eager else "CUDA-graph replay of the lowering"}
  if kernel_alone and n == 1:
    q, k, v = [ops.from_host(torch.from_numpy(_normal([ATTENTION_SEED, 9, i], (b, h, l, kv), 0.3))
                             .to(torch.bfloat16), mtf.bfloat16) for i in range(3)]
    alone = []
    for causal in (True, False):
      t = time_fn(lambda: ops.attention(q, k, v, causal), iters=5, warmup=2)
      work = attn_full * ((0.5 * (1 + 128.0 / l)) if causal else 1.0)
      alone.append({"kernel": "attn_fwd_tcgen05", "causal": causal, "launch_ms": t, "bound": "tensor",
                    "achieved": work / (t * 1e-3) / 1e12, "peak": pk["tflops"], "unit": "TFLOP/s",
                    "frac": work / (t * 1e-3) / 1e12 / pk["tflops"], "flops_executed": work})
    rec["roofline"] = alone
  impl.release_graphs()
  return rec


# ---------------------------------------------------------------- fp32 einsum
def measure_einsum_fp32(local_rank=0, iters=10):
  """x[4096,1024] . w[1024,4096] in fp32 on one GPU (the whole problem), with a
  check of the result against float64 (1e-5 relative)."""
  impl = CudaMeshImpl("all:1", "", [local_rank])
  ops = impl.slice_ops
  x = _normal([1234, 0], (4096, 1024))
  w = _normal([1234, 1], (1024, 4096), 1024 ** -0.5)
  dx, dw = ops.from_host(x, mtf.float32), ops.from_host(w, mtf.float32)
  ms = time_fn(lambda: ops.einsum("ab,bc->ac", dx, dw), iters=iters, flush=Flusher(ops))
  got = ops.to_host(ops.einsum("ab,bc->ac", dx, dw))[:64].astype(np.float64)
  ref = x[:64].astype(np.float64) @ w.astype(np.float64)
  return {"workload": "einsum x[4096,1024] . w[1024,4096] fp32", "ms": ms,
          "tflops": 2.0 * 4096 * 1024 * 4096 / (ms * 1e-3) / 1e12,
          "kernels": "split_bf16x3 x2 + einsum_gemm_tcgen05 over 6K",
          "parity": {"rows": 64, "rel_err": float(np.max(np.abs(got - ref)) / np.max(np.abs(ref)))}}


# ------------------------------------------------------------- command line
def _init(args):
  n = args.gpus
  rank = int(os.environ.get("RANK", "0"))
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local_rank)
  if n > 1:
    import torch.distributed as dist
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
  return n, rank, local_rank


def config_moe(args):
  n, rank, local_rank = _init(args)
  rec = measure_moe(n, rank, local_rank, args.iters, 3, eager=args.eager)
  if rank == 0:
    _emit(config="moe", **rec)
  if n > 1:
    leave()


def config_attention(args):
  n, rank, local_rank = _init(args)
  rec = measure_attention(n, rank, local_rank, args.iters, 3, batch=args.attention_batch, eager=args.eager)
  if rank == 0:
    _emit(config="attention", **rec)
  if n > 1:
    leave()


def config_einsum_fp32(args):
  torch.cuda.set_device(0)
  _emit(config="einsum_fp32", **measure_einsum_fp32(0, args.iters))


def measure_ffn_train(local_rank=0, iters=10, eager=False):
  """Forward and backward of the dense FFN (x[64,1024,1024], wi[1024,4096],
  wo[4096,1024], bf16) on one GPU: y, then dx, dwi, dwo from a given dy through
  mtf.gradients - three GEMM pairs with permuted operand roles and the ReLU
  mask, lowered onto the same kernels and replayed as a CUDA graph."""
  pk = peaks()
  torch.cuda.set_device(local_rank)
  impl = CudaMeshImpl("all:1", "", [local_rank])
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
  if not eager:
    _, run = impl.capture(step)
  ms = time_fn(run, iters=iters, warmup=3)
  flops = 3 * 2.0 * 2.0 * b * l * d * f     # forward + two gradient GEMMs per forward GEMM
  rec = dict(quantity="dense_relu_dense forward + backward (dx, dwi, dwo)", ms=ms,
             tflops=flops / (ms * 1e-3) / 1e12, frac_of_peak=flops / (ms * 1e-3) / 1e12 / pk["tflops"],
             peak_tflops=pk["tflops"], peak_source=pk["source"], libmtfc_launches_per_step=launches,
             stepping="eager" if eager else "cuda-graph replay")
  impl.release_graphs()
  return rec


def config_ffn_train(args):
  _emit(config="ffn_train", **measure_ffn_train(0, args.iters, args.eager))


def measure_moe_train(n, rank, local_rank, iters=10, eager=False):
  """Forward and backward of the top-2 MoE layer at the benchmark shape: the
  output, then dx, d(gate kernel), dwi, dwo from a given d(output) through
  mtf.gradients (gating, dispatch and combine gradients on their own kernels,
  six expert GEMMs per step instead of two), replayed as a CUDA graph."""
  c = MOE
  B, L, M, E, H, S, C = (c[k] for k in "BLMEHSC")
  pk = peaks()
  mesh_shape, layout = "all:%d" % n, "batch:all;experts:all"
  impl = CudaMeshImpl(mesh_shape, layout, list(range(n)) if n > 1 else [local_rank], distributed=n > 1)
  ops = impl.slice_ops
  b_loc, e_loc = B // n, E // n
  x, wg, wi, wo = moe_inputs(rows=list(range(rank * b_loc, (rank + 1) * b_loc)),
                             experts=range(rank * e_loc, (rank + 1) * e_loc))
  to_bf16 = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16)
  laid = lambda t, dt: impl.LaidOutTensor([ops.from_host(t, dt)])
  lx, lwg = laid(to_bf16(x), mtf.bfloat16), laid(wg, mtf.float32)
  ldy = laid(to_bf16(np.stack([_normal([MOE_SEED, 4, b], (L, M))
                               for b in range(rank * b_loc, (rank + 1) * b_loc)])), mtf.bfloat16)
  lwi, lwo = laid(to_bf16(np.stack(wi)), mtf.bfloat16), laid(to_bf16(np.stack(wo)), mtf.bfloat16)
  del x, wi, wo
  g = mtf.Graph()
  mesh = mtf.Mesh(g, "mesh")
  act = "batch:%d,length:%d,d_model:%d" % (B, L, M)
  X = mtf.import_laid_out_tensor(mesh, lx, act, mtf.bfloat16)
  DY = mtf.import_laid_out_tensor(mesh, ldy, act, mtf.bfloat16)
  WG = mtf.import_laid_out_tensor(mesh, lwg, "d_model:%d,expert_unsplit:%d" % (M, E), mtf.float32)
  WI = mtf.import_laid_out_tensor(mesh, lwi, "experts:%d,d_model:%d,d_ff:%d" % (E, M, H), mtf.bfloat16)
  WO = mtf.import_laid_out_tensor(mesh, lwo, "experts:%d,d_ff:%d,d_model:%d" % (E, H, M), mtf.bfloat16)
  hp = mtf.moe.HParams(moe_group_size=S, moe_second_policy_train="all")
  out, loss = mtf.moe.transformer_moe_layer_v1(X, mtf.Dimension("d_model", M), hp, True, mesh_shape,
                                               layout, WG, WI, WO)
  grads = mtf.gradients([out], [X, WG, WI, WO], grad_ys=[DY])

  def step():
    low = mtf.Lowering(g, {mesh: impl})
    return [low.tensors[t].to_laid_out_tensor() for t in [out] + grads]
  before = nat.launch_count()
  step()
  launches = nat.launch_count() - before
  impl.synchronize()
  run = step
  if not eager:
    _, run = impl.capture(step)
  ms, _ = time_steps(run, iters, 3, n)
  impl.synchronize()
  tokens = B * L
  flops = 3 * 2.0 * (E * (tokens // S) * C) * M * H * 2.0
  rec = dict(quantity="top-2 MoE layer forward + backward (dx, dwg, dwi, dwo)",
             mesh=mesh_shape, layout=layout, n_gpus=n, ms_per_step=ms, tokens_per_s=tokens / (ms * 1e-3),
             expert_tflops=flops / (ms * 1e-3) / 1e12, expert_flops_per_step=flops,
             frac_of_peak=flops / (ms * 1e-3) / 1e12 / (pk["tflops"] * n), peak_tflops=pk["tflops"],
             peak_source=pk["source"], libmtfc_launches_per_step=launches,
             stepping="eager" if eager else "cuda-graph replay")
  impl.release_graphs()
  return rec


def config_moe_train(args):
  n, rank, local_rank = _init(args)
  rec = measure_moe_train(n, rank, local_rank, args.iters, args.eager)
  if rank == 0:
    _emit(config="moe_train", **rec)
  if n > 1:
    leave()


def config_collectives(args):
  """allreduce / allconcat / alltoall bus bandwidth over one mesh axis.
  --mesh names the mesh (default all:N) and --axis the axis the collectives run
  along; on rows:2,cols:4 axis 1 gives two concurrent groups of four."""
  import torch.distributed as dist
  n, rank, local_rank = _init(args)
  mesh_shape = args.mesh or "all:%d" % n
  impl = CudaMeshImpl(mesh_shape, "", list(range(n)), distributed=True)
  axis = args.axis
  k = impl.shape.dims[axis].size
  ops = impl.slice_ops
  for dtype in (mtf.bfloat16, mtf.float32):
    for p in range(0, 11):
      nbytes = 1024 * 4 ** p
      if nbytes > args.max_bytes:
        break
      elems = nbytes // dtype.itemsize
      xs = impl.LaidOutTensor([ops.fill([k, elems // k], 0.5, dtype)])
      for name, fn, factor in (
          ("allreduce", lambda: impl.allreduce(xs, [axis], "SUM"), 2.0 * (k - 1) / k),
          ("allconcat", lambda: impl.allconcat(xs, axis, 0), float(k - 1)),
          ("alltoall", lambda: impl.alltoall(xs, axis, 0, 0), (k - 1) / k)):
        # recorded once and replayed, so that the host's work between the launches of
        # one collective does not count as device time
        if args.eager:
          ms = time_fn(fn, iters=5, warmup=2)
        else:
          _, replay = impl.capture(fn, warmup=2)
          ms = time_fn(replay, iters=5, warmup=1)
          impl.release_graphs()
        ms = _max_over_ranks(ms, n)
        if rank == 0:
          _emit(config="collectives", op=name, dtype=dtype.name, n_gpus=n, mesh=mesh_shape, axis=axis,
                group_size=k, stepping="eager" if args.eager else "cuda-graph replay", slice_bytes=nbytes, ms=ms, bus_gb_per_s=nbytes * factor / (ms * 1e-3) / 1e9)
  leave()


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--config", required=True, choices=["moe", "moe_train", "einsum_fp32", "attention", "collectives", "ffn_train"])
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--iters", type=int, default=10)
  ap.add_argument("--eager", action="store_true")
  ap.add_argument("--attention-batch", type=int, default=2)
  ap.add_argument("--max-bytes", type=int, default=1 << 30)
  ap.add_argument("--mesh", default=None)
  ap.add_argument("--axis", type=int, default=0)
  args = ap.parse_args()
  if not torch.cuda.is_available():
    sys.exit("needs a CUDA device")
  {"moe": config_moe, "einsum_fp32": config_einsum_fp32, "attention": config_attention,
   "ffn_train": config_ffn_train, "moe_train": config_moe_train,
   "collectives": config_collectives}[args.config](args)


if __name__ == "__main__":
  main()
