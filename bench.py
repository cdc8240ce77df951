"""Benchmark of the MeshImpl hot path: laid-out einsums of the dense FFN block,
with the top-2 MoE layer, the attention layer and the fp32 einsum beside it.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (the configuration the metric is quoted on): Transformer
dense_relu_dense, x[batch=64, length=1024, d_model=1024] ~ N(0,1),
wi[1024, 4096] ~ N(0, 1/1024), wo[4096, 1024] ~ N(0, 1/4096), bf16 weights and
activations, fp32 accumulation, ReLU between; 1.0995 TFLOP per step.  One step
is one lowering of that graph through `mtf.Lowering` on `CudaMeshImpl`.
At N GPUs the same global problem is laid out on a rows x cols mesh with
`batch:rows;d_ff:cols` (1: 1x1, 2: 2x1, 4: 2x2, 8: 2x4), so the second einsum
contracts a split dim and is followed by an allreduce over `cols` — strong
scaling.  Inputs are seeded synthetic data (no dataset is involved).

Rank 0 prints one JSON line.  `value` is einsum TFLOP/s with the inputs already
on the device; `e2e` is the same through host buffers (pinned-memory upload of
the step's activations and download of its output inside the timed region).
`parity` compares sampled rows of every rank's output slice, from the timed
device path and from the end-to-end host buffers, with a float64 product of
the same seeded inputs.  The `moe` record is the other half of the metric: the
top-2 mixture-of-experts layer (tokens/s, expert TFLOP/s, its routing kernels
against the HBM roofline, its own parity check, CPU baseline and end-to-end
number) on mesh all:N with `batch:all;experts:all`; `attention` and
`einsum_fp32` report the attention layer and the fp32 einsum.  `--only ffn`
skips those records.

`--impl reference` times the reference's CPU lowering of the same graphs: the
restated PlacementMeshImpl semantics on host cores (TensorFlow, and therefore
the reference itself, is not installable here).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
  sys.path.insert(0, ROOT)

BATCH, LENGTH, D_MODEL, D_FF = 64, 1024, 1024, 4096
SEED = 1235  # 1234 + configuration index
FLOPS_PER_STEP = 2.0 * BATCH * LENGTH * D_MODEL * D_FF * 2.0
MESHES = {1: "rows:1,cols:1", 2: "rows:2,cols:1", 4: "rows:2,cols:2", 8: "rows:2,cols:4"}
LAYOUT = "batch:rows;d_ff:cols"
METRIC = "einsum TFLOP/s (dense_relu_dense FFN, bf16, fp32 accumulate)"
CPU_SAMPLE_BATCH = 8  # sequences of the 64 the CPU arms run per step
CPU_MOE_GROUPS = 4    # groups of the 64 the CPU arms run per MoE step
NOMINAL_BF16_TFLOPS = 2250.0
PARITY_ROWS = 32

# DRAM bytes per launch of einsum_gemm_tcgen05_2cta on the GEMMs of this workload
# on one GPU: dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture, mean
# of the wi (625.3 MB) and wo (674.9 MB) launches; algorithmic bytes 679.5 MB each.
GEMM_DRAM_TRAFFIC_BYTES = 650.1e6


def measured_peaks():
  path = os.path.join(ROOT, "MEASURED_PEAKS.json")
  if os.path.exists(path):
    with open(path) as f:
      p = json.load(f)
    return {"tflops_sustained": p.get("bf16_tflops_sustained"), "tflops_burst": p.get("bf16_tflops"),
            "hbm_gbs": p.get("hbm_gbs"), "source": "measured"}
  return {"tflops_sustained": 1400.0, "tflops_burst": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler(object):
  """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

  FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
            "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

  def __init__(self, index):
    self._index = index
    self._proc = None
    self._lines = []
    self._thread = None

  def start(self):
    try:
      self._proc = subprocess.Popen(
          ["nvidia-smi", "-i", str(self._index), "--query-gpu=" + self.FIELDS,
           "--format=csv,noheader,nounits", "-lms", "100"],
          stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
    except OSError:
      self._proc = None
      return
    self._thread = threading.Thread(target=self._pump, daemon=True)
    self._thread.start()

  def _pump(self):
    for line in self._proc.stdout:
      self._lines.append(line.strip())

  def stop(self):
    if self._proc is None:
      return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
    self._proc.terminate()
    try:
      self._proc.wait(timeout=5)
    except subprocess.TimeoutExpired:
      self._proc.kill()
    clocks, max_clock, reasons = [], None, set()
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    for line in self._lines:
      parts = [p.strip() for p in line.split(",")]
      if len(parts) < 8:
        continue
      try:
        clocks.append(float(parts[0]))
        max_clock = float(parts[1])
      except ValueError:
        continue
      for name, flag in zip(names, parts[4:8]):
        if flag.lower().startswith("active"):
          reasons.add(name)
    return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_clock,
            "samples": len(clocks), "reasons": sorted(reasons)}


def run_reference(args):
  """The reference's CPU lowering of the same graphs, timed on the host cores."""
  rank = int(os.environ.get("RANK", "0"))
  if rank != 0:
    return
  import numpy as np
  from oracle import cpu_baseline
  cores = cpu_baseline.host_threads()
  seconds, _ = cpu_baseline.time_ffn(CPU_SAMPLE_BATCH, LENGTH, D_MODEL, D_FF, "", "",
                                     steps=max(1, args.steps), warmup=max(1, min(args.warmup, 1)))
  flops = cpu_baseline.ffn_flops(CPU_SAMPLE_BATCH, LENGTH, D_MODEL, D_FF)
  value = flops / seconds / 1e12
  sample = "%d of %d sequences per step (%.1f GFLOP)" % (CPU_SAMPLE_BATCH, BATCH, flops / 1e9)
  line = {
      "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s",
      "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
      "ms_per_step": seconds * 1e3, "higher_is_better": True, "scaling": "strong",
      "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
      "config": {"workload": "dense_relu_dense FFN x[64,1024,1024] wi[1024,4096] wo[4096,1024]",
                 "note": "restated PlacementMeshImpl lowering on host cores; TensorFlow absent, "
                         "so the reference package itself cannot be installed or run"},
      "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                       "sample": sample},
      "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
      "gpu_launches": 0,
  }
  if args.only != "ffn":
    line["moe"] = cpu_moe(cpu_baseline, np, steps=min(3, max(1, args.steps)))
  print(json.dumps(line), flush=True)


def cpu_moe(cpu_baseline, np, steps):
  """tokens/s of the reference's op-by-op MoE lowering on the host cores (a sample of groups)."""
  from mesh_b200 import bench_configs
  x, wg, wi, wo = bench_configs.moe_inputs(rows=range(CPU_MOE_GROUPS))
  sec, _ = cpu_baseline.time_moe(x, wg, np.stack(wi), np.stack(wo), bench_configs.MOE["S"], steps, 1)
  return {"value": CPU_MOE_GROUPS * bench_configs.MOE["S"] / sec, "unit": "tokens/s",
          "cores": cpu_baseline.host_threads(), "kind": "port", "ms_per_step": sec * 1e3,
          "sample": "%d of 64 groups per step with all 32 experts: the reference's op chain with the "
                    "dense one-hot dispatch/combine einsums and the triangular cumsum" % CPU_MOE_GROUPS}


def run_ours(args):
  import numpy as np
  import torch
  import torch.distributed as dist

  from mesh_b200 import _native as nat
  from mesh_b200 import bench_configs
  from mesh_b200 import mtf
  from mesh_b200.cuda_mesh_impl import CudaMeshImpl

  n = args.gpus
  if n not in MESHES:
    raise SystemExit("--gpus must be one of %s" % sorted(MESHES))
  rank = int(os.environ.get("RANK", "0"))
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))
  world = int(os.environ.get("WORLD_SIZE", "1"))
  if world != n:
    raise SystemExit("WORLD_SIZE=%d but --gpus %d: launch with torch.distributed.run" % (world, n))
  if not torch.cuda.is_available():
    raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
  torch.cuda.set_device(local_rank)
  device = torch.device("cuda", local_rank)
  if n > 1:
    dist.init_process_group("nccl", device_id=device)

  mesh_shape = args.mesh or MESHES[n]
  stall = args.stall_dump_s if args.stall_dump_s > 0 else (780 if n > 1 else 0)
  if stall > 0:
    # a rank that stops making progress dumps its Python stacks and exits, which
    # makes the launcher end the other ranks too
    import faulthandler
    faulthandler.dump_traceback_later(stall, exit=True)
  impl = CudaMeshImpl(mesh_shape, LAYOUT, devices=list(range(n)) if n > 1 else [local_rank],
                      distributed=(n > 1))
  rows = impl.shape.dims[0].size
  cols = impl.shape.dims[1].size
  coord = mtf.pnum_to_processor_coordinates(impl.shape, rank)

  # Seeded synthetic inputs, generated on the host and rounded to bf16 once.
  r = np.random.Generator(np.random.PCG64(SEED))
  x_full = r.standard_normal((BATCH, LENGTH, D_MODEL), dtype=np.float32)
  wi_full = r.standard_normal((D_MODEL, D_FF), dtype=np.float32) * np.float32(D_MODEL ** -0.5)
  wo_full = r.standard_normal((D_FF, D_MODEL), dtype=np.float32) * np.float32(D_FF ** -0.5)
  b_loc, f_loc = BATCH // rows, D_FF // cols
  x_full_host = torch.from_numpy(x_full).to(torch.bfloat16).pin_memory()
  x_host = x_full_host[coord[0] * b_loc:(coord[0] + 1) * b_loc]
  wi_bf16 = torch.from_numpy(wi_full).to(torch.bfloat16)
  wo_bf16 = torch.from_numpy(wo_full).to(torch.bfloat16)
  wi_host = wi_bf16[:, coord[1] * f_loc:(coord[1] + 1) * f_loc].contiguous()
  wo_host = wo_bf16[coord[1] * f_loc:(coord[1] + 1) * f_loc].contiguous()
  y_host = torch.empty((b_loc, LENGTH, D_MODEL), dtype=torch.bfloat16).pin_memory()
  del x_full, wi_full, wo_full

  ops = impl.slice_ops
  x_dev = impl.LaidOutTensor([ops.from_host(x_host, mtf.bfloat16)])
  wi_dev = impl.LaidOutTensor([ops.from_host(wi_host, mtf.bfloat16)])
  wo_dev = impl.LaidOutTensor([ops.from_host(wo_host, mtf.bfloat16)])

  x_shape = "batch:%d,length:%d,d_model:%d" % (BATCH, LENGTH, D_MODEL)
  wi_shape = "d_model:%d,d_ff:%d" % (D_MODEL, D_FF)
  wo_shape = "d_ff:%d,d_model:%d" % (D_FF, D_MODEL)

  def build(x_source):
    g = mtf.Graph()
    mesh = mtf.Mesh(g, "mesh")
    X = x_source(mesh)
    WI = mtf.import_laid_out_tensor(mesh, wi_dev, wi_shape, mtf.bfloat16)
    WO = mtf.import_laid_out_tensor(mesh, wo_dev, wo_shape, mtf.bfloat16)
    y = mtf.layers.dense_relu_dense(X, mtf.Dimension("d_ff", D_FF), wi=WI, wo=WO)
    return g, mesh, y

  # device-resident graph: activations already in HBM
  g_dev, mesh_dev, y_dev = build(lambda m: mtf.import_laid_out_tensor(m, x_dev, x_shape, mtf.bfloat16))

  def step_device():
    low = mtf.Lowering(g_dev, {mesh_dev: impl})
    return low.tensors[y_dev].to_laid_out_tensor()

  # End-to-end graph: the whole x sits in pinned host memory.  Each step's
  # import_tf_tensor cuts this rank's slice on the host; the ranks of a `cols`
  # group, which all need the same slice, upload a quarter (1/cols) of it each and
  # complete it with an allgather over NVLink; each downloads its 1/cols of the
  # replicated output slice.  Every byte crosses a host link once per step.
  g_e2e, mesh_e2e, y_e2e = build(lambda m: mtf.import_tf_tensor(m, x_full_host, x_shape, dtype=mtf.bfloat16))

  y_hosts = [y_host, torch.empty_like(y_host).pin_memory()]
  filled = [None, None]

  def make_step_e2e(slot):
    def step():
      low = mtf.Lowering(g_e2e, {mesh_e2e: impl})
      out = low.tensors[y_e2e].to_laid_out_tensor()
      res = impl.export_to_host_tensors(out, out=[y_hosts[slot]], tensor=y_e2e)
      filled[slot] = (res[0][1], res[0][2]) if isinstance(res[0], tuple) else (0, y_hosts[slot].numel())
    return step
  step_e2e = make_step_e2e(0)

  # The lowering is a fixed launch sequence: record it once as a CUDA graph and
  # replay it per step (eager lowering per step with --eager).  `launches_per_step`
  # counts the libmtfc kernels one lowering enqueues.
  before = nat.launch_count()
  step_device()
  launches_per_step = nat.launch_count() - before
  run_device, run_e2e = step_device, step_e2e
  join_e2e = None
  y_result = None
  if not args.eager:
    try:
      y_result, run_device = impl.capture(step_device)
    except Exception as e:  # e.g. a collective that cannot be stream-captured
      sys.stderr.write("bench: CUDA-graph capture failed (%r); stepping eagerly\n" % (e,))
      args.eager = True
      torch.cuda.synchronize()
  two_streams = not args.eager and not (n > 1 and cols > 1)
  if not args.eager:
    # End to end, consecutive steps are software-pipelined: two recorded copies of
    # the step (own device buffers, own pinned output) alternate on two streams, so
    # step i+1's upload overlaps step i's compute and download.  Every step still
    # uploads its input and downloads its output inside the timed region.  Steps
    # that contain collectives stay on one stream: two streams could run
    # communication kernels in different orders on different ranks.
    replays = [impl.capture(make_step_e2e(slot))[1] for slot in range(2)]
    streams = [torch.cuda.Stream(device=device) for _ in range(2)]
    if not two_streams:
      streams[1] = streams[0]
    turn = [0]

    def run_e2e():
      k = turn[0] & 1
      turn[0] += 1
      streams[k].wait_stream(torch.cuda.current_stream())
      with torch.cuda.stream(streams[k]):
        replays[k]()

    def join_e2e():
      for st in streams:
        torch.cuda.current_stream().wait_stream(st)

  # clocks are sampled across the timed regions (the GPU is under load throughout)
  sampler = ClockSampler(local_rank)
  if rank == 0:
    sampler.start()
  ms_step, launches = bench_configs.time_steps(run_device, args.steps, args.warmup, n)
  impl.synchronize()
  # the same loop long enough (>= 0.5 s) for clocks and power to settle
  long_steps = max(args.steps, int(500.0 / max(ms_step, 1e-3)))
  ms_long, _ = bench_configs.time_steps(run_device, long_steps, 0, n)
  impl.synchronize()
  ms_e2e, _ = bench_configs.time_steps(run_e2e, args.steps, max(3, args.warmup // 2), n,
                                       join=None if args.eager else join_e2e)
  impl.synchronize()
  if not args.eager:
    launches = launches_per_step * args.steps

  # dominant kernel: per-launch duration of the two GEMMs of this rank, each
  # launch timed on its own with events on the launching stream
  gemm_ms = []
  x_arr, wi_arr, wo_arr = x_dev.tensor_list[0], wi_dev.tensor_list[0], wo_dev.tensor_list[0]
  for _ in range(3):
    h = impl.einsum("abc,cd->abd", x_arr, wi_arr, epilogue="relu")
    impl.einsum("abc,cd->abd", h, wo_arr)
  torch.cuda.synchronize()
  for _ in range(max(5, args.steps)):
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    ev[0].record()
    h = impl.einsum("abc,cd->abd", x_arr, wi_arr, epilogue="relu")
    ev[1].record()
    impl.einsum("abc,cd->abd", h, wo_arr)
    ev[2].record()
    torch.cuda.synchronize()
    gemm_ms.append((ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2])))
  del h
  clocks = sampler.stop() if rank == 0 else None
  flops_per_launch = 2.0 * b_loc * LENGTH * D_MODEL * f_loc
  avg_launch_ms = statistics.mean([a + b for a, b in gemm_ms]) / 2.0
  achieved = flops_per_launch / (avg_launch_ms * 1e-3) / 1e12
  peaks = measured_peaks()

  # ---- parity: sampled rows of this rank's output slice against float64 ----
  def reference_rows(idx):
    xr = x_host.reshape(-1, D_MODEL)[idx].to(torch.float64).numpy()
    h_ref = np.maximum(xr @ wi_bf16.to(torch.float64).numpy(), 0)
    h_ref = torch.from_numpy(h_ref).to(torch.bfloat16).to(torch.float64).numpy()
    return h_ref @ wo_bf16.to(torch.float64).numpy()
  n_rows = b_loc * LENGTH
  pick = np.random.Generator(np.random.PCG64([SEED, rank]))
  lo, hi = filled[0] if filled[0] is not None else (0, n_rows * D_MODEL)
  row_lo, row_hi = -(-lo // D_MODEL), hi // D_MODEL
  idx_dev = np.unique(np.concatenate([[0, n_rows - 1], pick.integers(0, n_rows, PARITY_ROWS - 2)]))
  idx_e2e = np.unique(np.concatenate([[row_lo, row_hi - 1], pick.integers(row_lo, row_hi, PARITY_ROWS - 2)]))
  y_final = y_result if y_result is not None else step_device()
  got_dev = ops.to_host(y_final.tensor_list[0]).reshape(n_rows, D_MODEL)[idx_dev].astype(np.float64)
  torch.cuda.synchronize()
  got_e2e = y_hosts[0].reshape(n_rows, D_MODEL)[idx_e2e].to(torch.float64).numpy()

  def rel(got, ref):
    return float(np.max(np.abs(got - ref)) / max(float(np.max(np.abs(ref))), 1e-30))
  err_dev = bench_configs._max_over_ranks(rel(got_dev, reference_rows(idx_dev)), n)
  err_e2e = bench_configs._max_over_ranks(rel(got_e2e, reference_rows(idx_e2e)), n)
  parity = {"rel_err": max(err_dev, err_e2e), "rel_err_device_path": err_dev, "rel_err_e2e_path": err_e2e,
            "rows": (len(idx_dev) + len(idx_e2e)) * n, "tolerance": 2e-2, "ok": max(err_dev, err_e2e) < 2e-2,
            "checked": "every rank's slice, max over ranks; reference = float64 numpy on the bf16 inputs"}

  cpu = None
  if rank == 0 and n == 1 and not args.skip_cpu_baseline:
    from oracle import cpu_baseline
    cores = cpu_baseline.host_threads()
    seconds, _ = cpu_baseline.time_ffn(CPU_SAMPLE_BATCH, LENGTH, D_MODEL, D_FF, "", "", steps=3, warmup=1)
    flops = cpu_baseline.ffn_flops(CPU_SAMPLE_BATCH, LENGTH, D_MODEL, D_FF)
    cpu = {"value": flops / seconds / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
           "sample": "%d of %d sequences per step (%.1f GFLOP), median of 3"
                     % (CPU_SAMPLE_BATCH, BATCH, flops / 1e9)}

  line = None
  if rank == 0:
    shared = n > 1 and cols > 1
    h2d = x_host.numel() * 2 * (rows if shared else n)
    d2h = y_host.numel() * 2 * (rows if shared else n)
    if args.eager:
      overlap = "none (eager)"
    elif two_streams:
      overlap = "two recorded steps alternate on two streams (copies overlap compute)"
    else:
      overlap = ("one stream (steps hold collectives); each cols group uploads its x slice once, "
                 "1/cols per rank + NVLink allgather, and downloads 1/cols of y per rank")
    line = {
        "metric": METRIC, "value": FLOPS_PER_STEP / (ms_step * 1e-3) / 1e12, "unit": "TFLOP/s",
        "n_gpus": n, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "dense_relu_dense FFN x[64,1024,1024] wi[1024,4096] wo[4096,1024]",
                   "mesh": mesh_shape, "layout": LAYOUT,
                   "stepping": "eager lowering" if args.eager else "CUDA-graph replay of the lowering",
                   "l2": "working set per step (>=384 MiB of activations) exceeds the 126 MB L2"},
        "sustained": {"steps": long_steps, "ms_per_step": ms_long,
                      "value": FLOPS_PER_STEP / (ms_long * 1e-3) / 1e12, "unit": "TFLOP/s",
                      "note": "the same step loop run for at least 0.5 s"},
        "e2e": {"value": FLOPS_PER_STEP / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
                "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "overlap": overlap},
        "parity": parity,
        "gpu_launches": launches,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops_burst"],
                     "unit": "TFLOP/s", "frac": achieved / peaks["tflops_burst"],
                     "frac_of_sustained_peak": achieved / peaks["tflops_sustained"],
                     "frac_of_nominal_peak": achieved / NOMINAL_BF16_TFLOPS,
                     "peak_source": "%s bf16 GEMM, burst figure (each launch is timed on its own); "
                                    "sustained %.1f, nominal dense %.0f"
                                    % (peaks["source"], peaks["tflops_sustained"], NOMINAL_BF16_TFLOPS),
                     "kernel": "einsum_gemm_tcgen05_2cta", "launch_ms": avg_launch_ms,
                     "flops_per_launch": flops_per_launch,
                     # captured on the 1-GPU launch; a rank's launch at N GPUs moves 1/N of it
                     "traffic": GEMM_DRAM_TRAFFIC_BYTES / n,
                     "traffic_source": "one ncu capture at 1 GPU" + ("" if n == 1 else ", scaled by 1/N")},
        "cpu_baseline": cpu,
        "clocks": clocks,
    }
  # the FFN's recorded graphs and buffers are not needed any more
  impl.release_graphs()
  del run_device, run_e2e, y_result, y_final
  torch.cuda.empty_cache()

  if args.only != "ffn":
    extra = {}
    try:
      extra["moe"] = bench_configs.measure_moe(n, rank, local_rank, args.steps, args.warmup,
                                               eager=args.eager)
      if rank == 0 and n == 1 and not args.skip_cpu_baseline:
        from oracle import cpu_baseline
        extra["moe"]["cpu_baseline"] = cpu_moe(cpu_baseline, np, steps=2)
      torch.cuda.empty_cache()
      attn_steps = max(3, min(args.steps, 10))
      extra["attention"] = bench_configs.measure_attention(n, rank, local_rank, attn_steps, 3, batch=16,
                                                           eager=args.eager)
      torch.cuda.empty_cache()
      if n == 1:
        extra["einsum_fp32"] = bench_configs.measure_einsum_fp32(local_rank)
        torch.cuda.empty_cache()
        # forward + backward of the two layers (mtf.gradients lowered on the same kernels)
        extra["ffn_train"] = bench_configs.measure_ffn_train(local_rank, iters=10, eager=args.eager)
        torch.cuda.empty_cache()
        extra["moe_train"] = bench_configs.measure_moe_train(1, 0, local_rank, iters=10, eager=args.eager)
    except Exception as e:  # the headline line must still be printed
      import traceback
      traceback.print_exc()
      extra["error"] = repr(e)
    if line is not None:
      line.update(extra)
  if rank == 0:
    print(json.dumps(line), flush=True)
  sys.stdout.flush()
  sys.stderr.flush()
  if n > 1:
    # Recorded CUDA graphs that hold communication kernels keep their communicator
    # alive; they were released above (measure_* release their own), so the process
    # group can be torn down.  A watchdog ends the process should teardown stall.
    threading.Timer(30.0, lambda: os._exit(0)).start()
    bench_configs.barrier_all()
    dist.destroy_process_group()
    os._exit(0)


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=200)
  ap.add_argument("--warmup", type=int, default=10)
  ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
  ap.add_argument("--only", default="all", choices=["all", "ffn"],
                  help="ffn: only the headline dense-FFN measurement")
  ap.add_argument("--skip-cpu-baseline", action="store_true")
  ap.add_argument("--mesh", default=None,
                  help="override the rows x cols mesh, e.g. rows:1,cols:2 (size must equal --gpus)")
  ap.add_argument("--stall-dump-s", type=int, default=0,
                  help="dump all Python stacks and exit if the run takes longer than this")
  ap.add_argument("--eager", action="store_true",
                  help="lower the graph afresh every step instead of replaying a CUDA graph")
  args = ap.parse_args()
  if args.impl == "reference":
    run_reference(args)
  else:
    run_ours(args)


if __name__ == "__main__":
  main()
