"""mtfc_moe_dispatch_noalloc — the dispatch entry point for callers that must
not allocate device memory (a process whose GPU memory was planned and frozen
at start-up, or a latency-critical path where cudaMalloc's device-wide stall
is not acceptable).  Its routing table sits in a fixed array inside the
library instead of a caller-provided buffer.

Called through the C ABI and compared, bit for bit, with the existing two-call
form (mtfc_moe_slot_table + mtfc_moe_dispatch) on two calls in a row with
different problems, so that whatever the first call left in the shared array
cannot show up in the second result.  Collected last on purpose.
"""

import ctypes

import numpy as np
import pytest

from helpers import rng

pytestmark = pytest.mark.gpu


def _problem(dev, seed, outer, groups, s, e, cap, m):
  import torch
  from oracle import moe_spec
  r = rng(seed)
  logits = (r.standard_normal((outer * groups, s, e)) * 2).astype(np.float32)
  spec = moe_spec.gating_from_raw(moe_spec.softmax_f32(logits), cap, "all")
  x = torch.from_numpy(r.standard_normal((outer, groups, s, m)).astype(np.float32)).to(torch.bfloat16).to(dev)
  ints = [torch.from_numpy(spec[k].astype(np.int32)).to(dev)
          for k in ("index_1", "index_2", "position_1", "position_2")]
  gates = [torch.from_numpy(spec[k].astype(np.float32)).to(dev) for k in ("gate_1", "gate_2")]
  return x, ints + gates


def _both_paths(dev, seed, outer, groups, s, e, cap, m):
  import torch
  from mesh_b200 import _native as nat
  L = nat.lib()
  x, routing = _problem(dev, seed, outer, groups, s, e, cap, m)
  stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
  ptrs = [t.data_ptr() for t in routing]
  # existing entry points: the caller brings the table
  table = torch.empty(outer * groups * e * cap, dtype=torch.int32, device=dev)
  ref = torch.full((outer, e, groups, cap, m), 7.0, dtype=torch.bfloat16, device=dev)
  nat.check(L.mtfc_moe_slot_table(*ptrs, outer * groups, s, e, cap, 1, table.data_ptr(), stream))
  nat.check(L.mtfc_moe_dispatch(x.data_ptr(), table.data_ptr(), ref.data_ptr(), outer, groups, s,
                                e, cap, m * 2, stream))
  # the entry point under test: inputs and output only
  got = torch.full((outer, e, groups, cap, m), -7.0, dtype=torch.bfloat16, device=dev)
  torch.cuda.synchronize()
  free_before = torch.cuda.mem_get_info(dev)[0]
  torch_allocs_before = torch.cuda.memory_stats(dev).get("allocation.all.allocated", 0)
  nat.check(L.mtfc_moe_dispatch_noalloc(x.data_ptr(), *ptrs, got.data_ptr(), outer, groups, s, e,
                                        cap, m * 2, 1, stream))
  torch.cuda.synchronize()
  noalloc_deltas = (free_before - torch.cuda.mem_get_info(dev)[0],
                    torch.cuda.memory_stats(dev).get("allocation.all.allocated", 0) - torch_allocs_before)
  return got.float().cpu().numpy(), ref.float().cpu().numpy(), noalloc_deltas


def test_noalloc_dispatch_matches_two_call_form_twice_in_a_row(cuda_device):
  first = _both_paths(cuda_device, 41, outer=2, groups=6, s=256, e=16, cap=24, m=128)
  second = _both_paths(cuda_device, 42, outer=1, groups=3, s=96, e=8, cap=40, m=64)
  for got, ref, _ in (first, second):
    assert got.shape == ref.shape
    np.testing.assert_array_equal(got, ref)
    assert np.abs(ref).max() > 0
  # Nothing was allocated by the second call: the device's free memory and the count
  # of allocations made through torch are what they were just before it.  (The first
  # call on a device may load the kernels' module; that is set-up, not the steady state.)
  assert second[2] == (0, 0), "the no-alloc entry point changed device memory: %s" % (second[2],)
  # 320 slots per group for 192 (token, choice) pairs: empty slots must be zero rows
  assert (np.abs(second[1]).max(axis=-1) == 0).any()


def test_noalloc_dispatch_rejects_oversized_problems(cuda_device):
  import torch
  from mesh_b200 import _native as nat
  L = nat.lib()
  buf = torch.zeros(64, dtype=torch.int32, device=cuda_device)
  p = buf.data_ptr()
  launches = L.mtfc_launch_count()
  rc = L.mtfc_moe_dispatch_noalloc(p, p, p, p, p, p, p, p, 1, 4096, 64, 32, 40, 128, 1, None)
  assert rc == nat.ERR_SHAPE                      # 4096*32*40 entries > 1,048,576
  assert b"exceeds the built-in scratch" in L.mtfc_last_error()
  assert L.mtfc_launch_count() == launches        # nothing was launched
