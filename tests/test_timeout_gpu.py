"""The bounded waits of the kernels that wait on other ranks run out cleanly
(the fused GEMM + allreduce, the peer-memory alltoall).

One GPU plays rank 0 of a group of two whose second member never launches:
all "peer" buffers are ordinary local allocations that nobody ever signals.
With the wait limit lowered to a few milliseconds the kernel must return by
itself, report MTFC_ERR_TIMEOUT through the device status word, and leave the
context usable: the next ordinary GEMM on the device passes.  Nothing here
faults, traps or hangs - a wait simply gives up.
"""

import ctypes

import numpy as np
import pytest

from helpers import rel_err, rng

pytestmark = pytest.mark.gpu


def test_peer_wait_runs_out_and_context_survives(cuda_device):
  import torch
  from mesh_b200 import _native as nat
  from oracle.numpy_ops import round_to_bf16
  L = nat.lib()
  nat.device_status()   # clean slate
  m, n, k, nranks = 512, 256, 128, 2
  r = rng(61)
  A = round_to_bf16(r.standard_normal((m, k)).astype(np.float32))
  B = round_to_bf16((r.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32))
  At = torch.from_numpy(A).to(torch.bfloat16).to(cuda_device)
  Bt = torch.from_numpy(np.ascontiguousarray(B.T)).to(torch.bfloat16).to(cuda_device)   # K-major
  d = nat.GemmDesc()
  d.batch, d.m, d.n, d.k = 1, m, n, k
  d.a_batch, d.a_m, d.a_k = 0, k, 1
  d.b_batch, d.b_k, d.b_n = 0, 1, k
  d.c_batch, d.c_m, d.c_n = m * n, n, 1
  d.in_dtype = d.out_dtype = nat.BF16
  d.epilogue, d.force_path = nat.EPILOGUE_NONE, 0

  stage_bytes = int(L.mtfc_gemm_allreduce_stage_bytes(m, n, nranks))
  flag_bytes = int(L.mtfc_gemm_allreduce_flag_bytes())
  bufs = {name: [torch.zeros(size, dtype=torch.uint8, device=cuda_device) for _ in range(nranks)]
          for name, size in (("stage", stage_bytes), ("out", m * n * 2), ("flags", flag_bytes))}
  ctl = torch.zeros(4, dtype=torch.int32, device=cuda_device)

  def ptrs(ts):
    return (ctypes.c_void_p * nranks)(*[ctypes.c_void_p(t.data_ptr()) for t in ts])
  stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
  nat.check(L.mtfc_gemm_allreduce_set_wait_ms(5))
  try:
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    nat.check(L.mtfc_gemm_allreduce(ctypes.byref(d), At.data_ptr(), Bt.data_ptr(), ptrs(bufs["stage"]),
                                    ptrs(bufs["out"]), ptrs(bufs["flags"]), ctl.data_ptr(), 0, nranks,
                                    stream))
    t1.record()
    with pytest.raises(nat.MtfcError) as err:
      nat.device_status()     # synchronises, reads and clears the status word
    assert err.value.code == nat.ERR_TIMEOUT
    assert t0.elapsed_time(t1) < 2000.0    # gave up after milliseconds, not the 3 s default
  finally:
    nat.check(L.mtfc_gemm_allreduce_set_wait_ms(0))
  # rank 0's own partial tiles did reach the owners' staging buffers (block 0 is its own)
  own = bufs["stage"][0][:256 * n * 2].view(torch.bfloat16).float().cpu().numpy().reshape(256, n)
  ref = A.astype(np.float64) @ B.astype(np.float64)
  assert rel_err(own, ref[:256]) < 2e-2
  # the status word is clear again and the device still computes
  nat.device_status()
  C = torch.empty((m, n), dtype=torch.bfloat16, device=cuda_device)
  nat.check(L.mtfc_gemm(ctypes.byref(d), At.data_ptr(), Bt.data_ptr(), C.data_ptr(), stream))
  nat.device_status()
  assert rel_err(C.float().cpu().numpy(), ref) < 2e-2


def test_alltoall_peer_single_rank_and_wait_that_runs_out(cuda_device):
  """mtfc_alltoall_peer alone on one GPU.  A group of one is a strided copy (its
  own signals satisfy its waits); as rank 0 of a group of two whose peer never
  launches, the "buffer free" wait runs out: nothing is stored, the status word
  reads MTFC_ERR_TIMEOUT, the context stays usable."""
  import torch
  from mesh_b200 import _native as nat
  L = nat.lib()
  nat.device_status()
  stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
  i64s = lambda vals: (ctypes.c_int64 * max(1, len(vals)))(*vals)
  r = rng(62)
  x = torch.from_numpy(r.standard_normal((6, 5, 64)).astype(np.float32)).to(cuda_device)
  flag_bytes = int(L.mtfc_alltoall_peer_flag_bytes())

  def run(nranks, out, rows_as_dims):
    flags = [torch.zeros(flag_bytes, dtype=torch.uint8, device=cuda_device) for _ in range(nranks)]
    outs = [out] + [torch.zeros_like(out) for _ in range(nranks - 1)]
    ctl = torch.zeros(2, dtype=torch.int32, device=cuda_device)
    arr = lambda ts: (ctypes.c_void_p * nranks)(*[ctypes.c_void_p(t.data_ptr()) for t in ts])
    dims, ss, ds, row = rows_as_dims
    nat.check(L.mtfc_alltoall_peer(x.data_ptr(), arr(outs), arr(flags), nranks, 0, len(dims), i64s(dims),
                                   i64s(ss), i64s(ds), row, 0, 0, 0, 0, ctl.data_ptr(), stream))
    return ctl

  # one rank, twice on the same flags: [6, 5, 64] copied as 6 x 5 rows of 256 bytes into a
  # buffer whose rows are 512 bytes apart
  out = torch.full((6, 5, 128), -1.0, dtype=torch.float32, device=cuda_device)
  layout = ([6, 5], [5 * 256, 256], [5 * 512, 512], 256)
  ctl = run(1, out, layout)
  nat.device_status()
  np.testing.assert_array_equal(out[:, :, :64].cpu().numpy(), x.cpu().numpy())
  assert (out[:, :, 64:] == -1.0).all()
  assert ctl.cpu().tolist() == [1, 0]        # one launch completed, ticket back at zero

  nat.check(L.mtfc_alltoall_peer_set_wait_ms(5))
  try:
    out2 = torch.full((6, 5, 128), -1.0, dtype=torch.float32, device=cuda_device)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    run(2, out2, layout)
    t1.record()
    with pytest.raises(nat.MtfcError) as err:
      nat.device_status()
    assert err.value.code == nat.ERR_TIMEOUT
    assert t0.elapsed_time(t1) < 2000.0
    assert (out2 == -1.0).all()              # the peer never freed its buffer: nothing was stored
  finally:
    nat.check(L.mtfc_alltoall_peer_set_wait_ms(0))
  nat.device_status()
  y = x * 2
  assert torch.equal(y.cpu(), x.cpu() * 2)
