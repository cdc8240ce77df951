"""mtfc_gemm through the C ABI: tcgen05 path over operand layouts, tile edges,
batches and epilogues; FFMA path for fp32 / int32; against float64 numpy."""

import ctypes

import numpy as np
import pytest

from helpers import rel_err, rng

pytestmark = pytest.mark.gpu


def _run(dev, batch, m, n, k, a_mn, b_mn, out_f32, relu, in_dtype="bf16", force=0, b_batched=True, seed=0):
  import torch
  from mesh_b200 import _native as nat
  from oracle.numpy_ops import round_to_bf16
  L = nat.lib()
  r = rng(seed)
  A = r.standard_normal((batch, m, k)).astype(np.float32)
  B = (r.standard_normal((batch if b_batched else 1, k, n)) / np.sqrt(k)).astype(np.float32)
  if in_dtype == "bf16":
    A, B = round_to_bf16(A), round_to_bf16(B)
  elif in_dtype == "i32":
    A, B = np.round(A * 4), np.round(B * 16)
  ref = np.matmul(A.astype(np.float64), B.astype(np.float64))
  if relu:
    ref = np.maximum(ref, 0)
  tdt = {"bf16": torch.bfloat16, "f32": torch.float32, "i32": torch.int32}[in_dtype]
  code = {"bf16": nat.BF16, "f32": nat.F32, "i32": nat.I32}[in_dtype]
  At = torch.from_numpy(np.ascontiguousarray(A.transpose(0, 2, 1) if a_mn else A)).to(tdt).to(dev)
  Bt = torch.from_numpy(np.ascontiguousarray(B if b_mn else B.transpose(0, 2, 1))).to(tdt).to(dev)
  odt = torch.float32 if out_f32 else tdt
  C = torch.full((batch, m, n), -77, dtype=odt, device=dev)
  d = nat.GemmDesc()
  d.batch, d.m, d.n, d.k = batch, m, n, k
  d.a_m, d.a_k = (1, m) if a_mn else (k, 1)
  d.a_batch = m * k
  d.b_k, d.b_n = (n, 1) if b_mn else (1, k)
  d.b_batch = k * n if b_batched else 0
  d.c_batch, d.c_m, d.c_n = m * n, n, 1
  d.in_dtype = code
  d.out_dtype = nat.F32 if out_f32 else code
  d.epilogue = nat.EPILOGUE_RELU if relu else nat.EPILOGUE_NONE
  d.force_path = force
  used_tc = L.mtfc_gemm_uses_tensor_cores(ctypes.byref(d), At.data_ptr(), Bt.data_ptr(), C.data_ptr())
  st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
  nat.check(L.mtfc_gemm(ctypes.byref(d), At.data_ptr(), Bt.data_ptr(), C.data_ptr(), st))
  nat.device_status()
  return C.float().cpu().numpy(), ref, used_tc


@pytest.mark.parametrize("force", [3, 4], ids=["single-cta", "cta-pair"])
@pytest.mark.parametrize("a_mn", [0, 1])
@pytest.mark.parametrize("b_mn", [0, 1])
@pytest.mark.parametrize("shape", [(1, 128, 256, 64), (1, 200, 264, 72), (3, 136, 80, 200),
                                   (1, 1024, 512, 1024), (1, 9728, 512, 128), (2, 8, 8, 8),
                                   (2, 600, 520, 328)])
def test_tcgen05_layouts(cuda_device, shape, a_mn, b_mn, force):
  """Both tensor-core kernels (force_path 3: one CTA per 128x256 tile, 4: a CTA
  pair per 256x256 tile) over all four operand-majorness combinations."""
  batch, m, n, k = shape
  got, ref, used = _run(cuda_device, batch, m, n, k, a_mn, b_mn, out_f32=True, relu=False, force=force)
  assert used == 1
  assert rel_err(got, ref) < 1e-5   # exact bf16 products, fp32 accumulation
  got, ref, _ = _run(cuda_device, batch, m, n, k, a_mn, b_mn, out_f32=False, relu=True, force=force)
  assert rel_err(got, ref) < 2e-2


def test_tcgen05_broadcast_weights(cuda_device):
  got, ref, used = _run(cuda_device, 4, 130, 304, 96, 0, 1, True, True, force=1, b_batched=False)
  assert used == 1 and rel_err(got, ref) < 1e-5


def test_forced_tensor_cores_rejects_bad_strides(cuda_device):
  from mesh_b200 import _native as nat
  with pytest.raises(nat.MtfcError):
    _run(cuda_device, 1, 64, 300, 96, 0, 1, True, False, force=1)   # row stride 300 % 8 != 0


@pytest.mark.parametrize("in_dtype,tol", [("f32", 1e-5), ("bf16", 2e-2), ("i32", 0.0)])
@pytest.mark.parametrize("a_mn,b_mn", [(0, 1), (1, 0)])
def test_ffma_path(cuda_device, in_dtype, tol, a_mn, b_mn):
  got, ref, used = _run(cuda_device, 2, 131, 70, 33, a_mn, b_mn, out_f32=(in_dtype != "i32"), relu=False,
                        in_dtype=in_dtype, force=2)
  assert used == 0
  assert rel_err(got, ref) <= tol


def test_fp32_einsum_tolerance_cfg1_shape(cuda_device):
  """x[1024,1024] . w[1024,4096] in fp32: one processor's share of the 4-way
  batch-split einsum; 1e-5 relative."""
  got, ref, used = _run(cuda_device, 1, 1024, 4096, 1024, 0, 1, True, False, in_dtype="f32")
  assert used == 0 and rel_err(got, ref) < 1e-5
