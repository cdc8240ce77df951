"""ctypes binding of libmtfc.so, the C ABI declared in include/mtfc.h.

The library is loaded from the package directory.  There is no fallback: if
the shared object is missing or a call fails, an exception is raised.
"""

from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmtfc.so")

OK = 0
ERR_CUDA = -1
ERR_SHAPE = -2
ERR_TIMEOUT = -3
ERR_UNSUPPORTED = -4

F32 = 0
BF16 = 1
I32 = 2

EXCHANGE_PUSH, EXCHANGE_PULL, EXCHANGE_MULTIMEM = 0, 1, 2

EPILOGUE_NONE = 0
EPILOGUE_RELU = 1

MAX_DIMS = 8


class MtfcError(RuntimeError):
  """A libmtfc call returned a negative status."""

  def __init__(self, code, message):
    super().__init__("libmtfc error %d: %s" % (code, message))
    self.code = code


class GemmDesc(ctypes.Structure):
  """Mirror of mtfc_gemm_desc."""
  _fields_ = [
      ("batch", ctypes.c_int64), ("m", ctypes.c_int64), ("n", ctypes.c_int64),
      ("k", ctypes.c_int64),
      ("a_batch", ctypes.c_int64), ("a_m", ctypes.c_int64), ("a_k", ctypes.c_int64),
      ("b_batch", ctypes.c_int64), ("b_k", ctypes.c_int64), ("b_n", ctypes.c_int64),
      ("c_batch", ctypes.c_int64), ("c_m", ctypes.c_int64), ("c_n", ctypes.c_int64),
      ("in_dtype", ctypes.c_int32), ("out_dtype", ctypes.c_int32),
      ("epilogue", ctypes.c_int32), ("force_path", ctypes.c_int32),
  ]


_lib = None


def _declare(lib):
  vp = ctypes.c_void_p
  i32 = ctypes.c_int32
  i64 = ctypes.c_int64
  lib.mtfc_last_error.restype = ctypes.c_char_p
  lib.mtfc_last_error.argtypes = []
  lib.mtfc_version.restype = ctypes.c_int
  lib.mtfc_version.argtypes = []
  lib.mtfc_launch_count.restype = i64
  lib.mtfc_launch_count.argtypes = []
  lib.mtfc_device_status.restype = ctypes.c_int
  lib.mtfc_device_status.argtypes = []
  f32 = ctypes.c_float
  p_i64 = ctypes.POINTER(ctypes.c_int64)
  pp_i64 = ctypes.POINTER(p_i64)
  signatures = {
      "mtfc_gemm": [ctypes.POINTER(GemmDesc), vp, vp, vp, vp],
      "mtfc_gemm_uses_tensor_cores": [ctypes.POINTER(GemmDesc), vp, vp, vp],
      "mtfc_gemm_allreduce_flag_bytes": [],
      "mtfc_gemm_allreduce_set_wait_ms": [ctypes.c_int],
      "mtfc_gemm_allreduce_cooperative": [],
      "mtfc_gemm_allreduce_stage_bytes": [i64, i64, i32],
      "mtfc_gemm_allreduce": [ctypes.POINTER(GemmDesc), vp, vp, ctypes.POINTER(vp), ctypes.POINTER(vp),
                              ctypes.POINTER(vp), vp, i32, i32, vp],
      "mtfc_gemm_allreduce_ex": [ctypes.POINTER(GemmDesc), vp, vp, ctypes.POINTER(vp),
                                 ctypes.POINTER(vp), ctypes.POINTER(vp), vp, i32, i32, i32, vp, vp, vp],
      "mtfc_gemm_with_progress": [ctypes.POINTER(GemmDesc), vp, vp, vp, vp, vp],
      "mtfc_pipeline_set_wait_ms": [ctypes.c_int],
      "mtfc_wait_counters": [vp, i32, ctypes.c_uint32, vp, vp],
      "mtfc_signal_peers": [ctypes.POINTER(vp), i32, i64, vp],
      "mtfc_add_n_bf16": [ctypes.POINTER(vp), i32, vp, i64, vp],
      "mtfc_alltoall_peer_flag_bytes": [],
      "mtfc_alltoall_peer_set_wait_ms": [ctypes.c_int],
      "mtfc_alltoall_peer_set_ctas_per_sm": [ctypes.c_int],
      "mtfc_alltoall_peer": [vp, ctypes.POINTER(vp), ctypes.POINTER(vp), i32, i32, i32, p_i64, p_i64,
                             p_i64, i64, i64, i64, i32, i64, vp, vp],
      "mtfc_split_bf16x3": [vp, i64, i64, i64, vp, i64, i64, i64, i32, vp],
      "mtfc_attention_set_variant": [i32],
      "mtfc_attention_supported": [i64, p_i64, p_i64, p_i64, p_i64],
      "mtfc_attention_fwd": [vp, vp, vp, vp, i64, i64, i64, i64, i64, p_i64, p_i64, p_i64, p_i64,
                             i32, f32, vp],
      "mtfc_unary": [i32, vp, i32, vp, i32, i64, vp],
      "mtfc_binary": [i32, vp, p_i64, vp, p_i64, ctypes.c_double, vp, i32, i32, i32, p_i64, vp],
      "mtfc_broadcast_reduce": [i32, i32, ctypes.POINTER(vp), i32, vp, i32, i32, p_i64, pp_i64,
                                i32, p_i64, pp_i64, vp],
      "mtfc_topk_last": [vp, i32, i64, i32, i32, vp, vp, vp],
      "mtfc_gather_last": [vp, i32, vp, i64, i32, i32, vp, vp],
      "mtfc_one_hot": [vp, i64, i32, f32, f32, vp, i32, vp],
      "mtfc_fill": [vp, i32, i64, f32, f32, vp],
      "mtfc_copy_strided": [vp, p_i64, vp, p_i64, i32, p_i64, i32, vp],
      "mtfc_norm_rows": [vp, vp, vp, vp, i32, i64, i64, f32, i32, vp],
      "mtfc_random": [vp, i32, i64, i32, ctypes.c_uint64, f32, f32, vp],
      "mtfc_gather_rows": [vp, vp, vp, i64, i64, i32, i64, vp],
      "mtfc_xent_stats": [vp, i32, vp, i64, i64, i32, vp, vp, vp, vp],
      "mtfc_xent_grad": [vp, i32, vp, vp, vp, f32, i64, i64, i32, vp, vp],
      "mtfc_moe_split_gate_weights": [vp, i64, i32, vp, vp],
      "mtfc_moe_top2_gating": [vp, i32, i64, i32, i32, i32, i32, f32, vp, vp, vp, vp, vp, vp, vp,
                               vp, vp, vp],
      "mtfc_moe_gate_fused_supported": [i64, i32],
      "mtfc_moe_gate_padded_experts": [i32],
      "mtfc_moe_gate_scratch_bytes": [i64, i32, i32],
      "mtfc_moe_gate_prepare": [vp, i64, i32, vp, vp],
      "mtfc_moe_gate_top2": [vp, vp, i64, i32, i64, i32, i32, i32, f32, vp, vp, vp, vp, vp, vp, vp,
                             vp, vp, vp, i64, vp, i32, vp, i64, vp],
      "mtfc_moe_slot_table": [vp, vp, vp, vp, vp, vp, i64, i32, i32, i32, i32, vp, vp],
      "mtfc_moe_dispatch": [vp, vp, vp, i64, i64, i32, i32, i32, i64, vp],
      "mtfc_moe_dispatch_noalloc": [vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i32, i32, i32, i64,
                                    i32, vp],
      "mtfc_moe_dispatch_weighted": [vp, i32, vp, vp, vp, vp, vp, vp, i64, i64, i32, i32, i32, i64, vp],
      "mtfc_moe_gate_grad": [vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, i32, i64, i32, vp, vp],
      "mtfc_moe_combine_gate_grad": [vp, vp, i32, vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i32, i32,
                                     i32, i64, vp],
      "mtfc_moe_combine": [vp, i32, vp, vp, vp, vp, vp, vp, vp, i64, i64, i32, i32, i32, i64, vp],
  }
  for name, argtypes in signatures.items():
    fn = getattr(lib, name)
    fn.restype = i64 if name in ("mtfc_gemm_allreduce_stage_bytes", "mtfc_moe_gate_scratch_bytes",
                                 "mtfc_alltoall_peer_flag_bytes") else ctypes.c_int
    fn.argtypes = argtypes


def lib():
  """Returns the loaded library, loading it on first use."""
  global _lib
  if _lib is None:
    if not os.path.exists(LIB_PATH):
      raise MtfcError(
          ERR_CUDA,
          "%s is missing; build it with `python -m mesh_b200.csrc.build`" % LIB_PATH)
    loaded = ctypes.CDLL(LIB_PATH)
    _declare(loaded)
    _lib = loaded
  return _lib


def check(code):
  """Raises MtfcError for a negative status; returns the code otherwise."""
  if code < 0:
    raise MtfcError(code, lib().mtfc_last_error().decode("utf-8", "replace"))
  return code


def launch_count():
  return int(lib().mtfc_launch_count())


def device_status():
  """Synchronises the current device and raises if a kernel reported a timeout."""
  check(lib().mtfc_device_status())
