"""The C ABI without a GPU: libmtfc.so loads, exports every function declared in
include/mtfc.h, and rejects malformed calls with a status code and a message
instead of crashing.  No kernel is launched here."""

import ctypes
import os
import re

import pytest

from mesh_b200 import _native as nat

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
  from mesh_b200.csrc.build import build_library
  build_library()
  return nat.lib()


def _declared_functions():
  text = open(os.path.join(ROOT, "include", "mtfc.h")).read()
  text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
  return sorted(set(re.findall(r"\b(mtfc_[a-z0-9_]+)\s*\(", text)))


def test_header_functions_are_exported(lib):
  names = _declared_functions()
  assert len(names) >= 19
  for name in names:
    assert hasattr(lib, name), "libmtfc.so does not export %s" % name


def test_every_exported_function_has_a_python_signature(lib):
  for name in _declared_functions():
    fn = getattr(lib, name)
    assert fn.argtypes is not None, "%s has no ctypes signature" % name


def test_version_and_error_string(lib):
  assert lib.mtfc_version() >= 1
  assert isinstance(lib.mtfc_last_error(), bytes)
  assert lib.mtfc_launch_count() >= 0


def test_empty_problems_return_ok_without_a_device(lib):
  assert lib.mtfc_unary(1, None, nat.F32, None, nat.F32, 0, None) == nat.OK
  assert lib.mtfc_fill(None, nat.F32, 0, 0.0, 0.0, None) == nat.OK
  assert lib.mtfc_one_hot(None, 0, 8, 1.0, 0.0, None, nat.F32, None) == nat.OK
  d = nat.GemmDesc()
  d.batch, d.m, d.n, d.k = 1, 0, 4, 4
  d.in_dtype = d.out_dtype = nat.F32
  buf = ctypes.create_string_buffer(64)
  assert lib.mtfc_gemm(ctypes.byref(d), buf, buf, buf, None) == nat.OK


def test_bad_arguments_are_reported_not_fatal(lib):
  d = nat.GemmDesc()
  d.batch, d.m, d.n, d.k = 1, -1, 4, 4
  d.in_dtype = d.out_dtype = nat.F32
  buf = ctypes.create_string_buffer(64)
  assert lib.mtfc_gemm(ctypes.byref(d), buf, buf, buf, None) == nat.ERR_SHAPE
  assert b"negative" in lib.mtfc_last_error()
  d.m, d.in_dtype = 4, 99
  assert lib.mtfc_gemm(ctypes.byref(d), buf, buf, buf, None) == nat.ERR_UNSUPPORTED
  assert lib.mtfc_gemm(ctypes.byref(d), None, buf, buf, None) == nat.ERR_SHAPE
  with pytest.raises(nat.MtfcError) as info:
    nat.check(lib.mtfc_moe_top2_gating(buf, 1, 1, 16, 1, 4, 0, 0.2, None, buf, buf, buf, buf,
                                       buf, buf, None, buf, None))
  assert info.value.code == nat.ERR_SHAPE and "experts" in str(info.value)
  assert lib.mtfc_moe_dispatch(buf, buf, buf, 1, 1, 16, 4, 4, 24, None) == nat.ERR_SHAPE
  assert lib.mtfc_copy_strided(buf, None, buf, None, 0, None, 3, None) == nat.ERR_UNSUPPORTED


def test_cuda_mesh_impl_refuses_to_run_without_a_device():
  import torch
  if torch.cuda.is_available():
    pytest.skip("a CUDA device is visible")
  from mesh_b200.cuda_mesh_impl import CudaMeshImpl
  with pytest.raises(nat.MtfcError):
    CudaMeshImpl("all:2", "batch:all", [0, 0])
