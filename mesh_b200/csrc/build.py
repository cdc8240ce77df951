"""Builds libmtfc.so (the sm_100a kernels and their C ABI) in-tree with nvcc.

Usage: python -m mesh_b200.csrc.build [--force]

Each .cu file is compiled to an object file for sm_100a only and the objects
are linked into mesh_b200/libmtfc.so.  nvcc cross-compiles, so no GPU is needed.
"""

from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)
LIB_PATH = os.path.join(PKG, "libmtfc.so")
OBJ_DIR = os.path.join(HERE, "build")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + [
    "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
    "--expt-relaxed-constexpr", "-cudart", "shared",
]


def _nvcc() -> str:
  exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
  if not os.path.exists(exe):
    raise RuntimeError("nvcc not found; libmtfc.so cannot be built")
  return exe


def sources() -> list[str]:
  return sorted(
      os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith(".cu"))


def _deps_mtime() -> float:
  deps = sources() + [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith(".cuh")]
  deps.append(os.path.join(ROOT, "include", "mtfc.h"))
  return max(os.path.getmtime(p) for p in deps)


def _compile(src: str) -> tuple[str, str]:
  obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
  cmd = [_nvcc()] + NVCC_FLAGS + ["-c", src, "-o", obj]
  res = subprocess.run(cmd, capture_output=True, text=True)
  if res.returncode != 0:
    raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, res.stdout, res.stderr))
  return obj, res.stderr


def build_library(force: bool = False, verbose: bool = False) -> str:
  """Compiles and links libmtfc.so if it is missing or older than its sources."""
  if (not force and os.path.exists(LIB_PATH)
      and os.path.getmtime(LIB_PATH) >= _deps_mtime()):
    return LIB_PATH
  os.makedirs(OBJ_DIR, exist_ok=True)
  with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
    results = list(pool.map(_compile, sources()))
  objs = [o for o, _ in results]
  if verbose:
    for _, log in results:
      sys.stderr.write(log)
  cuda_lib = os.path.join(os.path.dirname(os.path.dirname(_nvcc())), "lib64")
  cmd = [_nvcc()] + ARCH_FLAGS + ["-shared", "-cudart", "shared", "-o", LIB_PATH] + objs + [
      "-Xlinker", "-rpath," + cuda_lib]
  res = subprocess.run(cmd, capture_output=True, text=True)
  if res.returncode != 0:
    raise RuntimeError("link failed:\n%s\n%s" % (res.stdout, res.stderr))
  return LIB_PATH


if __name__ == "__main__":
  path = build_library(force="--force" in sys.argv, verbose=True)
  print(path)
