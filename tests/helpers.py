"""Shared test helpers: seeded inputs, error metrics, and a CPU stand-in for
CudaMeshImpl's slice holder so the collective plumbing runs without a GPU."""

from __future__ import annotations

import numpy as np
import torch

from mesh_b200 import mtf
from mesh_b200.cuda_mesh_impl import SlicedMeshImpl
from oracle.numpy_ops import Arr, NumpyOps


def rng(seed):
  return np.random.Generator(np.random.PCG64(seed))


def rel_err(got, ref):
  """max |got - ref| / max |ref| — the parity metric for floating outputs."""
  got = np.asarray(got, dtype=np.float64)
  ref = np.asarray(ref, dtype=np.float64)
  return float(np.max(np.abs(got - ref)) / max(float(np.max(np.abs(ref))), 1e-30))


class NumpySlicedMeshImpl(SlicedMeshImpl):
  """SlicedMeshImpl over numpy slices: the same grouping / packing / process
  group code CudaMeshImpl runs, with the oracle's array library underneath."""

  def __init__(self, shape, layout, distributed=False, rank=0):
    mesh_shape = mtf.convert_to_shape(shape)
    local = [rank] if distributed else list(range(mesh_shape.size))
    super().__init__(mesh_shape, layout, local, distributed)
    self._ops = NumpyOps()

  @property
  def slice_ops(self):
    return self._ops

  def _ops_for(self, pnum):
    return self._ops

  def _is_slice(self, x):
    return isinstance(x, Arr)

  def _as_torch(self, s):
    return torch.from_numpy(np.ascontiguousarray(s.a).reshape(-1).copy())

  def _from_torch(self, t, shape, dtype, pnum):
    return Arr(t.numpy().reshape(shape), dtype)
