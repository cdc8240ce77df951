"""The training step of tests/test_training_loop.py (embedding, norms, causal attention,
top-2 MoE with its fused operations and their backward operations, vocabulary-split
cross-entropy, Adafactor) on the device kernels: losses of the first steps against the
oracle backend, on one processor and on a 2x2 mesh of slices sharing the GPU."""

import numpy as np
import pytest

from mesh_b200 import mtf
from helpers import rng
from test_training_loop import _training_graph

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mesh_shape,layout", [
    ("all:1", ""), ("rows:2,cols:2", "batch:rows;experts:rows;heads:cols;vocab:cols")])
def test_training_steps_match_oracle(cuda_device, mesh_shape, layout):
  from mesh_b200.cuda_mesh_impl import CudaMeshImpl
  from oracle.numpy_mesh_impl import NumpyMeshImpl
  n = mtf.convert_to_shape(mesh_shape).size

  def run(impl):
    g, m, loss, _ = _training_graph(mesh_shape, layout)
    return [float(mtf.Lowering(g, {m: impl}).export_to_tf_tensor(loss)) for _ in range(4)]
  ref = run(NumpyMeshImpl(mesh_shape, layout))
  got = run(CudaMeshImpl(mesh_shape, layout, [0] * n))
  assert ref[-1] < ref[0]
  np.testing.assert_allclose(got, ref, rtol=2e-3)
