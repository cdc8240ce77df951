"""Three Adafactor training steps on CudaMeshImpl against the oracle backend:
weights and optimizer slots stay on the device between lowerings."""

import numpy as np
import pytest

from mesh_b200 import mtf
from helpers import rel_err, rng

pytestmark = pytest.mark.gpu


def _train(impl, steps=3):
  r = rng(95)
  b, d, f = 64, 128, 256
  x = r.standard_normal((b, d)).astype(np.float32)
  t = r.standard_normal((b, d)).astype(np.float32)
  g = mtf.Graph()
  m = mtf.Mesh(g, "m")
  X = mtf.import_tf_tensor(m, x, "batch:%d,d_model:%d" % (b, d), dtype=mtf.float32)
  T = mtf.import_tf_tensor(m, t, "batch:%d,d_model:%d" % (b, d), dtype=mtf.float32)
  WI = mtf.get_variable(m, "wi", "d_model:%d,d_ff:%d" % (d, f),
                        initial_value=(r.standard_normal((d, f)) / np.sqrt(d)).astype(np.float32))
  WO = mtf.get_variable(m, "wo", "d_ff:%d,d_model:%d" % (f, d),
                        initial_value=(r.standard_normal((f, d)) / np.sqrt(f)).astype(np.float32))
  S = mtf.get_variable(m, "scale", "d_model:%d" % d, initial_value=np.ones(d, np.float32))
  y = mtf.layers.dense_relu_dense(mtf.layers.rms_norm(X, X.shape.dims[1], scale=S),
                                  mtf.Dimension("d_ff", f), wi=WI, wo=WO)
  loss = mtf.reduce_mean(mtf.square(y - T))
  variables = [WI, WO, S]
  grads = mtf.gradients([loss], variables)
  mtf.optimize.AdafactorOptimizer(learning_rate=0.05, decay_rate=0.8).apply_grads(grads, variables)
  losses = []
  for _ in range(steps):
    low = mtf.Lowering(g, {m: impl})
    losses.append(float(np.asarray(low.export_to_tf_tensor(loss))))
  low.copy_slices_to_masters()
  return losses, {v.name: np.asarray(v.get_master(), np.float64) for v in g.all_variables}


@pytest.mark.parametrize("mesh_shape,layout", [("all:1", ""), ("a:2,b:2", "batch:a;d_ff:b")])
def test_adafactor_steps_on_device(cuda_device, mesh_shape, layout):
  from mesh_b200.cuda_mesh_impl import CudaMeshImpl
  from oracle.numpy_mesh_impl import NumpyMeshImpl
  n = mtf.convert_to_shape(mesh_shape).size
  got_losses, got = _train(CudaMeshImpl(mesh_shape, layout, [0] * n))
  ref_losses, ref = _train(NumpyMeshImpl(mesh_shape, layout))
  assert got_losses[-1] < got_losses[0]
  np.testing.assert_allclose(got_losses, ref_losses, rtol=1e-4)
  assert sorted(got) == sorted(ref)
  for name in ref:
    assert rel_err(got[name], ref[name]) < 1e-4, name
