"""local_attention_1d on the oracle backend against sliding-window attention written
out in numpy; with the length split over a mesh axis the neighbours' margins travel
by MeshImpl.receive (halo exchange)."""

import numpy as np
import pytest

from mesh_b200 import mtf
from oracle.numpy_mesh_impl import NumpyMeshImpl
from helpers import rel_err, rng

BATCH, LENGTH, KEY, VALUE = 2, 256, 8, 6


def _window_attention(q, k, v, radius, autoregressive, sequence=None):
  out = np.zeros(q.shape[:-1] + (v.shape[-1],))
  for b in range(q.shape[0]):
    for p in range(LENGTH):
      lo, hi = p - radius + 1, (p if autoregressive else p + radius)
      cols = [j for j in range(max(lo, 0), min(hi, LENGTH - 1) + 1)
              if sequence is None or sequence[j] == sequence[p]]
      logits = q[b, p] @ k[b, cols].T
      w = np.exp(logits - logits.max())
      out[b, p] = (w / w.sum()) @ v[b, cols]
  return out


@pytest.mark.parametrize("mesh_shape,layout,splits", [("all:1", "", 1), ("all:2", "length:all", 2)])
@pytest.mark.parametrize("autoregressive", [True, False])
def test_local_attention_is_sliding_window_attention(mesh_shape, layout, splits, autoregressive):
  r = rng(61)
  q, k = [r.standard_normal((BATCH, LENGTH, KEY)).astype(np.float32) for _ in range(2)]
  v = r.standard_normal((BATCH, LENGTH, VALUE)).astype(np.float32)
  g = mtf.Graph()
  m = mtf.Mesh(g, "m")
  length, key, value = mtf.Dimension("length", LENGTH), mtf.Dimension("d_k", KEY), mtf.Dimension("d_v", VALUE)
  Q = mtf.import_tf_tensor(m, q, "batch:%d,length:%d,d_k:%d" % (BATCH, LENGTH, KEY))
  K = mtf.import_tf_tensor(m, k, "batch:%d,length:%d,d_k:%d" % (BATCH, LENGTH, KEY))
  V = mtf.import_tf_tensor(m, v, "batch:%d,length:%d,d_v:%d" % (BATCH, LENGTH, VALUE))
  out = mtf.layers.local_attention_1d(Q, K, V, length, key, value, fully_autoregressive=autoregressive,
                                      length_dim_num_splits=splits, radius=20)
  assert [d.name for d in out.shape.dims] == ["batch", "length", "d_v"]
  low = mtf.Lowering(g, {m: NumpyMeshImpl(mesh_shape, layout)})
  got = low.export_to_tf_tensor(out)
  assert rel_err(got, _window_attention(q, k, v, 20, autoregressive)) < 1e-5
  # the neighbours' margins are processor shifts (MeshImpl.receive when the length is split)
  assert any(type(op).__name__ == "ShiftOperation" for op in g.operations)


def test_local_attention_respects_sequence_boundaries_and_keys_as_values():
  r = rng(62)
  q, k = [r.standard_normal((BATCH, LENGTH, KEY)).astype(np.float32) for _ in range(2)]
  sequence = (np.arange(LENGTH) // 50 + 1).astype(np.int32)        # packed sequences of 50 positions
  g = mtf.Graph()
  m = mtf.Mesh(g, "m")
  length, key = mtf.Dimension("length", LENGTH), mtf.Dimension("d_k", KEY)
  Q = mtf.import_tf_tensor(m, q, "batch:%d,length:%d,d_k:%d" % (BATCH, LENGTH, KEY))
  K = mtf.import_tf_tensor(m, k, "batch:%d,length:%d,d_k:%d" % (BATCH, LENGTH, KEY))
  S = mtf.import_tf_tensor(m, sequence, "length:%d" % LENGTH, dtype=mtf.int32)
  out = mtf.layers.local_attention_1d(Q, K, None, length, key, key, radius=32, sequence_id=S)
  got = mtf.Lowering(g, {m: NumpyMeshImpl("all:1", "")}).export_to_tf_tensor(out)
  assert rel_err(got, _window_attention(q, k, k, 32, True, sequence)) < 1e-5
