"""CPU oracle for the MeshImpl hot path.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline and
reference arms may import this package; the product (mesh_b200) never does.

PARITY UNPINNED for values: TensorFlow is not installed here, so the reference
(mesh_tensorflow on PlacementMeshImpl) cannot be run to generate vectors, and
its own tests pin no einsum/MoE/collective values.  The few value tests the
reference does hold on this path (top-k on split dims, layout parsing) are
restated in tests/golden/ and checked against this oracle.
"""
