"""Layout algebra of the MeshImpl boundary: the behaviours the reference's own
tests pin (mesh_tensorflow/ops_test.py:40-102, 173-194) plus slice shapes,
offsets and processor groups on the meshes of the benchmark configurations."""

import pytest

from mesh_b200 import mtf


@pytest.mark.parametrize("inputs", [mtf.Dimension("x", 5), ("x", 5)])
def test_convert_to_dimension(inputs):
  d = mtf.convert_to_dimension(inputs)
  assert (d.name, d.size) == ("x", 5)


def test_convert_to_dimension_generic_inputs():
  assert mtf.convert_to_dimension(None) is None
  with pytest.raises(TypeError):
    mtf.convert_to_dimension(5)


@pytest.mark.parametrize("inputs", [
    mtf.Shape([mtf.Dimension("x", 4), mtf.Dimension("y", 8)]), "x:4;y:8", "x:4.y:8", "x:4 y:8", "x:4,y:8"])
def test_convert_to_shape(inputs):
  assert mtf.convert_to_shape(inputs) == mtf.Shape([mtf.Dimension("x", 4), mtf.Dimension("y", 8)])


def test_convert_to_shape_generic_inputs():
  assert mtf.convert_to_shape([]).dims == []
  assert mtf.convert_to_shape(None) is None
  with pytest.raises(ValueError):
    mtf.convert_to_shape("x;4")


@pytest.mark.parametrize("inputs", [
    mtf.LayoutRules([("d_ff", "model"), ("heads", "model")]), "d_ff:model;heads:model",
    "d_ff:model.heads:model", "d_ff:model heads:model", "d_ff:model,heads:model",
    [("d_ff", "model"), ("heads", "model")]])
def test_convert_to_layout_rules(inputs):
  assert mtf.convert_to_layout_rules(inputs).pairs == {("d_ff", "model"), ("heads", "model")}


def test_convert_to_layout_rules_generic_inputs():
  with pytest.raises(ValueError):
    mtf.convert_to_layout_rules("d_ff;heads")


def test_tensor_layout():
  tl = mtf.TensorLayout([0, 2, 1])
  assert tl.mesh_axis_to_tensor_axis(0) == ()
  assert tl.mesh_axis_to_tensor_axis(1) == (0,)
  assert tl.mesh_axis_to_tensor_axis(2) == (0, 2)
  assert not mtf.TensorLayout([None, 0]).is_fully_replicated
  assert mtf.TensorLayout([None, None, None]).is_fully_replicated


def test_mesh_impl_layout_queries():
  shape = mtf.Shape([mtf.Dimension("batch", 4), mtf.Dimension("model", 8)])
  rules = mtf.LayoutRules([("batch", "batch"), ("d_ff", "model"), ("heads", "model")])
  impl = mtf.MeshImpl(shape=shape, layout_rules=rules)
  assert impl.shape == shape and impl.ndims == 2 and impl.size == 32
  assert impl.layout_rules is rules and impl.supports_control_dependencies
  batch, length = mtf.Dimension("batch", 128), mtf.Dimension("length", 500)
  d_ff, heads = mtf.Dimension("d_ff", 2048), mtf.Dimension("heads", 8)
  assert impl.tensor_dimension_to_mesh_axis(batch) == 0
  assert impl.tensor_dimension_to_mesh_axis(d_ff) == 1
  assert impl.tensor_dimension_to_mesh_axis(heads) == 1
  assert impl.tensor_layout(mtf.Shape([batch, length, d_ff])) == mtf.TensorLayout([0, None, 1])


def test_layout_errors():
  impl = mtf.MeshImpl("rows:2,cols:4", "batch:rows;d_ff:cols;heads:cols;x:rows;x:cols")
  with pytest.raises(ValueError):   # two tensor dims on one mesh dim
    impl.tensor_layout(mtf.convert_to_shape("d_ff:8,heads:8"))
  with pytest.raises(ValueError):   # one tensor dim on two mesh dims
    impl.tensor_layout(mtf.convert_to_shape("x:8"))
  with pytest.raises(ValueError):   # not divisible
    impl.slice_shape(mtf.convert_to_shape("batch:3,d_ff:8"))


def test_slices_and_groups_on_2x4():
  impl = mtf.MeshImpl("rows:2,cols:4", "batch:rows;d_ff:cols")
  h = mtf.convert_to_shape("batch:64,length:1024,d_ff:4096")
  assert impl.slice_shape(h) == [32, 1024, 1024]
  assert impl.slice_begin(h, 0) == [0, 0, 0]
  assert impl.slice_begin(h, 3) == [0, 0, 3072]
  assert impl.slice_begin(h, 6) == [32, 0, 2048]
  assert impl.laid_out_size(h) == 32 * 1024 * 1024 * 8
  assert impl.mesh_axis_to_cumprod(h) == [1, 64 * 1024]
  assert mtf.processor_groups(impl.shape, [0]) == [[0, 4], [1, 5], [2, 6], [3, 7]]
  assert mtf.processor_groups(impl.shape, [1]) == [[0, 1, 2, 3], [4, 5, 6, 7]]
  assert mtf.processor_groups(impl.shape, [0, 1]) == [list(range(8))]
  assert mtf.pnum_to_processor_coordinates(impl.shape, 6) == [1, 2]
  assert mtf.processor_coordinates_to_pnum(impl.shape, [1, 2]) == 6


def test_cumprod_to_tensor_axis_prefers_last():
  s = mtf.convert_to_shape("outer:1,experts:32,groups:8,cap:40,d:16")
  assert s.cumprod == [1, 1, 32, 256, 10240]
  assert s.cumprod_to_tensor_axis(1) == 1
  assert s.cumprod_to_tensor_axis(32) == 2
  assert s.cumprod_to_tensor_axis(7) is None


def test_moe_grouping_and_capacity():
  assert mtf.moe._split_into_groups(65536, 1024, 8) == (64, 1024)
  assert mtf.moe._split_into_groups(100, 30, 4) == (4, 25)
  with pytest.raises(ValueError):
    mtf.moe._split_into_groups(10, 4, 4)
  assert mtf.moe.expert_capacity(1024, 32, 1.25, 4) == 40
  assert mtf.moe.expert_capacity(16, 32, 1.25, 4) == 4
