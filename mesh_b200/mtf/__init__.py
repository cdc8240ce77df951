"""A minimal Mesh TensorFlow front-end: named shapes, layouts, graph, lowering.

The names mirror `import mesh_tensorflow as mtf` so graphs written against the
reference read the same here.
"""

from mesh_b200.mtf.graph import (DType, Graph, Lowering, Mesh, Operation, Tensor, bfloat16,
                                 bool_, float32, int32)
from mesh_b200.mtf.layout import (LayoutRules, TensorLayout, convert_to_layout_rules,
                                  pnum_to_group, pnum_to_processor_coordinates,
                                  processor_coordinates_to_pnum, processor_groups,
                                  tensor_dim_to_mesh_dim_size)
from mesh_b200.mtf.mesh_impl import (LazyAllreduceSum, LazyLaidOutTensor, MeshImpl, compatible_lazy_allreduce_sums,
                                     convert_args_to_laid_out_tensors, expand_dims_to)
from mesh_b200.mtf.ops import *  # noqa: F401,F403
from mesh_b200.mtf.ops import mtf_range as range  # noqa: A001
from mesh_b200.mtf.shapes import (Dimension, Shape, convert_to_dimension, convert_to_shape,
                                  list_product, parse_pairs, shape_union)
from mesh_b200.mtf import layers, moe, optimize  # noqa: E402
