"""CubReduction::analyzeGeometry on dense tensors and on strided views, restated from the reference's own
test/Utilities/TensorOperations/CubReductionGeometryTest.cpp:12-397 as data (same shapes, strides, axes and expected
fields).  No GPU needed."""
import itertools

import pytest

from thor_b200.reductions import CubReductionPath as P
from thor_b200.reductions import analyze_geometry_full as geom
from thor_b200.reductions import map_logical_reduction_index as map_index

NATURAL, PERMUTED = 0, 1


def _check(g, **want):
    for key, value in want.items():
        assert g[key] == value, (key, g[key], value)


def test_selects_the_best_single_axis_path():  # CubReductionGeometryTest.cpp:12-40
    _check(geom([257], [0]), path=P.DeviceTransformReduce, reduced_axes_are_contiguous=1, outer_size=1, reduction_size=257, inner_size=1,
           output_elements=1, output_dimensions=[1])
    _check(geom([2, 3, 4], [2]), path=P.ContiguousFixedSegment, outer_size=6, reduction_size=4, inner_size=1, output_elements=6, output_dimensions=[2, 3, 1])
    _check(geom([2, 3, 4], [1]), path=P.TiledFixedSegment, outer_size=2, reduction_size=3, inner_size=4, output_elements=8, output_dimensions=[2, 1, 4])


def test_rejects_invalid_geometry():  # :42-46, :122-137
    for dims, axes in (([], [0]), ([2, 3], [2]), ([2, 0, 3], [1]), ([2, 3], []), ([2, 3], [0, 0]), ([2, 3], [1, 0]), ([2, 3], [0, 2]), ([2, 0, 3], [0, 2])):
        with pytest.raises(Exception):
            geom(dims, axes)


def test_selects_the_best_multi_axis_path_and_shapes():  # :48-120
    _check(geom([2, 3, 4], [0, 1, 2]), path=P.DeviceTransformReduce, outer_size=1, inner_size=1, input_elements=24, reduction_size=24, output_elements=1,
           output_dimensions=[1, 1, 1], squeezed_output_dimensions=[1])
    _check(geom([2, 3, 4, 5], [2, 3]), path=P.ContiguousFixedSegment, outer_size=6, reduction_size=20, inner_size=1, output_elements=6,
           output_dimensions=[2, 3, 1, 1], squeezed_output_dimensions=[2, 3])
    _check(geom([2, 3, 4, 5], [1, 2]), path=P.TiledFixedSegment, outer_size=2, reduction_size=12, inner_size=5, output_elements=10,
           output_dimensions=[2, 1, 1, 5], squeezed_output_dimensions=[2, 5])
    _check(geom([2, 3, 4, 5], [1, 3]), path=P.StridedFixedSegment, reduced_axes_are_contiguous=0, outer_size=0, reduction_size=15, inner_size=0,
           output_elements=8, output_dimensions=[2, 1, 4, 1], squeezed_output_dimensions=[2, 4])
    _check(geom([2, 3, 4], [0, 1]), path=P.TiledFixedSegment, outer_size=1, reduction_size=6, inner_size=4, output_dimensions=[1, 1, 4], squeezed_output_dimensions=[4])
    _check(geom([2, 3, 1], [1]), path=P.ContiguousFixedSegment, outer_size=2, reduction_size=3, inner_size=1, output_elements=2)
    _check(geom([1, 3, 1], [1]), path=P.DeviceTransformReduce, outer_size=1, reduction_size=3, inner_size=1, output_elements=1)


def test_rank_nine_and_the_logical_index_map():  # :139-156
    dims, axes = [2, 1, 2, 1, 2, 1, 2, 1, 2], [0, 2, 4, 6]
    _check(geom(dims, axes), rank=9, path=P.StridedFixedSegment, input_elements=32, reduction_size=16, output_elements=2,
           output_dimensions=[1, 1, 1, 1, 1, 1, 1, 1, 2], reduced_axes=axes)
    assert map_index(dims, axes, 0, 15) == 30 and map_index(dims, axes, 1, 15) == 31


def test_the_logical_index_map_is_a_bijection_onto_row_major_coordinates():  # :158-222
    for dims in ([2], [2, 3], [2, 1, 3], [2, 3, 2, 1]):
        rank = len(dims)
        for mask in range(1, 1 << rank):
            axes = [a for a in range(rank) if mask & (1 << a)]
            kept = [a for a in range(rank) if not mask & (1 << a)]
            g = geom(dims, axes)
            seen = set()
            for out, red in itertools.product(range(g["output_elements"]), range(g["reduction_size"])):
                coords = [0] * rank
                o, r = out, red
                for a in reversed(kept):
                    coords[a], o = o % dims[a], o // dims[a]
                for a in reversed(axes):
                    coords[a], r = r % dims[a], r // dims[a]
                want = 0
                for a in range(rank):
                    want = want * dims[a] + coords[a]
                got = map_index(dims, axes, out, red)
                assert got == want and got not in seen
                seen.add(got)
            assert len(seen) == g["input_elements"]
    with pytest.raises(Exception):
        map_index([2, 3, 4], [0, 2], 3, 0)
    with pytest.raises(Exception):
        map_index([2, 3, 4], [0, 2], 0, 8)


def test_permutation_aware_tiled_path_for_a_dense_physical_permutation():  # :224-254
    I, J, K = 7, 5, 32
    g = geom([K, I, J], [2], strides=[1, J * K, K])  # logical [K, I, J] over physically dense [I, J, K]
    _check(g, path=P.TiledFixedSegment, device_transform_uses_affine_stride=0, physical_layout_is_dense_permutation=1,
           physical_non_singleton_axis_order=[1, 2, 0], outer_size=I, reduction_size=J, inner_size=K, tiled_output_permuted=1,
           tiled_output_shared_transpose=1, tiled_output_outer_stride=1, tiled_output_inner_stride=I)
    _check(g["permutation_aware_tiled_geometry"], physical_outer_axes=[1], physical_reduction_axes=[2], physical_inner_axes=[0],
           logical_non_singleton_retained_axes=[0, 1], outer_size=I, reduction_size=J, inner_size=K, retained_output_order=PERMUTED)


def test_natural_retained_order_for_a_dense_physical_permutation():  # :256-276
    g = geom([5, 7, 32], [0], strides=[32, 160, 1])
    _check(g, path=P.TiledFixedSegment, physical_layout_is_dense_permutation=1, physical_non_singleton_axis_order=[1, 0, 2], outer_size=7, reduction_size=5,
           inner_size=32, tiled_output_permuted=0, tiled_output_shared_transpose=0, tiled_output_outer_stride=32, tiled_output_inner_stride=1)
    _check(g["permutation_aware_tiled_geometry"], physical_outer_axes=[1], physical_reduction_axes=[0], physical_inner_axes=[2], retained_output_order=NATURAL)


def test_planning_does_not_depend_on_the_storage_offset():  # :278-297 (the offset lives in the pointer, not in the geometry)
    g = geom([32, 7, 5], [2], strides=[1, 160, 32])
    _check(g, path=P.TiledFixedSegment, physical_layout_is_dense_permutation=1, tiled_output_shared_transpose=1, tiled_output_outer_stride=1, tiled_output_inner_stride=7)
    _check(g["permutation_aware_tiled_geometry"], outer_size=7, reduction_size=5, inner_size=32, retained_output_order=PERMUTED)


def test_singleton_axes_do_not_hide_a_dense_permutation():  # :299-322
    g = geom([4, 1, 2, 3], [3], strides=[1, 12, 12, 4])
    _check(g, path=P.TiledFixedSegment, physical_layout_is_dense_permutation=1, physical_non_singleton_axis_order=[2, 3, 0], outer_size=2, reduction_size=3,
           inner_size=4, tiled_output_permuted=1, tiled_output_shared_transpose=1, tiled_output_outer_stride=1, tiled_output_inner_stride=2)
    _check(g["permutation_aware_tiled_geometry"], physical_outer_axes=[2], physical_reduction_axes=[3], physical_inner_axes=[0],
           logical_non_singleton_retained_axes=[0, 2], retained_output_order=PERMUTED)


def test_logically_disjoint_axes_that_are_one_physical_block_use_the_tiled_path():  # :324-341
    g = geom([3, 2, 5, 7], [0, 2], strides=[35, 105, 7, 1])
    _check(g, reduced_axes_are_contiguous=0, path=P.TiledFixedSegment, outer_size=2, reduction_size=15, inner_size=7, tiled_output_permuted=0)
    _check(g["permutation_aware_tiled_geometry"], physical_outer_axes=[1], physical_reduction_axes=[0, 2], physical_inner_axes=[3])


def test_gapped_overlapping_and_broadcast_storage_are_not_dense_permutations():  # :343-361
    for strides in ([1, 7, 2], [1, 1, 2], [0, 6, 2]):
        g = geom([2, 2, 3], [2], strides=strides)
        _check(g, path=P.StridedFixedSegment, physical_layout_is_dense_permutation=0, permutation_aware_tiled_geometry=None)


def test_split_reduction_blocks_and_unsupported_retained_orders_fall_back():  # :363-378
    g = geom([3, 5, 2, 7], [1, 2], strides=[35, 7, 105, 1])
    _check(g, physical_layout_is_dense_permutation=1, physical_non_singleton_axis_order=[2, 0, 1, 3], permutation_aware_tiled_geometry=None, path=P.StridedFixedSegment)
    g = geom([3, 5, 2, 7], [0], strides=[35, 7, 105, 1])
    _check(g, physical_layout_is_dense_permutation=1, permutation_aware_tiled_geometry=None, path=P.StridedFixedSegment)


def test_dense_and_affine_path_selection():  # :380-397
    _check(geom([2, 3, 4], [1]), path=P.TiledFixedSegment, physical_layout_is_dense_permutation=1, permutation_aware_tiled_geometry=None)
    g = geom([3], [0], strides=[4])
    _check(g, path=P.DeviceTransformReduce, device_transform_uses_affine_stride=1, affine_input_stride=4, physical_layout_is_dense_permutation=0,
           permutation_aware_tiled_geometry=None)
    assert map_index([3], [0], 0, 2, strides=[4]) == 8


def test_arg_reductions_take_dense_tensors_only():
    """The reference's CubArgReduction::stamp starts with requireDenseContiguousGpuTensor (CubReduction.cpp:1310): a
    view is refused before anything touches a device."""
    import torch

    from thor_b200 import ThorB200InvalidArgument
    from thor_b200.reductions import CubArgReduction, CubArgReductionOp

    with pytest.raises(ThorB200InvalidArgument, match="dense contiguous"):
        CubArgReduction(CubArgReductionOp.ArgMax, [1]).stamp(torch.zeros(4, 6).t())
