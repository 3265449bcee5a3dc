#include "CubReduction.h"

#include <algorithm>
#include <cmath>
#include <limits>
#include <stdexcept>
#include <string>

#include "thor_b200.h"

namespace ThorB200 {

namespace {
void check(int status, const char* what) {
    if (status == THOR_B200_OK) return;
    const std::string msg = std::string(what) + ": " + thor_b200_last_error();
    if (status == THOR_B200_INVALID_ARGUMENT || status == THOR_B200_UNSUPPORTED) throw std::logic_error(msg);
    throw std::runtime_error(msg);
}
}  // namespace

CubReduction::CubReduction(CubReductionOp op, std::vector<uint32_t> axes, std::optional<DataType> output_dtype, float output_scale)
    : op_(op), axes_(std::move(axes)), output_dtype_(output_dtype), output_scale_(output_scale) {
    // axes must be non-empty, unique and strictly increasing (CubReduction.h:178-180)
    if (axes_.empty()) throw std::invalid_argument("CubReduction requires at least one axis.");
    for (size_t i = 1; i < axes_.size(); ++i)
        if (axes_[i] <= axes_[i - 1]) throw std::invalid_argument("CubReduction axes must be unique and strictly increasing.");
    if (!std::isfinite(output_scale_)) throw std::invalid_argument("CubReduction output scale must be finite.");
}

float CubReduction::getFp32EmptyReductionValue(CubReductionOp op) {
    switch (op) {
        case CubReductionOp::Product: return 1.0f;
        case CubReductionOp::Min: return std::numeric_limits<float>::infinity();
        case CubReductionOp::Max: return -std::numeric_limits<float>::infinity();
        default: return 0.0f;
    }
}

namespace {
std::vector<uint64_t> denseStrides(const std::vector<uint64_t>& dims) {
    std::vector<uint64_t> s(dims.size(), 1);
    for (size_t i = dims.size(); i-- > 1;) s[i - 1] = s[i] * dims[i];
    return s;
}

// Is the view a permutation of dense storage?  Axes of extent > 1, ordered by decreasing stride, must tile the storage
// without gap, overlap or broadcast (CubReduction.cpp:91-131).
void detectDensePermutation(const std::vector<uint64_t>& dims, const std::vector<uint64_t>& strides, CubReductionGeometry& g) {
    std::vector<uint32_t> order;
    for (uint32_t ax = 0; ax < dims.size(); ++ax)
        if (dims[ax] > 1) {
            if (strides[ax] == 0) return;
            order.push_back(ax);
        }
    std::sort(order.begin(), order.end(), [&](uint32_t l, uint32_t r) { return strides[l] != strides[r] ? strides[l] > strides[r] : l < r; });
    uint64_t expect = 1;
    for (size_t k = order.size(); k-- > 0;) {
        if (strides[order[k]] != expect) return;
        expect *= dims[order[k]];
    }
    if (expect != g.input_elements) return;
    g.physical_layout_is_dense_permutation = true;
    g.physical_non_singleton_axis_order = std::move(order);
}

// A dense permutation whose reduced axes are ONE physical block with something behind it, and whose retained axes come
// out either in physical order or as the (inner, outer) rotation of it, can use the dense tiled kernels on the storage
// as it lies (CubReduction.cpp:133-223).
void detectPermutedTiledCandidate(const std::vector<uint64_t>& dims, const std::vector<uint32_t>& axes, CubReductionGeometry& g) {
    if (!g.physical_layout_is_dense_permutation || g.output_elements <= 1) return;
    std::vector<bool> reduced(dims.size(), false);
    for (uint32_t ax : axes) reduced[ax] = true;
    const auto& order = g.physical_non_singleton_axis_order;
    size_t first = order.size(), last = 0;
    bool any = false;
    for (size_t k = 0; k < order.size(); ++k)
        if (reduced[order[k]]) {
            if (!any) first = k;
            last = k;
            any = true;
        }
    if (!any) return;
    for (size_t k = first; k <= last; ++k)
        if (!reduced[order[k]]) return;
    CubReductionPermutationAwareTiledGeometry c;
    c.physical_outer_axes.assign(order.begin(), order.begin() + first);
    c.physical_reduction_axes.assign(order.begin() + first, order.begin() + last + 1);
    c.physical_inner_axes.assign(order.begin() + last + 1, order.end());
    auto product = [&](const std::vector<uint32_t>& ax) {
        uint64_t p = 1;
        for (uint32_t a : ax) p *= dims[a];
        return p;
    };
    c.outer_size = product(c.physical_outer_axes);
    c.reduction_size = g.reduction_size;
    c.inner_size = product(c.physical_inner_axes);
    if (c.inner_size <= 1) return;  // a physically trailing reduction belongs to the contiguous-segment family
    for (uint32_t ax = 0; ax < dims.size(); ++ax)
        if (!reduced[ax] && dims[ax] > 1) c.logical_non_singleton_retained_axes.push_back(ax);
    std::vector<uint32_t> natural = c.physical_outer_axes, rotated = c.physical_inner_axes;
    natural.insert(natural.end(), c.physical_inner_axes.begin(), c.physical_inner_axes.end());
    rotated.insert(rotated.end(), c.physical_outer_axes.begin(), c.physical_outer_axes.end());
    if (c.logical_non_singleton_retained_axes == natural) c.retained_output_order = CubReductionTiledRetainedOutputOrder::NaturalOuterInner;
    else if (c.logical_non_singleton_retained_axes == rotated) c.retained_output_order = CubReductionTiledRetainedOutputOrder::PermutedInnerOuter;
    else return;
    g.permutation_aware_tiled_geometry = std::move(c);
}
}  // namespace

CubReductionGeometry CubReduction::analyzeGeometry(const std::vector<uint64_t>& dims, const std::vector<uint32_t>& axes) {
    return analyzeGeometry(dims, denseStrides(dims), axes);
}

CubReductionGeometry CubReduction::analyzeGeometry(const std::vector<uint64_t>& dims, const std::vector<uint64_t>& strides, const std::vector<uint32_t>& axes) {
    CubReductionGeometry g;
    g.axes = axes;
    g.rank = static_cast<uint32_t>(dims.size());
    if (dims.empty()) throw std::invalid_argument("CubReduction input must have at least one dimension.");
    if (dims.size() != strides.size()) throw std::invalid_argument("CubReduction input stride rank must match the input rank.");
    if (axes.empty()) throw std::invalid_argument("CubReduction requires at least one reduction axis.");
    if (axes.size() > dims.size()) throw std::invalid_argument("CubReduction has more reduction axes than input dimensions.");
    std::vector<bool> reduced(dims.size(), false);
    for (size_t i = 0; i < axes.size(); ++i) {
        if (axes[i] >= dims.size()) throw std::invalid_argument("CubReduction axis is out of range.");
        if (i > 0 && axes[i] <= axes[i - 1]) throw std::invalid_argument("CubReduction axes must be unique and strictly increasing.");
        reduced[axes[i]] = true;
    }
    g.input_elements = 1;
    g.reduction_size = 1;
    g.indexing.input_strides = strides;
    for (size_t i = 0; i < dims.size(); ++i) {
        if (dims[i] == 0) throw std::invalid_argument("CubReduction does not accept zero-sized dimensions.");
        if (g.input_elements > std::numeric_limits<uint64_t>::max() / dims[i]) throw std::invalid_argument("CubReduction input element count overflows uint64_t.");
        g.input_elements *= dims[i];
        if (reduced[i]) g.reduction_size *= dims[i];
        g.output_dimensions.push_back(reduced[i] ? 1 : dims[i]);
        if (!reduced[i]) g.squeezed_output_dimensions.push_back(dims[i]);
        (reduced[i] ? g.indexing.reduced_axes : g.indexing.retained_axes).push_back(static_cast<uint32_t>(i));
        (reduced[i] ? g.indexing.reduced_dimensions : g.indexing.retained_dimensions).push_back(dims[i]);
    }
    if (g.squeezed_output_dimensions.empty()) g.squeezed_output_dimensions.push_back(1);
    g.output_elements = g.input_elements / g.reduction_size;
    // one block of adjacent axis numbers, as the reference defines it (CubReduction.cpp:843-866)
    bool block = true;
    for (size_t i = 1; i < axes.size(); ++i) block = block && axes[i] == axes[i - 1] + 1;
    uint64_t outer = 1, inner = 1;
    g.reduced_axes_are_contiguous = block;
    if (block) {
        for (uint32_t i = 0; i < axes.front(); ++i) outer *= dims[i];
        for (size_t i = axes.back() + 1; i < dims.size(); ++i) inner *= dims[i];
        g.outer_size = outer;
        g.inner_size = inner;
        g.tiled_output_outer_stride = inner;
        g.tiled_output_inner_stride = 1;
    }
    bool dense = true;
    {
        const std::vector<uint64_t> want = denseStrides(dims);
        for (size_t i = 0; i < dims.size(); ++i) dense = dense && (dims[i] == 1 || strides[i] == want[i]);
    }
    detectDensePermutation(dims, strides, g);
    if (!dense) detectPermutedTiledCandidate(dims, axes, g);

    if (dense) {
        if (g.output_elements == 1) g.path = CubReductionPath::DeviceTransformReduce;
        else if (!block) g.path = CubReductionPath::StridedFixedSegment;
        else if (inner == 1) g.path = CubReductionPath::ContiguousFixedSegment;
        else g.path = CubReductionPath::TiledFixedSegment;
    } else if (g.permutation_aware_tiled_geometry) {
        const auto& c = *g.permutation_aware_tiled_geometry;
        g.path = CubReductionPath::TiledFixedSegment;
        g.outer_size = c.outer_size;
        g.reduction_size = c.reduction_size;
        g.inner_size = c.inner_size;
        const bool rotated = c.retained_output_order == CubReductionTiledRetainedOutputOrder::PermutedInnerOuter;
        g.tiled_output_permuted = rotated;
        g.tiled_output_shared_transpose = rotated;
        g.tiled_output_outer_stride = rotated ? 1 : c.inner_size;
        g.tiled_output_inner_stride = rotated ? c.outer_size : 1;
    } else if (g.output_elements == 1 && dims.size() == 1) {
        g.path = CubReductionPath::DeviceTransformReduce;  // a rank-1 view is affine: diagonals, broadcast aliases
        g.device_transform_uses_affine_stride = true;
        g.affine_input_stride = strides[0];
    } else {
        g.path = CubReductionPath::StridedFixedSegment;  // never materialise a view to regain a dense path
    }
    return g;
}

uint64_t CubReduction::mapLogicalReductionIndexToPhysicalIndex(const CubReductionGeometry& g, uint64_t output_index, uint64_t reduction_index) {
    if (output_index >= g.output_elements) throw std::out_of_range("CubReduction output index is outside the output.");
    if (reduction_index >= g.reduction_size) throw std::out_of_range("CubReduction reduction index is outside the reduction domain.");
    uint64_t physical = 0;
    for (size_t k = g.indexing.retained_axes.size(); k-- > 0;) {
        physical += (output_index % g.indexing.retained_dimensions[k]) * g.indexing.input_strides[g.indexing.retained_axes[k]];
        output_index /= g.indexing.retained_dimensions[k];
    }
    for (size_t k = g.indexing.reduced_axes.size(); k-- > 0;) {
        physical += (reduction_index % g.indexing.reduced_dimensions[k]) * g.indexing.input_strides[g.indexing.reduced_axes[k]];
        reduction_index /= g.indexing.reduced_dimensions[k];
    }
    return physical;
}

namespace {
thor_b200_strided_reduce_desc stridedDesc(const Tensor& input, const std::vector<uint32_t>& axes, int op, int arg_op, DataType output_dtype) {
    thor_b200_strided_reduce_desc d{};
    const auto& dims = input.getDimensions();
    if (dims.size() > THOR_B200_MAX_RANK) throw std::invalid_argument("reductions over non-adjacent axes support rank <= 8");
    d.op = op;
    d.arg_op = arg_op;
    d.input_dtype = static_cast<int>(input.getDataType());
    d.output_dtype = static_cast<int>(output_dtype);
    d.rank = static_cast<uint32_t>(dims.size());
    for (size_t i = 0; i < dims.size(); ++i) d.dims[i] = dims[i];
    for (uint32_t ax : axes) d.reduced[ax] = 1;
    if (!input.isDenseRowMajor()) {
        d.has_strides = 1;
        const std::vector<uint64_t> strides = input.getStridesElements();
        for (size_t i = 0; i < dims.size(); ++i) d.strides[i] = strides[i];
    }
    return d;
}
}  // namespace

StampedCubReduction CubReduction::stamp(const Tensor& input, const Stream& stream) const {
    const CubReductionGeometry g = analyzeGeometry(input.getDimensions(), input.getStridesElements(), axes_);
    Tensor out = Tensor::allocate(resolveOutputDataType(input.getDataType()), g.output_dimensions, input.getGpuNum());
    return stamp(input, out, stream);
}

StampedCubReduction CubReduction::stamp(const Tensor& input, const Tensor& output, const Stream& stream) const {
    if (!input.isInitialized() || !output.isInitialized()) throw std::invalid_argument("CubReduction::stamp requires initialized tensors.");
    StampedCubReduction s;
    s.geometry_ = analyzeGeometry(input.getDimensions(), input.getStridesElements(), axes_);
    if (output.getTotalNumElements() != s.geometry_.output_elements) throw std::invalid_argument("CubReduction::stamp output has the wrong number of elements.");
    if (!output.isDenseRowMajor()) throw std::invalid_argument("CubReduction::stamp writes a dense output.");
    // genuine views (gapped, broadcast, overlapping, permutations the dense kernels cannot walk) and rank-1 affine views
    // go to the strided kernel, which reads the view through its strides: nothing is materialised
    if (s.geometry_.path == CubReductionPath::StridedFixedSegment || s.geometry_.device_transform_uses_affine_stride) {
        s.strided_ = std::make_shared<thor_b200_strided_reduce_desc>(stridedDesc(input, axes_, static_cast<int>(op_), -1, output.getDataType()));
        s.input_ = input;
        s.output_ = output;
        s.stream_ = stream;
        s.output_scale_ = output_scale_;
        return s;
    }
    thor_b200_reduce_desc d{};
    d.op = static_cast<int>(op_);
    d.input_dtype = static_cast<int>(input.getDataType());
    d.output_dtype = static_cast<int>(output.getDataType());
    d.outer = s.geometry_.outer_size;
    d.reduction = s.geometry_.reduction_size;
    d.inner = s.geometry_.inner_size;
    if (s.geometry_.tiled_output_permuted) {
        // a permuted view whose retained axes come out as [inner, outer]: the dense kernel walks the storage as it lies
        // and writes each result where the logical output order wants it
        d.out_stride_outer = s.geometry_.tiled_output_outer_stride;
        d.out_stride_inner = s.geometry_.tiled_output_inner_stride;
    }
    thor_b200_reduce_plan* plan = nullptr;
    size_t ws = 1;
    check(thor_b200_reduce_plan_create(&d, &plan, &ws), "CubReduction::stamp");
    s.plan_ = std::shared_ptr<thor_b200_reduce_plan>(plan, [](thor_b200_reduce_plan* p) { thor_b200_reduce_plan_destroy(p); });
    s.input_ = input;
    s.output_ = output;
    s.workspace_bytes_ = ws;
    s.workspace_ = Tensor::allocate(DataType::UINT8, {static_cast<uint64_t>(ws)}, input.getGpuNum());
    s.stream_ = stream;
    s.output_scale_ = output_scale_;
    return s;
}

void StampedCubReduction::run() { runOn(stream_, output_scale_); }

void StampedCubReduction::runOn(const Stream& stream, float output_scale) {
    if (strided_) {
        check(thor_b200_strided_reduce_launch(strided_.get(), input_.getMemPtr(), output_.getMemPtr(), output_scale, stream.handle), "StampedCubReduction::run");
        return;
    }
    check(thor_b200_reduce_launch(plan_.get(), input_.getMemPtr(), output_.getMemPtr(), workspace_.getMemPtr(), workspace_bytes_, output_scale,
                                  stream.handle),
          "StampedCubReduction::run");
}

const char* StampedCubReduction::kernelKind() const { return strided_ ? "strided" : thor_b200_reduce_plan_kind(plan_.get()); }

CubArgReduction::CubArgReduction(CubArgReductionOp op, std::vector<uint32_t> axes, CubArgReductionOutputOptions options)
    : op_(op), axes_(std::move(axes)), options_(options) {
    if (axes_.empty()) throw std::invalid_argument("CubArgReduction requires at least one axis.");
    for (size_t i = 1; i < axes_.size(); ++i)
        if (axes_[i] <= axes_[i - 1]) throw std::invalid_argument("CubArgReduction axes must be unique and strictly increasing.");
    if (!options_.produce_index && !options_.produce_value) throw std::invalid_argument("CubArgReduction must produce an index or a value.");
    if (options_.index_output_dtype != DataType::UINT32 && options_.index_output_dtype != DataType::UINT64)
        throw std::invalid_argument("CubArgReduction index dtype must be UINT32 or UINT64.");
}

StampedCubArgReduction CubArgReduction::stamp(const Tensor& input, const Stream& stream) const {
    // views are for value reductions; arg reductions take dense tensors only, like the reference's
    // (CubReduction.cpp:1310, requireDenseContiguousGpuTensor)
    if (!input.isInitialized()) throw std::invalid_argument("input must be initialized.");
    if (!input.isDenseRowMajor()) throw std::invalid_argument("input must be dense contiguous.");
    const CubReductionGeometry g = CubReduction::analyzeGeometry(input.getDimensions(), axes_);
    StampedCubArgReduction s;
    if (g.path == CubReductionPath::StridedFixedSegment) {
        const DataType vdt = options_.value_output_dtype.value_or(input.getDataType());
        s.input_ = input;
        s.stream_ = stream;
        if (options_.produce_index) {
            s.index_ = Tensor::allocate(options_.index_output_dtype, g.output_dimensions, input.getGpuNum());
            s.strided_index_ = std::make_shared<thor_b200_strided_reduce_desc>(stridedDesc(input, axes_, 0, static_cast<int>(op_), options_.index_output_dtype));
        }
        if (options_.produce_value) {
            // the winner's value is the NaN-propagating min / max of the segment
            s.value_ = Tensor::allocate(vdt, g.output_dimensions, input.getGpuNum());
            s.strided_value_ = std::make_shared<thor_b200_strided_reduce_desc>(
                stridedDesc(input, axes_, op_ == CubArgReductionOp::ArgMax ? THOR_B200_REDUCE_MAX : THOR_B200_REDUCE_MIN, -1, vdt));
        }
        return s;
    }
    thor_b200_argreduce_desc d{};
    d.op = static_cast<int>(op_);
    d.input_dtype = static_cast<int>(input.getDataType());
    const DataType value_dtype = options_.value_output_dtype.value_or(input.getDataType());
    d.value_dtype = options_.produce_value ? static_cast<int>(value_dtype) : 0;
    d.index_dtype = static_cast<int>(options_.index_output_dtype);
    d.outer = g.outer_size;
    d.reduction = g.reduction_size;
    d.inner = g.inner_size;
    thor_b200_argreduce_plan* plan = nullptr;
    size_t ws = 1;
    check(thor_b200_argreduce_plan_create(&d, &plan, &ws), "CubArgReduction::stamp");
    s.plan_ = std::shared_ptr<thor_b200_argreduce_plan>(plan, [](thor_b200_argreduce_plan* p) { thor_b200_argreduce_plan_destroy(p); });
    s.input_ = input;
    if (options_.produce_index) s.index_ = Tensor::allocate(options_.index_output_dtype, g.output_dimensions, input.getGpuNum());
    if (options_.produce_value) s.value_ = Tensor::allocate(value_dtype, g.output_dimensions, input.getGpuNum());
    s.workspace_bytes_ = ws;
    s.workspace_ = Tensor::allocate(DataType::UINT8, {static_cast<uint64_t>(ws)}, input.getGpuNum());
    s.stream_ = stream;
    return s;
}

void StampedCubArgReduction::run() {
    if (strided_index_ || strided_value_) {
        if (strided_index_) check(thor_b200_strided_reduce_launch(strided_index_.get(), input_.getMemPtr(), index_.getMemPtr(), 1.0f, stream_.handle), "StampedCubArgReduction::run");
        if (strided_value_) check(thor_b200_strided_reduce_launch(strided_value_.get(), input_.getMemPtr(), value_.getMemPtr(), 1.0f, stream_.handle), "StampedCubArgReduction::run");
        return;
    }
    check(thor_b200_argreduce_launch(plan_.get(), input_.getMemPtr(), value_.getMemPtr(), index_.getMemPtr(), workspace_.getMemPtr(), workspace_bytes_,
                                     stream_.handle),
          "StampedCubArgReduction::run");
}

void TypeConverter::convertType(void* source, void* dest, DataType source_dtype, DataType dest_dtype, long num_elements, const Stream& stream) {
    check(thor_b200_cast_launch(source, dest, static_cast<int>(source_dtype), static_cast<int>(dest_dtype), num_elements, stream.handle),
          "TypeConverter::convertType");
}

}  // namespace ThorB200
