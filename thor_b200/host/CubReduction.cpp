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

CubReductionGeometry CubReduction::analyzeGeometry(const std::vector<uint64_t>& dims, const std::vector<uint32_t>& axes) {
    CubReductionGeometry g;
    g.axes = axes;
    g.rank = static_cast<uint32_t>(dims.size());
    if (dims.empty()) throw std::invalid_argument("CubReduction input must have at least one dimension.");
    std::vector<bool> reduced(dims.size(), false);
    for (uint32_t ax : axes) {
        if (ax >= dims.size()) throw std::invalid_argument("CubReduction axis is out of range.");
        reduced[ax] = true;
    }
    g.input_elements = 1;
    g.reduction_size = 1;
    for (size_t i = 0; i < dims.size(); ++i) {
        if (dims[i] == 0) throw std::invalid_argument("CubReduction does not accept zero-sized dimensions.");
        g.input_elements *= dims[i];
        if (reduced[i]) g.reduction_size *= dims[i];
        g.output_dimensions.push_back(reduced[i] ? 1 : dims[i]);
        if (!reduced[i]) g.squeezed_output_dimensions.push_back(dims[i]);
    }
    if (g.squeezed_output_dimensions.empty()) g.squeezed_output_dimensions.push_back(1);
    g.output_elements = g.input_elements / g.reduction_size;
    // contiguity of the non-singleton reduced axes
    uint64_t outer = 1, inner = 1;
    int phase = 0;
    bool contiguous = true;
    for (size_t i = 0; i < dims.size(); ++i) {
        if (dims[i] == 1) continue;
        if (reduced[i]) {
            if (phase == 2) contiguous = false;
            phase = 1;
        } else if (phase == 0) {
            outer *= dims[i];
        } else {
            phase = 2;
            inner *= dims[i];
        }
    }
    g.reduced_axes_are_contiguous = contiguous;
    if (contiguous) {
        g.outer_size = outer;
        g.inner_size = inner;
    }
    if (g.output_elements == 1) g.path = CubReductionPath::DeviceTransformReduce;
    else if (!contiguous) g.path = CubReductionPath::StridedFixedSegment;
    else if (inner == 1) g.path = CubReductionPath::ContiguousFixedSegment;
    else g.path = CubReductionPath::TiledFixedSegment;
    return g;
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
    return d;
}
}  // namespace

StampedCubReduction CubReduction::stamp(const Tensor& input, const Stream& stream) const {
    const CubReductionGeometry g = analyzeGeometry(input.getDimensions(), axes_);
    Tensor out = Tensor::allocate(resolveOutputDataType(input.getDataType()), g.output_dimensions, input.getGpuNum());
    return stamp(input, out, stream);
}

StampedCubReduction CubReduction::stamp(const Tensor& input, const Tensor& output, const Stream& stream) const {
    if (!input.isInitialized() || !output.isInitialized()) throw std::invalid_argument("CubReduction::stamp requires initialized tensors.");
    StampedCubReduction s;
    s.geometry_ = analyzeGeometry(input.getDimensions(), axes_);
    if (output.getTotalNumElements() != s.geometry_.output_elements) throw std::invalid_argument("CubReduction::stamp output has the wrong number of elements.");
    if (s.geometry_.path == CubReductionPath::StridedFixedSegment) {
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
