// CubReduction / CubArgReduction / TypeConverter with the reference's call surface
// (Utilities/TensorOperations/Cub/CubReduction.h:176-537 and
// Utilities/TensorOperations/DataTypeConversions/TypeConverter.h:17-34), implemented on the C ABI.
#pragma once

#include <memory>
#include <optional>
#include <vector>

#include "Tensor.h"

struct thor_b200_reduce_plan;
struct thor_b200_argreduce_plan;
struct thor_b200_strided_reduce_desc;

namespace ThorB200 {

enum class CubReductionOp : uint8_t { Sum = 0, Min = 1, Max = 2, Product = 3, Mean = 4, L1Norm = 5, L2Norm = 6 };
enum class CubArgReductionOp : uint8_t { ArgMin = 0, ArgMax = 1 };
enum class CubReductionPath : uint8_t { DeviceTransformReduce = 0, ContiguousFixedSegment = 1, TiledFixedSegment = 2, StridedFixedSegment = 3 };

// How the two retained axis groups of a permuted view land in the dense output (CubReduction.h:93-105).
enum class CubReductionTiledRetainedOutputOrder : uint8_t { NaturalOuterInner = 0, PermutedInnerOuter = 1 };

// A logical permutation view over physically dense storage whose reduced axes form one physical block: the dense
// [outer, reduction, inner] kernels walk the storage as it lies, no copy is made (CubReduction.h:107-126).
struct CubReductionPermutationAwareTiledGeometry {
    std::vector<uint32_t> physical_outer_axes, physical_reduction_axes, physical_inner_axes;  // logical axis numbers, physical order
    std::vector<uint32_t> logical_non_singleton_retained_axes;
    uint64_t outer_size = 0, reduction_size = 0, inner_size = 0;
    CubReductionTiledRetainedOutputOrder retained_output_order = CubReductionTiledRetainedOutputOrder::NaturalOuterInner;
};

struct CubReductionIndexing {
    std::vector<uint64_t> input_strides;  // element strides of the (possibly strided) input view
    std::vector<uint32_t> reduced_axes, retained_axes;
    std::vector<uint64_t> reduced_dimensions, retained_dimensions;
};

struct CubReductionGeometry {
    std::vector<uint32_t> axes;
    uint32_t rank = 0;
    bool reduced_axes_are_contiguous = false;
    uint64_t outer_size = 0, reduction_size = 0, inner_size = 0;
    uint64_t input_elements = 0, output_elements = 0;
    std::vector<uint64_t> output_dimensions;           // reduced axes kept as 1
    std::vector<uint64_t> squeezed_output_dimensions;  // reduced axes removed ([1] if nothing is left)
    CubReductionPath path = CubReductionPath::DeviceTransformReduce;
    CubReductionIndexing indexing;
    // views (CubReduction.h:127-153)
    bool physical_layout_is_dense_permutation = false;
    std::vector<uint32_t> physical_non_singleton_axis_order;  // logical axes with extent > 1, slowest varying first
    std::optional<CubReductionPermutationAwareTiledGeometry> permutation_aware_tiled_geometry;
    bool tiled_output_permuted = false;          // the dense output is [inner, outer], not [outer, inner]
    bool tiled_output_shared_transpose = false;  // the reference's kernel stages that transposition in shared memory
    uint64_t tiled_output_outer_stride = 0, tiled_output_inner_stride = 0;
    bool device_transform_uses_affine_stride = false;  // rank-1 view (diagonal, broadcast) reduced to one value
    uint64_t affine_input_stride = 1;
};

class StampedCubReduction {
   public:
    // Launches the stamped reduction; performs no allocation and no planning (CubReduction.h:160-174).
    void run();
    void runOn(const Stream& stream, float output_scale);
    Tensor getOutput() const { return output_; }
    const CubReductionGeometry& getGeometry() const { return geometry_; }
    const char* kernelKind() const;
    size_t workspaceBytes() const { return workspace_bytes_; }

   private:
    friend class CubReduction;
    std::shared_ptr<thor_b200_reduce_plan> plan_;
    std::shared_ptr<thor_b200_strided_reduce_desc> strided_;  // StridedFixedSegment path: stateless launch, no plan
    Tensor input_, output_, workspace_;
    size_t workspace_bytes_ = 1;
    Stream stream_;
    float output_scale_ = 1.0f;
    CubReductionGeometry geometry_;
};

class CubReduction {
   public:
    CubReduction(CubReductionOp op, uint32_t axis, std::optional<DataType> output_dtype = std::nullopt, float output_scale = 1.0f)
        : CubReduction(op, std::vector<uint32_t>{axis}, output_dtype, output_scale) {}
    CubReduction(CubReductionOp op, std::vector<uint32_t> axes, std::optional<DataType> output_dtype = std::nullopt, float output_scale = 1.0f);

    CubReductionOp getOperation() const { return op_; }
    const std::vector<uint32_t>& getAxes() const { return axes_; }
    float getOutputScale() const { return output_scale_; }
    // Output storage dtype defaults to the input storage dtype (CubReduction.h:188-190).
    DataType resolveOutputDataType(DataType input_dtype) const { return output_dtype_.value_or(input_dtype); }
    // FP32 result defined for an empty reduction domain (CubReduction.cpp:718-734).
    static float getFp32EmptyReductionValue(CubReductionOp op);
    // Classifies the reduction like CubReduction::analyzeGeometry (CubReduction.cpp:755-912).
    static CubReductionGeometry analyzeGeometry(const std::vector<uint64_t>& input_dims, const std::vector<uint32_t>& axes);
    // The same for a strided view (element strides): dense permutations whose reduced axes are one physical block keep the
    // dense tiled kernels, rank-1 views keep the full reduction, everything else takes the strided fallback.
    static CubReductionGeometry analyzeGeometry(const std::vector<uint64_t>& input_dims, const std::vector<uint64_t>& input_strides,
                                                const std::vector<uint32_t>& axes);
    // Element offset (from the view's first element) of reduction element `reduction_index` of output `output_index`,
    // both counted row-major over the reduced / retained axes (CubReduction.cpp:914-960).
    static uint64_t mapLogicalReductionIndexToPhysicalIndex(const CubReductionGeometry& geometry, uint64_t output_index, uint64_t reduction_index);

    // Validates, plans, allocates output (unless given) and workspace.
    StampedCubReduction stamp(const Tensor& input, const Stream& stream) const;
    StampedCubReduction stamp(const Tensor& input, const Tensor& output, const Stream& stream) const;

   private:
    CubReductionOp op_;
    std::vector<uint32_t> axes_;
    std::optional<DataType> output_dtype_;
    float output_scale_;
};

class StampedCubArgReduction {
   public:
    void run();
    Tensor getIndexOutput() const { return index_; }
    Tensor getValueOutput() const { return value_; }

   private:
    friend class CubArgReduction;
    std::shared_ptr<thor_b200_argreduce_plan> plan_;
    std::shared_ptr<thor_b200_strided_reduce_desc> strided_index_, strided_value_;  // StridedFixedSegment path
    Tensor input_, index_, value_, workspace_;
    size_t workspace_bytes_ = 1;
    Stream stream_;
};

struct CubArgReductionOutputOptions {
    bool produce_value = true;
    bool produce_index = true;
    std::optional<DataType> value_output_dtype = std::nullopt;
    DataType index_output_dtype = DataType::UINT32;
};

class CubArgReduction {
   public:
    CubArgReduction(CubArgReductionOp op, std::vector<uint32_t> axes, CubArgReductionOutputOptions options = {});
    StampedCubArgReduction stamp(const Tensor& input, const Stream& stream) const;

   private:
    CubArgReductionOp op_;
    std::vector<uint32_t> axes_;
    CubArgReductionOutputOptions options_;
};

class TypeConverter {
   public:
    // TypeConverter::convertType on device memory (TypeConverter.h:28-34): asynchronous on `stream`.
    static void convertType(void* source, void* dest, DataType source_dtype, DataType dest_dtype, long num_elements, const Stream& stream);
};

}  // namespace ThorB200
