// Wrapper that exposes the REFERENCE's own reduction device path behind C symbols.
//
// TEST AND BASELINE INFRASTRUCTURE ONLY (never shipped, never linked by the product).  No reference
// source is copied here: this translation unit #includes the reference's CubReductionOperation.cuh
// where it lies in the reference checkout and calls its templates -- the fp32 transform / reduce
// operators (:60-129), the finalise-and-store output iterator (:186-207), the contiguous input
// iterator (:232-236) and the tiled dispatcher launchTiledFixedSegmentReduction (:2482-2876) -- with
// the arguments launchReductionForInput (:2966-3054) passes for the three dense paths:
//   path 0  DeviceTransformReduce   cub::DeviceReduce::TransformReduce over the whole input
//   path 1  ContiguousFixedSegment  cub::DeviceSegmentedReduce::Reduce, fixed segment size
//   path 2  TiledFixedSegment       the reference's own [outer, reduction, inner] kernels
// Arg reductions the same way from CubArgReductionOperation.cuh: candidate operators (:24-73), the store functor
// (:89-105), the candidate input functors (:115-134) wrapped in the iterators its helper functions build from them
// (:107-113, :152-162), the tiled dispatcher launchTiledFixedSegmentArgReduction (:1030-1060) and the initial
// candidates of CubArgReductionMax.cu / CubArgReductionMin.cu, as launchArgReductionForInput (:1119-1178) calls them.
// launchReductionForInput itself takes the reference's Tensor objects, whose implementation drags in
// the whole runtime, so the three calls are made on raw pointers instead.  The reference needs
// <cuda/iterator> (CCCL 3.x); the build points the compiler at a CCCL copy of that generation.
#include <algorithm>
#include <any>
#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <optional>
#include <set>
#include <sstream>
#include <string>
#include <thread>
#include <unordered_map>
#include <unordered_set>
#include <variant>
#include <vector>

#include <cublasLt.h>
#include <cublas_v2.h>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <cudnn.h>
#include <nlohmann/json.hpp>
#include <omp.h>

#include "Utilities/TensorOperations/Cub/CubReductionOperation.cuh"
#include "Utilities/TensorOperations/Cub/CubArgReductionOperation.cuh"

#include <cuda/std/functional>

namespace {

using namespace ThorImplementation;
using namespace ThorImplementation::CubReductionInternal;

template <typename InputT, typename ReductionOpT, typename FinalizeT>
int reduceTyped(int path, const void* input, void* output, DataType output_dtype, uint64_t outer, uint64_t reduction, uint64_t inner, ReductionOpT op, float init,
                FinalizeT finalize, void* temp, size_t* temp_bytes, cudaStream_t stream) {
    const InputT* in = static_cast<const InputT*>(input);
    auto out_it = makeRuntimeFp32OutputIterator(output, output_dtype, finalize, 1.0f);
    size_t bytes = temp ? *temp_bytes : 0;
    cudaError_t st = cudaSuccess;
    if (path == 0) {
        const ConvertAndTransformInputToFp32<InputT, IdentityFp32> transform{IdentityFp32{}};
        st = cub::DeviceReduce::TransformReduce(temp, bytes, in, out_it, static_cast<int64_t>(outer * reduction * inner), op, transform, init, stream);
    } else if (path == 1) {
        auto in_it = makeContiguousFp32Iterator(in, IdentityFp32{});
        st = cub::DeviceSegmentedReduce::Reduce(temp, bytes, in_it, out_it, static_cast<int64_t>(outer), static_cast<int>(reduction), op, init, stream);
    } else {
        if (temp == nullptr) {
            *temp_bytes = 1;
            return 0;
        }
        CubReductionGeometry g;
        g.rank = 3;
        g.axes = {1};
        g.reduced_axes_are_contiguous = true;
        g.outer_size = outer;
        g.reduction_size = reduction;
        g.inner_size = inner;
        g.input_elements = outer * reduction * inner;
        g.output_elements = outer * inner;
        g.tiled_output_outer_stride = inner;
        g.tiled_output_inner_stride = 1;
        g.path = CubReductionPath::TiledFixedSegment;
        launchTiledFixedSegmentReduction<InputT>(in, output, output_dtype, g, op, init, IdentityFp32{}, finalize, 1.0f, stream);
        st = cudaGetLastError();
    }
    if (temp == nullptr) *temp_bytes = std::max<size_t>(bytes, 1);
    return st == cudaSuccess ? 0 : 2;
}

template <typename InputT>
int reduceOp(int op, int path, const void* input, void* output, DataType output_dtype, uint64_t outer, uint64_t reduction, uint64_t inner, void* temp, size_t* temp_bytes,
             cudaStream_t stream) {
    // operators, identities and finalisers of the reference's per-op wrappers (CubReductionSum.cu, CubReductionMean.cu,
    // CubReductionMax.cu, CubReductionMin.cu)
    switch (op) {
        case 0: return reduceTyped<InputT>(path, input, output, output_dtype, outer, reduction, inner, cuda::std::plus<float>{}, 0.0f, AdditiveFinalizeFp32{1.0f}, temp, temp_bytes, stream);
        case 1:
            return reduceTyped<InputT>(path, input, output, output_dtype, outer, reduction, inner, cuda::std::plus<float>{}, 0.0f,
                                       AdditiveFinalizeFp32{static_cast<float>(reduction)}, temp, temp_bytes, stream);
        case 2:
            return reduceTyped<InputT>(path, input, output, output_dtype, outer, reduction, inner, PropagatingMaximumFp32{}, -std::numeric_limits<float>::infinity(), IdentityFp32{}, temp,
                                       temp_bytes, stream);
        case 3:
            return reduceTyped<InputT>(path, input, output, output_dtype, outer, reduction, inner, PropagatingMinimumFp32{}, std::numeric_limits<float>::infinity(), IdentityFp32{}, temp,
                                       temp_bytes, stream);
        default: return 3;
    }
}

template <typename InputT, typename ReductionOpT>
int argReduceTyped(int path, const void* input, void* value_output, DataType value_dtype, void* index_output, DataType index_dtype, uint64_t outer, uint64_t reduction, uint64_t inner,
                   ReductionOpT op, ArgReductionCandidateFp32 init, void* temp, size_t* temp_bytes, cudaStream_t stream) {
    const InputT* in = static_cast<const InputT*>(input);
    auto out_it = cuda::make_tabulate_output_iterator(StoreArgReductionResultRuntime{value_output, value_dtype, index_output, index_dtype});
    size_t bytes = temp ? *temp_bytes : 0;
    cudaError_t st = cudaSuccess;
    if (path == 0) {
        auto in_it = thrust::make_transform_iterator(thrust::counting_iterator<int64_t>(0), DeviceArgCandidateInput<InputT>{in});
        st = cub::DeviceReduce::Reduce(temp, bytes, in_it, out_it, static_cast<int64_t>(outer * reduction * inner), op, init, stream);
    } else if (path == 1) {
        auto in_it = thrust::make_transform_iterator(thrust::counting_iterator<int64_t>(0), ContiguousArgCandidateInput<InputT>{in, reduction});
        st = cub::DeviceSegmentedReduce::Reduce(temp, bytes, in_it, out_it, static_cast<int64_t>(outer), static_cast<int>(reduction), op, init, stream);
    } else {
        if (temp == nullptr) {
            *temp_bytes = 1;
            return 0;
        }
        CubReductionGeometry g;
        g.rank = 3;
        g.axes = {1};
        g.reduced_axes_are_contiguous = true;
        g.outer_size = outer;
        g.reduction_size = reduction;
        g.inner_size = inner;
        g.input_elements = outer * reduction * inner;
        g.output_elements = outer * inner;
        g.tiled_output_outer_stride = inner;
        g.tiled_output_inner_stride = 1;
        g.path = CubReductionPath::TiledFixedSegment;
        launchTiledFixedSegmentArgReduction<InputT>(in, value_output, value_dtype, index_output, index_dtype, g, op, init, stream);
        st = cudaGetLastError();
    }
    if (temp == nullptr) *temp_bytes = std::max<size_t>(bytes, 1);
    return st == cudaSuccess ? 0 : 2;
}

template <typename InputT>
int argReduceOp(int is_max, int path, const void* input, void* value_output, DataType value_dtype, void* index_output, DataType index_dtype, uint64_t outer, uint64_t reduction,
                uint64_t inner, void* temp, size_t* temp_bytes, cudaStream_t stream) {
    if (is_max)
        return argReduceTyped<InputT>(path, input, value_output, value_dtype, index_output, index_dtype, outer, reduction, inner, ArgMaximumCandidateFp32{},
                                      ArgReductionCandidateFp32{std::numeric_limits<uint64_t>::max(), -std::numeric_limits<float>::infinity()}, temp, temp_bytes, stream);
    return argReduceTyped<InputT>(path, input, value_output, value_dtype, index_output, index_dtype, outer, reduction, inner, ArgMinimumCandidateFp32{},
                                  ArgReductionCandidateFp32{std::numeric_limits<uint64_t>::max(), std::numeric_limits<float>::infinity()}, temp, temp_bytes, stream);
}

}  // namespace

// op: 0 sum, 1 mean, 2 max, 3 min.  path: see the header of this file.  input dtype: the reference's DataType value of
// FP32, FP16 or BF16; output dtype likewise.  With temp == NULL the call only stores the workspace size in *temp_bytes.
extern "C" __attribute__((visibility("default"))) int thor_ref_cub_reduce(int op, int path, const void* input, int input_dtype, void* output, int output_dtype, unsigned long long outer,
                                                                          unsigned long long reduction, unsigned long long inner, void* temp, size_t* temp_bytes, void* stream) {
    try {
        const DataType out = static_cast<DataType>(output_dtype);
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        switch (static_cast<DataType>(input_dtype)) {
            case DataType::FP32: return reduceOp<float>(op, path, input, output, out, outer, reduction, inner, temp, temp_bytes, s);
            case DataType::BF16: return reduceOp<__nv_bfloat16>(op, path, input, output, out, outer, reduction, inner, temp, temp_bytes, s);
            case DataType::FP16: return reduceOp<__half>(op, path, input, output, out, outer, reduction, inner, temp, temp_bytes, s);
            default: return 3;
        }
    } catch (...) {
        return 1;
    }
}

// Arg reduction over the middle axis of a dense [outer, reduction, inner] input: value_output (fp32 / fp16 / bf16) and / or
// index_output (the reference's UINT32 or UINT64 DataType value) may be NULL.  Same path and workspace conventions.
extern "C" __attribute__((visibility("default"))) int thor_ref_cub_argreduce(int is_max, int path, const void* input, int input_dtype, void* value_output, int value_dtype,
                                                                             void* index_output, int index_dtype, unsigned long long outer, unsigned long long reduction,
                                                                             unsigned long long inner, void* temp, size_t* temp_bytes, void* stream) {
    try {
        const DataType vd = static_cast<DataType>(value_dtype), id = static_cast<DataType>(index_dtype);
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        switch (static_cast<DataType>(input_dtype)) {
            case DataType::FP32: return argReduceOp<float>(is_max, path, input, value_output, vd, index_output, id, outer, reduction, inner, temp, temp_bytes, s);
            case DataType::BF16: return argReduceOp<__nv_bfloat16>(is_max, path, input, value_output, vd, index_output, id, outer, reduction, inner, temp, temp_bytes, s);
            case DataType::FP16: return argReduceOp<__half>(is_max, path, input, value_output, vd, index_output, id, outer, reduction, inner, temp, temp_bytes, s);
            default: return 3;
        }
    } catch (...) {
        return 1;
    }
}
