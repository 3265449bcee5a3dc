// Wrapper that exposes the REFERENCE's own GPU cast path behind a C symbol.
//
// TEST AND BASELINE INFRASTRUCTURE ONLY (never shipped, never linked by the product).  No reference
// source is copied here: this translation unit #includes the reference's TypeConverterKernels.cu
// where it lies in the reference checkout (the build passes that checkout as an include directory)
// and calls TypeConverter::gpuConvertType (Utilities/TensorOperations/DataTypeConversions/
// TypeConverter.h:61-66, TypeConverterKernels.cu:39-823) on caller-provided device buffers.  Access
// control is lifted for the reference headers only, after every standard and third-party header has
// been included with normal access.
//
// The reference's Stream / ScopedGpu classes are declared by its headers; their three member
// functions that the cast path calls are defined here against the caller's raw stream, because the
// reference's Stream.cpp drags in the whole runtime (events, cuDNN / cuBLAS handles, topology).
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

#define private public
#define protected public
#include "Utilities/TensorOperations/DataTypeConversions/TypeConverterKernels.cu"
#undef private
#undef protected

namespace {
thread_local cudaStream_t g_stream = nullptr;
thread_local int g_device = 0;
}  // namespace

// The stream every launch of this call goes to and the device it belongs to.
cudaStream_t Stream::getStream() const { return g_stream; }
int Stream::getGpuNum() const { return g_device; }
// Makes `newDeviceNum` current and reports the device that was current (ScopedGpu.h:27).
int ScopedGpu::swapActiveDevice(int newDeviceNum) {
    int previous = 0;
    cudaGetDevice(&previous);
    if (previous != newDeviceNum) cudaSetDevice(newDeviceNum);
    return previous;
}

extern "C" __attribute__((visibility("default"))) int thor_ref_gpu_convert(void* source_d, void* dest_d, int source_dtype, int dest_dtype, long num_elements,
                                                                           void* stream) {
    try {
        g_stream = static_cast<cudaStream_t>(stream);
        cudaGetDevice(&g_device);
        ThorImplementation::TypeConverter::gpuConvertType(source_d, dest_d, static_cast<ThorImplementation::DataType>(source_dtype),
                                                          static_cast<ThorImplementation::DataType>(dest_dtype), num_elements, Stream());
        return cudaGetLastError() == cudaSuccess ? 0 : 2;
    } catch (...) {
        return 1;
    }
}
