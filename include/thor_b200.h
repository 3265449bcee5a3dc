/*
 * thor_b200.h — C ABI of libthor_b200.so
 *
 * B200 (sm_100a) kernels for the data-parallel hot path of Thor's expression engine:
 * dtype casts, dense value/arg reductions, and fused elementwise/broadcast expression stages.
 * Every entry point takes plain pointers and sizes, returns an int status (0 = ok) and is
 * asynchronous on the cudaStream_t that it is given (passed as void*).  After a non-zero
 * status thor_b200_last_error() returns a thread-local message; a C++ adapter turns that
 * into the std::runtime_error / std::logic_error that Thor's callers expect.
 *
 * No entry point here falls back to the CPU: without a CUDA device every launch fails.
 *
 * Each declaration cites the reference interface (path within the Thor project) it replaces.
 */
#ifndef THOR_B200_H
#define THOR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define THOR_B200_ABI_VERSION 1

#if defined(__GNUC__)
#define THOR_B200_API __attribute__((visibility("default")))
#else
#define THOR_B200_API
#endif

/* Same integers as ThorImplementation::DataType (DeepLearning/Implementation/Tensor/DataType.h:7-26). */
typedef enum thor_b200_dtype {
    THOR_B200_FP16 = 10,
    THOR_B200_FP32 = 11,
    THOR_B200_FP64 = 12,
    THOR_B200_INT8 = 13,
    THOR_B200_INT16 = 14,
    THOR_B200_INT32 = 15,
    THOR_B200_INT64 = 16,
    THOR_B200_UINT8 = 17,
    THOR_B200_UINT16 = 18,
    THOR_B200_UINT32 = 19,
    THOR_B200_UINT64 = 20,
    THOR_B200_BOOLEAN = 21,
    THOR_B200_FP8_E4M3 = 22,
    THOR_B200_FP8_E5M2 = 23,
    THOR_B200_BF16 = 24
} thor_b200_dtype;

/* Status codes.  INVALID_ARGUMENT maps to std::logic_error in the adapter (THOR_THROW_IF_FALSE,
 * DeepLearning/Implementation/ThorError.h:47-53), CUDA_ERROR / JIT_ERROR to std::runtime_error
 * (CUDA_CHECK / CU_CHECK, Utilities/Common/CudaHelpers.h:42-80). */
typedef enum thor_b200_status {
    THOR_B200_OK = 0,
    THOR_B200_INVALID_ARGUMENT = 1,
    THOR_B200_CUDA_ERROR = 2,
    THOR_B200_JIT_ERROR = 3,
    THOR_B200_UNSUPPORTED = 4
} thor_b200_status;

THOR_B200_API int thor_b200_abi_version(void);
/* Message for the last non-zero status returned on the calling thread ("" if none). */
THOR_B200_API const char* thor_b200_last_error(void);
/* Size in bytes of one stored element of `dtype`, 0 for an unknown dtype. */
THOR_B200_API size_t thor_b200_dtype_size(int dtype);
/* Number of kernels this library has launched from the calling process (all threads). */
THOR_B200_API uint64_t thor_b200_launch_count(void);

/* ---------------------------------------------------------------------------------------------
 * S1  dtype cast
 * Replaces TypeConverter::gpuConvertType (Utilities/TensorOperations/DataTypeConversions/
 * TypeConverter.h:61-66; launcher TypeConverterKernels.cu:1340-1433).
 * Converts n elements from src (src_dtype) to dst (dst_dtype) with the C++ static_cast rule of
 * the CUDA element types (fp8-e4m3 destinations saturate to +-448).  Both pointers are device
 * memory of the stream's device.  src == dst requests an in-place conversion; otherwise the two
 * ranges must not overlap.  n == 0 is a no-op.  src_dtype == dst_dtype is a caller bug and is
 * rejected, as in the reference.  Reads and writes exactly n elements: no tail padding needed.
 * ------------------------------------------------------------------------------------------- */
THOR_B200_API int thor_b200_cast_launch(const void* src, void* dst, int src_dtype, int dst_dtype, int64_t n, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* THOR_B200_H */
