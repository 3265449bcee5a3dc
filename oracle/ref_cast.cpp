// Wrapper that exposes the REFERENCE's own CPU cast path behind a C symbol.
//
// TEST INFRASTRUCTURE ONLY (never shipped, never linked by the product).  No reference source is
// copied here: this translation unit #includes the reference's TypeConverter.cpp where it lies
// in the reference checkout (the build passes that checkout as an include directory) and calls
// TypeConverter::cpuConvertType (Utilities/TensorOperations/DataTypeConversions/
// TypeConverter.cpp:110, dispatching to cpuConvertTypeImpl :899-942) on a caller-provided
// buffer pair.  Access control is lifted for the reference headers only, after every standard
// and third-party header has already been included with normal access.
//
// The GPU and stream-callback halves of TypeConverter stay undefined; they are unreachable from
// the exported symbol and are dropped by --gc-sections (the link uses -z defs to prove it).
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
#include "Utilities/TensorOperations/DataTypeConversions/TypeConverter.cpp"
#undef private
#undef protected

extern "C" __attribute__((visibility("default"))) int thor_ref_cpu_convert(void* source, void* dest, int source_dtype, int dest_dtype,
                                                                           long num_elements) {
    try {
        ThorImplementation::TypeConverter::Args args(source, dest, static_cast<ThorImplementation::DataType>(source_dtype),
                                                     static_cast<ThorImplementation::DataType>(dest_dtype), num_elements);
        ThorImplementation::TypeConverter::cpuConvertType(&args);
        return 0;
    } catch (...) {
        return 1;
    }
}

extern "C" __attribute__((visibility("default"))) int thor_ref_omp_threads_for(long num_elements) {
    // The reference's own thread-count rule (TypeConverter.cpp:917-919), evaluated on this host.
    return static_cast<int>(std::max(std::min(static_cast<long>(omp_get_num_procs()), num_elements / 500000), 1L));
}
