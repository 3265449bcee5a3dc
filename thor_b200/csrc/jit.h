// NVRTC compile cache + cudaLibrary loader shared by the fused-stage and row-program seams.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <memory>
#include <mutex>
#include <string>

namespace tb::jit {

struct Module {
    std::string cubin;
    std::string kernel_name;
    // `library` is written before `kernel` is published; readers that see a non-null kernel (acquire) see the library too
    cudaLibrary_t library = nullptr;
    std::atomic<cudaKernel_t> kernel{nullptr};
    std::mutex load_mutex;
    ~Module();  // unloads the library (a module leaves the cache by eviction; handles that still use it keep it alive)
};

// Compiles `source` (which may #include "tb_prelude.cuh") for sm_100a; identical (source, flags)
// pairs share one module process-wide.  Needs NVRTC but neither a GPU nor a driver.
int compileSource(const std::string& source, bool fast_math, const char* kernel_name, std::shared_ptr<Module>* out);
// Loads the cubin on first use (needs a device).
int ensureLoaded(Module& m);
// The compile cache keeps the most recently used modules, at most this many (the reference's LRU caches hold 10 000
// compiled stages, EquationCompiler.cpp:123-157).  Returns the previous capacity; 0 entries = caching off.
size_t setCacheCapacity(size_t entries);
size_t cacheSize();

}  // namespace tb::jit
