// NVRTC compile cache + cudaLibrary loader shared by the fused-stage and row-program seams.
#pragma once

#include <cuda_runtime.h>

#include <memory>
#include <mutex>
#include <string>

namespace tb::jit {

struct Module {
    std::string cubin;
    std::string kernel_name;
    cudaLibrary_t library = nullptr;
    cudaKernel_t kernel = nullptr;
    std::mutex load_mutex;
};

// Compiles `source` (which may #include "tb_prelude.cuh") for sm_100a; identical (source, flags)
// pairs share one module process-wide.  Needs NVRTC but neither a GPU nor a driver.
int compileSource(const std::string& source, bool fast_math, const char* kernel_name, std::shared_ptr<Module>* out);
// Loads the cubin on first use (needs a device).
int ensureLoaded(Module& m);

}  // namespace tb::jit
