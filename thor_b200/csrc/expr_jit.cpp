// Fused-stage seam of the C ABI: emit -> NVRTC (sm_100a cubin) -> cudaLibrary -> launch.
//
// NVRTC is dlopen'ed on first use so that libthor_b200 itself loads on a machine that has
// neither a driver nor the toolkit; compiled modules are cached process-wide by source text.
#include <dlfcn.h>
#include <nvrtc.h>

#include <cstdlib>
#include <cstring>
#include <list>
#include <memory>
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "expr_emit.h"
#include "expr_prelude.h"
#include "jit.h"

namespace tb::expr {

namespace {

struct Nvrtc {
    void* handle = nullptr;
    std::string path;
    decltype(&nvrtcCreateProgram) createProgram = nullptr;
    decltype(&nvrtcCompileProgram) compileProgram = nullptr;
    decltype(&nvrtcDestroyProgram) destroyProgram = nullptr;
    decltype(&nvrtcGetProgramLogSize) getLogSize = nullptr;
    decltype(&nvrtcGetProgramLog) getLog = nullptr;
    decltype(&nvrtcGetCUBINSize) getCubinSize = nullptr;
    decltype(&nvrtcGetCUBIN) getCubin = nullptr;
    decltype(&nvrtcGetErrorString) errorString = nullptr;
    std::string include_dir;
};

std::string dirOf(const std::string& path) {
    const size_t slash = path.rfind('/');
    return slash == std::string::npos ? std::string(".") : path.substr(0, slash);
}

bool fileExists(const std::string& p) {
    FILE* f = fopen(p.c_str(), "rb");
    if (!f) return false;
    fclose(f);
    return true;
}

// Finds the CUDA include directory that holds cuda_fp16.h: $THOR_B200_CUDA_INCLUDE_DIR, $CUDA_HOME,
// next to the loaded libnvrtc, then the conventional install prefix.
std::string findIncludeDir(const std::string& nvrtc_path) {
    std::vector<std::string> candidates;
    if (const char* e = getenv("THOR_B200_CUDA_INCLUDE_DIR")) candidates.push_back(e);
    if (const char* e = getenv("CUDA_HOME")) candidates.push_back(std::string(e) + "/include");
    if (const char* e = getenv("CUDA_PATH")) candidates.push_back(std::string(e) + "/include");
    if (!nvrtc_path.empty()) {
        const std::string libdir = dirOf(nvrtc_path);
        candidates.push_back(libdir + "/../include");
        candidates.push_back(libdir + "/../../include");
        candidates.push_back(libdir + "/../../cuda_runtime/include");  // pip layout: nvidia/cuda_nvrtc/lib -> nvidia/cuda_runtime/include
    }
    candidates.push_back("/usr/local/cuda/include");
    for (const auto& c : candidates)
        if (fileExists(c + "/cuda_fp16.h")) return c;
    return "";
}

int loadNvrtc(Nvrtc** out) {
    static Nvrtc lib;
    static std::once_flag once;
    static std::string error;
    std::call_once(once, [&]() {
        std::vector<std::string> names;
        if (const char* e = getenv("THOR_B200_NVRTC")) names.push_back(e);
        names.insert(names.end(), {"libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so.12", "libnvrtc.so.13", "/usr/local/cuda/lib64/libnvrtc.so", "libnvrtc.so"});
        for (const auto& n : names) {
            lib.handle = dlopen(n.c_str(), RTLD_NOW | RTLD_LOCAL);
            if (lib.handle) break;
        }
        if (!lib.handle) {
            error = "NVRTC not found (set THOR_B200_NVRTC to libnvrtc.so): ";
            error += dlerror() ? dlerror() : "dlopen failed";
            return;
        }
#define TB_SYM(field, name)                                                        \
    lib.field = reinterpret_cast<decltype(lib.field)>(dlsym(lib.handle, name));    \
    if (!lib.field) { error = std::string("NVRTC symbol missing: ") + name; return; }
        TB_SYM(createProgram, "nvrtcCreateProgram")
        TB_SYM(compileProgram, "nvrtcCompileProgram")
        TB_SYM(destroyProgram, "nvrtcDestroyProgram")
        TB_SYM(getLogSize, "nvrtcGetProgramLogSize")
        TB_SYM(getLog, "nvrtcGetProgramLog")
        TB_SYM(getCubinSize, "nvrtcGetCUBINSize")
        TB_SYM(getCubin, "nvrtcGetCUBIN")
        TB_SYM(errorString, "nvrtcGetErrorString")
#undef TB_SYM
        Dl_info info;
        if (dladdr(reinterpret_cast<void*>(lib.createProgram), &info) && info.dli_fname) lib.path = info.dli_fname;
        lib.include_dir = findIncludeDir(lib.path);
        if (lib.include_dir.empty()) error = "CUDA headers (cuda_fp16.h) not found: set THOR_B200_CUDA_INCLUDE_DIR";
    });
    if (!error.empty()) return fail(THOR_B200_JIT_ERROR, "%s", error.c_str());
    *out = &lib;
    return THOR_B200_OK;
}

// Least-recently-used cache of compiled modules, key: fast-math flag + source.  Heap-allocated and never destroyed: at
// process exit no module destructor runs against a CUDA runtime that is already shutting down.
struct ModuleCache {
    std::mutex mutex;
    size_t capacity = 10000;
    std::list<std::string> order;  // most recently used first
    std::unordered_map<std::string, std::pair<std::shared_ptr<jit::Module>, std::list<std::string>::iterator>> entries;
};
ModuleCache& cache() {
    static ModuleCache* c = new ModuleCache();
    return *c;
}

}  // namespace
}  // namespace tb::expr

namespace tb::jit {
using namespace tb::expr;

int compileSource(const std::string& source, bool fast_math, const char* kernel_name, std::shared_ptr<Module>* out) {
    const std::string key = (fast_math ? "F" : "P") + source;
    ModuleCache& mc = cache();
    {
        std::lock_guard<std::mutex> lock(mc.mutex);
        auto it = mc.entries.find(key);
        if (it != mc.entries.end()) {
            mc.order.splice(mc.order.begin(), mc.order, it->second.second);
            *out = it->second.first;
            return THOR_B200_OK;
        }
    }
    Nvrtc* rt = nullptr;
    if (int st = loadNvrtc(&rt)) return st;
    nvrtcProgram prog = nullptr;
    const char* header_src[] = {kPrelude, kRowProgPrelude};
    const char* header_name[] = {"tb_prelude.cuh", "tb_rowprog.cuh"};
    nvrtcResult r = rt->createProgram(&prog, source.c_str(), "thor_b200_fused_stage.cu", 2, header_src, header_name);
    if (r != NVRTC_SUCCESS) return fail(THOR_B200_JIT_ERROR, "nvrtcCreateProgram: %s", rt->errorString(r));
    const std::string inc = "--include-path=" + rt->include_dir;
    std::vector<const char*> opts = {"--gpu-architecture=sm_100a", "--std=c++17", "-fmad=true", "-default-device", inc.c_str()};
    if (fast_math) opts.push_back("--use_fast_math");
    r = rt->compileProgram(prog, static_cast<int>(opts.size()), opts.data());
    if (r != NVRTC_SUCCESS) {
        size_t log_size = 0;
        rt->getLogSize(prog, &log_size);
        std::string log(log_size, '\0');
        if (log_size) rt->getLog(prog, log.data());
        rt->destroyProgram(&prog);
        if (log.size() > 1500) log.resize(1500);
        return fail(THOR_B200_JIT_ERROR, "NVRTC compilation failed (%s): %s", rt->errorString(r), log.c_str());
    }
    auto mod = std::make_shared<Module>();
    mod->kernel_name = kernel_name;
    size_t size = 0;
    r = rt->getCubinSize(prog, &size);
    if (r == NVRTC_SUCCESS && size) {
        mod->cubin.resize(size);
        r = rt->getCubin(prog, mod->cubin.data());
    }
    rt->destroyProgram(&prog);
    if (r != NVRTC_SUCCESS || mod->cubin.empty()) return fail(THOR_B200_JIT_ERROR, "nvrtcGetCUBIN: %s", rt->errorString(r));
    std::vector<std::shared_ptr<Module>> evicted;  // released after the lock: unloading a library is slow
    {
        std::lock_guard<std::mutex> lock(mc.mutex);
        auto it = mc.entries.find(key);
        if (it != mc.entries.end()) {  // another thread compiled the same source meanwhile: share its module
            *out = it->second.first;
            return THOR_B200_OK;
        }
        *out = mod;
        if (mc.capacity > 0) {
            mc.order.push_front(key);
            mc.entries.emplace(key, std::make_pair(mod, mc.order.begin()));
            while (mc.entries.size() > mc.capacity) {
                auto victim = mc.entries.find(mc.order.back());
                evicted.push_back(victim->second.first);
                mc.entries.erase(victim);
                mc.order.pop_back();
            }
        }
    }
    return THOR_B200_OK;
}

size_t setCacheCapacity(size_t entries) {
    ModuleCache& mc = cache();
    std::vector<std::shared_ptr<Module>> evicted;
    std::lock_guard<std::mutex> lock(mc.mutex);
    const size_t before = mc.capacity;
    mc.capacity = entries;
    while (mc.entries.size() > mc.capacity) {
        auto victim = mc.entries.find(mc.order.back());
        evicted.push_back(victim->second.first);
        mc.entries.erase(victim);
        mc.order.pop_back();
    }
    return before;
}
size_t cacheSize() {
    ModuleCache& mc = cache();
    std::lock_guard<std::mutex> lock(mc.mutex);
    return mc.entries.size();
}

Module::~Module() {
    if (library != nullptr) (void)cudaLibraryUnload(library);
}

int ensureLoaded(Module& m) {
    if (m.kernel.load(std::memory_order_acquire) != nullptr) return THOR_B200_OK;
    std::lock_guard<std::mutex> lock(m.load_mutex);
    if (m.kernel.load(std::memory_order_relaxed) != nullptr) return THOR_B200_OK;
    TB_CUDA(cudaFree(nullptr));  // make sure the primary context exists
    cudaLibrary_t lib = nullptr;
    TB_CUDA(cudaLibraryLoadData(&lib, m.cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0));
    cudaKernel_t k = nullptr;
    TB_CUDA(cudaLibraryGetKernel(&k, lib, m.kernel_name.c_str()));
    m.library = lib;
    m.kernel.store(k, std::memory_order_release);
    return THOR_B200_OK;
}

}  // namespace tb::jit

namespace tb::expr {

struct Variant {
    Emitted em;
    std::shared_ptr<jit::Module> module;
};

}  // namespace tb::expr

struct thor_b200_expr {
    tb::expr::Stage stage;
    tb::expr::Variant fast;
    tb::expr::Variant safe;  // generic kernel, compiled on the first launch that needs it
    bool safe_ready = false;
    bool fast_is_generic = false;
    bool compile_only = false;
    std::mutex safe_mutex;
    std::vector<int64_t> strides_storage;
};

namespace tb::expr {

namespace {

int launchVariant(const thor_b200_expr& e, const Variant& v, const void* const* input_ptrs, const float* runtime_scalars, void* const* output_ptrs,
                  uint64_t numel, cudaStream_t stream) {
    const Stage& st = e.stage;
    jit::Module& m = *v.module;
    if (int s = jit::ensureLoaded(m)) return s;
    // kernel parameters: inputs in slot order, outputs, then numel for flat kernels
    constexpr size_t kMaxArgs = 64;
    void* args[kMaxArgs];
    const void* ptr_store[kMaxArgs];
    float scalar_store[kMaxArgs];
    size_t n = 0;
    if (st.inputs.size() + st.outputs.size() + 1 > kMaxArgs) return fail(THOR_B200_UNSUPPORTED, "stage has too many kernel arguments");
    for (size_t s = 0; s < st.inputs.size(); ++s) {
        if (st.inputs[s].kind == THOR_B200_INPUT_RUNTIME_SCALAR_FP32) {
            scalar_store[n] = runtime_scalars[s];
            args[n] = &scalar_store[n];
        } else {
            ptr_store[n] = input_ptrs[s];
            args[n] = &ptr_store[n];
        }
        ++n;
    }
    for (size_t o = 0; o < st.outputs.size(); ++o) {
        ptr_store[n] = output_ptrs[o];
        args[n] = &ptr_store[n];
        ++n;
    }
    unsigned long long numel_arg = numel;
    dim3 grid(1, 1, 1), block(static_cast<unsigned>(v.em.threads), 1, 1);
    switch (v.em.kind) {
        case Kind::FlatV2:
        case Kind::FlatScalar: {
            args[n++] = &numel_arg;
            const uint64_t per_cta = static_cast<uint64_t>(v.em.threads) * v.em.unroll;
            uint64_t blocks = (numel / v.em.vec + per_cta - 1) / per_cta;
            if (blocks == 0) blocks = 1;
            if (blocks > 0x7FFFFFFFull) return fail(THOR_B200_UNSUPPORTED, "stage of %llu elements exceeds the launch grid", numel_arg);
            grid.x = static_cast<unsigned>(blocks);
        } break;
        case Kind::TiledV2:
        case Kind::TiledScalar: {
            const uint64_t rows_per_cta = static_cast<uint64_t>(v.em.ty) * v.em.unroll;
            const uint64_t gx = (v.em.rows + rows_per_cta - 1) / rows_per_cta;
            const uint64_t ppr = v.em.cols / v.em.vec;
            const uint64_t gy = (ppr + v.em.tx - 1) / v.em.tx;
            if (gx > 0x7FFFFFFFull || gy > 65535ull) return fail(THOR_B200_UNSUPPORTED, "broadcast stage exceeds the launch grid");
            grid.x = static_cast<unsigned>(gx);
            grid.y = static_cast<unsigned>(gy);
            if (v.em.linear_grid) {
                grid.x = static_cast<unsigned>(gx * gy);
                grid.y = 1;
            }
        } break;
        case Kind::Generic: {
            const uint64_t total = st.broadcast ? v.em.numel : numel;
            if (!st.broadcast) args[n++] = &numel_arg;
            const uint64_t blocks = (total + 255) / 256;
            if (blocks > 0x7FFFFFFFull) return fail(THOR_B200_UNSUPPORTED, "stage exceeds the launch grid");
            grid.x = static_cast<unsigned>(blocks == 0 ? 1 : blocks);
        } break;
    }
    TB_CUDA(launchDependentC(reinterpret_cast<const void*>(m.kernel.load()), grid, block, args, 0, stream));
    countLaunch();
    return THOR_B200_OK;
}

}  // namespace
}  // namespace tb::expr

extern "C" {

int thor_b200_expr_compile(const thor_b200_expr_node* nodes, uint32_t n_nodes, const thor_b200_expr_input* inputs, uint32_t n_inputs,
                           const thor_b200_expr_output* outputs, uint32_t n_outputs, const thor_b200_expr_broadcast* broadcast,
                           const thor_b200_expr_options* options, thor_b200_expr** out_expr) {
    using namespace tb;
    using namespace tb::expr;
    TB_REQUIRE(out_expr != nullptr, "expr_compile: out_expr is null");
    *out_expr = nullptr;
    TB_REQUIRE(nodes != nullptr && n_nodes > 0, "expr_compile: empty node list");
    TB_REQUIRE(outputs != nullptr && n_outputs > 0, "expr_compile: no outputs");
    TB_REQUIRE(n_inputs == 0 || inputs != nullptr, "expr_compile: inputs is null");
    if (options)
        for (int r : options->reserved) TB_REQUIRE(r == 0, "expr_compile: reserved option fields must be zero");
    auto e = std::make_unique<thor_b200_expr>();
    e->stage.nodes.assign(nodes, nodes + n_nodes);
    e->stage.inputs.assign(inputs, inputs + n_inputs);
    e->stage.outputs.assign(outputs, outputs + n_outputs);
    e->stage.fast_math = options && options->use_fast_math;
    e->compile_only = options && options->compile_only;
    if (options) {
        e->stage.rows_per_thread = options->rows_per_thread;
        e->stage.min_ctas_per_sm = options->min_ctas_per_sm;
        e->stage.packs_per_thread = options->packs_per_thread;
    }
    if (broadcast) {
        TB_REQUIRE(broadcast->rank >= 1 && broadcast->rank <= THOR_B200_MAX_RANK, "expr_compile: broadcast rank %u out of range", broadcast->rank);
        TB_REQUIRE(broadcast->input_strides != nullptr || n_inputs == 0, "expr_compile: broadcast strides missing");
        e->stage.broadcast = true;
        e->stage.rank = broadcast->rank;
        e->stage.dims.assign(broadcast->dims, broadcast->dims + broadcast->rank);
        e->stage.strides.resize(n_inputs);
        for (uint32_t s = 0; s < n_inputs; ++s)
            e->stage.strides[s].assign(broadcast->input_strides + static_cast<size_t>(s) * THOR_B200_MAX_RANK,
                                       broadcast->input_strides + static_cast<size_t>(s) * THOR_B200_MAX_RANK + broadcast->rank);
    }
    const std::string why = emit(e->stage, false, &e->fast.em);
    if (!why.empty()) return fail(THOR_B200_INVALID_ARGUMENT, "expr_compile: %s", why.c_str());
    e->fast_is_generic = e->fast.em.kind == Kind::Generic;
    if (int st = jit::compileSource(e->fast.em.source, e->stage.fast_math, "fused_kernel", &e->fast.module)) return st;
    if (!e->compile_only)
        if (int st = jit::ensureLoaded(*e->fast.module)) return st;
    *out_expr = e.release();
    return THOR_B200_OK;
}

int thor_b200_expr_launch(thor_b200_expr* e, const void* const* input_ptrs, const float* runtime_scalars, void* const* output_ptrs, uint64_t numel,
                          void* stream_v) {
    using namespace tb;
    using namespace tb::expr;
    TB_REQUIRE(e != nullptr, "expr_launch: null handle");
    TB_REQUIRE(!e->compile_only, "expr_launch: handle was compiled with compile_only");
    TB_REQUIRE(output_ptrs != nullptr, "expr_launch: output_ptrs is null");
    const Stage& st = e->stage;
    bool need_scalars = false, need_ptrs = false;
    for (const auto& in : st.inputs) (in.kind == THOR_B200_INPUT_RUNTIME_SCALAR_FP32 ? need_scalars : need_ptrs) = true;
    TB_REQUIRE(!need_ptrs || input_ptrs != nullptr, "expr_launch: input_ptrs is null");
    TB_REQUIRE(!need_scalars || runtime_scalars != nullptr, "expr_launch: runtime_scalars is null");
    for (size_t s = 0; s < st.inputs.size(); ++s)
        if (st.inputs[s].kind != THOR_B200_INPUT_RUNTIME_SCALAR_FP32) TB_REQUIRE(input_ptrs[s] != nullptr, "expr_launch: input %zu is null", s);
    for (size_t o = 0; o < st.outputs.size(); ++o) TB_REQUIRE(output_ptrs[o] != nullptr, "expr_launch: output %zu is null", o);
    if (!st.broadcast && numel == 0) return THOR_B200_OK;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    bool aligned = true;
    for (size_t s = 0; s < st.inputs.size() && aligned; ++s)
        if (st.inputs[s].kind == THOR_B200_INPUT_TENSOR) aligned = isAligned(input_ptrs[s], e->fast.em.input_align[s]);
    for (size_t o = 0; o < st.outputs.size() && aligned; ++o) aligned = isAligned(output_ptrs[o], e->fast.em.output_align[o]);
    if (aligned) return launchVariant(*e, e->fast, input_ptrs, runtime_scalars, output_ptrs, numel, stream);
    {
        std::lock_guard<std::mutex> lock(e->safe_mutex);
        if (!e->safe_ready) {
            const std::string why = emit(st, true, &e->safe.em);
            if (!why.empty()) return fail(THOR_B200_INVALID_ARGUMENT, "expr_launch: %s", why.c_str());
            if (int s = jit::compileSource(e->safe.em.source, st.fast_math, "fused_kernel", &e->safe.module)) return s;
            e->safe_ready = true;
        }
    }
    return launchVariant(*e, e->safe, input_ptrs, runtime_scalars, output_ptrs, numel, stream);
}

// Exhaustive comparison of the lean pair routines of the device prelude with the toolkit's routines.
static const char* const kSelfCheckSource = R"TBCHECK(
#include "tb_prelude.cuh"
__device__ __forceinline__ unsigned int tb_half2bits(const __half2 v) { return *reinterpret_cast<const unsigned int*>(&v); }
extern "C" __global__ void __launch_bounds__(256) selfcheck_kernel(unsigned long long* counters) {
    const unsigned int a16 = blockIdx.x;  // 65536 blocks: one per fp16 bit pattern
    unsigned long long bad_exp = 0, bad_expn = 0, bad_div = 0, checks = 0;
    // division: lane x computes a / b, lane y computes b / a, for every b: all 2^32 ordered pairs in both lanes
    for (unsigned int b16 = threadIdx.x; b16 < 65536u; b16 += blockDim.x) {
        const __half2 A = tb_bits2half2(a16 | (b16 << 16)), B = tb_bits2half2(b16 | (a16 << 16));
        bad_div += tb_half2bits(__h2div(A, B)) != tb_half2bits(tb_h2div(A, B));
        ++checks;
    }
    if (threadIdx.x == 0) {
        // exp: every pattern in lane x, its complement in lane y
        const __half2 X = tb_bits2half2(a16 | ((65535u - a16) << 16));
        bad_exp += tb_half2bits(h2exp(X)) != tb_half2bits(tb_h2exp(X));
        // exp of arguments that are <= 0 or NaN: every pattern with the sign bit set in lane x; +0 and the
        // positive NaN patterns in lane y
        const unsigned int y = (a16 & 0x3FFu) ? (0x7C00u | (a16 & 0x3FFu)) : 0u;
        const __half2 N = tb_bits2half2((a16 | 0x8000u) | (y << 16));
        bad_expn += tb_half2bits(h2exp(N)) != tb_half2bits(tb_h2exp_nonpos(N));
    }
    atomicAdd(&counters[0], bad_exp);
    atomicAdd(&counters[1], bad_expn);
    atomicAdd(&counters[2], bad_div);
    atomicAdd(&counters[3], checks);
}
)TBCHECK";

int thor_b200_selfcheck_pair_math(unsigned long long* device_counters, void* stream_v) {
    using namespace tb;
    TB_REQUIRE(device_counters != nullptr, "selfcheck_pair_math: device_counters is null");
    std::shared_ptr<jit::Module> mod;
    if (int st = jit::compileSource(kSelfCheckSource, false, "selfcheck_kernel", &mod)) return st;
    if (int st = jit::ensureLoaded(*mod)) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    TB_CUDA(cudaMemsetAsync(device_counters, 0, 4 * sizeof(unsigned long long), stream));
    void* args[] = {&device_counters};
    TB_CUDA(cudaLaunchKernel(reinterpret_cast<const void*>(mod->kernel.load()), dim3(65536), dim3(256), args, 0, stream));
    countLaunch();
    return THOR_B200_OK;
}

const char* thor_b200_expr_source(const thor_b200_expr* e) { return e ? e->fast.em.source.c_str() : ""; }

const char* thor_b200_expr_launch_kind(const thor_b200_expr* e) { return e ? tb::expr::kindName(e->fast.em.kind) : ""; }

void thor_b200_expr_destroy(thor_b200_expr* e) { delete e; }

size_t thor_b200_jit_cache_capacity(size_t entries) { return tb::jit::setCacheCapacity(entries); }
size_t thor_b200_jit_cache_size(void) { return tb::jit::cacheSize(); }

}  // extern "C"
