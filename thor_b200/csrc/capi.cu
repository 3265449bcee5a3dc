// Status plumbing of the C ABI: thread-local error text, launch counter, per-device properties.
#include "common.cuh"

#include <cstdlib>

#include <mutex>

namespace tb {

std::string& lastErrorSlot() {
    thread_local std::string slot;
    return slot;
}

int fail(int status, const char* fmt, ...) {
    char buf[2048];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    lastErrorSlot() = buf;
    return status;
}

void clearError() { lastErrorSlot().clear(); }

static std::atomic<uint64_t> g_launches{0};
void countLaunch(uint64_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

static std::atomic<bool> g_dependent_launch{true};
bool dependentLaunchEnabled() { return g_dependent_launch.load(std::memory_order_relaxed); }

int currentDeviceInfo(const DeviceInfo** out) {
    static DeviceInfo table[64];
    static std::once_flag once[64];
    int dev = -1;
    TB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(THOR_B200_CUDA_ERROR, "device ordinal %d out of range", dev);
    cudaError_t err = cudaSuccess;
    std::call_once(once[dev], [&]() {
        int v = 0;
        DeviceInfo& d = table[dev];
        if ((err = cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return;
        d.sm_count = v;
        if ((err = cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess) return;
        d.cc_major = v;
        if ((err = cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMinor, dev)) != cudaSuccess) return;
        d.cc_minor = v;
        if ((err = cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess) return;
        d.smem_optin = static_cast<size_t>(v);
    });
    if (err != cudaSuccess) return fail(THOR_B200_CUDA_ERROR, "device attribute query failed: %s", cudaGetErrorString(err));
    if (table[dev].sm_count == 0) return fail(THOR_B200_CUDA_ERROR, "device %d properties unavailable", dev);
    *out = &table[dev];
    return THOR_B200_OK;
}

const char* dtypeName(int dt) {
    switch (dt) {
        case THOR_B200_FP16: return "fp16";
        case THOR_B200_FP32: return "fp32";
        case THOR_B200_FP64: return "fp64";
        case THOR_B200_INT8: return "int8";
        case THOR_B200_INT16: return "int16";
        case THOR_B200_INT32: return "int32";
        case THOR_B200_INT64: return "int64";
        case THOR_B200_UINT8: return "uint8";
        case THOR_B200_UINT16: return "uint16";
        case THOR_B200_UINT32: return "uint32";
        case THOR_B200_UINT64: return "uint64";
        case THOR_B200_BOOLEAN: return "boolean";
        case THOR_B200_FP8_E4M3: return "fp8_e4m3";
        case THOR_B200_FP8_E5M2: return "fp8_e5m2";
        case THOR_B200_BF16: return "bf16";
        default: return "unknown";
    }
}

}  // namespace tb

extern "C" {

int thor_b200_abi_version(void) { return THOR_B200_ABI_VERSION; }

const char* thor_b200_last_error(void) { return tb::lastErrorSlot().c_str(); }

size_t thor_b200_dtype_size(int dtype) { return tb::dtypeSize(dtype); }

uint64_t thor_b200_launch_count(void) { return tb::g_launches.load(std::memory_order_relaxed); }

void thor_b200_set_dependent_launch(int on) { tb::g_dependent_launch.store(on != 0, std::memory_order_relaxed); }
int thor_b200_dependent_launch(void) { return tb::g_dependent_launch.load(std::memory_order_relaxed) ? 1 : 0; }

// Helper streams and events for stamped plans whose independent branches run beside the caller's stream.
int thor_b200_stream_create(void** out_stream) {
    using namespace tb;
    TB_REQUIRE(out_stream != nullptr, "stream_create: null output");
    cudaStream_t s = nullptr;
    TB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *out_stream = s;
    return THOR_B200_OK;
}
void thor_b200_stream_destroy(void* stream) {
    if (stream) (void)cudaStreamDestroy(static_cast<cudaStream_t>(stream));
}
int thor_b200_event_create(void** out_event) {
    using namespace tb;
    TB_REQUIRE(out_event != nullptr, "event_create: null output");
    cudaEvent_t e = nullptr;
    TB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    *out_event = e;
    return THOR_B200_OK;
}
void thor_b200_event_destroy(void* event) {
    if (event) (void)cudaEventDestroy(static_cast<cudaEvent_t>(event));
}
int thor_b200_event_record(void* event, void* stream) {
    using namespace tb;
    TB_REQUIRE(event != nullptr, "event_record: null event");
    TB_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)));
    return THOR_B200_OK;
}
int thor_b200_stream_wait_event(void* stream, void* event) {
    using namespace tb;
    TB_REQUIRE(event != nullptr, "stream_wait_event: null event");
    TB_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(event), 0));
    return THOR_B200_OK;
}

}  // extern "C"
