// Shared host/device helpers of libthor_b200: status + thread-local error text, the launch
// counter, dtype traits and the vector load/store primitives every streaming kernel uses.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>

#include "thor_b200.h"

namespace tb {

// B200: 148 SMs.  Persistent grids are sized as a multiple of the SM count read from the device;
// this constant only sizes static tables.
constexpr int kMaxSms = 160;

// ---- status ------------------------------------------------------------------------------------
std::string& lastErrorSlot();
int fail(int status, const char* fmt, ...);
void clearError();
void countLaunch(uint64_t n = 1);

#define TB_REQUIRE(cond, ...)                                          \
    do {                                                               \
        if (!(cond)) return ::tb::fail(THOR_B200_INVALID_ARGUMENT, __VA_ARGS__); \
    } while (0)

#define TB_CUDA(expr)                                                                          \
    do {                                                                                       \
        cudaError_t _e = (expr);                                                               \
        if (_e != cudaSuccess)                                                                 \
            return ::tb::fail(THOR_B200_CUDA_ERROR, "%s failed: %s (%s:%d)", #expr,            \
                              cudaGetErrorString(_e), __FILE__, __LINE__);                     \
    } while (0)

// ---- programmatic dependent launch ---------------------------------------------------------------
// Every streaming kernel of the library is launched with stream serialization relaxed: its CTAs may
// be placed on SMs while the tail of the previous kernel of the stream is still draining, which hides
// most of the launch latency between back-to-back kernels.  The kernel's first statement is
// gridDependencyWait(): it returns only once the previous kernel has completed and its writes are
// visible, so stream-order semantics are unchanged (a predecessor that never signals counts as
// signalling when it exits).  gridLaunchDependents() right after lets the next kernel do the same.
#ifdef __CUDACC__
__device__ __forceinline__ void gridDependencyWait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void gridLaunchDependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif
bool dependentLaunchEnabled();  // thor_b200_set_dependent_launch(0) turns the launch attribute off

template <class... KArgs, class... Args>
cudaError_t launchDependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependentLaunchEnabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Same for a kernel handle with an argument-pointer array (generated kernels).
inline cudaError_t launchDependentC(const void* kernel, dim3 grid, dim3 block, void** args, size_t smem, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependentLaunchEnabled() ? 1 : 0;
    return cudaLaunchKernelExC(&cfg, kernel, args);
}

// Device properties that launch geometry needs, cached per device.
struct DeviceInfo {
    int sm_count = 0;
    int cc_major = 0;
    int cc_minor = 0;
    size_t smem_optin = 0;
};
int currentDeviceInfo(const DeviceInfo** out);

// ---- dtype traits ------------------------------------------------------------------------------
template <int DT> struct CType;
template <> struct CType<THOR_B200_FP16> { using type = __half; };
template <> struct CType<THOR_B200_BF16> { using type = __nv_bfloat16; };
template <> struct CType<THOR_B200_FP32> { using type = float; };
template <> struct CType<THOR_B200_FP64> { using type = double; };
template <> struct CType<THOR_B200_INT8> { using type = int8_t; };
template <> struct CType<THOR_B200_INT16> { using type = int16_t; };
template <> struct CType<THOR_B200_INT32> { using type = int32_t; };
template <> struct CType<THOR_B200_INT64> { using type = int64_t; };
template <> struct CType<THOR_B200_UINT8> { using type = uint8_t; };
template <> struct CType<THOR_B200_UINT16> { using type = uint16_t; };
template <> struct CType<THOR_B200_UINT32> { using type = uint32_t; };
template <> struct CType<THOR_B200_UINT64> { using type = uint64_t; };
template <> struct CType<THOR_B200_BOOLEAN> { using type = bool; };
template <> struct CType<THOR_B200_FP8_E4M3> { using type = __nv_fp8_e4m3; };
template <> struct CType<THOR_B200_FP8_E5M2> { using type = __nv_fp8_e5m2; };

inline size_t dtypeSize(int dt) {
    switch (dt) {
        case THOR_B200_FP16: case THOR_B200_BF16: case THOR_B200_INT16: case THOR_B200_UINT16: return 2;
        case THOR_B200_FP32: case THOR_B200_INT32: case THOR_B200_UINT32: return 4;
        case THOR_B200_FP64: case THOR_B200_INT64: case THOR_B200_UINT64: return 8;
        case THOR_B200_INT8: case THOR_B200_UINT8: case THOR_B200_BOOLEAN:
        case THOR_B200_FP8_E4M3: case THOR_B200_FP8_E5M2: return 1;
        default: return 0;
    }
}

inline bool isFloatDtype(int dt) {
    return dt == THOR_B200_FP16 || dt == THOR_B200_BF16 || dt == THOR_B200_FP32 || dt == THOR_B200_FP64 ||
           dt == THOR_B200_FP8_E4M3 || dt == THOR_B200_FP8_E5M2;
}

const char* dtypeName(int dt);

// ---- vector I/O --------------------------------------------------------------------------------
// A pack of BYTES bytes moved with the widest accesses the size allows (16-byte LDG/STG.128).
// Streaming data is touched once, so loads bypass L1 allocation (ld.global.nc / __ldg is not
// used because in-place callers alias src and dst) and stores are plain.
template <int BYTES>
struct alignas(BYTES >= 16 ? 16 : BYTES) Pack {
    static_assert(BYTES == 1 || BYTES == 2 || BYTES == 4 || BYTES == 8 || (BYTES % 16) == 0, "pack size");
    unsigned char b[BYTES];
};

// 256-bit global load (sm_100 LDG.256); the address must be 32-byte aligned.
__device__ __forceinline__ void load256(uint4& lo, uint4& hi, const void* p) {
    asm volatile("ld.global.cs.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w), "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w)
                 : "l"(p));
}

template <int BYTES, bool WIDE = false>
__device__ __forceinline__ void loadPack(Pack<BYTES>& dst, const void* src) {
    if constexpr (WIDE && (BYTES % 32) == 0) {
#pragma unroll
        for (int i = 0; i < BYTES / 32; ++i)
            load256(reinterpret_cast<uint4*>(&dst)[2 * i], reinterpret_cast<uint4*>(&dst)[2 * i + 1], reinterpret_cast<const char*>(src) + 32 * i);
    } else if constexpr (BYTES >= 16) {
#pragma unroll
        for (int i = 0; i < BYTES / 16; ++i)
            reinterpret_cast<uint4*>(&dst)[i] = __ldcs(reinterpret_cast<const uint4*>(src) + i);
    } else if constexpr (BYTES == 8) {
        *reinterpret_cast<uint2*>(&dst) = __ldcs(reinterpret_cast<const uint2*>(src));
    } else if constexpr (BYTES == 4) {
        *reinterpret_cast<uint32_t*>(&dst) = __ldcs(reinterpret_cast<const uint32_t*>(src));
    } else if constexpr (BYTES == 2) {
        *reinterpret_cast<uint16_t*>(&dst) = __ldcs(reinterpret_cast<const uint16_t*>(src));
    } else {
        *reinterpret_cast<uint8_t*>(&dst) = __ldcs(reinterpret_cast<const uint8_t*>(src));
    }
}

template <int BYTES>
__device__ __forceinline__ void storePack(void* dst, const Pack<BYTES>& src) {
    if constexpr (BYTES >= 16) {
#pragma unroll
        for (int i = 0; i < BYTES / 16; ++i)
            __stcs(reinterpret_cast<uint4*>(dst) + i, reinterpret_cast<const uint4*>(&src)[i]);
    } else if constexpr (BYTES == 8) {
        __stcs(reinterpret_cast<uint2*>(dst), *reinterpret_cast<const uint2*>(&src));
    } else if constexpr (BYTES == 4) {
        __stcs(reinterpret_cast<uint32_t*>(dst), *reinterpret_cast<const uint32_t*>(&src));
    } else if constexpr (BYTES == 2) {
        __stcs(reinterpret_cast<uint16_t*>(dst), *reinterpret_cast<const uint16_t*>(&src));
    } else {
        __stcs(reinterpret_cast<uint8_t*>(dst), *reinterpret_cast<const uint8_t*>(&src));
    }
}

inline bool isAligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

}  // namespace tb
