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
