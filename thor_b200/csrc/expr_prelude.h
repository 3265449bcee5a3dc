// Device prelude of every generated fused-stage kernel, handed to NVRTC as the in-memory header
// "tb_prelude.cuh".  Hand-written for sm_100a: 16-byte packs, streaming (evict-first) loads and
// stores for data touched once, cached loads for operands that are re-used across rows.
#pragma once

namespace tb::expr {

static const char* const kPrelude = R"TBPRELUDE(
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>

typedef unsigned long long tb_u64;
typedef unsigned int tb_u32;

template <int BYTES>
struct __align__(BYTES >= 16 ? 16 : BYTES) tb_pack {
    unsigned char b[BYTES];
};

// Streaming load: the data is read exactly once by the whole grid (ld.global.cs).
template <int BYTES>
__device__ __forceinline__ void tb_load_stream(tb_pack<BYTES>& dst, const void* src) {
    if constexpr (BYTES >= 16) {
#pragma unroll
        for (int i = 0; i < BYTES / 16; ++i) reinterpret_cast<uint4*>(&dst)[i] = __ldcs(reinterpret_cast<const uint4*>(src) + i);
    } else if constexpr (BYTES == 8) {
        *reinterpret_cast<uint2*>(&dst) = __ldcs(reinterpret_cast<const uint2*>(src));
    } else if constexpr (BYTES == 4) {
        *reinterpret_cast<unsigned int*>(&dst) = __ldcs(reinterpret_cast<const unsigned int*>(src));
    } else if constexpr (BYTES == 2) {
        *reinterpret_cast<unsigned short*>(&dst) = __ldcs(reinterpret_cast<const unsigned short*>(src));
    } else {
        *reinterpret_cast<unsigned char*>(&dst) = __ldcs(reinterpret_cast<const unsigned char*>(src));
    }
}

// Cached load: operands shared by many CTAs (per-column vectors) should stay in L1/L2.
template <int BYTES>
__device__ __forceinline__ void tb_load_keep(tb_pack<BYTES>& dst, const void* src) {
    if constexpr (BYTES >= 16) {
#pragma unroll
        for (int i = 0; i < BYTES / 16; ++i) reinterpret_cast<uint4*>(&dst)[i] = __ldca(reinterpret_cast<const uint4*>(src) + i);
    } else if constexpr (BYTES == 8) {
        *reinterpret_cast<uint2*>(&dst) = __ldca(reinterpret_cast<const uint2*>(src));
    } else if constexpr (BYTES == 4) {
        *reinterpret_cast<unsigned int*>(&dst) = __ldca(reinterpret_cast<const unsigned int*>(src));
    } else if constexpr (BYTES == 2) {
        *reinterpret_cast<unsigned short*>(&dst) = __ldca(reinterpret_cast<const unsigned short*>(src));
    } else {
        *reinterpret_cast<unsigned char*>(&dst) = __ldca(reinterpret_cast<const unsigned char*>(src));
    }
}

template <int BYTES>
__device__ __forceinline__ void tb_store_stream(void* dst, const tb_pack<BYTES>& src) {
    if constexpr (BYTES >= 16) {
#pragma unroll
        for (int i = 0; i < BYTES / 16; ++i) __stcs(reinterpret_cast<uint4*>(dst) + i, reinterpret_cast<const uint4*>(&src)[i]);
    } else if constexpr (BYTES == 8) {
        __stcs(reinterpret_cast<uint2*>(dst), *reinterpret_cast<const uint2*>(&src));
    } else if constexpr (BYTES == 4) {
        __stcs(reinterpret_cast<unsigned int*>(dst), *reinterpret_cast<const unsigned int*>(&src));
    } else if constexpr (BYTES == 2) {
        __stcs(reinterpret_cast<unsigned short*>(dst), *reinterpret_cast<const unsigned short*>(&src));
    } else {
        __stcs(reinterpret_cast<unsigned char*>(dst), *reinterpret_cast<const unsigned char*>(&src));
    }
}

// fp8 e4m3 stores saturate to the largest finite value (+-448).
__device__ __forceinline__ __nv_fp8_e4m3 tb_to_e4m3(float v) {
    __nv_fp8_e4m3 r;
    r.__x = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
    return r;
}

// digamma(x): reflection for x < 0.5, upward recurrence to x >= 6, then the asymptotic series
// ln x - 1/(2x) - sum B_2k / (2k x^2k).
__device__ __forceinline__ float tb_digammaf(float x) {
    const float pi = 3.14159265358979323846f;
    if (x != x) return x;
    float reflect = 0.0f;
    bool reflected = false;
    if (x < 0.5f) {
        if (x == floorf(x)) return __int_as_float(0x7fffffff);  // poles at 0, -1, -2, ...
        reflect = pi / tanf(pi * x);
        x = 1.0f - x;
        reflected = true;
    }
    float acc = 0.0f;
    while (x < 6.0f) {
        acc -= 1.0f / x;
        x += 1.0f;
    }
    const float inv = 1.0f / x;
    const float inv2 = inv * inv;
    const float series = inv2 * (1.0f / 12.0f - inv2 * (1.0f / 120.0f - inv2 * (1.0f / 252.0f - inv2 * (1.0f / 240.0f - inv2 * (1.0f / 132.0f)))));
    const float r = acc + logf(x) - 0.5f * inv - series;
    return reflected ? r - reflect : r;
}
)TBPRELUDE";

// Team-wide reductions of the row-program kernels ("tb_rowprog.cuh").
static const char* const kRowProgPrelude = R"TBROWPROG(
__device__ __forceinline__ float tb_add(float a, float b) { return a + b; }
__device__ __forceinline__ float tb_mul(float a, float b) { return a * b; }
// NaN-propagating min / max, the rule of the reduction seam.
__device__ __forceinline__ float tb_nanmin(float a, float b) { return a != a ? a : (b != b ? b : fminf(a, b)); }
__device__ __forceinline__ float tb_nanmax(float a, float b) { return a != a ? a : (b != b ? b : fmaxf(a, b)); }

// Stage 1: xor butterfly inside each warp (every lane ends with the warp's value, bit-identical
// across lanes because the operators are commutative); warp leaders of wide teams publish it.
template <int TEAM, float (*OP)(float, float)>
__device__ __forceinline__ float tb_team_reduce_stage1(float v, float* smem) {
    constexpr int SPAN = TEAM < 32 ? TEAM : 32;
#pragma unroll
    for (int off = SPAN / 2; off > 0; off >>= 1) v = OP(v, __shfl_xor_sync(0xffffffffu, v, off, SPAN));
    if (TEAM > 32 && (threadIdx.x & 31) == 0) smem[(threadIdx.x % TEAM) >> 5] = v;
    return v;
}
// Stage 2 (after a __syncthreads): every thread folds the warp values in warp order.
template <int TEAM, float (*OP)(float, float)>
__device__ __forceinline__ float tb_team_reduce_stage2(float v, const float* smem) {
    if (TEAM <= 32) return v;
    float r = smem[0];
#pragma unroll
    for (int w = 1; w < TEAM / 32; ++w) r = OP(r, smem[w]);
    return r;
}
)TBROWPROG";

}  // namespace tb::expr
