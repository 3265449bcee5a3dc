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

// First statements of every generated kernel: wait until the previous kernel of the stream has completed
// and its writes are visible (the kernel is launched with stream serialization relaxed, so its CTAs may
// already sit on the SMs while that kernel drains), then let the next kernel be placed the same way.
__device__ __forceinline__ void tb_grid_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
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

// ---- lean pair math -------------------------------------------------------------------------------
// Bit-identical replacements for two cuda_fp16.hpp pair routines that dominate the instruction count
// of 16-bit stages (h2exp, __h2div).  Same arithmetic per lane (fp32 multiply by log2(e),
// ex2.approx.ftz.f32, one round-to-nearest conversion, the same special-input corrections; fp32
// reciprocal-multiply with the same refinement for tiny quotients), but packed conversions and a
// packed test for the rare refinement.  thor_b200_selfcheck_pair_math compares them with the toolkit
// routines over every input (exp) and every input pair (div).
__device__ __forceinline__ __half2 tb_bits2half2(unsigned int v) {
    __half2 r;
    *reinterpret_cast<unsigned int*>(&r) = v;
    return r;
}
__device__ __forceinline__ __half2 tb_h2exp_core(const __half2 a) {
    const float2 f = __half22float2(a);
    float lo, hi;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(lo) : "f"(__fmaf_rn(f.x, __int_as_float(0x3fb8aa3b), __int_as_float(0x80000000))));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(hi) : "f"(__fmaf_rn(f.y, __int_as_float(0x3fb8aa3b), __int_as_float(0x80000000))));
    return __floats2half2_rn(lo, hi);
}
__device__ __forceinline__ __half2 tb_h2exp_fix(const __half2 a, const __half2 r, unsigned int special, unsigned int ulp) {
    return __hfma2(__heq2(a, tb_bits2half2(special)), tb_bits2half2(ulp), r);
}
__device__ __forceinline__ __half2 tb_h2exp(const __half2 a) {
    __half2 r = tb_h2exp_core(a);
    r = tb_h2exp_fix(a, r, 0x1F791F79u, 0x94009400u);
    r = tb_h2exp_fix(a, r, 0x25CF25CFu, 0x94009400u);
    r = tb_h2exp_fix(a, r, 0xC13BC13Bu, 0x04000400u);
    r = tb_h2exp_fix(a, r, 0xC1EFC1EFu, 0x02000200u);
    return r;
}
// Argument known to be <= 0 (or NaN): the two corrections for positive inputs can never fire.
__device__ __forceinline__ __half2 tb_h2exp_nonpos(const __half2 a) {
    __half2 r = tb_h2exp_core(a);
    r = tb_h2exp_fix(a, r, 0xC13BC13Bu, 0x04000400u);
    r = tb_h2exp_fix(a, r, 0xC1EFC1EFu, 0x02000200u);
    return r;
}
// Lane-wise z < 0 ? if_negative : otherwise (false for -0 and NaN, like the comparison).
__device__ __forceinline__ __half2 tb_h2sel_neg(const __half2 z, const __half2 if_negative, const __half2 otherwise) {
    const unsigned int m = __hlt2_mask(z, __half2half2(__ushort_as_half((unsigned short)0)));
    const unsigned int a = *reinterpret_cast<const unsigned int*>(&if_negative), b = *reinterpret_cast<const unsigned int*>(&otherwise);
    const unsigned int r = (a & m) | (b & ~m);
    return *reinterpret_cast<const __half2*>(&r);
}
__device__ __forceinline__ __nv_bfloat162 tb_h2sel_neg(const __nv_bfloat162 z, const __nv_bfloat162 if_negative, const __nv_bfloat162 otherwise) {
    const unsigned int m = __hlt2_mask(z, __bfloat162bfloat162(__ushort_as_bfloat16((unsigned short)0)));
    const unsigned int a = *reinterpret_cast<const unsigned int*>(&if_negative), b = *reinterpret_cast<const unsigned int*>(&otherwise);
    const unsigned int r = (a & m) | (b & ~m);
    return *reinterpret_cast<const __nv_bfloat162*>(&r);
}
__device__ __forceinline__ __half2 tb_h2div(const __half2 a, const __half2 b) {
    const float2 fa = __half22float2(a), fb = __half22float2(b);
    float rx, ry;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rx) : "f"(fb.x));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(ry) : "f"(fb.y));
    const __half2 v = __floats2half2_rn(rx * fa.x, ry * fa.y);
    // the toolkit routine refines a lane whose quotient q satisfies 0 < |q| < 0x008F (as fp16 bits)
    const unsigned int bits = *reinterpret_cast<const unsigned int*>(&v) & 0x7fff7fffu;
    if (((bits & 0xffffu) - 1u) < 0x8Eu || ((bits >> 16) - 1u) < 0x8Eu) return __h2div(a, b);
    return v;
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
// NaN-propagating min / max in one instruction (the result for a NaN operand is the canonical NaN 0x7fffffff).
__device__ __forceinline__ float tb_max_nan(float a, float b) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ float tb_min_nan(float a, float b) {
    float r;
    asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
// Three values: two instructions (the three-input form of sm_100 needs a newer PTX version than every NVRTC that may be
// loaded at run time accepts, so generated code stays with the two-input form).
__device__ __forceinline__ float tb_max3_nan(float a, float b, float c) { return tb_max_nan(a, tb_max_nan(b, c)); }
__device__ __forceinline__ float tb_min3_nan(float a, float b, float c) { return tb_min_nan(a, tb_min_nan(b, c)); }
// NaN-propagating min / max, the rule of the reduction seam.
__device__ __forceinline__ float tb_nanmin(float a, float b) { return a != a ? a : (b != b ? b : fminf(a, b)); }
__device__ __forceinline__ float tb_nanmax(float a, float b) { return a != a ? a : (b != b ? b : fmaxf(a, b)); }

// ---- bulk copies through the TMA engine (no tensor map) into a ring of row buffers, completion on an mbarrier ----
// Every wait is bounded by wall-clock time: a wait that runs out counts in tb_wait_expired (read by the host),
// raises the CTA's flag so that later waits give up quickly, and lets the kernel run to its end on stale data.
#ifdef TB_BULK_RING
#ifndef TB_WAIT_LIMIT_NS
#define TB_WAIT_LIMIT_NS 2000000000ull  // two seconds: far beyond any copy, short enough that the device keeps answering
#endif
__device__ unsigned int tb_wait_expired = 0;
__device__ __forceinline__ unsigned tb_smem_addr(const void* ptr) { return static_cast<unsigned>(__cvta_generic_to_shared(ptr)); }
__device__ __forceinline__ void tb_mbar_init(tb_u64* bar, unsigned arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tb_smem_addr(bar)), "r"(arrivals) : "memory");
}
__device__ __forceinline__ void tb_mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tb_mbar_expect(tb_u64* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tb_smem_addr(bar)), "r"(bytes) : "memory");
}
// source and destination 16-byte aligned, size a multiple of 16 bytes
__device__ __forceinline__ void tb_bulk_load(void* smem, const void* gmem, unsigned bytes, tb_u64* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(tb_smem_addr(smem)), "l"(gmem), "r"(bytes),
                 "r"(tb_smem_addr(bar))
                 : "memory");
}
__device__ __forceinline__ void tb_mbar_arrive(tb_u64* bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tb_smem_addr(bar)) : "memory"); }
// Barrier among the first THREADS threads of the CTA (a multiple of 32), leaving __syncthreads' barrier 0 alone.
template <int ID, int THREADS>
__device__ __forceinline__ void tb_named_barrier() { asm volatile("bar.sync %0, %1;" ::"n"(ID), "n"(THREADS) : "memory"); }
// Register hand-over between warpgroups (every warp of a warpgroup must execute the same one): the copy warpgroup keeps
// 24 registers per thread, the two team warpgroups grow to 240 (per SM sub-partition: 2 x 240 + 24 <= 512 per lane).
__device__ __forceinline__ void tb_release_registers() { asm volatile("setmaxnreg.dec.sync.aligned.u32 24;"); }
__device__ __forceinline__ void tb_claim_registers() { asm volatile("setmaxnreg.inc.sync.aligned.u32 240;"); }
__device__ __forceinline__ tb_u64 tb_now_ns() {
    tb_u64 ns;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns));
    return ns;
}
__device__ __forceinline__ void tb_mbar_wait(tb_u64* bar, unsigned parity, volatile int* gave_up) {
    const unsigned addr = tb_smem_addr(bar);
    unsigned done = 0;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return;
    const tb_u64 start = tb_now_ns();
    const tb_u64 limit_ns = *gave_up ? 100000ull : (tb_u64)TB_WAIT_LIMIT_NS;
    while (tb_now_ns() - start < limit_ns) {
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return;
    }
    if (!*gave_up) atomicAdd(&tb_wait_expired, 1u);
    *gave_up = 1;
}
#endif

// 16-byte asynchronous global -> shared copy (LDGSTS, bypasses registers and L1) and its group fences.
__device__ __forceinline__ void tb_cp_async16(void* smem, const void* gmem) {
    const unsigned addr = static_cast<unsigned>(__cvta_generic_to_shared(smem));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(addr), "l"(gmem) : "memory");
}
__device__ __forceinline__ void tb_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// two-lane value of a type without a native pair type; tb_both broadcasts a float to both lanes of a float2
template <class T>
struct tb_pr {
    T x, y;
};
__device__ __forceinline__ float2 tb_both(float v) { return make_float2(v, v); }
__device__ __forceinline__ void tb_prefetch_l2(const void* gmem) { asm volatile("prefetch.global.L2 [%0];" ::"l"(gmem)); }
template <int N>
__device__ __forceinline__ void tb_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

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
// Arg reductions: candidates are (value, index); NaN beats numbers, then the better value, then the lower index
// (the rule of the arg-reduction seam).  index 0xffffffff marks "no candidate".
template <bool IS_MAX>
__device__ __forceinline__ bool tb_arg_better(float v, tb_u32 i, float bv, tb_u32 bi) {
    if (bi == 0xffffffffu) return true;
    if (i == 0xffffffffu) return false;
    const bool vn = v != v, bn = bv != bv;
    if (vn != bn) return vn;
    if (!vn && v != bv) return IS_MAX ? v > bv : v < bv;
    return i < bi;
}
template <bool IS_MAX>
__device__ __forceinline__ void tb_arg_update(float& bv, tb_u32& bi, float v, tb_u32 i) {
    if (tb_arg_better<IS_MAX>(v, i, bv, bi)) {
        bv = v;
        bi = i;
    }
}
// Scan of one thread's elements, which it visits in increasing column order: a strict compare keeps the lowest
// index among equals, the first NaN is remembered on the side.  tb_arg_scan_finish turns the pair into a candidate:
// a NaN wins; a thread whose values never beat the starting value (all -inf for max / +inf for min) offers its first one.
template <bool IS_MAX>
__device__ __forceinline__ void tb_arg_scan(float& bv, tb_u32& bi, tb_u32& nan_i, float v, tb_u32 col) {
    if (IS_MAX ? v > bv : v < bv) {
        bv = v;
        bi = col;
    }
    nan_i = min(nan_i, v != v ? col : 0xffffffffu);
}
template <bool IS_MAX>
__device__ __forceinline__ void tb_arg_scan_finish(float& bv, tb_u32& bi, tb_u32 nan_i, bool has_elements, tb_u32 first_col) {
    if (nan_i != 0xffffffffu) {
        bv = __int_as_float(0x7fffffff);
        bi = nan_i;
    } else if (bi == 0xffffffffu && has_elements) {
        bi = first_col;
    }
}
// Team combine of arg candidates: each thread's candidate becomes one 64-bit key whose unsigned order is the
// arg rule -- NaN above everything, then the value in its float order (reversed for arg-min, -0 and +0 equal),
// then the LOWER index (stored complemented) -- so lanes and warps combine with a plain 64-bit max.
// 0 means "no candidate".  Only the team's first thread needs the result: it folds the warp keys.
template <bool IS_MAX>
__device__ __forceinline__ tb_u64 tb_arg_key(float v, tb_u32 i) {
    if (i == 0xffffffffu) return 0ull;
    tb_u32 b = v == 0.0f ? 0u : __float_as_uint(v);
    tb_u32 k = (b & 0x80000000u) ? ~b : (b | 0x80000000u);  // ascending with the float order
    if (!IS_MAX) k = ~k;
    if (v != v) k = 0xffffffffu;
    return ((tb_u64)k << 32) | (tb_u64)(tb_u32)~i;
}
template <int TEAM>
__device__ __forceinline__ tb_u64 tb_team_arg_stage1(tb_u64 key, tb_u64* smem) {
    constexpr int SPAN = TEAM < 32 ? TEAM : 32;
#pragma unroll
    for (int off = SPAN / 2; off > 0; off >>= 1) {
        const tb_u64 other = __shfl_xor_sync(0xffffffffu, key, off, SPAN);
        key = other > key ? other : key;
    }
    if (TEAM > 32 && (threadIdx.x & 31) == 0) smem[(threadIdx.x % TEAM) >> 5] = key;
    return key;
}
template <int TEAM>
__device__ __forceinline__ tb_u32 tb_team_arg_stage2(tb_u64 key, const tb_u64* smem) {
    if (TEAM > 32) {
        key = smem[0];
#pragma unroll
        for (int w = 1; w < TEAM / 32; ++w) key = smem[w] > key ? smem[w] : key;
    }
    return ~(tb_u32)key;
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
