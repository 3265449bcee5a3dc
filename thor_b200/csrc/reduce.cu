// Dense value reductions over a tensor viewed as [outer, reduction, inner].
//
// Kernel families (all accumulate in fp32, one store conversion at the end):
//   rows   inner == 1.  A team of 8, 32 or 256 threads owns one row and streams it with 16-byte
//          loads (scalar head/tail peel, so no alignment or padding is required).  When there are
//          too few rows to fill the GPU, every row is cut into S contiguous splits (one CTA each),
//          fp32 partials go to the workspace and a second small kernel folds them in a fixed order
//          -- the two-phase full reduction is the outer == 1 case of this.
//   cols   inner > 1.  A CTA owns a [reduction chunk x inner tile] slab: threads are laid out
//          TX along inner (16-byte packs) x TY along the reduction axis, each thread keeps one fp32
//          accumulator per pack lane, the TY partials are combined through shared memory.  The
//          reduction axis is split across CTAs (the reference walks it serially per CTA, which
//          leaves a [1, 32768, 8192] column sum on 2 CTAs); partials are folded by a second kernel.
// The fold order never depends on timing, so results are bit-reproducible run to run.
#include "common.cuh"

#include <cfloat>
#include <memory>
#include <mutex>

namespace tb {

namespace {

constexpr int kThreads = 256;
constexpr int kAssumedSms = 148;  // used for planning when no device is present

// ---- op traits -----------------------------------------------------------------------------------
template <int OP> struct OpTraits;
template <> struct OpTraits<THOR_B200_REDUCE_SUM> {
    __device__ static float identity() { return 0.0f; }
    __device__ static float transform(float v) { return v; }
    __device__ static float combine(float a, float b) { return a + b; }
};
template <> struct OpTraits<THOR_B200_REDUCE_MEAN> : OpTraits<THOR_B200_REDUCE_SUM> {};
template <> struct OpTraits<THOR_B200_REDUCE_L1NORM> : OpTraits<THOR_B200_REDUCE_SUM> {
    __device__ static float transform(float v) { return fabsf(v); }
};
template <> struct OpTraits<THOR_B200_REDUCE_L2NORM> : OpTraits<THOR_B200_REDUCE_SUM> {
    __device__ static float transform(float v) { return v * v; }
};
template <> struct OpTraits<THOR_B200_REDUCE_PRODUCT> {
    __device__ static float identity() { return 1.0f; }
    __device__ static float transform(float v) { return v; }
    __device__ static float combine(float a, float b) { return a * b; }
};
// NaN-propagating min / max (CubReductionOperation.cuh:106-129) as ONE instruction, min.NaN / max.NaN; the result for a NaN
// operand is the canonical NaN (the two compares and selects around fminf / fmaxf kept the payload of the first NaN).
__device__ __forceinline__ float minNaN(float a, float b) {
    float r;
    asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ float maxNaN(float a, float b) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
template <> struct OpTraits<THOR_B200_REDUCE_MIN> {
    __device__ static float identity() { return __int_as_float(0x7f800000); }
    __device__ static float transform(float v) { return v; }
    __device__ static float combine(float a, float b) { return minNaN(a, b); }
};
template <> struct OpTraits<THOR_B200_REDUCE_MAX> {
    __device__ static float identity() { return __int_as_float(0xff800000); }
    __device__ static float transform(float v) { return v; }
    __device__ static float combine(float a, float b) { return maxNaN(a, b); }
};

template <class T> __device__ __forceinline__ float toFloat(T v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ float toFloat<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float toFloat<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// Finalise (CubReductionOperation.cuh:81-103), scale, convert once, store.
__device__ __forceinline__ float finalizeValue(int op, float v, float divisor, float scale) {
    if (op == THOR_B200_REDUCE_MEAN) v = divisor == 0.0f ? 0.0f : (divisor == 1.0f ? v : v / divisor);
    else if (op == THOR_B200_REDUCE_L2NORM) v = sqrtf(v);
    return v * scale;
}
__device__ __forceinline__ void storeAs(void* out, int dtype, uint64_t idx, float v) {
    switch (dtype) {
        case THOR_B200_FP32: static_cast<float*>(out)[idx] = v; break;
        case THOR_B200_FP16: static_cast<__half*>(out)[idx] = __float2half_rn(v); break;
        case THOR_B200_BF16: static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v); break;
        case THOR_B200_FP8_E4M3: static_cast<__nv_fp8_storage_t*>(out)[idx] = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3); break;
        case THOR_B200_FP8_E5M2: static_cast<__nv_fp8_storage_t*>(out)[idx] = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E5M2); break;
        default: break;
    }
}

// Combine across a team of TEAM consecutive threads (TEAM = 8, 32 or 256); the result is valid in
// the team's first thread.  The shuffle / shared-memory tree has a fixed shape.
template <int OP, int TEAM>
__device__ __forceinline__ float teamCombine(float v, float* smem) {
    using Tr = OpTraits<OP>;
    constexpr int kWarpSpan = TEAM < 32 ? TEAM : 32;
#pragma unroll
    for (int off = kWarpSpan / 2; off > 0; off >>= 1) v = Tr::combine(v, __shfl_down_sync(0xffffffffu, v, off, kWarpSpan));
    if constexpr (TEAM > 32) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        if (lane == 0) smem[warp] = v;
        __syncthreads();
        if (warp == 0) {
            v = lane < TEAM / 32 ? smem[lane] : Tr::identity();
#pragma unroll
            for (int off = TEAM / 64; off > 0; off >>= 1) v = Tr::combine(v, __shfl_down_sync(0xffffffffu, v, off));
        }
    }
    return v;
}

struct RowsArgs {
    const void* in;
    void* out;
    float* partials;  // [outer][splits] when splits > 1
    uint64_t outer, reduction, out_stride;
    uint32_t splits;
    int op, out_dtype;
    float divisor, scale;
};

// One team per (row, split).  blockIdx.x = row_group * splits + split.
template <class T, int OP, int TEAM>
__global__ void __launch_bounds__(kThreads) rowsKernel(RowsArgs a) {
    gridDependencyWait();
    gridLaunchDependents();
    using Tr = OpTraits<OP>;
    constexpr int VEC = 16 / sizeof(T);
    constexpr int U = 4;
    constexpr int kTeamsPerCta = kThreads / TEAM;
    __shared__ float smem[32];
    const uint32_t split = blockIdx.x % a.splits;
    const uint64_t row = static_cast<uint64_t>(blockIdx.x / a.splits) * kTeamsPerCta + threadIdx.x / TEAM;
    const int t = threadIdx.x % TEAM;
    float acc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = Tr::identity();
    if (row < a.outer) {
        // element range of this split inside the row
        const uint64_t per = (a.reduction + a.splits - 1) / a.splits;
        const uint64_t lo = static_cast<uint64_t>(split) * per;
        const uint64_t hi = lo + per < a.reduction ? lo + per : a.reduction;
        const T* p = static_cast<const T*>(a.in) + row * a.reduction;
        if (lo < hi) {
            // peel to a 16-byte boundary, stream aligned packs, finish the ragged tail one by one
            const uintptr_t addr = reinterpret_cast<uintptr_t>(p + lo);
            uint64_t head = ((16 - (addr & 15)) & 15) / sizeof(T);
            if (head > hi - lo) head = hi - lo;
            const uint64_t body0 = lo + head;
            const uint64_t n_packs = (hi - body0) / VEC;
            const uint64_t tail0 = body0 + n_packs * VEC;
            for (uint64_t i = lo + t; i < body0; i += TEAM) acc[0] = Tr::combine(acc[0], Tr::transform(toFloat(p[i])));
            for (uint64_t i = tail0 + t; i < hi; i += TEAM) acc[0] = Tr::combine(acc[0], Tr::transform(toFloat(p[i])));
            const T* body = p + body0;
            for (uint64_t q = t; q < n_packs; q += static_cast<uint64_t>(TEAM) * U) {
                Pack<16> pk[U];
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (q + static_cast<uint64_t>(u) * TEAM < n_packs) loadPack(pk[u], body + (q + static_cast<uint64_t>(u) * TEAM) * VEC);
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (q + static_cast<uint64_t>(u) * TEAM < n_packs) {
#pragma unroll
                        for (int j = 0; j < VEC; ++j) acc[j] = Tr::combine(acc[j], Tr::transform(toFloat(reinterpret_cast<const T*>(&pk[u])[j])));
                    }
            }
        }
    }
    float v = acc[0];
#pragma unroll
    for (int j = 1; j < VEC; ++j) v = Tr::combine(v, acc[j]);
    v = teamCombine<OP, TEAM>(v, smem);
    if (t == 0 && row < a.outer) {
        if (a.splits == 1) storeAs(a.out, a.out_dtype, row * a.out_stride, finalizeValue(a.op, v, a.divisor, a.scale));
        else a.partials[row * a.splits + split] = v;
    }
}

// Folds the per-split partials of each row: one CTA per row, thread t takes partials t, t+256, ...
template <int OP>
__global__ void __launch_bounds__(kThreads) rowsFoldKernel(RowsArgs a) {
    gridDependencyWait();
    gridLaunchDependents();
    using Tr = OpTraits<OP>;
    __shared__ float smem[32];
    const uint64_t row = blockIdx.x;
    float v = Tr::identity();
    for (uint32_t s = threadIdx.x; s < a.splits; s += kThreads) v = Tr::combine(v, a.partials[row * a.splits + s]);
    v = teamCombine<OP, 256>(v, smem);
    if (threadIdx.x == 0) storeAs(a.out, a.out_dtype, row * a.out_stride, finalizeValue(a.op, v, a.divisor, a.scale));
}

struct ColsArgs {
    const void* in;
    void* out;
    float* partials;  // [outer][splits][inner] when splits > 1
    uint64_t outer, reduction, inner;
    uint64_t out_stride_outer, out_stride_inner;
    uint32_t splits;
    int op, out_dtype;
    float divisor, scale;
};

// grid = (inner tiles, splits, outer); block = TX x TY threads, thread (tx, ty) owns pack tx of the
// tile and rows ty, ty + TY, ... of the split.
template <class T, int OP, int VEC, int TX>
__global__ void __launch_bounds__(kThreads) colsKernel(ColsArgs a) {
    gridDependencyWait();
    gridLaunchDependents();
    using Tr = OpTraits<OP>;
    constexpr int TY = kThreads / TX;
    constexpr int U = 4;
    __shared__ float smem[TY][TX * VEC + 1];
    const int tx = threadIdx.x % TX, ty = threadIdx.x / TX;
    const uint64_t col = (static_cast<uint64_t>(blockIdx.x) * TX + tx) * VEC;
    const uint64_t o = blockIdx.z;
    const uint64_t per = (a.reduction + a.splits - 1) / a.splits;
    const uint64_t lo = static_cast<uint64_t>(blockIdx.y) * per;
    const uint64_t hi = lo + per < a.reduction ? lo + per : a.reduction;
    float acc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = Tr::identity();
    if (col < a.inner) {
        const T* base = static_cast<const T*>(a.in) + o * a.reduction * a.inner + col;
        for (uint64_t r = lo + ty; r < hi; r += static_cast<uint64_t>(TY) * U) {
            Pack<VEC * sizeof(T)> pk[U];
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (r + static_cast<uint64_t>(u) * TY < hi) loadPack(pk[u], base + (r + static_cast<uint64_t>(u) * TY) * a.inner);
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (r + static_cast<uint64_t>(u) * TY < hi) {
#pragma unroll
                    for (int j = 0; j < VEC; ++j) acc[j] = Tr::combine(acc[j], Tr::transform(toFloat(reinterpret_cast<const T*>(&pk[u])[j])));
                }
        }
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) smem[ty][tx * VEC + j] = acc[j];
    __syncthreads();
    // thread k of the CTA folds column k of the tile over ty = 0 .. TY-1 (fixed order)
    for (int c = threadIdx.x; c < TX * VEC; c += kThreads) {
        const uint64_t i = static_cast<uint64_t>(blockIdx.x) * TX * VEC + c;
        if (i >= a.inner) continue;
        float v = smem[0][c];
#pragma unroll 4
        for (int y = 1; y < TY; ++y) v = Tr::combine(v, smem[y][c]);
        if (a.splits == 1) storeAs(a.out, a.out_dtype, o * a.out_stride_outer + i * a.out_stride_inner, finalizeValue(a.op, v, a.divisor, a.scale));
        else a.partials[(o * a.splits + blockIdx.y) * a.inner + i] = v;
    }
}

template <int OP>
__global__ void __launch_bounds__(kThreads) colsFoldKernel(ColsArgs a) {
    gridDependencyWait();
    gridLaunchDependents();
    using Tr = OpTraits<OP>;
    const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
    if (idx >= a.outer * a.inner) return;
    const uint64_t o = idx / a.inner, i = idx % a.inner;
    float v = Tr::identity();
    for (uint32_t s = 0; s < a.splits; ++s) v = Tr::combine(v, a.partials[(o * a.splits + s) * a.inner + i]);
    storeAs(a.out, a.out_dtype, o * a.out_stride_outer + i * a.out_stride_inner, finalizeValue(a.op, v, a.divisor, a.scale));
}

enum class Family { Rows, Cols };

}  // namespace
}  // namespace tb

struct thor_b200_reduce_plan {
    thor_b200_reduce_desc desc;
    tb::Family family;
    int team = 256;       // rows
    uint32_t splits = 1;  // rows / cols
    int cols_vec = 1, cols_tx = 32;
    size_t workspace_bytes = 1;
    const char* kind = "";
};

namespace tb {
namespace {

bool isReduceFloat(int dt) {
    return dt == THOR_B200_FP32 || dt == THOR_B200_FP16 || dt == THOR_B200_BF16 || dt == THOR_B200_FP8_E4M3 || dt == THOR_B200_FP8_E5M2;
}

template <class T, int OP>
int launchRowsT(const thor_b200_reduce_plan& p, const RowsArgs& a, cudaStream_t stream) {
    const uint64_t teams_per_cta = kThreads / p.team;
    const uint64_t groups = (a.outer + teams_per_cta - 1) / teams_per_cta;
    const uint64_t blocks = groups * a.splits;
    if (blocks > 0x7FFFFFFFull) return fail(THOR_B200_UNSUPPORTED, "reduce: grid too large");
    switch (p.team) {
        case 8: (void)launchDependent(rowsKernel<T, OP, 8>, dim3(static_cast<unsigned>(blocks)), dim3(kThreads), 0, stream, a); break;
        case 32: (void)launchDependent(rowsKernel<T, OP, 32>, dim3(static_cast<unsigned>(blocks)), dim3(kThreads), 0, stream, a); break;
        default: (void)launchDependent(rowsKernel<T, OP, 256>, dim3(static_cast<unsigned>(blocks)), dim3(kThreads), 0, stream, a); break;
    }
    countLaunch();
    TB_CUDA(cudaGetLastError());
    if (a.splits > 1) {
        (void)launchDependent(rowsFoldKernel<OP>, dim3(static_cast<unsigned>(a.outer)), dim3(kThreads), 0, stream, a);
        countLaunch();
        TB_CUDA(cudaGetLastError());
    }
    return THOR_B200_OK;
}

template <class T, int OP>
int launchColsT(const thor_b200_reduce_plan& p, const ColsArgs& a, cudaStream_t stream) {
    constexpr int VEC = 16 / sizeof(T);
    const uint64_t tile = static_cast<uint64_t>(p.cols_tx) * p.cols_vec;
    const uint64_t tiles = (a.inner + tile - 1) / tile;
    if (tiles > 0x7FFFFFFFull || a.splits > 65535u || a.outer > 65535ull) return fail(THOR_B200_UNSUPPORTED, "reduce: grid too large");
    dim3 grid(static_cast<unsigned>(tiles), a.splits, static_cast<unsigned>(a.outer));
    if (p.cols_vec == 1) {
        (void)launchDependent(colsKernel<T, OP, 1, 32>, dim3(grid), dim3(kThreads), 0, stream, a);
    } else {
        switch (p.cols_tx) {
            case 1: (void)launchDependent(colsKernel<T, OP, VEC, 1>, dim3(grid), dim3(kThreads), 0, stream, a); break;
            case 2: (void)launchDependent(colsKernel<T, OP, VEC, 2>, dim3(grid), dim3(kThreads), 0, stream, a); break;
            case 4: (void)launchDependent(colsKernel<T, OP, VEC, 4>, dim3(grid), dim3(kThreads), 0, stream, a); break;
            case 8: (void)launchDependent(colsKernel<T, OP, VEC, 8>, dim3(grid), dim3(kThreads), 0, stream, a); break;
            case 16: (void)launchDependent(colsKernel<T, OP, VEC, 16>, dim3(grid), dim3(kThreads), 0, stream, a); break;
            default: (void)launchDependent(colsKernel<T, OP, VEC, 32>, dim3(grid), dim3(kThreads), 0, stream, a); break;
        }
    }
    countLaunch();
    TB_CUDA(cudaGetLastError());
    if (a.splits > 1) {
        const uint64_t n = a.outer * a.inner;
        (void)launchDependent(colsFoldKernel<OP>, dim3(static_cast<unsigned>((n + kThreads - 1) / kThreads)), dim3(kThreads), 0, stream, a);
        countLaunch();
        TB_CUDA(cudaGetLastError());
    }
    return THOR_B200_OK;
}

template <class T>
int launchOp(const thor_b200_reduce_plan& p, const RowsArgs* ra, const ColsArgs* ca, cudaStream_t stream) {
#define TB_OP(OPV) \
    case OPV: return ra ? launchRowsT<T, OPV>(p, *ra, stream) : launchColsT<T, OPV>(p, *ca, stream);
    switch (p.desc.op) {
        TB_OP(THOR_B200_REDUCE_SUM)
        TB_OP(THOR_B200_REDUCE_MIN)
        TB_OP(THOR_B200_REDUCE_MAX)
        TB_OP(THOR_B200_REDUCE_PRODUCT)
        TB_OP(THOR_B200_REDUCE_MEAN)
        TB_OP(THOR_B200_REDUCE_L1NORM)
        TB_OP(THOR_B200_REDUCE_L2NORM)
        default: break;
    }
#undef TB_OP
    return fail(THOR_B200_INVALID_ARGUMENT, "reduce: unknown op %d", p.desc.op);
}

}  // namespace
}  // namespace tb

extern "C" {

int thor_b200_device_alloc(size_t bytes, void** out_ptr) {
    using namespace tb;
    TB_REQUIRE(out_ptr != nullptr, "device_alloc: out_ptr is null");
    *out_ptr = nullptr;
    TB_CUDA(cudaMalloc(out_ptr, bytes == 0 ? 1 : bytes));
    return THOR_B200_OK;
}

int thor_b200_device_free(void* ptr) {
    using namespace tb;
    if (ptr) TB_CUDA(cudaFree(ptr));
    return THOR_B200_OK;
}

int thor_b200_reduce_plan_create(const thor_b200_reduce_desc* d, thor_b200_reduce_plan** out_plan, size_t* workspace_bytes) {
    using namespace tb;
    TB_REQUIRE(d != nullptr && out_plan != nullptr && workspace_bytes != nullptr, "reduce_plan_create: null argument");
    *out_plan = nullptr;
    TB_REQUIRE(d->op >= THOR_B200_REDUCE_SUM && d->op <= THOR_B200_REDUCE_L2NORM, "reduce: unknown op %d", d->op);
    TB_REQUIRE(isReduceFloat(d->input_dtype), "reduce: unsupported input dtype %s", dtypeName(d->input_dtype));
    TB_REQUIRE(isReduceFloat(d->output_dtype), "reduce: unsupported output dtype %s", dtypeName(d->output_dtype));
    TB_REQUIRE(d->flags == 0, "reduce: flags must be zero");
    // zero-sized dimensions are rejected like CubReduction::analyzeGeometry does (CubReduction.cpp:789-793)
    TB_REQUIRE(d->outer > 0 && d->reduction > 0 && d->inner > 0, "reduce: zero-sized dimension");
    TB_REQUIRE((d->out_stride_outer == 0) == (d->out_stride_inner == 0), "reduce: output strides must both be zero or both be set");
    auto p = std::make_unique<thor_b200_reduce_plan>();
    p->desc = *d;
    if (p->desc.out_stride_outer == 0) {
        p->desc.out_stride_outer = d->inner;
        p->desc.out_stride_inner = 1;
    }
    int sms = kAssumedSms;
    {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) sms = v;
        else (void)cudaGetLastError();
    }
    const size_t esize = dtypeSize(d->input_dtype);
    const uint64_t vec = 16 / esize;
    if (d->inner == 1) {
        p->family = Family::Rows;
        const uint64_t packs = (d->reduction + vec - 1) / vec;
        p->team = packs <= 16 ? 8 : (packs <= 512 ? 32 : 256);
        const uint64_t ctas = (d->outer + (kThreads / p->team) - 1) / (kThreads / p->team);
        p->splits = 1;
        if (p->team == 256 && ctas < static_cast<uint64_t>(2 * sms)) {
            // too few rows to fill the GPU: cut each row so that one CTA streams >= 64 KiB
            const uint64_t chunk_packs = 4096;
            uint64_t s = (packs + chunk_packs - 1) / chunk_packs;
            const uint64_t cap = 1u << 20;
            if (s > cap) s = cap;
            if (s * d->outer > (1ull << 24)) s = (1ull << 24) / d->outer;
            p->splits = static_cast<uint32_t>(s < 1 ? 1 : s);
        }
        p->kind = p->splits > 1 ? (d->outer == 1 ? "full" : "rows_split") : (p->team == 256 ? "rows_cta" : (p->team == 32 ? "rows_warp" : "rows_subwarp"));
        p->workspace_bytes = p->splits > 1 ? static_cast<size_t>(d->outer) * p->splits * sizeof(float) : 1;
    } else {
        p->family = Family::Cols;
        const bool vec_ok = (d->inner % vec) == 0;
        p->cols_vec = vec_ok ? static_cast<int>(vec) : 1;
        if (vec_ok) {
            const uint64_t packs = d->inner / vec;
            int tx = 32;
            while (tx > 1 && static_cast<uint64_t>(tx / 2) >= packs) tx /= 2;
            p->cols_tx = tx;
        } else {
            p->cols_tx = 32;
        }
        const uint64_t tile = static_cast<uint64_t>(p->cols_tx) * p->cols_vec;
        const uint64_t tiles = (d->inner + tile - 1) / tile;
        const uint64_t ty = kThreads / p->cols_tx;
        const uint64_t ctas = tiles * d->outer;
        uint64_t s = 1;
        if (ctas < static_cast<uint64_t>(4 * sms)) {
            s = (static_cast<uint64_t>(4 * sms) + ctas - 1) / ctas;
            const uint64_t max_s = (d->reduction + ty * 8 - 1) / (ty * 8);  // keep >= 8 rows per thread
            if (s > max_s) s = max_s;
            if (s > 4096) s = 4096;
            if (s < 1) s = 1;
        }
        p->splits = static_cast<uint32_t>(s);
        p->kind = s > 1 ? "cols_split" : "cols";
        p->workspace_bytes = s > 1 ? static_cast<size_t>(d->outer) * s * d->inner * sizeof(float) : 1;
    }
    *workspace_bytes = p->workspace_bytes;
    *out_plan = p.release();
    return THOR_B200_OK;
}

int thor_b200_reduce_launch(const thor_b200_reduce_plan* p, const void* input, void* output, void* workspace, size_t workspace_bytes,
                            float output_scale, void* stream_v) {
    using namespace tb;
    TB_REQUIRE(p != nullptr, "reduce_launch: null plan");
    TB_REQUIRE(input != nullptr && output != nullptr, "reduce_launch: null tensor pointer");
    TB_REQUIRE(workspace_bytes >= p->workspace_bytes, "reduce_launch: workspace of %zu bytes is smaller than the planned %zu", workspace_bytes,
               p->workspace_bytes);
    TB_REQUIRE(p->splits == 1 || (workspace != nullptr && isAligned(workspace, 16)), "reduce_launch: workspace must be a 16-byte aligned device pointer");
    TB_REQUIRE(output_scale == output_scale && output_scale - output_scale == 0.0f, "reduce_launch: output_scale must be finite");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const thor_b200_reduce_desc& d = p->desc;
    const float divisor = d.op == THOR_B200_REDUCE_MEAN ? static_cast<float>(d.reduction) : 1.0f;
    RowsArgs ra{};
    ColsArgs ca{};
    const bool rows = p->family == Family::Rows;
    if (rows) {
        ra = RowsArgs{input, output, static_cast<float*>(workspace), d.outer, d.reduction, d.out_stride_outer, p->splits, d.op, d.output_dtype, divisor, output_scale};
    } else {
        if (p->cols_vec > 1) TB_REQUIRE(isAligned(input, 16), "reduce_launch: input must be 16-byte aligned for this geometry");
        ca = ColsArgs{input, output, static_cast<float*>(workspace), d.outer, d.reduction, d.inner, d.out_stride_outer, d.out_stride_inner,
                      p->splits, d.op, d.output_dtype, divisor, output_scale};
    }
    switch (d.input_dtype) {
        case THOR_B200_FP32: return launchOp<float>(*p, rows ? &ra : nullptr, rows ? nullptr : &ca, stream);
        case THOR_B200_FP16: return launchOp<__half>(*p, rows ? &ra : nullptr, rows ? nullptr : &ca, stream);
        case THOR_B200_BF16: return launchOp<__nv_bfloat16>(*p, rows ? &ra : nullptr, rows ? nullptr : &ca, stream);
        case THOR_B200_FP8_E4M3: return launchOp<__nv_fp8_e4m3>(*p, rows ? &ra : nullptr, rows ? nullptr : &ca, stream);
        case THOR_B200_FP8_E5M2: return launchOp<__nv_fp8_e5m2>(*p, rows ? &ra : nullptr, rows ? nullptr : &ca, stream);
        default: break;
    }
    return fail(THOR_B200_INVALID_ARGUMENT, "reduce_launch: unsupported input dtype");
}

const char* thor_b200_reduce_plan_kind(const thor_b200_reduce_plan* p) { return p ? p->kind : ""; }

void thor_b200_reduce_plan_destroy(thor_b200_reduce_plan* p) { delete p; }

}  // extern "C"

// ---------------------------------------------------------------------------------------------------
// Full reduction without any allocation by anybody.
//
// thor_b200_reduce_launch needs a workspace that somebody allocated beforehand.  Some callers have no
// such moment: code that runs under a fixed device-memory budget where every byte was handed out at
// start-up, a plug-in that its host application does not allow to call the allocator, and code on a
// latency-critical path where cudaMalloc's implicit device synchronisation is not acceptable.  For
// them the per-CTA partials of the two-phase full reduction
// live in the fixed array below, which is part of the library image: every GPU that loads the
// library carries these 256 KiB until the process exits.
// ---------------------------------------------------------------------------------------------------
namespace tb {
namespace {

constexpr uint32_t kNoAllocMaxPartials = 65536;  // 256 KiB of fp32 partials
static __device__ __align__(256) float g_noalloc_partials[kNoAllocMaxPartials];

// Device address of g_noalloc_partials per device ordinal.  In host code the array's name is only a
// handle for the runtime, never a pointer a kernel could use, so the address is looked up once per
// device with cudaGetSymbolAddress while that device is current (the first call on a device does this;
// make it before any stream capture begins).  The cached address belongs to the device's context: a
// process that calls cudaDeviceReset must not use this entry point on that device afterwards.
std::mutex g_noalloc_mutex;
float* g_noalloc_ptr[64] = {};

int noAllocScratch(float** out) {
    int dev = -1;
    TB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(THOR_B200_CUDA_ERROR, "reduce_full_noalloc: device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_ptr[dev]) {
        void* p = nullptr;
        TB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_partials));
        g_noalloc_ptr[dev] = static_cast<float*>(p);
    }
    *out = g_noalloc_ptr[dev];
    return THOR_B200_OK;
}

}  // namespace
}  // namespace tb

extern "C" int thor_b200_reduce_full_noalloc(int op, const void* input, int input_dtype, uint64_t n, void* output, int output_dtype, float output_scale,
                                             void* stream_v) {
    using namespace tb;
    TB_REQUIRE(op >= THOR_B200_REDUCE_SUM && op <= THOR_B200_REDUCE_L2NORM, "reduce_full_noalloc: unknown op %d", op);
    TB_REQUIRE(isReduceFloat(input_dtype), "reduce_full_noalloc: unsupported input dtype %s", dtypeName(input_dtype));
    TB_REQUIRE(isReduceFloat(output_dtype), "reduce_full_noalloc: unsupported output dtype %s", dtypeName(output_dtype));
    TB_REQUIRE(input != nullptr && output != nullptr, "reduce_full_noalloc: null tensor pointer");
    TB_REQUIRE(n > 0, "reduce_full_noalloc: zero-sized dimension");
    TB_REQUIRE(output_scale == output_scale && output_scale - output_scale == 0.0f, "reduce_full_noalloc: output_scale must be finite");
    // same cut as the planned path: one CTA per 4096 sixteen-byte packs
    const uint64_t vec = 16 / dtypeSize(input_dtype);
    const uint64_t packs = (n + vec - 1) / vec;
    const uint64_t splits = (packs + 4095) / 4096;
    const uint64_t max_elements = static_cast<uint64_t>(kNoAllocMaxPartials) * 4096 * vec;
    if (splits > kNoAllocMaxPartials)
        return fail(THOR_B200_INVALID_ARGUMENT,
                    "reduce_full_noalloc: %llu elements of %s exceed the fixed scratch of %u partials (limit %llu elements); use thor_b200_reduce_launch with a workspace",
                    static_cast<unsigned long long>(n), dtypeName(input_dtype), kNoAllocMaxPartials, static_cast<unsigned long long>(max_elements));
    float* scratch = nullptr;
    if (int st = noAllocScratch(&scratch)) return st;
    thor_b200_reduce_plan plan{};
    plan.desc.op = op;
    plan.desc.input_dtype = input_dtype;
    plan.desc.output_dtype = output_dtype;
    plan.desc.outer = 1;
    plan.desc.reduction = n;
    plan.desc.inner = 1;
    plan.family = Family::Rows;
    plan.team = 256;
    plan.splits = static_cast<uint32_t>(splits);
    const float divisor = op == THOR_B200_REDUCE_MEAN ? static_cast<float>(n) : 1.0f;
    // Every partial the fold kernel reads is written by the first kernel of this same call, so nothing
    // in the array has to start at zero and stale values of earlier calls are never observed.
    const RowsArgs ra{input, output, scratch, 1, n, 1, plan.splits, op, output_dtype, divisor, output_scale};
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    switch (input_dtype) {
        case THOR_B200_FP32: return launchOp<float>(plan, &ra, nullptr, stream);
        case THOR_B200_FP16: return launchOp<__half>(plan, &ra, nullptr, stream);
        case THOR_B200_BF16: return launchOp<__nv_bfloat16>(plan, &ra, nullptr, stream);
        case THOR_B200_FP8_E4M3: return launchOp<__nv_fp8_e4m3>(plan, &ra, nullptr, stream);
        case THOR_B200_FP8_E5M2: return launchOp<__nv_fp8_e5m2>(plan, &ra, nullptr, stream);
        default: break;
    }
    return fail(THOR_B200_INVALID_ARGUMENT, "reduce_full_noalloc: unsupported input dtype");
}
