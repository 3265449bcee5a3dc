// Dense argmin / argmax over a tensor viewed as [outer, reduction, inner].
//
// Candidates are (fp32 value, index inside the reduction domain).  Ordering rule of the reference
// (CubArgReductionOperation.cuh:31-73): NaN beats every number, and among equal candidates -- two
// NaNs included -- the lower index wins, so the result does not depend on how the domain was cut.
// Kernel families mirror reduce.cu: rows (team per row, optional split of long rows with a fold
// kernel) and cols (TX x TY slab per CTA, shared-memory fold over TY).
#include "common.cuh"

#include <memory>

namespace tb {
namespace {

constexpr int kThreads = 256;
constexpr int kAssumedSms = 148;
constexpr unsigned long long kNoIndex = ~0ull;

struct Cand {
    float v;
    unsigned long long i;
};

template <bool IS_MAX>
__device__ __forceinline__ bool better(const Cand& a, const Cand& b) {
    // true when a must replace b
    if (a.i == kNoIndex) return false;
    if (b.i == kNoIndex) return true;
    const bool an = a.v != a.v, bn = b.v != b.v;
    if (an || bn) return an && (!bn || a.i < b.i);
    if (a.v == b.v) return a.i < b.i;
    return IS_MAX ? a.v > b.v : a.v < b.v;
}

template <class T> __device__ __forceinline__ float toFloat(T v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ float toFloat<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float toFloat<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ void storeValue(void* out, int dtype, uint64_t idx, float v) {
    switch (dtype) {
        case THOR_B200_FP32: static_cast<float*>(out)[idx] = v; break;
        case THOR_B200_FP16: static_cast<__half*>(out)[idx] = __float2half_rn(v); break;
        case THOR_B200_BF16: static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v); break;
        case THOR_B200_FP8_E4M3: static_cast<__nv_fp8_storage_t*>(out)[idx] = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3); break;
        case THOR_B200_FP8_E5M2: static_cast<__nv_fp8_storage_t*>(out)[idx] = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E5M2); break;
        default: break;
    }
}

struct ArgArgs {
    const void* in;
    void* value_out;  // may be null
    void* index_out;  // may be null
    float* part_v;    // [outer][splits]
    unsigned long long* part_i;
    uint64_t outer, reduction, inner;
    uint32_t splits;
    int value_dtype, index_dtype;
};

__device__ __forceinline__ void storeResult(const ArgArgs& a, uint64_t out_idx, const Cand& c) {
    if (a.index_out) {
        if (a.index_dtype == THOR_B200_UINT64) static_cast<unsigned long long*>(a.index_out)[out_idx] = c.i;
        else static_cast<unsigned int*>(a.index_out)[out_idx] = static_cast<unsigned int>(c.i);
    }
    if (a.value_out) storeValue(a.value_out, a.value_dtype, out_idx, c.v);
}

// IDX32: every index of the reduction domain fits 32 bits (kNoIndex travels as 0xffffffff), which halves
// the shuffle traffic of the combine.
template <bool IDX32>
__device__ __forceinline__ unsigned long long shflIndex(unsigned long long i, int off, int span) {
    if (IDX32) {
        const unsigned int lo = __shfl_down_sync(0xffffffffu, static_cast<unsigned int>(i), off, span);
        return lo == 0xffffffffu ? kNoIndex : static_cast<unsigned long long>(lo);
    }
    return __shfl_down_sync(0xffffffffu, i, off, span);
}

template <bool IS_MAX, int TEAM, bool IDX32 = false>
__device__ __forceinline__ Cand teamBest(Cand c, float* sv, unsigned long long* si) {
    constexpr int kSpan = TEAM < 32 ? TEAM : 32;
#pragma unroll
    for (int off = kSpan / 2; off > 0; off >>= 1) {
        Cand o;
        o.v = __shfl_down_sync(0xffffffffu, c.v, off, kSpan);
        o.i = shflIndex<IDX32>(c.i, off, kSpan);
        if (better<IS_MAX>(o, c)) c = o;
    }
    if constexpr (TEAM > 32) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        if (lane == 0) {
            sv[warp] = c.v;
            si[warp] = c.i;
        }
        __syncthreads();
        if (warp == 0) {
            if (lane < TEAM / 32) {
                c.v = sv[lane];
                c.i = si[lane];
            } else {
                c.v = 0.0f;
                c.i = kNoIndex;
            }
#pragma unroll
            for (int off = TEAM / 64; off > 0; off >>= 1) {
                Cand o;
                o.v = __shfl_down_sync(0xffffffffu, c.v, off);
                o.i = __shfl_down_sync(0xffffffffu, c.i, off);
                if (better<IS_MAX>(o, c)) c = o;
            }
        }
    }
    return c;
}

// NaN-propagating extreme of two / three values in one instruction (three-input max / min exists from sm_100 on): a pack
// of sixteen bytes is summarised by its extreme in VEC / 2 instructions instead of a compare-and-select per element.
template <bool IS_MAX>
__device__ __forceinline__ float extreme2(float a, float b) {
    float r;
    if constexpr (IS_MAX) asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    else asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
template <bool IS_MAX>
__device__ __forceinline__ float extreme3(float a, float b, float c) {
    float r;
    if constexpr (IS_MAX) asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    else asm("min.NaN.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

template <class T, bool IS_MAX, int TEAM, bool IDX32>
__global__ void __launch_bounds__(kThreads) argRowsKernel(ArgArgs a) {
    gridDependencyWait();
    gridLaunchDependents();
    constexpr int VEC = 16 / sizeof(T);
    constexpr int U = 4;
    constexpr int kTeamsPerCta = kThreads / TEAM;
    __shared__ float sv[32];
    __shared__ unsigned long long si[32];
    const uint32_t split = blockIdx.x % a.splits;
    const uint64_t row = static_cast<uint64_t>(blockIdx.x / a.splits) * kTeamsPerCta + threadIdx.x / TEAM;
    const int t = threadIdx.x % TEAM;
    Cand best{0.0f, kNoIndex};
    if (row < a.outer) {
        const uint64_t per = (a.reduction + a.splits - 1) / a.splits;
        const uint64_t lo = static_cast<uint64_t>(split) * per;
        const uint64_t hi = lo + per < a.reduction ? lo + per : a.reduction;
        const T* p = static_cast<const T*>(a.in) + row * a.reduction;
        if (lo < hi) {
            const uintptr_t addr = reinterpret_cast<uintptr_t>(p + lo);
            uint64_t head = ((16 - (addr & 15)) & 15) / sizeof(T);
            if (head > hi - lo) head = hi - lo;
            const uint64_t body0 = lo + head;
            const uint64_t n_packs = (hi - body0) / VEC;
            const uint64_t tail0 = body0 + n_packs * VEC;
            // A thread visits its elements in increasing index order, so inside a thread a strict comparison keeps
            // the earliest of equal values and the first NaN sticks; the full ordering rule is only needed when
            // candidates of different threads meet.
            // Packs are compared through their extreme alone; a pack that wins is remembered by its first index and looked
            // into once, after the loops (`in_pack`): the first element equal to the extreme -- or the first NaN -- is
            // the candidate, with the value it really holds (the extreme of {-0, +0} may carry either sign).
            float bv = 0.0f;
            uint64_t bi = kNoIndex;
            bool have = false, in_pack = false;
            auto consider = [&](uint64_t idx, float v, bool pack) {
                const bool take = !have || (bv == bv && (v != v || (IS_MAX ? v > bv : v < bv)));
                if (take) {
                    bv = v;
                    bi = idx;
                    in_pack = pack;
                    have = true;
                }
            };
            for (uint64_t i = lo + t; i < body0; i += TEAM) consider(i, toFloat(p[i]), false);
            for (uint64_t q = t; q < n_packs; q += static_cast<uint64_t>(TEAM) * U) {
                Pack<16> pk[U];
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (q + static_cast<uint64_t>(u) * TEAM < n_packs) loadPack(pk[u], p + body0 + (q + static_cast<uint64_t>(u) * TEAM) * VEC);
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (q + static_cast<uint64_t>(u) * TEAM < n_packs) {
                        const T* e = reinterpret_cast<const T*>(&pk[u]);
                        float m = toFloat(e[0]);
#pragma unroll
                        for (int j = 1; j + 1 < VEC; j += 2) m = extreme3<IS_MAX>(m, toFloat(e[j]), toFloat(e[j + 1]));
                        if constexpr (VEC % 2 == 0) m = extreme2<IS_MAX>(m, toFloat(e[VEC - 1]));
                        consider(body0 + (q + static_cast<uint64_t>(u) * TEAM) * VEC, m, true);
                    }
            }
            for (uint64_t i = tail0 + t; i < hi; i += TEAM) consider(i, toFloat(p[i]), false);
            if (in_pack) {
                Pack<16> pk;
                loadPack(pk, p + bi);
                const T* e = reinterpret_cast<const T*>(&pk);
                const bool want_nan = bv != bv;
                int pos = 0;
                float val = bv;
#pragma unroll
                for (int j = VEC - 1; j >= 0; --j) {  // descending, so the lowest matching position is what remains
                    const float v = toFloat(e[j]);
                    const bool match = want_nan ? v != v : v == bv;
                    pos = match ? j : pos;
                    val = match ? v : val;
                }
                bi += static_cast<uint64_t>(pos);
                bv = val;
            }
            best = Cand{bv, bi};
        }
    }
    best = teamBest<IS_MAX, TEAM, IDX32>(best, sv, si);
    if (t == 0 && row < a.outer) {
        if (a.splits == 1) storeResult(a, row, best);
        else {
            a.part_v[row * a.splits + split] = best.v;
            a.part_i[row * a.splits + split] = best.i;
        }
    }
}

template <bool IS_MAX>
__global__ void __launch_bounds__(kThreads) argRowsFoldKernel(ArgArgs a) {
    gridDependencyWait();
    gridLaunchDependents();
    __shared__ float sv[32];
    __shared__ unsigned long long si[32];
    const uint64_t row = blockIdx.x;
    Cand best{0.0f, kNoIndex};
    for (uint32_t s = threadIdx.x; s < a.splits; s += kThreads) {
        const Cand c{a.part_v[row * a.splits + s], a.part_i[row * a.splits + s]};
        if (better<IS_MAX>(c, best)) best = c;
    }
    best = teamBest<IS_MAX, 256>(best, sv, si);
    if (threadIdx.x == 0) storeResult(a, row, best);
}

// grid = (inner tiles, outer); block = TX x TY; thread (tx, ty) owns pack tx and rows ty, ty+TY, ...
template <class T, bool IS_MAX, int VEC, int TX>
__global__ void __launch_bounds__(kThreads) argColsKernel(ArgArgs a) {
    gridDependencyWait();
    gridLaunchDependents();
    constexpr int TY = kThreads / TX;
    constexpr int U = 4;
    __shared__ float sv[TY][TX * VEC + 1];
    __shared__ unsigned int si[TY][TX * VEC + 1];
    const int tx = threadIdx.x % TX, ty = threadIdx.x / TX;
    const uint64_t col = (static_cast<uint64_t>(blockIdx.x) * TX + tx) * VEC;
    const uint64_t o = blockIdx.y;
    Cand best[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) best[j] = Cand{0.0f, kNoIndex};
    if (col < a.inner) {
        const T* base = static_cast<const T*>(a.in) + o * a.reduction * a.inner + col;
        for (uint64_t r = ty; r < a.reduction; r += static_cast<uint64_t>(TY) * U) {
            Pack<VEC * sizeof(T)> pk[U];
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (r + static_cast<uint64_t>(u) * TY < a.reduction) loadPack(pk[u], base + (r + static_cast<uint64_t>(u) * TY) * a.inner);
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (r + static_cast<uint64_t>(u) * TY < a.reduction) {
#pragma unroll
                    for (int j = 0; j < VEC; ++j) {
                        const Cand c{toFloat(reinterpret_cast<const T*>(&pk[u])[j]), r + static_cast<uint64_t>(u) * TY};
                        if (better<IS_MAX>(c, best[j])) best[j] = c;
                    }
                }
        }
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
        sv[ty][tx * VEC + j] = best[j].v;
        si[ty][tx * VEC + j] = best[j].i == kNoIndex ? 0xffffffffu : static_cast<unsigned int>(best[j].i);
    }
    __syncthreads();
    for (int c = threadIdx.x; c < TX * VEC; c += kThreads) {
        const uint64_t i = static_cast<uint64_t>(blockIdx.x) * TX * VEC + c;
        if (i >= a.inner) continue;
        Cand b{sv[0][c], si[0][c] == 0xffffffffu ? kNoIndex : si[0][c]};
        for (int y = 1; y < TY; ++y) {
            const Cand k{sv[y][c], si[y][c] == 0xffffffffu ? kNoIndex : si[y][c]};
            if (better<IS_MAX>(k, b)) b = k;
        }
        storeResult(a, o * a.inner + i, b);
    }
}

}  // namespace
}  // namespace tb

struct thor_b200_argreduce_plan {
    thor_b200_argreduce_desc desc;
    bool rows = true;
    int team = 256;
    uint32_t splits = 1;
    int cols_vec = 1, cols_tx = 32;
    size_t workspace_bytes = 1;
};

namespace tb {
namespace {

template <class T, bool IS_MAX>
int launchArg(const thor_b200_argreduce_plan& p, const ArgArgs& a, cudaStream_t stream) {
    if (p.rows) {
        const uint64_t teams = kThreads / p.team;
        const uint64_t blocks = ((a.outer + teams - 1) / teams) * a.splits;
        if (blocks > 0x7FFFFFFFull) return fail(THOR_B200_UNSUPPORTED, "argreduce: grid too large");
        const bool idx32 = a.reduction < 0xffffffffull;
#define TB_ARG_ROWS(TEAMV)                                                                                              \
    if (idx32) (void)launchDependent(argRowsKernel<T, IS_MAX, TEAMV, true>, dim3(static_cast<unsigned>(blocks)), dim3(kThreads), 0, stream, a);        \
    else (void)launchDependent(argRowsKernel<T, IS_MAX, TEAMV, false>, dim3(static_cast<unsigned>(blocks)), dim3(kThreads), 0, stream, a);
        switch (p.team) {
            case 8: TB_ARG_ROWS(8) break;
            case 32: TB_ARG_ROWS(32) break;
            default: TB_ARG_ROWS(256) break;
        }
#undef TB_ARG_ROWS
        countLaunch();
        TB_CUDA(cudaGetLastError());
        if (a.splits > 1) {
            (void)launchDependent(argRowsFoldKernel<IS_MAX>, dim3(static_cast<unsigned>(a.outer)), dim3(kThreads), 0, stream, a);
            countLaunch();
            TB_CUDA(cudaGetLastError());
        }
        return THOR_B200_OK;
    }
    constexpr int VEC = 16 / sizeof(T);
    const uint64_t tile = static_cast<uint64_t>(p.cols_tx) * p.cols_vec;
    const uint64_t tiles = (a.inner + tile - 1) / tile;
    if (tiles > 0x7FFFFFFFull || a.outer > 65535ull) return fail(THOR_B200_UNSUPPORTED, "argreduce: grid too large");
    if (a.reduction > 0xfffffffeull) return fail(THOR_B200_UNSUPPORTED, "argreduce: reduction axis of the tiled path is limited to 2^32 - 2 elements");
    dim3 grid(static_cast<unsigned>(tiles), static_cast<unsigned>(a.outer));
    if (p.cols_vec == 1) {
        (void)launchDependent(argColsKernel<T, IS_MAX, 1, 32>, dim3(grid), dim3(kThreads), 0, stream, a);
    } else {
        switch (p.cols_tx) {
            case 1: (void)launchDependent(argColsKernel<T, IS_MAX, VEC, 1>, dim3(grid), dim3(kThreads), 0, stream, a); break;
            case 2: (void)launchDependent(argColsKernel<T, IS_MAX, VEC, 2>, dim3(grid), dim3(kThreads), 0, stream, a); break;
            case 4: (void)launchDependent(argColsKernel<T, IS_MAX, VEC, 4>, dim3(grid), dim3(kThreads), 0, stream, a); break;
            case 8: (void)launchDependent(argColsKernel<T, IS_MAX, VEC, 8>, dim3(grid), dim3(kThreads), 0, stream, a); break;
            case 16: (void)launchDependent(argColsKernel<T, IS_MAX, VEC, 16>, dim3(grid), dim3(kThreads), 0, stream, a); break;
            default: (void)launchDependent(argColsKernel<T, IS_MAX, VEC, 32>, dim3(grid), dim3(kThreads), 0, stream, a); break;
        }
    }
    countLaunch();
    TB_CUDA(cudaGetLastError());
    return THOR_B200_OK;
}

bool isArgFloat(int dt) {
    return dt == THOR_B200_FP32 || dt == THOR_B200_FP16 || dt == THOR_B200_BF16 || dt == THOR_B200_FP8_E4M3 || dt == THOR_B200_FP8_E5M2;
}

}  // namespace
}  // namespace tb

extern "C" {

int thor_b200_argreduce_plan_create(const thor_b200_argreduce_desc* d, thor_b200_argreduce_plan** out_plan, size_t* workspace_bytes) {
    using namespace tb;
    TB_REQUIRE(d != nullptr && out_plan != nullptr && workspace_bytes != nullptr, "argreduce_plan_create: null argument");
    *out_plan = nullptr;
    TB_REQUIRE(d->op == 0 || d->op == 1, "argreduce: op must be 0 (argmin) or 1 (argmax)");
    TB_REQUIRE(isArgFloat(d->input_dtype), "argreduce: unsupported input dtype %s", dtypeName(d->input_dtype));
    TB_REQUIRE(d->value_dtype == 0 || isArgFloat(d->value_dtype), "argreduce: unsupported value dtype %s", dtypeName(d->value_dtype));
    TB_REQUIRE(d->index_dtype == THOR_B200_UINT32 || d->index_dtype == THOR_B200_UINT64, "argreduce: index dtype must be uint32 or uint64");
    TB_REQUIRE(d->outer > 0 && d->reduction > 0 && d->inner > 0, "argreduce: zero-sized dimension");
    TB_REQUIRE(d->index_dtype == THOR_B200_UINT64 || d->reduction <= 0x100000000ull, "argreduce: uint32 indices cannot address %llu elements",
               static_cast<unsigned long long>(d->reduction));
    auto p = std::make_unique<thor_b200_argreduce_plan>();
    p->desc = *d;
    int sms = kAssumedSms;
    {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) sms = v;
        else (void)cudaGetLastError();
    }
    const uint64_t vec = 16 / dtypeSize(d->input_dtype);
    if (d->inner == 1) {
        p->rows = true;
        const uint64_t packs = (d->reduction + vec - 1) / vec;
        // one warp per row up to 2048 packs: the (value, index) combine then needs no shared memory and no
        // barrier, which matters because it costs far more than a plain sum
        p->team = packs <= 16 ? 8 : (packs <= 2048 && d->outer >= static_cast<uint64_t>(16 * sms) ? 32 : (packs <= 512 ? 32 : 256));
        const uint64_t ctas = (d->outer + (kThreads / p->team) - 1) / (kThreads / p->team);
        if (p->team == 256 && ctas < static_cast<uint64_t>(2 * sms)) {
            uint64_t s = (packs + 4095) / 4096;
            if (s > (1u << 20)) s = 1u << 20;
            if (s * d->outer > (1ull << 24)) s = (1ull << 24) / d->outer;
            p->splits = static_cast<uint32_t>(s < 1 ? 1 : s);
        }
        // partial values (float) then partial indices (u64), the latter 16-byte aligned
        const size_t n = static_cast<size_t>(d->outer) * p->splits;
        p->workspace_bytes = p->splits > 1 ? ((n * sizeof(float) + 15) / 16) * 16 + n * sizeof(unsigned long long) : 1;
    } else {
        p->rows = false;
        const bool vec_ok = (d->inner % vec) == 0;
        p->cols_vec = vec_ok ? static_cast<int>(vec) : 1;
        if (vec_ok) {
            const uint64_t packs = d->inner / vec;
            int tx = 32;
            while (tx > 1 && static_cast<uint64_t>(tx / 2) >= packs) tx /= 2;
            p->cols_tx = tx;
        }
    }
    *workspace_bytes = p->workspace_bytes;
    *out_plan = p.release();
    return THOR_B200_OK;
}

int thor_b200_argreduce_launch(const thor_b200_argreduce_plan* p, const void* input, void* value_output, void* index_output, void* workspace,
                               size_t workspace_bytes, void* stream_v) {
    using namespace tb;
    TB_REQUIRE(p != nullptr, "argreduce_launch: null plan");
    TB_REQUIRE(input != nullptr, "argreduce_launch: null input");
    TB_REQUIRE(value_output != nullptr || index_output != nullptr, "argreduce_launch: no output requested");
    TB_REQUIRE(value_output == nullptr || p->desc.value_dtype != 0, "argreduce_launch: plan was created without a value output");
    TB_REQUIRE(workspace_bytes >= p->workspace_bytes, "argreduce_launch: workspace too small");
    TB_REQUIRE(p->splits == 1 || (workspace != nullptr && isAligned(workspace, 16)), "argreduce_launch: workspace must be a 16-byte aligned device pointer");
    if (!p->rows && p->cols_vec > 1) TB_REQUIRE(isAligned(input, 16), "argreduce_launch: input must be 16-byte aligned for this geometry");
    const thor_b200_argreduce_desc& d = p->desc;
    ArgArgs a{};
    a.in = input;
    a.value_out = value_output;
    a.index_out = index_output;
    a.outer = d.outer;
    a.reduction = d.reduction;
    a.inner = d.inner;
    a.splits = p->splits;
    a.value_dtype = d.value_dtype;
    a.index_dtype = d.index_dtype;
    if (p->splits > 1) {
        const size_t n = static_cast<size_t>(d.outer) * p->splits;
        a.part_v = static_cast<float*>(workspace);
        a.part_i = reinterpret_cast<unsigned long long*>(static_cast<char*>(workspace) + ((n * sizeof(float) + 15) / 16) * 16);
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
#define TB_ARG(T) return d.op == 1 ? launchArg<T, true>(*p, a, stream) : launchArg<T, false>(*p, a, stream);
    switch (d.input_dtype) {
        case THOR_B200_FP32: TB_ARG(float)
        case THOR_B200_FP16: TB_ARG(__half)
        case THOR_B200_BF16: TB_ARG(__nv_bfloat16)
        case THOR_B200_FP8_E4M3: TB_ARG(__nv_fp8_e4m3)
        case THOR_B200_FP8_E5M2: TB_ARG(__nv_fp8_e5m2)
        default: break;
    }
#undef TB_ARG
    return fail(THOR_B200_INVALID_ARGUMENT, "argreduce_launch: unsupported input dtype");
}

void thor_b200_argreduce_plan_destroy(thor_b200_argreduce_plan* p) { delete p; }

}  // extern "C"
