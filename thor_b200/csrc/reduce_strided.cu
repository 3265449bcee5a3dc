// Value and arg reductions over non-adjacent axes of a dense tensor.
//
// Adjacent axes of the same kind (kept / reduced) are merged on the host, which leaves alternating
// groups.  Two kernels:
//   lanes-on-reduction  the innermost group is reduced: a warp (short segments) or a CTA (long ones)
//                       owns one output element; its lanes walk the innermost reduced group, which
//                       is contiguous in memory, and step through the outer reduced groups together;
//   lanes-on-output     the innermost group is kept: one thread owns one output element and
//                       consecutive threads own consecutive elements of the innermost kept group, so
//                       every step of the (serial) reduction loop is a coalesced access.
// Accumulation is fp32 in a fixed order, finalisation and the single store conversion follow the
// planned reductions.  This is the general fallback: index arithmetic per outer step, no splitting
// of long reductions across CTAs.
#include <algorithm>

#include "common.cuh"

namespace tb {
namespace {

constexpr int kMaxGroups = THOR_B200_MAX_RANK;

struct Groups {
    uint32_t n_kept, n_red;
    uint64_t kept_dim[kMaxGroups], kept_stride[kMaxGroups];  // outermost first
    uint64_t red_dim[kMaxGroups], red_stride[kMaxGroups];
    uint64_t n_out, n_red_total;
};

struct StridedArgs {
    const void* in;
    void* out;
    Groups g;
    int in_dtype, out_dtype, op, arg_op;
    float divisor, scale;
};

__device__ __forceinline__ float loadAsFloat(const void* p, int dtype, uint64_t i) {
    switch (dtype) {
        case THOR_B200_FP32: return static_cast<const float*>(p)[i];
        case THOR_B200_FP16: return __half2float(static_cast<const __half*>(p)[i]);
        case THOR_B200_BF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
        case THOR_B200_FP8_E4M3: return static_cast<float>(static_cast<const __nv_fp8_e4m3*>(p)[i]);
        default: return static_cast<float>(static_cast<const __nv_fp8_e5m2*>(p)[i]);
    }
}

__device__ __forceinline__ float transformValue(int op, float v) {
    return op == THOR_B200_REDUCE_L1NORM ? fabsf(v) : (op == THOR_B200_REDUCE_L2NORM ? v * v : v);
}
__device__ __forceinline__ float identityValue(int op) {
    return op == THOR_B200_REDUCE_PRODUCT ? 1.0f : (op == THOR_B200_REDUCE_MIN ? __int_as_float(0x7f800000) : (op == THOR_B200_REDUCE_MAX ? __int_as_float(0xff800000) : 0.0f));
}
__device__ __forceinline__ float combineValue(int op, float a, float b) {
    switch (op) {
        case THOR_B200_REDUCE_PRODUCT: return a * b;
        case THOR_B200_REDUCE_MIN: {  // NaN-propagating, one instruction
            float r;
            asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
            return r;
        }
        case THOR_B200_REDUCE_MAX: {
            float r;
            asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
            return r;
        }
        default: return a + b;
    }
}
// Arg candidates: NaN beats numbers, then the better value, then the lower index.
__device__ __forceinline__ bool argBetter(int is_max, float v, uint64_t i, float bv, uint64_t bi) {
    const bool vn = v != v, bn = bv != bv;
    if (vn != bn) return vn;
    if (!vn && v != bv) return is_max ? v > bv : v < bv;
    return i < bi;
}

__device__ __forceinline__ void storeResult(const StridedArgs& a, uint64_t o, float v, uint64_t idx) {
    if (a.arg_op >= 0) {
        if (a.out_dtype == THOR_B200_UINT32) static_cast<uint32_t*>(a.out)[o] = static_cast<uint32_t>(idx);
        else static_cast<unsigned long long*>(a.out)[o] = idx;
        return;
    }
    if (a.op == THOR_B200_REDUCE_MEAN) v = v / a.divisor;
    else if (a.op == THOR_B200_REDUCE_L2NORM) v = sqrtf(v);
    v *= a.scale;
    switch (a.out_dtype) {
        case THOR_B200_FP32: static_cast<float*>(a.out)[o] = v; break;
        case THOR_B200_FP16: static_cast<__half*>(a.out)[o] = __float2half_rn(v); break;
        case THOR_B200_BF16: static_cast<__nv_bfloat16*>(a.out)[o] = __float2bfloat16_rn(v); break;
        case THOR_B200_FP8_E4M3: static_cast<__nv_fp8_storage_t*>(a.out)[o] = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3); break;
        default: static_cast<__nv_fp8_storage_t*>(a.out)[o] = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E5M2); break;
    }
}

__device__ __forceinline__ uint64_t keptOffset(const Groups& g, uint64_t o) {
    uint64_t off = 0;
    for (uint32_t k = g.n_kept; k-- > 0;) {
        off += (o % g.kept_dim[k]) * g.kept_stride[k];
        o /= g.kept_dim[k];
    }
    return off;
}
// Offset of outer reduction step `step` (all reduced groups but the innermost).
__device__ __forceinline__ uint64_t redOuterOffset(const Groups& g, uint64_t step) {
    uint64_t off = 0;
    for (uint32_t k = g.n_red - 1; k-- > 0;) {
        off += (step % g.red_dim[k]) * g.red_stride[k];
        step /= g.red_dim[k];
    }
    return off;
}

// TEAM lanes (32: a warp, 256: the CTA) own one output element; the innermost group is reduced.
template <int TEAM>
__global__ void __launch_bounds__(256) stridedLanesOnReductionKernel(StridedArgs a) {
    gridDependencyWait();
    gridLaunchDependents();
    __shared__ float s_val[8];
    __shared__ unsigned long long s_idx[8];
    const Groups& g = a.g;
    const int lane = threadIdx.x % TEAM;
    const uint64_t o = static_cast<uint64_t>(blockIdx.x) * (256 / TEAM) + threadIdx.x / TEAM;
    const bool live = o < g.n_out;
    const uint64_t inner = g.red_dim[g.n_red - 1], inner_stride = g.red_stride[g.n_red - 1];
    const uint64_t steps = g.n_red_total / inner;
    const uint64_t base = live ? keptOffset(g, o) : 0;
    const bool arg = a.arg_op >= 0;
    float acc = arg ? 0.0f : identityValue(a.op);
    uint64_t best = ~0ull;  // arg: no candidate yet
    if (live) {
        for (uint64_t s = 0; s < steps; ++s) {
            const uint64_t off = base + redOuterOffset(g, s);
            for (uint64_t i = lane; i < inner; i += TEAM) {
                const float v = loadAsFloat(a.in, a.in_dtype, off + i * inner_stride);
                if (arg) {
                    const uint64_t idx = s * inner + i;
                    if (best == ~0ull || argBetter(a.arg_op, v, idx, acc, best)) {
                        acc = v;
                        best = idx;
                    }
                } else {
                    acc = combineValue(a.op, acc, transformValue(a.op, v));
                }
            }
        }
    }
    // combine the lanes: xor butterfly inside the warp, then (TEAM == 256) the 8 warp results in warp order
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, acc, off);
        const unsigned long long oi = __shfl_xor_sync(0xffffffffu, static_cast<unsigned long long>(best), off);
        if (arg) {
            if (oi != ~0ull && (best == ~0ull || argBetter(a.arg_op, ov, oi, acc, best))) {
                acc = ov;
                best = oi;
            }
        } else {
            acc = combineValue(a.op, acc, ov);
        }
    }
    if (TEAM == 256) {
        const int warp = threadIdx.x >> 5;
        if ((threadIdx.x & 31) == 0) {
            s_val[warp] = acc;
            s_idx[warp] = best;
        }
        __syncthreads();
        acc = s_val[0];
        best = s_idx[0];
        for (int w = 1; w < 8; ++w) {
            if (arg) {
                if (s_idx[w] != ~0ull && (best == ~0ull || argBetter(a.arg_op, s_val[w], s_idx[w], acc, best))) {
                    acc = s_val[w];
                    best = s_idx[w];
                }
            } else {
                acc = combineValue(a.op, acc, s_val[w]);
            }
        }
    }
    if (live && lane == 0) storeResult(a, o, acc, best);
}

// One thread per output element; the innermost group is kept, so neighbouring threads read neighbouring addresses.
__global__ void __launch_bounds__(256) stridedLanesOnOutputKernel(StridedArgs a) {
    gridDependencyWait();
    gridLaunchDependents();
    const Groups& g = a.g;
    const uint64_t o = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (o >= g.n_out) return;
    const uint64_t inner = g.red_dim[g.n_red - 1], inner_stride = g.red_stride[g.n_red - 1];
    const uint64_t steps = g.n_red_total / inner;
    const uint64_t base = keptOffset(g, o);
    const bool arg = a.arg_op >= 0;
    float acc = arg ? 0.0f : identityValue(a.op);
    uint64_t best = ~0ull;
    for (uint64_t s = 0; s < steps; ++s) {
        const uint64_t off = base + redOuterOffset(g, s);
        for (uint64_t i = 0; i < inner; ++i) {
            const float v = loadAsFloat(a.in, a.in_dtype, off + i * inner_stride);
            if (arg) {
                const uint64_t idx = s * inner + i;
                if (best == ~0ull || argBetter(a.arg_op, v, idx, acc, best)) {
                    acc = v;
                    best = idx;
                }
            } else {
                acc = combineValue(a.op, acc, transformValue(a.op, v));
            }
        }
    }
    storeResult(a, o, acc, best);
}

bool isStridedFloat(int dt) {
    return dt == THOR_B200_FP32 || dt == THOR_B200_FP16 || dt == THOR_B200_BF16 || dt == THOR_B200_FP8_E4M3 || dt == THOR_B200_FP8_E5M2;
}

}  // namespace
}  // namespace tb

extern "C" int thor_b200_strided_reduce_launch(const thor_b200_strided_reduce_desc* d, const void* input, void* output, float output_scale, void* stream_v) {
    using namespace tb;
    TB_REQUIRE(d != nullptr && input != nullptr && output != nullptr, "strided_reduce: null argument");
    TB_REQUIRE(d->rank >= 1 && d->rank <= THOR_B200_MAX_RANK, "strided_reduce: rank must be 1..%d", THOR_B200_MAX_RANK);
    TB_REQUIRE(d->arg_op >= -1 && d->arg_op <= 1, "strided_reduce: arg_op must be -1, 0 or 1");
    TB_REQUIRE(isStridedFloat(d->input_dtype), "strided_reduce: unsupported input dtype %s", dtypeName(d->input_dtype));
    if (d->arg_op < 0) {
        TB_REQUIRE(d->op >= THOR_B200_REDUCE_SUM && d->op <= THOR_B200_REDUCE_L2NORM, "strided_reduce: unknown op %d", d->op);
        TB_REQUIRE(isStridedFloat(d->output_dtype), "strided_reduce: unsupported output dtype %s", dtypeName(d->output_dtype));
        TB_REQUIRE(output_scale == output_scale && output_scale - output_scale == 0.0f, "strided_reduce: output_scale must be finite");
    } else {
        TB_REQUIRE(d->output_dtype == THOR_B200_UINT32 || d->output_dtype == THOR_B200_UINT64, "strided_reduce: index dtype must be uint32 or uint64");
    }
    // merge adjacent axes of one kind (singleton axes join whatever surrounds them)
    StridedArgs a{};
    Groups& g = a.g;
    TB_REQUIRE(d->has_strides <= 1, "strided_reduce: has_strides must be 0 or 1");
    uint64_t stride[THOR_B200_MAX_RANK];
    uint64_t s = 1;
    for (uint32_t i = d->rank; i-- > 0;) {
        TB_REQUIRE(d->dims[i] > 0, "strided_reduce: zero-sized dimension");
        stride[i] = d->has_strides ? d->strides[i] : s;
        s *= d->dims[i];
    }
    g.n_out = g.n_red_total = 1;
    int last_kind = -1;
    bool innermost_reduced = false;
    for (uint32_t i = 0; i < d->rank; ++i) {
        if (d->dims[i] == 1) continue;
        const int kind = d->reduced[i] ? 1 : 0;
        uint64_t* dim = kind ? g.red_dim : g.kept_dim;
        uint64_t* str = kind ? g.red_stride : g.kept_stride;
        uint32_t& n = kind ? g.n_red : g.n_kept;
        // an axis joins the group before it when it is of the same kind and continues it in memory
        if (kind == last_kind && str[n - 1] == d->dims[i] * stride[i]) {
            dim[n - 1] *= d->dims[i];
            str[n - 1] = stride[i];
        } else {
            dim[n] = d->dims[i];
            str[n] = stride[i];
            ++n;
        }
        (kind ? g.n_red_total : g.n_out) *= d->dims[i];
        last_kind = kind;
        innermost_reduced = kind == 1;
    }
    if (g.n_red == 0) {  // nothing (but singletons) is reduced: a reduction group of one element keeps the kernels uniform
        g.red_dim[0] = 1;
        g.red_stride[0] = 1;
        g.n_red = 1;
        innermost_reduced = false;
    }
    if (d->arg_op >= 0 && d->output_dtype == THOR_B200_UINT32) TB_REQUIRE(g.n_red_total <= 0x100000000ull, "strided_reduce: uint32 indices cannot address the reduction");
    a.in = input;
    a.out = output;
    a.in_dtype = d->input_dtype;
    a.out_dtype = d->output_dtype;
    a.op = d->op;
    a.arg_op = d->arg_op;
    a.divisor = static_cast<float>(g.n_red_total);
    a.scale = output_scale;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    if (innermost_reduced) {
        const bool cta = g.red_dim[g.n_red - 1] >= 2048;
        const uint64_t per_cta = cta ? 1 : 8;
        const uint64_t blocks = (g.n_out + per_cta - 1) / per_cta;
        TB_REQUIRE(blocks <= 0x7FFFFFFFull, "strided_reduce: too many outputs for one grid");
        if (cta) TB_CUDA(launchDependent(stridedLanesOnReductionKernel<256>, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, a));
        else TB_CUDA(launchDependent(stridedLanesOnReductionKernel<32>, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, a));
    } else {
        const uint64_t blocks = (g.n_out + 255) / 256;
        TB_REQUIRE(blocks <= 0x7FFFFFFFull, "strided_reduce: too many outputs for one grid");
        TB_CUDA(launchDependent(stridedLanesOnOutputKernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, a));
    }
    countLaunch();
    return THOR_B200_OK;
}
