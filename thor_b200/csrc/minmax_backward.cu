// Backward of dense min / max reductions: arg reduction + one streaming route kernel.
//
// The route kernel writes grad_input [outer, reduction, inner] once, 16 bytes per store: element
// (o, r, i) is grad_output[o, i] when r is the winner of segment (o, i) and zero otherwise.  It
// never reads the forward input (the arg reduction did), so the pair of kernels moves
// input + grad_input bytes, the least a gather-free formulation can move.
#include <algorithm>

#include "common.cuh"

namespace tb {
namespace {

template <class T>
__device__ __forceinline__ float gradToFloat(T v) {
    return static_cast<float>(v);
}
template <class T>
__device__ __forceinline__ T gradFromFloat(float v) {
    return static_cast<T>(v);
}

// Where a segment's gradient comes from: one value per segment, one value for all, or a literal.
struct GradSource {
    int mode;
    float value;
};
template <class G>
__device__ __forceinline__ float segmentGrad(const G* grad_output, uint64_t seg, GradSource gs) {
    return gs.mode == 2 ? gs.value : gradToFloat(grad_output[gs.mode == 1 ? 0 : seg]);
}

// inner == 1: rows of `reduction` elements, P elements per pack, reduction % P == 0.
template <class G, class O, int P>
__global__ void __launch_bounds__(256) routeRowsKernel(const G* __restrict__ grad_output, const uint32_t* __restrict__ winners, O* __restrict__ grad_input,
                                                        uint64_t packs_per_row, uint64_t n_packs, GradSource gs) {
    gridDependencyWait();
    gridLaunchDependents();
    const uint64_t p = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (p >= n_packs) return;
    const uint64_t row = p / packs_per_row;
    const uint32_t first = static_cast<uint32_t>((p - row * packs_per_row) * P);
    const uint32_t hit = winners[row] - first;  // < P exactly when the winner lies in this pack
    Pack<P * sizeof(O)> out;
    O* lanes = reinterpret_cast<O*>(&out);
    const O zero = gradFromFloat<O>(0.0f);
#pragma unroll
    for (int e = 0; e < P; ++e) lanes[e] = zero;
    if (hit < static_cast<uint32_t>(P)) {
        const O g = gradFromFloat<O>(segmentGrad(grad_output, row, gs));
#pragma unroll
        for (int e = 0; e < P; ++e)
            if (static_cast<uint32_t>(e) == hit) lanes[e] = g;
    }
    storePack(grad_input + p * P, out);
}

// inner > 1, inner % P == 0: a pack covers P neighbouring `inner` positions of one (outer, r) line.
template <class G, class O, int P>
__global__ void __launch_bounds__(256) routeInnerKernel(const G* __restrict__ grad_output, const uint32_t* __restrict__ winners, O* __restrict__ grad_input,
                                                         uint64_t reduction, uint64_t packs_per_line, uint64_t n_packs, GradSource gs) {
    gridDependencyWait();
    gridLaunchDependents();
    const uint64_t p = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (p >= n_packs) return;
    const uint64_t line = p / packs_per_line;  // = outer index * reduction + r
    const uint64_t i0 = (p - line * packs_per_line) * P;
    const uint64_t o = line / reduction;
    const uint32_t r = static_cast<uint32_t>(line - o * reduction);
    const uint64_t seg = o * packs_per_line * P + i0;  // first (outer, inner) segment of this pack
    Pack<P * sizeof(O)> out;
    O* lanes = reinterpret_cast<O*>(&out);
#pragma unroll
    for (int e = 0; e < P; ++e) {
        const bool hit = winners[seg + e] == r;
        lanes[e] = gradFromFloat<O>(hit ? segmentGrad(grad_output, seg + e, gs) : 0.0f);
    }
    storePack(grad_input + p * P, out);
}

// Any shape: one element per thread step, index arithmetic per element.
template <class G, class O>
__global__ void __launch_bounds__(256) routeGenericKernel(const G* __restrict__ grad_output, const uint32_t* __restrict__ winners, O* __restrict__ grad_input,
                                                           uint64_t reduction, uint64_t inner, uint64_t n, GradSource gs) {
    gridDependencyWait();
    gridLaunchDependents();
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * 256;
    for (uint64_t f = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x; f < n; f += stride) {
        const uint64_t line = f / inner;
        const uint64_t i = f - line * inner;
        const uint64_t o = line / reduction;
        const uint32_t r = static_cast<uint32_t>(line - o * reduction);
        const uint64_t seg = o * inner + i;
        grad_input[f] = gradFromFloat<O>(winners[seg] == r ? segmentGrad(grad_output, seg, gs) : 0.0f);
    }
}

template <class G, class O>
int launchRoute(const thor_b200_minmax_backward_desc& d, const void* grad_output_v, const uint32_t* winners, void* grad_input_v, cudaStream_t stream) {
    const G* grad_output = static_cast<const G*>(grad_output_v);
    O* grad_input = static_cast<O*>(grad_input_v);
    constexpr int P = 16 / sizeof(O);
    const uint64_t n = d.outer * d.reduction * d.inner;
    const bool aligned = isAligned(grad_input_v, 16);
    const GradSource gs{d.grad_mode, d.grad_value};
    if (aligned && d.inner == 1 && d.reduction % P == 0) {
        const uint64_t packs = n / P;
        const uint64_t blocks = (packs + 255) / 256;
        TB_REQUIRE(blocks <= 0x7FFFFFFFull, "minmax_backward: too many elements for one grid");
        TB_CUDA(launchDependent(routeRowsKernel<G, O, P>, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, grad_output, winners, grad_input,
                                d.reduction / P, packs, gs));
    } else if (aligned && d.inner > 1 && d.inner % P == 0) {
        const uint64_t packs = n / P;
        const uint64_t blocks = (packs + 255) / 256;
        TB_REQUIRE(blocks <= 0x7FFFFFFFull, "minmax_backward: too many elements for one grid");
        TB_CUDA(launchDependent(routeInnerKernel<G, O, P>, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, grad_output, winners, grad_input,
                                d.reduction, d.inner / P, packs, gs));
    } else {
        const uint64_t blocks = std::min<uint64_t>((n + 255) / 256, 148ull * 32);
        TB_CUDA(launchDependent(routeGenericKernel<G, O>, dim3(static_cast<unsigned>(std::max<uint64_t>(1, blocks))), dim3(256), 0, stream, grad_output, winners,
                                grad_input, d.reduction, d.inner, n, gs));
    }
    countLaunch();
    return THOR_B200_OK;
}

template <class G>
int dispatchOut(const thor_b200_minmax_backward_desc& d, const void* grad_output, const uint32_t* winners, void* grad_input, cudaStream_t stream) {
    switch (d.grad_input_dtype) {
        case THOR_B200_FP32: return launchRoute<G, float>(d, grad_output, winners, grad_input, stream);
        case THOR_B200_FP16: return launchRoute<G, __half>(d, grad_output, winners, grad_input, stream);
        case THOR_B200_BF16: return launchRoute<G, __nv_bfloat16>(d, grad_output, winners, grad_input, stream);
        default: return fail(THOR_B200_INVALID_ARGUMENT, "minmax_backward: grad_input dtype must be fp32, fp16 or bf16");
    }
}

bool gradDtypeOk(int dt) { return dt == THOR_B200_FP32 || dt == THOR_B200_FP16 || dt == THOR_B200_BF16; }

}  // namespace
}  // namespace tb

struct thor_b200_minmax_backward_plan {
    thor_b200_minmax_backward_desc desc{};
    thor_b200_argreduce_plan* arg = nullptr;
    size_t arg_workspace = 0;   // bytes, rounded up to 256
    size_t winners_bytes = 0;
};

extern "C" {

int thor_b200_minmax_backward_plan_create(const thor_b200_minmax_backward_desc* d, thor_b200_minmax_backward_plan** out_plan, size_t* workspace_bytes) {
    using namespace tb;
    TB_REQUIRE(d != nullptr && out_plan != nullptr && workspace_bytes != nullptr, "minmax_backward_plan_create: null argument");
    *out_plan = nullptr;
    TB_REQUIRE(d->outer > 0 && d->reduction > 0 && d->inner > 0, "minmax_backward_plan_create: zero-sized dimension");
    TB_REQUIRE(d->reduction <= 0xFFFFFFFFull, "minmax_backward_plan_create: reduction length exceeds the 32-bit winner index");
    TB_REQUIRE(d->grad_mode >= 0 && d->grad_mode <= 2, "minmax_backward_plan_create: grad_mode must be 0, 1 or 2");
    TB_REQUIRE((d->grad_mode == 2 || gradDtypeOk(d->grad_output_dtype)) && gradDtypeOk(d->grad_input_dtype),
               "minmax_backward_plan_create: gradient dtypes must be fp32, fp16 or bf16");
    thor_b200_argreduce_desc a{};
    a.op = d->is_max ? 1 : 0;
    a.input_dtype = d->input_dtype;
    a.value_dtype = 0;
    a.index_dtype = THOR_B200_UINT32;
    a.outer = d->outer;
    a.reduction = d->reduction;
    a.inner = d->inner;
    auto plan = new thor_b200_minmax_backward_plan();
    plan->desc = *d;
    size_t ws = 0;
    if (int st = thor_b200_argreduce_plan_create(&a, &plan->arg, &ws)) {
        delete plan;
        return st;
    }
    plan->arg_workspace = (ws + 255) / 256 * 256;
    plan->winners_bytes = static_cast<size_t>(d->outer * d->inner) * sizeof(uint32_t);
    *workspace_bytes = plan->arg_workspace + plan->winners_bytes;
    *out_plan = plan;
    return THOR_B200_OK;
}

int thor_b200_minmax_backward_launch(const thor_b200_minmax_backward_plan* plan, const void* input, const void* grad_output, void* grad_input, void* workspace,
                                     size_t workspace_bytes, void* stream_v) {
    using namespace tb;
    TB_REQUIRE(plan != nullptr, "minmax_backward_launch: null plan");
    TB_REQUIRE(input != nullptr && grad_input != nullptr && (grad_output != nullptr || plan->desc.grad_mode == 2), "minmax_backward_launch: null tensor pointer");
    TB_REQUIRE(workspace != nullptr && workspace_bytes >= plan->arg_workspace + plan->winners_bytes, "minmax_backward_launch: workspace too small");
    TB_REQUIRE(isAligned(workspace, 256), "minmax_backward_launch: workspace must be 256-byte aligned");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    uint32_t* winners = reinterpret_cast<uint32_t*>(static_cast<char*>(workspace) + plan->arg_workspace);
    if (int st = thor_b200_argreduce_launch(plan->arg, input, nullptr, winners, workspace, plan->arg_workspace, stream)) return st;
    switch (plan->desc.grad_mode == 2 ? THOR_B200_FP32 : plan->desc.grad_output_dtype) {
        case THOR_B200_FP32: return dispatchOut<float>(plan->desc, grad_output, winners, grad_input, stream);
        case THOR_B200_FP16: return dispatchOut<__half>(plan->desc, grad_output, winners, grad_input, stream);
        case THOR_B200_BF16: return dispatchOut<__nv_bfloat16>(plan->desc, grad_output, winners, grad_input, stream);
        default: return fail(THOR_B200_INVALID_ARGUMENT, "minmax_backward_launch: grad_output dtype must be fp32, fp16 or bf16");
    }
}

void thor_b200_minmax_backward_plan_destroy(thor_b200_minmax_backward_plan* plan) {
    if (!plan) return;
    thor_b200_argreduce_plan_destroy(plan->arg);
    delete plan;
}

}  // extern "C"
