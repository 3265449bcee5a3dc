// dtype casts: one streaming kernel template over all 15 x 15 storage pairs.
//
// Design for B200: the cast is pure HBM traffic.  Each thread moves one or two packs of P
// elements (the narrower side of a pack is 16 bytes, the wider side 32..128 bytes, read with
// 256-bit loads where the address allows) and each CTA owns a contiguous run of packs.  A plain
// one-wave-after-another grid measured ~10 % faster on B200 than a persistent grid-stride loop
// for this access pattern (6.7-6.8 TB/s against 6.0-6.2 TB/s at 1.5 GB of traffic), so the grid
// is sized to the tensor.  The last n % P elements are converted one by one by the first CTA,
// which means the kernel touches exactly n elements on both sides.
#include <cooperative_groups.h>

#include "common.cuh"

namespace tb {

// Element conversion = the C++ static_cast of the CUDA element types, the rule the reference
// states for TypeConverter (TypeConverter.h:24-27, TypeConverterKernels.cu:23-37); fp8-e4m3
// destinations saturate to the largest finite value (Utilities/Common/LowPrecisionFloat.h:18-46).
template <class F, class T>
struct Cvt {
    __device__ __forceinline__ static T run(F x) { return static_cast<T>(x); }
};
template <class F>
struct Cvt<F, __nv_fp8_e4m3> {
    __device__ __forceinline__ static __nv_fp8_e4m3 run(F x) {
        __nv_fp8_e4m3 r;
        if constexpr (std::is_same_v<F, double>) {
            r.__x = __nv_cvt_double_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
        } else if constexpr (std::is_integral_v<F>) {
            r.__x = __nv_cvt_double_to_fp8(static_cast<double>(x), __NV_SATFINITE, __NV_E4M3);
        } else if constexpr (std::is_same_v<F, __half>) {
            r.__x = __nv_cvt_float_to_fp8(__half2float(x), __NV_SATFINITE, __NV_E4M3);
        } else if constexpr (std::is_same_v<F, __nv_bfloat16>) {
            r.__x = __nv_cvt_float_to_fp8(__bfloat162float(x), __NV_SATFINITE, __NV_E4M3);
        } else if constexpr (std::is_same_v<F, __nv_fp8_e5m2>) {
            r.__x = __nv_cvt_float_to_fp8(static_cast<float>(x), __NV_SATFINITE, __NV_E4M3);
        } else {
            r.__x = __nv_cvt_float_to_fp8(static_cast<float>(x), __NV_SATFINITE, __NV_E4M3);
        }
        return r;
    }
};
template <>
struct Cvt<__nv_fp8_e4m3, __nv_fp8_e5m2> {
    __device__ __forceinline__ static __nv_fp8_e5m2 run(__nv_fp8_e4m3 x) { return __nv_fp8_e5m2(static_cast<float>(x)); }
};

// Pack width: P elements per pack so that the narrower side moves 16 bytes (the wider side then
// moves 32, 64 or 128 bytes as consecutive 16-byte accesses).
template <class F, class T>
struct CastGeom {
    static constexpr int kMin = sizeof(F) < sizeof(T) ? sizeof(F) : sizeof(T);
    static constexpr int kMax = sizeof(F) < sizeof(T) ? sizeof(T) : sizeof(F);
    static constexpr int P = 16 / kMin;
    // Packs per thread: one when a pack already loads >= 32 bytes, else two.
    static constexpr int U = (P * sizeof(F) >= 32) ? 1 : 2;
};

template <class F, class T, int P, int U, bool WIDE>
__global__ void __launch_bounds__(256) castPackedKernel(const F* __restrict__ src, T* __restrict__ dst, int64_t n_packs, int64_t n) {
    gridDependencyWait();
    gridLaunchDependents();
    // One CTA owns a contiguous run of 256 * U packs; thread t takes packs t, t + 256, ...
    const int64_t base = static_cast<int64_t>(blockIdx.x) * (256 * U) + threadIdx.x;
    Pack<P * sizeof(F)> in[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t p = base + u * 256;
        if (p < n_packs) loadPack<P * sizeof(F), WIDE>(in[u], src + p * P);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t p = base + u * 256;
        if (p < n_packs) {
            Pack<P * sizeof(T)> out;
            const F* fi = reinterpret_cast<const F*>(&in[u]);
            T* to = reinterpret_cast<T*>(&out);
#pragma unroll
            for (int e = 0; e < P; ++e) to[e] = Cvt<F, T>::run(fi[e]);
            storePack(dst + p * P, out);
        }
    }
    // Ragged tail (< P elements).
    if (blockIdx.x == 0) {
        const int64_t i = n_packs * P + threadIdx.x;
        if (i < n) dst[i] = Cvt<F, T>::run(src[i]);
    }
}

// Fallback for pointers that are not aligned to the pack width (foreign sub-views).
template <class F, class T>
__global__ void __launch_bounds__(256) castScalarKernel(const F* __restrict__ src, T* __restrict__ dst, int64_t n) {
    gridDependencyWait();
    gridLaunchDependents();
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = Cvt<F, T>::run(src[i]);
}

// Same-address conversion between types of one size: every thread reads its pack before it
// writes it, so the packed kernel is safe; this variant only drops __restrict__.
template <class F, class T, int P>
__global__ void __launch_bounds__(256) castInPlaceSameSizeKernel(void* buf, int64_t n_packs, int64_t n) {
    gridDependencyWait();
    gridLaunchDependents();
    static_assert(sizeof(F) == sizeof(T), "same-size in-place only");
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t p = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; p < n_packs; p += stride) {
        Pack<P * sizeof(F)> in;
        loadPack(in, reinterpret_cast<const F*>(buf) + p * P);
        Pack<P * sizeof(T)> out;
#pragma unroll
        for (int e = 0; e < P; ++e) reinterpret_cast<T*>(&out)[e] = Cvt<F, T>::run(reinterpret_cast<const F*>(&in)[e]);
        storePack(reinterpret_cast<T*>(buf) + p * P, out);
    }
    if (blockIdx.x == 0) {
        const int64_t i = n_packs * P + threadIdx.x;
        if (i < n) {
            const F v = reinterpret_cast<const F*>(buf)[i];
            reinterpret_cast<T*>(buf)[i] = Cvt<F, T>::run(v);
        }
    }
}

// Same-address conversion between element sizes, first block of elements: one CTA reads its (at
// most kHeadElements) values into registers, meets at a barrier, then writes them; reads and writes
// of this block overlap each other but nothing else.
constexpr int kHeadElements = 8192;
template <class F, class T>
__global__ void __launch_bounds__(256) castInPlaceHeadKernel(void* buf, int count) {
    gridDependencyWait();
    gridLaunchDependents();
    constexpr int PER = kHeadElements / 256;
    F held[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = threadIdx.x + i * 256;
        if (e < count) held[i] = reinterpret_cast<const F*>(buf)[e];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = threadIdx.x + i * 256;
        if (e < count) reinterpret_cast<T*>(buf)[e] = Cvt<F, T>::run(held[i]);
    }
}

// Same-address conversion between element sizes in ONE launch.  All CTAs of the grid are resident together (cooperative
// launch) and walk the buffer in waves of gridDim.x * 256 * UW packs: every thread reads its packs of the wave into
// registers, the grid meets at a barrier, every thread writes.  Waves go upwards when the elements shrink and downwards
// when they grow, so the bytes a wave writes hold only values that this or an earlier wave has already read, and the
// next wave's reads never touch bytes that a straggler of this wave still writes: one barrier per wave is enough
// (4 waves for 2^24 fp32 -> fp16 on 148 SMs).  The last, partial pack is moved element by element by its thread.
template <class F, class T, int P, int UW>
__global__ void __launch_bounds__(256) castInPlaceWavesKernel(void* buf, int64_t n) {
    namespace cg = cooperative_groups;
    cg::grid_group grid = cg::this_grid();
    const int64_t threads = static_cast<int64_t>(gridDim.x) * 256, tid = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    const int64_t packs = (n + P - 1) / P, wave_packs = threads * UW, waves = (packs + wave_packs - 1) / wave_packs;
    const F* src = static_cast<const F*>(buf);
    T* dst = static_cast<T*>(buf);
    for (int64_t w = 0; w < waves; ++w) {
        const int64_t wave = sizeof(F) > sizeof(T) ? w : waves - 1 - w;
        Pack<P * sizeof(F)> in[UW];
#pragma unroll
        for (int u = 0; u < UW; ++u) {
            const int64_t p = wave * wave_packs + static_cast<int64_t>(u) * threads + tid;
            if (p >= packs) continue;
            if ((p + 1) * P <= n) {
                loadPack<P * sizeof(F), false>(in[u], src + p * P);
            } else {
                for (int e = 0; e < P; ++e)
                    if (p * P + e < n) reinterpret_cast<F*>(&in[u])[e] = src[p * P + e];
            }
        }
        grid.sync();
#pragma unroll
        for (int u = 0; u < UW; ++u) {
            const int64_t p = wave * wave_packs + static_cast<int64_t>(u) * threads + tid;
            if (p >= packs) continue;
            Pack<P * sizeof(T)> out;
#pragma unroll
            for (int e = 0; e < P; ++e) reinterpret_cast<T*>(&out)[e] = Cvt<F, T>::run(reinterpret_cast<const F*>(&in[u])[e]);
            if ((p + 1) * P <= n) {
                storePack(dst + p * P, out);
            } else {
                for (int e = 0; e < P; ++e)
                    if (p * P + e < n) dst[p * P + e] = reinterpret_cast<const T*>(&out)[e];
            }
        }
    }
}

template <class F, class T>
int launchCast(const void* src_v, void* dst_v, int64_t n, cudaStream_t stream);

// Grid of the wave kernel: as many CTAs as are resident at once, but no more than one wave needs.
template <class F, class T>
int launchInPlaceWaves(void* buf, int64_t n, cudaStream_t stream) {
    using G = CastGeom<F, T>;
    constexpr int P = G::P, UW = 2;
    const DeviceInfo* dev = nullptr;
    if (int st = currentDeviceInfo(&dev)) return st;
    static int per_sm = 0;  // the same for every device this library supports (one architecture)
    if (per_sm == 0) {
        int v = 0;
        TB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&v, castInPlaceWavesKernel<F, T, P, UW>, 256, 0));
        TB_REQUIRE(v > 0, "in-place cast: the wave kernel does not fit an SM");
        per_sm = v;
    }
    const int64_t packs = (n + P - 1) / P;
    int64_t blocks = (packs + 256 * UW - 1) / (256 * UW);
    const int64_t resident = static_cast<int64_t>(dev->sm_count) * per_sm;
    blocks = blocks < 1 ? 1 : (blocks > resident ? resident : blocks);
    void* args[] = {&buf, &n};
    TB_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(castInPlaceWavesKernel<F, T, P, UW>), dim3(static_cast<unsigned>(blocks)), dim3(256), args, 0, stream));
    countLaunch();
    return THOR_B200_OK;
}

// Same-address conversion between element sizes (element i of the source view becomes element i of
// the destination view; TypeConverterKernels.cu:846-904 has the reference's semantics).  The range
// is cut into stream-ordered passes whose writes land only on bytes that no later pass reads:
//   narrowing: [0, head) by the head kernel, then [s, e) with e * sizeof(T) <= s * sizeof(F), upwards;
//   widening:  [s, n) with s * sizeof(T) >= n * sizeof(F), then downwards, the head block last.
// Each pass is the ordinary out-of-place kernel on disjoint byte ranges; pass boundaries are
// multiples of 2048 elements so 16-byte packs stay aligned.  The number of launches grows with
// log(n / head) to the base of the size ratio (12 for 2^24 fp32 -> fp16).
template <class F, class T>
int launchInPlaceResize(void* buf, int64_t n, cudaStream_t stream) {
    constexpr int64_t S = sizeof(F), D = sizeof(T), kAlign = 2048;
    F* src = static_cast<F*>(buf);
    T* dst = static_cast<T*>(buf);
    auto head = [&](int64_t count) -> int {
        TB_CUDA(launchDependent(castInPlaceHeadKernel<F, T>, dim3(1), dim3(256), 0, stream, buf, static_cast<int>(count)));
        countLaunch();
        return THOR_B200_OK;
    };
    if constexpr (sizeof(F) > sizeof(T)) {
        int64_t s = n < kHeadElements ? n : kHeadElements;
        if (int st = head(s)) return st;
        while (s < n) {
            int64_t e = s * S / D;
            e = e / kAlign * kAlign;
            if (e > n) e = n;
            if (int st = launchCast<F, T>(src + s, dst + s, e - s, stream)) return st;
            s = e;
        }
    } else {
        int64_t e = n;
        while (e > kHeadElements) {
            int64_t s = (e * S + D - 1) / D;
            s = (s + kAlign - 1) / kAlign * kAlign;  // s < e because e > kHeadElements >= 2 * kAlign and S <= D / 2
            if (int st = launchCast<F, T>(src + s, dst + s, e - s, stream)) return st;
            e = s;
        }
        if (int st = head(e)) return st;
    }
    return THOR_B200_OK;
}

template <class F, class T>
int launchCast(const void* src_v, void* dst_v, int64_t n, cudaStream_t stream) {
    using G = CastGeom<F, T>;
    constexpr int P = G::P;
    constexpr int U = G::U;
    const DeviceInfo* dev = nullptr;
    if (int st = currentDeviceInfo(&dev)) return st;
    const F* src = static_cast<const F*>(src_v);
    T* dst = static_cast<T*>(dst_v);
    const int64_t resident = static_cast<int64_t>(dev->sm_count) * 8;  // 8 x 256 threads = 2048 per SM

    if (src_v == dst_v) {
        if constexpr (sizeof(F) == sizeof(T)) {
            if (!isAligned(src_v, 16)) return fail(THOR_B200_UNSUPPORTED, "in-place cast needs a 16-byte aligned buffer");
            const int64_t n_packs = n / P;
            int64_t blocks = (n_packs + 255) / 256;
            blocks = blocks < 1 ? 1 : (blocks > resident ? resident : blocks);
            (void)launchDependent(castInPlaceSameSizeKernel<F, T, P>, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, dst_v, n_packs, n);
            countLaunch();
            TB_CUDA(cudaGetLastError());
            return THOR_B200_OK;
        } else {
            // one cooperative launch when the buffer allows 16-byte packs (every allocation does); a foreign sub-view
            // that is not aligned takes the chain of out-of-place passes
            if (isAligned(dst_v, 16)) return launchInPlaceWaves<F, T>(dst_v, n, stream);
            return launchInPlaceResize<F, T>(dst_v, n, stream);
        }
    }

    const bool aligned = isAligned(src_v, sizeof(F) * P >= 16 ? 16 : sizeof(F) * P) && isAligned(dst_v, sizeof(T) * P >= 16 ? 16 : sizeof(T) * P);
    if (aligned) {
        const int64_t n_packs = n / P;
        int64_t blocks = (n_packs + 256 * U - 1) / (256 * U);
        blocks = blocks < 1 ? 1 : blocks;
        if (blocks > 0x7FFFFFFF) return fail(THOR_B200_UNSUPPORTED, "cast: %lld elements exceed the launch grid", static_cast<long long>(n));
        if ((P * sizeof(F)) % 32 == 0 && isAligned(src_v, 32))
            TB_CUDA(launchDependent(castPackedKernel<F, T, P, U, true>, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, src, dst, n_packs, n));
        else
            TB_CUDA(launchDependent(castPackedKernel<F, T, P, U, false>, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, src, dst, n_packs, n));
    } else {
        int64_t blocks = (n + 255) / 256;
        blocks = blocks < 1 ? 1 : (blocks > resident ? resident : blocks);
        (void)launchDependent(castScalarKernel<F, T>, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, src, dst, n);
    }
    countLaunch();
    TB_CUDA(cudaGetLastError());
    return THOR_B200_OK;
}

template <class F>
int dispatchDst(const void* src, void* dst, int dst_dtype, int64_t n, cudaStream_t stream) {
#define TB_DST(DT)                                                                  \
    case DT:                                                                        \
        if constexpr (std::is_same_v<F, typename CType<DT>::type>) break;           \
        else return launchCast<F, typename CType<DT>::type>(src, dst, n, stream);
    switch (dst_dtype) {
        TB_DST(THOR_B200_FP16)
        TB_DST(THOR_B200_BF16)
        TB_DST(THOR_B200_FP32)
        TB_DST(THOR_B200_FP64)
        TB_DST(THOR_B200_INT8)
        TB_DST(THOR_B200_INT16)
        TB_DST(THOR_B200_INT32)
        TB_DST(THOR_B200_INT64)
        TB_DST(THOR_B200_UINT8)
        TB_DST(THOR_B200_UINT16)
        TB_DST(THOR_B200_UINT32)
        TB_DST(THOR_B200_UINT64)
        TB_DST(THOR_B200_BOOLEAN)
        TB_DST(THOR_B200_FP8_E4M3)
        TB_DST(THOR_B200_FP8_E5M2)
        default: break;
    }
#undef TB_DST
    return fail(THOR_B200_INVALID_ARGUMENT, "cast: unsupported destination dtype %d", dst_dtype);
}

}  // namespace tb

extern "C" int thor_b200_cast_launch(const void* src, void* dst, int src_dtype, int dst_dtype, int64_t n, void* stream_v) {
    using namespace tb;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    TB_REQUIRE(n >= 0, "cast: numElements must be >= 0 (got %lld)", static_cast<long long>(n));
    const size_t ss = dtypeSize(src_dtype), ds = dtypeSize(dst_dtype);
    TB_REQUIRE(ss != 0, "cast: unknown source dtype %d", src_dtype);
    TB_REQUIRE(ds != 0, "cast: unknown destination dtype %d", dst_dtype);
    TB_REQUIRE(src_dtype != dst_dtype, "cast: source and destination dtype are both %s", dtypeName(src_dtype));
    if (n == 0) return THOR_B200_OK;
    TB_REQUIRE(src != nullptr && dst != nullptr, "cast: null pointer");
    if (src != dst) {
        // Out of place: the two byte ranges must be disjoint (TypeConverterKernels.cu:915-924).
        const uintptr_t s0 = reinterpret_cast<uintptr_t>(src), s1 = s0 + static_cast<uintptr_t>(n) * ss;
        const uintptr_t d0 = reinterpret_cast<uintptr_t>(dst), d1 = d0 + static_cast<uintptr_t>(n) * ds;
        TB_REQUIRE(s1 <= d0 || d1 <= s0, "cast: source and destination ranges overlap");
    }
#define TB_SRC(DT) \
    case DT: return dispatchDst<typename CType<DT>::type>(src, dst, dst_dtype, n, stream);
    switch (src_dtype) {
        TB_SRC(THOR_B200_FP16)
        TB_SRC(THOR_B200_BF16)
        TB_SRC(THOR_B200_FP32)
        TB_SRC(THOR_B200_FP64)
        TB_SRC(THOR_B200_INT8)
        TB_SRC(THOR_B200_INT16)
        TB_SRC(THOR_B200_INT32)
        TB_SRC(THOR_B200_INT64)
        TB_SRC(THOR_B200_UINT8)
        TB_SRC(THOR_B200_UINT16)
        TB_SRC(THOR_B200_UINT32)
        TB_SRC(THOR_B200_UINT64)
        TB_SRC(THOR_B200_BOOLEAN)
        TB_SRC(THOR_B200_FP8_E4M3)
        TB_SRC(THOR_B200_FP8_E5M2)
        default: break;
    }
#undef TB_SRC
    return fail(THOR_B200_INVALID_ARGUMENT, "cast: unsupported source dtype %d", src_dtype);
}

// Tensor::copyFromAsync across placements with a dtype change (Tensor.cpp:769-792, 842-851): the bytes travel in the
// SOURCE dtype into the destination buffer, which is then converted where it lies.  Only destinations whose array is
// at least as large as the source's are accepted, as in the reference: shrinking would need a hidden temporary.
extern "C" int thor_b200_copy_convert_launch(void* dst, int dst_dtype, int dst_device, const void* src, int src_dtype, int src_device, int64_t n,
                                             void* stream_v) {
    using namespace tb;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    TB_REQUIRE(n >= 0, "copy_convert: numElements must be >= 0 (got %lld)", static_cast<long long>(n));
    const size_t ss = dtypeSize(src_dtype), ds = dtypeSize(dst_dtype);
    TB_REQUIRE(ss != 0 && ds != 0, "copy_convert: unknown dtype (%d -> %d)", src_dtype, dst_dtype);
    if (n == 0) return THOR_B200_OK;
    TB_REQUIRE(dst != nullptr && src != nullptr, "copy_convert: null pointer");
    TB_REQUIRE(dst_device >= -1 && src_device >= -1, "copy_convert: a device is -1 (host memory) or a GPU ordinal");
    const bool same_place = dst_device == src_device;
    if (dst_device < 0 && (src_device < 0 || src_dtype != dst_dtype))
        return fail(THOR_B200_UNSUPPORTED, "copy_convert: conversions into host memory run on the CPU, which this library does not do");
    if (src_dtype == dst_dtype) {
        const size_t bytes = static_cast<size_t>(n) * ss;
        if (dst_device >= 0 && src_device >= 0 && !same_place) TB_CUDA(cudaMemcpyPeerAsync(dst, dst_device, src, src_device, bytes, stream));
        else TB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, stream));
        return THOR_B200_OK;
    }
    if (same_place) return thor_b200_cast_launch(src, dst, src_dtype, dst_dtype, n, stream_v);  // on one GPU: the cast seam, possibly in place
    TB_REQUIRE(ss <= ds, "copy_convert: a copy across placements into a smaller dtype (%s -> %s) would need a hidden temporary; stage it explicitly",
               dtypeName(src_dtype), dtypeName(dst_dtype));
    const size_t bytes = static_cast<size_t>(n) * ss;
    if (src_device >= 0) TB_CUDA(cudaMemcpyPeerAsync(dst, dst_device, src, src_device, bytes, stream));
    else TB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, stream));
    return thor_b200_cast_launch(dst, dst, src_dtype, dst_dtype, n, stream_v);
}
