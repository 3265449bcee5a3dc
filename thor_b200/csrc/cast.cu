// dtype casts: one streaming kernel template over all 15 x 15 storage pairs.
//
// Design for B200: the cast is pure HBM traffic.  Each thread moves one or two packs of P
// elements (the narrower side of a pack is 16 bytes, the wider side 32..128 bytes, read with
// 256-bit loads where the address allows) and each CTA owns a contiguous run of packs.  A plain
// one-wave-after-another grid measured ~10 % faster on B200 than a persistent grid-stride loop
// for this access pattern (6.7-6.8 TB/s against 6.0-6.2 TB/s at 1.5 GB of traffic), so the grid
// is sized to the tensor.  The last n % P elements are converted one by one by the first CTA,
// which means the kernel touches exactly n elements on both sides.
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

template <class F, class T>
int launchCast(const void* src_v, void* dst_v, int64_t n, cudaStream_t stream);

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
