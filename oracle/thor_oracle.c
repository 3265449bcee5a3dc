/*
 * thor_oracle.c — CPU restatement of the reference semantics of the hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the product (libthor_b200, the host layer, the Python
 * package) links, imports or executes this file; it is the checker that the tests, the smoke
 * run and the benchmark's cpu_baseline leg compare the CUDA path against.
 *
 * Pinning: the cast routines are checked bit-for-bit against the reference's own CPU converter
 * (TypeConverter::cpuConvertTypeImpl compiled from the reference tree into oracle/_ref, see
 * ref_cast.cpp) and against the golden fixtures in tests/golden; the reductions against the
 * hand-computed vectors of the reference's CubReduction*Test.cpp files restated in the tests.
 *
 * Every function cites the reference file:line (path inside the Thor project) it follows.
 * Build: gcc -O3 -fopenmp -fPIC -shared thor_oracle.c -o _build/libthor_oracle.so -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define API __attribute__((visibility("default")))

/* DataType integers: DeepLearning/Implementation/Tensor/DataType.h:7-26 */
enum { DT_FP16 = 10, DT_FP32, DT_FP64, DT_INT8, DT_INT16, DT_INT32, DT_INT64, DT_UINT8, DT_UINT16, DT_UINT32, DT_UINT64,
       DT_BOOL, DT_E4M3, DT_E5M2, DT_BF16 };

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint64_t f64_bits(double f) { uint64_t u; memcpy(&u, &f, 8); return u; }

/* ------------------------------------------------------------------------------------------
 * Narrow float formats.  One generic round-to-nearest-even encoder from double: a double holds
 * every float/half/bf16/fp8 input exactly, so encoding from the double is a single rounding,
 * which is what static_cast<half>(float) = __float2half_rn, __double2half, __float2bfloat16_rn,
 * __double2bfloat16 do (TypeConverterKernels.cu:23-27 applies static_cast per element).
 * NaN maps to the canonical 0x7FFF of the CUDA conversions; overflow goes to infinity.
 * ---------------------------------------------------------------------------------------- */
static uint32_t encode_rne(double x, int exp_bits, int man_bits, int has_inf, int satfinite, uint32_t nan_code, uint32_t max_finite) {
    uint64_t b = f64_bits(x);
    uint32_t sign = (uint32_t)(b >> 63) << (exp_bits + man_bits);
    if (x != x) return nan_code;
    double a = fabs(x);
    if (a == 0.0) return sign;
    int bias = (1 << (exp_bits - 1)) - 1;
    int emin = 1 - bias; /* exponent of the smallest normal */
    if (isinf(a)) {
        if (satfinite) return sign | max_finite;
        return has_inf ? (sign | ((uint32_t)((1 << exp_bits) - 1) << man_bits)) : nan_code;
    }
    int e;
    double m = frexp(a, &e); /* a = m * 2^e, m in [0.5, 1) */
    e -= 1;                  /* a = (2m) * 2^e, 2m in [1, 2) */
    int q = (e < emin ? emin : e) - man_bits; /* exponent of one ulp at this magnitude */
    double scaled = ldexp(a, -q);             /* exact: power-of-two scaling */
    double r = nearbyint(scaled);             /* default rounding mode = ties to even */
    (void)m;
    /* r is an integer < 2^(man_bits+2); rebuild the encoding by adding it to the ulp grid origin */
    uint64_t ri = (uint64_t)r;
    uint32_t code;
    if (e < emin) {
        code = (uint32_t)ri; /* subnormal (may round up into the smallest normal, which is the right code) */
    } else {
        uint32_t biased = (uint32_t)(e + bias);
        code = (biased << man_bits) + (uint32_t)(ri - ((uint64_t)1 << man_bits));
    }
    /* overflow check against the format's largest finite code */
    if (code > max_finite) {
        if (satfinite) return sign | max_finite;
        return has_inf ? (sign | ((uint32_t)((1 << exp_bits) - 1) << man_bits)) : nan_code;
    }
    return sign | code;
}

API uint16_t tor_f64_to_f16(double x) { return (uint16_t)encode_rne(x, 5, 10, 1, 0, 0x7FFF, 0x7BFF); }
API uint16_t tor_f32_to_f16(float x) { return tor_f64_to_f16((double)x); }
API uint16_t tor_f64_to_bf16(double x) { return (uint16_t)encode_rne(x, 8, 7, 1, 0, 0x7FFF, 0x7F7F); }
API uint16_t tor_f32_to_bf16(float x) { return tor_f64_to_bf16((double)x); }
/* fp8 class constructors and Thor's e4m3 helper both use __NV_SATFINITE
 * (Utilities/Common/LowPrecisionFloat.h:18-46): finite overflow and infinities clamp to the
 * largest finite value, NaN encodes as 0x7F. */
API uint8_t tor_f64_to_e4m3(double x) { return (uint8_t)encode_rne(x, 4, 3, 0, 1, 0x7F, 0x7E); }
API uint8_t tor_f64_to_e5m2(double x) { return (uint8_t)encode_rne(x, 5, 2, 1, 1, 0x7F, 0x7B); }

static double decode(uint32_t code, int exp_bits, int man_bits, int e4m3_nan_rule) {
    uint32_t sign = (code >> (exp_bits + man_bits)) & 1u;
    uint32_t ex = (code >> man_bits) & ((1u << exp_bits) - 1);
    uint32_t man = code & ((1u << man_bits) - 1);
    int bias = (1 << (exp_bits - 1)) - 1;
    double v;
    if (e4m3_nan_rule) {
        if (ex == 15 && man == 7) return NAN;
    } else if (ex == (1u << exp_bits) - 1) {
        v = man ? NAN : INFINITY;
        return sign ? -v : v;
    }
    if (ex == 0) v = ldexp((double)man, 1 - bias - man_bits);
    else v = ldexp((double)(man | (1u << man_bits)), (int)ex - bias - man_bits);
    return sign ? -v : v;
}
API float tor_f16_to_f32(uint16_t h) { return (float)decode(h, 5, 10, 0); }
API float tor_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }
API float tor_e4m3_to_f32(uint8_t v) { return (float)decode(v, 4, 3, 1); }
API float tor_e5m2_to_f32(uint8_t v) { return (float)decode(v, 5, 2, 0); }

API void tor_round_f32_to_f16_array(const float* x, float* y, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) y[i] = tor_f16_to_f32(tor_f32_to_f16(x[i]));
}
API void tor_round_f32_to_bf16_array(const float* x, float* y, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) y[i] = tor_bf16_to_f32(tor_f32_to_bf16(x[i]));
}

/* ------------------------------------------------------------------------------------------
 * Cast, all storage pairs.  Follows TypeConverter::cpuConvertTypeImpl
 * (Utilities/TensorOperations/DataTypeConversions/TypeConverter.cpp:899-942): one static_cast per
 * element.  Every source value is first widened exactly (to double, or to a 64-bit integer),
 * then narrowed once.  Float -> integer truncates toward zero and, like the GPU's cvt.rzi,
 * saturates and sends NaN to 0 (C++ leaves out-of-range undefined; the tests stay in range).
 * Integer -> e5m2 goes through float first, as the __nv_fp8_e5m2 integer constructors do
 * (cuda_fp8.hpp); integer -> e4m3 goes through double (LowPrecisionFloat.h:42-47).
 * ---------------------------------------------------------------------------------------- */
typedef struct { int is_float; int is_signed; double f; int64_t i; uint64_t u; } wide_t;

static inline wide_t load_wide(const void* p, int dt, int64_t k) {
    wide_t w; w.is_float = 0; w.is_signed = 1; w.f = 0; w.i = 0; w.u = 0;
    switch (dt) {
        case DT_FP16: w.is_float = 1; w.f = tor_f16_to_f32(((const uint16_t*)p)[k]); break;
        case DT_BF16: w.is_float = 1; w.f = tor_bf16_to_f32(((const uint16_t*)p)[k]); break;
        case DT_FP32: w.is_float = 1; w.f = ((const float*)p)[k]; break;
        case DT_FP64: w.is_float = 1; w.f = ((const double*)p)[k]; break;
        case DT_E4M3: w.is_float = 1; w.f = tor_e4m3_to_f32(((const uint8_t*)p)[k]); break;
        case DT_E5M2: w.is_float = 1; w.f = tor_e5m2_to_f32(((const uint8_t*)p)[k]); break;
        case DT_INT8: w.i = ((const int8_t*)p)[k]; break;
        case DT_INT16: w.i = ((const int16_t*)p)[k]; break;
        case DT_INT32: w.i = ((const int32_t*)p)[k]; break;
        case DT_INT64: w.i = ((const int64_t*)p)[k]; break;
        case DT_UINT8: w.is_signed = 0; w.u = ((const uint8_t*)p)[k]; break;
        case DT_UINT16: w.is_signed = 0; w.u = ((const uint16_t*)p)[k]; break;
        case DT_UINT32: w.is_signed = 0; w.u = ((const uint32_t*)p)[k]; break;
        case DT_UINT64: w.is_signed = 0; w.u = ((const uint64_t*)p)[k]; break;
        case DT_BOOL: w.is_signed = 0; w.u = ((const uint8_t*)p)[k] != 0; break;
    }
    return w;
}

static inline int64_t sat_i64(double f, double lo, double hi, int64_t ilo, int64_t ihi) {
    if (f != f) return 0;
    double t = trunc(f);
    if (t <= lo) return ilo;
    if (t >= hi) return ihi;
    return (int64_t)t;
}
static inline uint64_t sat_u64(double f, double hi, uint64_t ihi) {
    if (f != f) return 0;
    double t = trunc(f);
    if (t <= 0.0) return 0;
    if (t >= hi) return ihi;
    return (uint64_t)t;
}

/* int64/uint64 -> float formats need a single rounding from the integer, not via double. */
static double wide_as_double_exactish(wide_t w, int* exact) {
    if (w.is_float) { *exact = 1; return w.f; }
    if (w.is_signed) { *exact = (w.i > -(1LL << 53) && w.i < (1LL << 53)); return (double)w.i; }
    *exact = (w.u < (1ULL << 53)); return (double)w.u;
}
/* Round-to-odd reduction of a 64-bit integer to a double, so that a later RNE to <= 24 bits is
 * still a single correct rounding. */
static double int_to_double_round_odd(wide_t w) {
    uint64_t mag; int neg = 0;
    if (w.is_signed) { neg = w.i < 0; mag = neg ? (uint64_t)(-(w.i + 1)) + 1u : (uint64_t)w.i; } else mag = w.u;
    if (mag < (1ULL << 53)) return neg ? -(double)mag : (double)mag;
    int shift = 0; uint64_t m = mag;
    while ((m >> shift) >= (1ULL << 53)) ++shift;
    uint64_t kept = m >> shift, lost = m & ((1ULL << shift) - 1);
    if (lost) kept |= 1;
    double d = ldexp((double)kept, shift);
    return neg ? -d : d;
}

static inline void store_narrow(void* p, int dt, int64_t k, wide_t w) {
    int exact;
    switch (dt) {
        case DT_FP16: ((uint16_t*)p)[k] = tor_f64_to_f16(w.is_float ? w.f : int_to_double_round_odd(w)); break;
        case DT_BF16: ((uint16_t*)p)[k] = tor_f64_to_bf16(w.is_float ? w.f : int_to_double_round_odd(w)); break;
        case DT_FP32:
            if (w.is_float) ((float*)p)[k] = (float)w.f;
            else ((float*)p)[k] = w.is_signed ? (float)w.i : (float)w.u;
            break;
        case DT_FP64:
            if (w.is_float) ((double*)p)[k] = w.f;
            else ((double*)p)[k] = w.is_signed ? (double)w.i : (double)w.u;
            break;
        case DT_E4M3: ((uint8_t*)p)[k] = tor_f64_to_e4m3(w.is_float ? w.f : wide_as_double_exactish(w, &exact)); break;
        case DT_E5M2: {
            double v = w.is_float ? w.f : (double)(w.is_signed ? (float)w.i : (float)w.u);
            ((uint8_t*)p)[k] = tor_f64_to_e5m2(v);
        } break;
        case DT_INT8: ((int8_t*)p)[k] = (int8_t)(w.is_float ? sat_i64(w.f, -128, 127, -128, 127) : (w.is_signed ? w.i : (int64_t)w.u)); break;
        case DT_INT16: ((int16_t*)p)[k] = (int16_t)(w.is_float ? sat_i64(w.f, -32768, 32767, -32768, 32767) : (w.is_signed ? w.i : (int64_t)w.u)); break;
        case DT_INT32: ((int32_t*)p)[k] = (int32_t)(w.is_float ? sat_i64(w.f, -2147483648.0, 2147483647.0, INT32_MIN, INT32_MAX) : (w.is_signed ? w.i : (int64_t)w.u)); break;
        case DT_INT64: ((int64_t*)p)[k] = w.is_float ? sat_i64(w.f, -9223372036854775808.0, 9223372036854775808.0, INT64_MIN, INT64_MAX) : (w.is_signed ? w.i : (int64_t)w.u); break;
        case DT_UINT8: ((uint8_t*)p)[k] = (uint8_t)(w.is_float ? sat_u64(w.f, 255, 255) : (w.is_signed ? (uint64_t)w.i : w.u)); break;
        case DT_UINT16: ((uint16_t*)p)[k] = (uint16_t)(w.is_float ? sat_u64(w.f, 65535, 65535) : (w.is_signed ? (uint64_t)w.i : w.u)); break;
        case DT_UINT32: ((uint32_t*)p)[k] = (uint32_t)(w.is_float ? sat_u64(w.f, 4294967295.0, UINT32_MAX) : (w.is_signed ? (uint64_t)w.i : w.u)); break;
        case DT_UINT64: ((uint64_t*)p)[k] = w.is_float ? sat_u64(w.f, 18446744073709551616.0, UINT64_MAX) : (w.is_signed ? (uint64_t)w.i : w.u); break;
        case DT_BOOL: ((uint8_t*)p)[k] = w.is_float ? (w.f != 0.0) : (w.is_signed ? (w.i != 0) : (w.u != 0)); break;
    }
}

API int tor_cast(const void* src, void* dst, int src_dt, int dst_dt, int64_t n) {
    if (src_dt < DT_FP16 || src_dt > DT_BF16 || dst_dt < DT_FP16 || dst_dt > DT_BF16 || n < 0) return 1;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) store_narrow(dst, dst_dt, i, load_wide(src, src_dt, i));
    return 0;
}

/* Dedicated fp32 -> fp16 loop with the reference's threading rule (TypeConverter.cpp:917-925:
 * min(cores, n / 500000) threads, static schedule); used as the timed CPU baseline "port". */
API void tor_cast_f32_f16(const float* src, uint16_t* dst, int64_t n, int threads) {
    if (threads < 1) threads = 1;
#pragma omp parallel for schedule(static) num_threads(threads)
    for (int64_t i = 0; i < n; ++i) dst[i] = tor_f32_to_f16(src[i]);
}

/* ------------------------------------------------------------------------------------------
 * Fast fp32 <-> fp16 / bf16 for the workload-sized loops below (bit tricks, RNE, NaN -> 0x7FFF);
 * checked against encode_rne / decode over all inputs classes by tests/test_oracle_cast.py.
 * ---------------------------------------------------------------------------------------- */
static inline uint16_t fast_f32_to_f16(float f) {
    uint32_t x = f32_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t a = x & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return 0x7FFF;                    /* NaN */
    if (a >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* >= 65520 rounds to inf (also inf) */
    if (a < 0x38800000u) {                                   /* below the smallest normal half: subnormal or zero */
        if (a < 0x33000000u) return (uint16_t)sign;          /* < 2^-25: rounds to zero (2^-25 itself ties to even = 0) */
        /* add the magic constant 0.5f: the float adder performs the RNE rounding to the 2^-24 grid */
        float m = bits_f32(a) + 0.5f;
        return (uint16_t)(sign | (f32_bits(m) - 0x3F000000u));
    }
    uint32_t mant_odd = (a >> 13) & 1u;
    a += 0xC8000FFFu + mant_odd; /* rebias exponent (-112 << 23) and round to nearest even */
    return (uint16_t)(sign | (a >> 13));
}
static inline float fast_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t em = h & 0x7FFFu;
    if (em >= 0x7C00u) return bits_f32(sign | 0x7F800000u | ((em & 0x3FFu) << 13));
    if (em < 0x0400u) { /* subnormal: value = em * 2^-24 */
        float v = (float)em * 5.9604644775390625e-8f;
        return sign ? -v : v;
    }
    return bits_f32(sign | ((em + 0x1C000u) << 13));
}
static inline uint16_t fast_f32_to_bf16(float f) {
    uint32_t x = f32_bits(f);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFF;
    x += 0x7FFFu + ((x >> 16) & 1u);
    return (uint16_t)(x >> 16);
}
static inline float rh(float v) { return fast_f16_to_f32(fast_f32_to_f16(v)); }   /* round through fp16 */
static inline float rb(float v) { return bits_f32((uint32_t)fast_f32_to_bf16(v) << 16); } /* round through bf16 */

API uint16_t tor_fast_f32_to_f16(float f) { return fast_f32_to_f16(f); }
API float tor_fast_f16_to_f32(uint16_t h) { return fast_f16_to_f32(h); }
API uint16_t tor_fast_f32_to_bf16(float f) { return fast_f32_to_bf16(f); }

/* ------------------------------------------------------------------------------------------
 * Configuration 2: y = relu(a*x + b) * sigmoid(z) with every node in fp16
 * (dtype assignment ExpressionDTypeResolution.cpp:1012-1128; sigmoid composite Expression.h:1077-1088;
 * relu = max(x, 0), DeepLearning/Api/Layers/Activations/Relu.h:21-22).  Every node result is rounded
 * to fp16; b is first rounded to fp16 (scalars take the stage's 16-bit compute type,
 * CudaSourceEmitter.cpp:4034-4043).  fuse_mul_add = 1 evaluates a*x+b as one fused multiply-add
 * (what -fmad=true lets the compiler do with __hmul2 + __hadd2); 0 rounds the product first.
 * x, z, y: [rows, cols]; a: [cols].
 * ---------------------------------------------------------------------------------------- */
API void tor_c2_fused(const uint16_t* a, const uint16_t* x, float b, const uint16_t* z, uint16_t* y, int64_t rows, int64_t cols, int fuse_mul_add,
                      int threads) {
    const float bh = rh(b);
    if (threads < 1) threads = 1;
#pragma omp parallel for schedule(static) num_threads(threads)
    for (int64_t r = 0; r < rows; ++r) {
        for (int64_t c = 0; c < cols; ++c) {
            const float av = fast_f16_to_f32(a[c]), xv = fast_f16_to_f32(x[r * cols + c]), zv = fast_f16_to_f32(z[r * cols + c]);
            float lin;
            if (fuse_mul_add) lin = rh((float)((double)av * (double)xv + (double)bh)); /* exact product + one rounding */
            else lin = rh(rh(av * xv) + bh);
            const float relu = lin > 0.0f ? lin : 0.0f;             /* max(lin, 0) */
            const float neg = -zv;
            const float num = rh(expf(-(neg > 0.0f ? neg : 0.0f))); /* exp(-max(-z, 0)) */
            const float den = rh(1.0f + rh(expf(-fabsf(zv))));      /* 1 + exp(-|z|) */
            const float sig = rh(num / den);
            y[r * cols + c] = fast_f32_to_f16(relu * sig);
        }
    }
}

/* ------------------------------------------------------------------------------------------
 * Configuration 3: composed softmax over the last axis of fp32 [rows, cols] plus row argmax.
 * m = reduce_max (exact), e = expf(x - m) per element in fp32, s = sum(e) accumulated in fp64
 * (CubReductionOperation.cuh:60-129 accumulates in fp32; the fp64 sum is the accuracy reference
 * both are compared to), y = e / s in fp32.  argmax: NaN wins, lowest index wins ties
 * (CubArgReductionOperation.cuh:31-73).
 * ---------------------------------------------------------------------------------------- */
API void tor_softmax_rows_f32(const float* x, float* y, uint32_t* argmax, int64_t rows, int64_t cols, int threads) {
    if (threads < 1) threads = 1;
#pragma omp parallel for schedule(static) num_threads(threads)
    for (int64_t r = 0; r < rows; ++r) {
        const float* p = x + r * cols;
        float m = -INFINITY;
        int64_t best = 0;
        int has_nan = 0;
        for (int64_t c = 0; c < cols; ++c) {
            const float v = p[c];
            if (v != v) { if (!has_nan) { has_nan = 1; best = c; m = v; } continue; }
            if (!has_nan && (c == 0 || v > m)) { m = v; best = c; }
        }
        if (argmax) argmax[r] = (uint32_t)best;
        if (!y) continue;
        double s = 0.0;
        for (int64_t c = 0; c < cols; ++c) { const float e = expf(p[c] - m); y[r * cols + c] = e; s += e; }
        const float sf = (float)s;
        for (int64_t c = 0; c < cols; ++c) y[r * cols + c] = y[r * cols + c] / sf;
    }
}

/* ------------------------------------------------------------------------------------------
 * Configuration 4: sum, sum of squares and max of a bf16 vector.  sum-of-squares is spelled
 * (x*x).reduce_sum() (cf. DeepLearning/Implementation/Layers/Optimizers/Lamb.cpp:106): the product
 * node is a bf16 node, so it is rounded to bf16 before the fp32 conversion of the reduction.
 * Accumulation here is fp64 over those rounded operands.
 * ---------------------------------------------------------------------------------------- */
API void tor_c4_stats_bf16(const uint16_t* x, int64_t n, double* sum, double* sumsq, float* maxv, int threads) {
    double s = 0.0, q = 0.0;
    float m = -INFINITY;
    int has_nan = 0;
    if (threads < 1) threads = 1;
#pragma omp parallel for schedule(static) num_threads(threads) reduction(+ : s, q) reduction(max : m) reduction(| : has_nan)
    for (int64_t i = 0; i < n; ++i) {
        const float v = bits_f32((uint32_t)x[i] << 16);
        s += v;
        q += rb(v * v);
        if (v != v) has_nan = 1;
        else if (v > m) m = v;
    }
    *sum = s;
    *sumsq = q;
    *maxv = has_nan ? NAN : m;
}

/* ------------------------------------------------------------------------------------------
 * Configuration 5: LayerNorm written as an Expression DAG over bf16 [rows, cols]:
 *   mean = x.reduce_mean({1}); xc = x - mean; var = (xc*xc).reduce_mean({1});
 *   rstd = 1 / sqrt(var + eps); y = (xc * rstd * gamma + beta).cast(BF16)
 * Everything from xc onward is fp32 (bf16 - fp32 promotes, ExpressionDTypeResolution.cpp:277-307);
 * reductions accumulate here in fp64 and are rounded to fp32 like every reduction output.
 * Backward (reverse-mode of that DAG, AutoDiff.cpp:3690-5930), with g = dy * gamma, xhat = xc * rstd:
 *   dx = rstd * (g - mean_row(g) - xhat * mean_row(g * xhat)),
 *   dgamma = sum_rows(dy * xhat), dbeta = sum_rows(dy)       (fp32 outputs)
 * ---------------------------------------------------------------------------------------- */
API void tor_layernorm_fwd_bf16(const uint16_t* x, const uint16_t* gamma, const uint16_t* beta, float eps, uint16_t* y, float* mean_out,
                                float* rstd_out, int64_t rows, int64_t cols, int threads) {
    if (threads < 1) threads = 1;
#pragma omp parallel for schedule(static) num_threads(threads)
    for (int64_t r = 0; r < rows; ++r) {
        const uint16_t* p = x + r * cols;
        double s = 0.0;
        for (int64_t c = 0; c < cols; ++c) s += bits_f32((uint32_t)p[c] << 16);
        const float mean = (float)s / (float)cols;
        double q = 0.0;
        for (int64_t c = 0; c < cols; ++c) { const float xc = bits_f32((uint32_t)p[c] << 16) - mean; q += (double)(xc * xc); }
        const float var = (float)q / (float)cols;
        const float rstd = 1.0f / sqrtf(var + eps);
        if (mean_out) mean_out[r] = mean;
        if (rstd_out) rstd_out[r] = rstd;
        if (y)
            for (int64_t c = 0; c < cols; ++c) {
                const float xc = bits_f32((uint32_t)p[c] << 16) - mean;
                const float v = xc * rstd * bits_f32((uint32_t)gamma[c] << 16) + bits_f32((uint32_t)beta[c] << 16);
                y[r * cols + c] = fast_f32_to_bf16(v);
            }
    }
}

API void tor_layernorm_bwd_bf16(const uint16_t* x, const uint16_t* gamma, const uint16_t* dy, float eps, uint16_t* dx, double* dgamma, double* dbeta,
                                int64_t rows, int64_t cols, int threads) {
    if (threads < 1) threads = 1;
    for (int64_t c = 0; c < cols; ++c) { dgamma[c] = 0.0; dbeta[c] = 0.0; }
#pragma omp parallel num_threads(threads)
    {
        double* lg = (double*)calloc((size_t)cols, sizeof(double));
        double* lb = (double*)calloc((size_t)cols, sizeof(double));
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            const uint16_t* p = x + r * cols;
            const uint16_t* d = dy + r * cols;
            double s = 0.0;
            for (int64_t c = 0; c < cols; ++c) s += bits_f32((uint32_t)p[c] << 16);
            const float mean = (float)s / (float)cols;
            double q = 0.0;
            for (int64_t c = 0; c < cols; ++c) { const float xc = bits_f32((uint32_t)p[c] << 16) - mean; q += (double)(xc * xc); }
            const float rstd = 1.0f / sqrtf((float)q / (float)cols + eps);
            double sg = 0.0, sgx = 0.0;
            for (int64_t c = 0; c < cols; ++c) {
                const double xhat = (double)(bits_f32((uint32_t)p[c] << 16) - mean) * rstd;
                const double dyv = bits_f32((uint32_t)d[c] << 16);
                const double g = dyv * bits_f32((uint32_t)gamma[c] << 16);
                sg += g;
                sgx += g * xhat;
                lg[c] += dyv * xhat;
                lb[c] += dyv;
            }
            const double mg = sg / (double)cols, mgx = sgx / (double)cols;
            if (dx)
                for (int64_t c = 0; c < cols; ++c) {
                    const double xhat = (double)(bits_f32((uint32_t)p[c] << 16) - mean) * rstd;
                    const double g = (double)bits_f32((uint32_t)d[c] << 16) * bits_f32((uint32_t)gamma[c] << 16);
                    dx[r * cols + c] = fast_f32_to_bf16((float)(rstd * (g - mg - xhat * mgx)));
                }
        }
#pragma omp critical
        for (int64_t c = 0; c < cols; ++c) { dgamma[c] += lg[c]; dbeta[c] += lb[c]; }
        free(lg);
        free(lb);
    }
}
