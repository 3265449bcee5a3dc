/*
 * thor_b200.h — C ABI of libthor_b200.so
 *
 * B200 (sm_100a) kernels for the data-parallel hot path of Thor's expression engine:
 * dtype casts, dense value/arg reductions, and fused elementwise/broadcast expression stages.
 * Every entry point takes plain pointers and sizes, returns an int status (0 = ok) and is
 * asynchronous on the cudaStream_t that it is given (passed as void*).  After a non-zero
 * status thor_b200_last_error() returns a thread-local message; a C++ adapter turns that
 * into the std::runtime_error / std::logic_error that Thor's callers expect.
 *
 * No entry point here falls back to the CPU: without a CUDA device every launch fails.
 *
 * Each declaration cites the reference interface (path within the Thor project) it replaces.
 */
#ifndef THOR_B200_H
#define THOR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define THOR_B200_ABI_VERSION 1

#if defined(__GNUC__)
#define THOR_B200_API __attribute__((visibility("default")))
#else
#define THOR_B200_API
#endif

/* Same integers as ThorImplementation::DataType (DeepLearning/Implementation/Tensor/DataType.h:7-26). */
typedef enum thor_b200_dtype {
    THOR_B200_FP16 = 10,
    THOR_B200_FP32 = 11,
    THOR_B200_FP64 = 12,
    THOR_B200_INT8 = 13,
    THOR_B200_INT16 = 14,
    THOR_B200_INT32 = 15,
    THOR_B200_INT64 = 16,
    THOR_B200_UINT8 = 17,
    THOR_B200_UINT16 = 18,
    THOR_B200_UINT32 = 19,
    THOR_B200_UINT64 = 20,
    THOR_B200_BOOLEAN = 21,
    THOR_B200_FP8_E4M3 = 22,
    THOR_B200_FP8_E5M2 = 23,
    THOR_B200_BF16 = 24
} thor_b200_dtype;

/* Status codes.  INVALID_ARGUMENT maps to std::logic_error in the adapter (THOR_THROW_IF_FALSE,
 * DeepLearning/Implementation/ThorError.h:47-53), CUDA_ERROR / JIT_ERROR to std::runtime_error
 * (CUDA_CHECK / CU_CHECK, Utilities/Common/CudaHelpers.h:42-80). */
typedef enum thor_b200_status {
    THOR_B200_OK = 0,
    THOR_B200_INVALID_ARGUMENT = 1,
    THOR_B200_CUDA_ERROR = 2,
    THOR_B200_JIT_ERROR = 3,
    THOR_B200_UNSUPPORTED = 4
} thor_b200_status;

THOR_B200_API int thor_b200_abi_version(void);
/* Message for the last non-zero status returned on the calling thread ("" if none). */
THOR_B200_API const char* thor_b200_last_error(void);
/* Size in bytes of one stored element of `dtype`, 0 for an unknown dtype. */
THOR_B200_API size_t thor_b200_dtype_size(int dtype);
/* Number of kernels this library has launched from the calling process (all threads). */
THOR_B200_API uint64_t thor_b200_launch_count(void);
/* Programmatic dependent launch: every kernel of this library is launched with stream serialisation relaxed and opens
 * with griddepcontrol.wait, so its CTAs are placed while the previous kernel of the stream drains; stream-order
 * semantics are unchanged.  On by default; set_dependent_launch(0) launches without the attribute (process-wide, for
 * comparison runs and for tools that cannot follow overlapped launches).  dependent_launch() returns the setting. */
THOR_B200_API void thor_b200_set_dependent_launch(int on);
THOR_B200_API int thor_b200_dependent_launch(void);

/* ---------------------------------------------------------------------------------------------
 * S1  dtype cast
 * Replaces TypeConverter::gpuConvertType (Utilities/TensorOperations/DataTypeConversions/
 * TypeConverter.h:61-66; launcher TypeConverterKernels.cu:1340-1433).
 * Converts n elements from src (src_dtype) to dst (dst_dtype) with the C++ static_cast rule of
 * the CUDA element types (fp8-e4m3 destinations saturate to +-448).  Both pointers are device
 * memory of the stream's device.  src == dst requests an in-place conversion (element i of the
 * source view becomes element i of the destination view; between different element sizes the
 * buffer must hold the larger view, TypeConverterKernels.cu:846-904); otherwise the two
 * ranges must not overlap.  n == 0 is a no-op.  src_dtype == dst_dtype is a caller bug and is
 * rejected, as in the reference.  Reads and writes exactly n elements: no tail padding needed.
 * ------------------------------------------------------------------------------------------- */
THOR_B200_API int thor_b200_cast_launch(const void* src, void* dst, int src_dtype, int dst_dtype, int64_t n, void* stream);

/* Copy with an optional dtype change between placements: the data path of Tensor::copyFromAsync
 * (DeepLearning/Implementation/Tensor/Tensor.cpp:769-792, 842-851).  A device of -1 means host memory (pinned for a truly
 * asynchronous copy), otherwise a GPU ordinal; the destination's GPU is current and owns `stream`.  Same dtype: one
 * copy.  Same GPU, different dtypes: thor_b200_cast_launch.  Different placements and dtypes: the bytes travel in the
 * SOURCE dtype into the destination buffer and are converted there in place (one more launch), which requires the
 * destination array to be at least as large as the source's -- the reference refuses the shrinking case too because it
 * would need a hidden temporary (THOR_B200_INVALID_ARGUMENT).  Conversions INTO host memory are CPU work and are not
 * done here (THOR_B200_UNSUPPORTED). */
THOR_B200_API int thor_b200_copy_convert_launch(void* dst, int dst_dtype, int dst_device, const void* src, int src_dtype, int src_device, int64_t n,
                                                void* stream);

/* ---------------------------------------------------------------------------------------------
 * S3  fused elementwise / broadcast expression stage
 * Replaces EquationCompiler::compileFusedStage / compileSpecializedBroadcastStage
 * (Utilities/Expression/EquationCompiler.h:36-75; emitter CudaSourceEmitter.cpp:6749-6859 and
 * :7794-7944) and EquationRunner::run (Utilities/Expression/EquationRunner.h:14-18,
 * EquationRunner.cpp:34-290).
 *
 * A stage is a topologically ordered SSA node list, as in ThorImplementation::PhysicalExpression
 * (Expression.h:231-371): node k may only name parents < k.  `op` carries the integer value of
 * ThorImplementation::ExprOp (Expression.h:32-148); the subset a fused stage may contain is
 * listed in thor_b200_expr_op.  Every node arrives with its dtypes already resolved by the
 * caller (ExpressionDTypeResolution.cpp:1012-1148): the node computes in compute_dtype and
 * materialises its value in output_dtype; parents are converted to the consumer's compute dtype.
 * ------------------------------------------------------------------------------------------- */
typedef enum thor_b200_expr_op {
    THOR_B200_OP_INPUT = 3, THOR_B200_OP_RUNTIME_SCALAR = 4, THOR_B200_OP_TENSOR_RUNTIME_SCALAR = 5, THOR_B200_OP_SCALAR_FP = 6,
    THOR_B200_OP_ADD = 7, THOR_B200_OP_SUB = 8, THOR_B200_OP_MUL = 9, THOR_B200_OP_DIV = 10, THOR_B200_OP_POW = 11,
    THOR_B200_OP_EQUAL = 12, THOR_B200_OP_NOT_EQUAL = 13, THOR_B200_OP_LESS = 14, THOR_B200_OP_LESS_EQUAL = 15,
    THOR_B200_OP_GREATER = 16, THOR_B200_OP_GREATER_EQUAL = 17, THOR_B200_OP_LOGICAL_AND = 18, THOR_B200_OP_LOGICAL_OR = 19,
    THOR_B200_OP_LOGICAL_NOT = 20, THOR_B200_OP_CAST = 21, THOR_B200_OP_WHERE = 22, THOR_B200_OP_NEG = 23, THOR_B200_OP_ABS = 24,
    THOR_B200_OP_CEIL = 25, THOR_B200_OP_FLOOR = 26, THOR_B200_OP_ROUND = 27, THOR_B200_OP_TRUNC = 28, THOR_B200_OP_SIN = 29,
    THOR_B200_OP_COS = 30, THOR_B200_OP_TAN = 31, THOR_B200_OP_ASIN = 32, THOR_B200_OP_ACOS = 33, THOR_B200_OP_ATAN = 34,
    THOR_B200_OP_SINH = 35, THOR_B200_OP_COSH = 36, THOR_B200_OP_ASINH = 37, THOR_B200_OP_ACOSH = 38, THOR_B200_OP_ATANH = 39,
    THOR_B200_OP_ERF = 40, THOR_B200_OP_ERFC = 41, THOR_B200_OP_ERFCX = 42, THOR_B200_OP_ERFINV = 43, THOR_B200_OP_ERFCINV = 44,
    THOR_B200_OP_TGAMMA = 45, THOR_B200_OP_LGAMMA = 46, THOR_B200_OP_DIGAMMA = 47, THOR_B200_OP_EXP = 48, THOR_B200_OP_EXPM1 = 49,
    THOR_B200_OP_EXP2 = 50, THOR_B200_OP_EXP10 = 51, THOR_B200_OP_LN = 52, THOR_B200_OP_LOG1P = 53, THOR_B200_OP_LOG2 = 54,
    THOR_B200_OP_LOG10 = 55, THOR_B200_OP_SQRT = 56, THOR_B200_OP_TANH = 57, THOR_B200_OP_NORMCDF = 58,
    THOR_B200_OP_MIN = 69, THOR_B200_OP_MAX = 70, THOR_B200_OP_MIN_GRAD_LEFT = 71, THOR_B200_OP_MIN_GRAD_RIGHT = 72,
    THOR_B200_OP_MAX_GRAD_LEFT = 73, THOR_B200_OP_MAX_GRAD_RIGHT = 74,
    /* stage-boundary ops: never inside a fused stage, listed for the host layer and the reduction seam */
    THOR_B200_OP_REDUCE_SUM = 83, THOR_B200_OP_REDUCE_PROD = 84, THOR_B200_OP_REDUCE_MIN = 85, THOR_B200_OP_REDUCE_MAX = 86,
    THOR_B200_OP_REDUCE_ARGMIN = 87, THOR_B200_OP_REDUCE_ARGMAX = 88, THOR_B200_OP_REDUCE_AVG = 95, THOR_B200_OP_REDUCE_NORM1 = 96,
    THOR_B200_OP_REDUCE_NORM2 = 97
} thor_b200_expr_op;

#define THOR_B200_NO_NODE 0xFFFFFFFFu
#define THOR_B200_MAX_RANK 8

typedef struct thor_b200_expr_node {
    uint16_t op;            /* thor_b200_expr_op */
    uint16_t output_dtype;  /* thor_b200_dtype the node's value is stored in */
    uint16_t compute_dtype; /* thor_b200_dtype the node computes in */
    uint16_t input_dtype;   /* INPUT / *_RUNTIME_SCALAR nodes: dtype of the bound value; 0 otherwise */
    uint32_t lhs, rhs, aux; /* parent node indices, THOR_B200_NO_NODE when unused (WHERE: lhs=cond, rhs=true, aux=false) */
    uint32_t input_slot;    /* INPUT / *_RUNTIME_SCALAR nodes: index into the stage's input list */
    double scalar_fp;       /* SCALAR_FP nodes: the literal */
} thor_b200_expr_node;

typedef enum thor_b200_input_kind {
    THOR_B200_INPUT_TENSOR = 0,               /* device pointer to a tensor of the stage's shape (or a broadcast view of it) */
    THOR_B200_INPUT_RUNTIME_SCALAR_FP32 = 1,  /* float passed by value at launch (Expression::runtimeScalar) */
    THOR_B200_INPUT_TENSOR_RUNTIME_SCALAR = 2 /* device pointer to one element (Expression::tensorRuntimeScalar) */
} thor_b200_input_kind;

typedef struct thor_b200_expr_input {
    int32_t kind;  /* thor_b200_input_kind */
    int32_t dtype; /* thor_b200_dtype of the bound value */
} thor_b200_expr_input;

typedef struct thor_b200_expr_output {
    uint32_t node;  /* node whose value is written */
    int32_t dtype;  /* must equal that node's output_dtype */
} thor_b200_expr_output;

/* Broadcast geometry of a stage, the information the reference bakes into specialised broadcast
 * kernels (SpecializedBroadcastGroup, FusedEquation.cpp:5802-6020).  Outputs are dense row-major
 * tensors of shape dims[0..rank).  input_strides[slot][d] is the element stride of tensor input
 * `slot` along output axis d, 0 where that input is broadcast (ignored for scalar inputs). */
typedef struct thor_b200_expr_broadcast {
    uint32_t rank;
    uint64_t dims[THOR_B200_MAX_RANK];
    const int64_t* input_strides; /* [n_inputs][THOR_B200_MAX_RANK], row-major */
} thor_b200_expr_broadcast;

typedef struct thor_b200_expr_options {
    int32_t use_fast_math; /* NVRTC --use_fast_math, off by default like FusedEquation::compile (FusedEquation.cpp:7014-7016) */
    int32_t compile_only;  /* 1: emit + compile to a cubin but do not load it (usable without a GPU or driver) */
    int32_t rows_per_thread;  /* tiled broadcast kernels: rows each thread walks (1, 2, 4 or 8); 0 = chosen by the emitter */
    int32_t min_ctas_per_sm;  /* second argument of __launch_bounds__ (caps registers per thread); 0 = none */
    int32_t packs_per_thread; /* flat kernels: 16-byte packs each thread handles (1, 2 or 4); 0 = chosen by the emitter */
    int32_t reserved[3];      /* must be zero */
} thor_b200_expr_options;

typedef struct thor_b200_expr thor_b200_expr;

/* Emits CUDA C++ for the stage, compiles it with NVRTC for sm_100a and (unless compile_only) loads
 * it on the current device.  broadcast == NULL compiles a flat stage: every tensor input and
 * output has the same number of elements, given at launch.  Identical stages share one compiled
 * module (process-wide cache keyed by the emitted source), like the reference's LRU caches
 * (EquationCompiler.cpp:123-157).  Thread-safe.  The handle is immutable and may be launched
 * from any thread on any stream of the device it was compiled on. */
THOR_B200_API int thor_b200_expr_compile(const thor_b200_expr_node* nodes, uint32_t n_nodes, const thor_b200_expr_input* inputs,
                                         uint32_t n_inputs, const thor_b200_expr_output* outputs, uint32_t n_outputs,
                                         const thor_b200_expr_broadcast* broadcast, const thor_b200_expr_options* options,
                                         thor_b200_expr** out_expr);
/* Launches the stage.  input_ptrs[slot] is the device pointer for tensor and tensor-runtime-scalar
 * inputs (ignored for fp32 runtime scalars, whose values are read from runtime_scalars[slot]).
 * numel is the element count of a flat stage (ignored for broadcast stages, whose shape is baked
 * in).  Performs no allocation and no compilation except the first use of the unaligned-pointer
 * variant of a stage.  An output may alias an input only if it is that input's whole tensor. */
THOR_B200_API int thor_b200_expr_launch(thor_b200_expr* expr, const void* const* input_ptrs, const float* runtime_scalars,
                                        void* const* output_ptrs, uint64_t numel, void* stream);
/* The CUDA C++ source emitted for the stage (owned by the handle). */
THOR_B200_API const char* thor_b200_expr_source(const thor_b200_expr* expr);
/* "flat_v2", "flat_scalar", "bcast_tiled_v2", "bcast_tiled_scalar" or "bcast_generic": which kernel shape was chosen. */
THOR_B200_API const char* thor_b200_expr_launch_kind(const thor_b200_expr* expr);
THOR_B200_API void thor_b200_expr_destroy(thor_b200_expr* expr);
/* The process-wide cache of compiled stages and row programs keeps the most recently used modules, at most `entries`
 * (default 10 000, the bound of the reference's LRU caches, EquationCompiler.cpp:123-157; 0 turns caching off).  A module
 * that leaves the cache is unloaded once the last handle that uses it is destroyed.  Returns the previous bound. */
THOR_B200_API size_t thor_b200_jit_cache_capacity(size_t entries);
THOR_B200_API size_t thor_b200_jit_cache_size(void);
/* 16-bit stages evaluate exp and division with leaner routines than cuda_fp16.hpp's h2exp / __h2div, the
 * intrinsics the reference emits (CudaSourceEmitter.cpp:4376-4377).  This self-check runs both over every fp16
 * input (exp) and every ordered input pair in both lanes (division) and writes four counters to device
 * memory: [0] exp mismatches, [1] mismatches of the variant used for arguments known to be <= 0, [2] division
 * mismatches, [3] division pairs checked (2^32).  Bit parity with the reference requires [0..2] == 0. */
THOR_B200_API int thor_b200_selfcheck_pair_math(unsigned long long* device_counters, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Device memory for stamped plans.  Replaces the allocation half of ThorImplementation::Tensor
 * (DeepLearning/Implementation/Tensor/Tensor.cpp:232-281) for the intermediates and outputs that
 * FusedEquation::stamp / CubReduction::stamp create; run-time entry points never allocate.
 * ------------------------------------------------------------------------------------------- */
THOR_B200_API int thor_b200_device_alloc(size_t bytes, void** out_ptr);
THOR_B200_API int thor_b200_device_free(void* ptr);

/* Helper streams (non-blocking) and events (no timing) for a stamped plan whose independent branches run beside the
 * caller's stream (StampedExecutionPlan::runOn, Utilities/Expression/StampedEquation.cpp:4057-4205): created at stamp
 * time on the current device, reused by every run; recording and waiting are stream-ordered and never block the host. */
THOR_B200_API int thor_b200_stream_create(void** out_stream);
THOR_B200_API void thor_b200_stream_destroy(void* stream);
THOR_B200_API int thor_b200_event_create(void** out_event);
THOR_B200_API void thor_b200_event_destroy(void* event);
THOR_B200_API int thor_b200_event_record(void* event, void* stream);
THOR_B200_API int thor_b200_stream_wait_event(void* stream, void* event);

/* ---------------------------------------------------------------------------------------------
 * S2  dense value reductions and arg reductions
 * Replaces CubReductionInternal::query*ReductionBytes / launch*Reduction and the ArgMin/ArgMax
 * variants (Utilities/TensorOperations/Cub/CubReductionInternal.h:9-176; dispatch
 * CubReductionOperation.cuh:2966-3054, CubArgReductionOperation.cuh:1119-1178), i.e. what
 * CubReduction::stampValidated (CubReduction.cpp:935-968) and StampedCub{,Arg}Reduction::runOn
 * (CubReduction.cpp:1405,1441) call.
 *
 * The input is a dense tensor viewed as [outer, reduction, inner]: the geometry that
 * CubReduction::analyzeGeometry (CubReduction.cpp:755-912) produces for the DeviceTransformReduce
 * (outer = inner = 1), ContiguousFixedSegment (inner = 1) and TiledFixedSegment paths.  Every
 * input element is converted to fp32, transformed (identity / |x| / x^2), combined in fp32
 * (NaN-propagating min / max), finalised in fp32 (mean divides by the count, L2 takes the square
 * root), multiplied by output_scale and converted once to the output dtype
 * (CubReductionOperation.cuh:60-129,186-198).  Results are deterministic: a given plan combines
 * partial results in a fixed order.
 * ------------------------------------------------------------------------------------------- */
typedef enum thor_b200_reduce_op { /* = ThorImplementation::CubReductionOp (CubReduction.h:17-25) */
    THOR_B200_REDUCE_SUM = 0, THOR_B200_REDUCE_MIN = 1, THOR_B200_REDUCE_MAX = 2, THOR_B200_REDUCE_PRODUCT = 3,
    THOR_B200_REDUCE_MEAN = 4, THOR_B200_REDUCE_L1NORM = 5, THOR_B200_REDUCE_L2NORM = 6
} thor_b200_reduce_op;

typedef struct thor_b200_reduce_desc {
    int32_t op;           /* thor_b200_reduce_op */
    int32_t input_dtype;  /* fp8 / fp16 / bf16 / fp32 */
    int32_t output_dtype; /* fp8 / fp16 / bf16 / fp32 */
    uint32_t flags;       /* must be zero */
    uint64_t outer, reduction, inner;
    /* Element strides of output[o, i]; both zero selects the natural dense [outer, inner] layout.
     * (outer_stride = 1, inner_stride = outer) writes the permuted [inner, outer] layout of
     * CubReductionGeometry::tiled_output_permuted (CubReduction.h:139-147). */
    uint64_t out_stride_outer, out_stride_inner;
} thor_b200_reduce_desc;

typedef struct thor_b200_reduce_plan thor_b200_reduce_plan;

/* Plans the reduction (kernel choice, split of the reduction axis, workspace size).  May be
 * called without a GPU.  workspace_bytes is always >= 1, like the reference's convention
 * (CubReductionOperation.cuh:2941-2945). */
THOR_B200_API int thor_b200_reduce_plan_create(const thor_b200_reduce_desc* desc, thor_b200_reduce_plan** out_plan, size_t* workspace_bytes);
/* Runs the planned reduction; no allocation, no planning.  `workspace` must hold workspace_bytes
 * bytes, be 16-byte aligned and must not be shared by launches that overlap in time. */
THOR_B200_API int thor_b200_reduce_launch(const thor_b200_reduce_plan* plan, const void* input, void* output, void* workspace,
                                          size_t workspace_bytes, float output_scale, void* stream);
/* "full", "rows_warp", "rows_cta", "rows_split", "cols" ...: the kernel family the plan selected. */
THOR_B200_API const char* thor_b200_reduce_plan_kind(const thor_b200_reduce_plan* plan);
THOR_B200_API void thor_b200_reduce_plan_destroy(thor_b200_reduce_plan* plan);

typedef struct thor_b200_argreduce_desc {
    int32_t op;          /* 0 = argmin, 1 = argmax (CubArgReductionOp, CubReduction.h:27-30) */
    int32_t input_dtype; /* fp8 / fp16 / bf16 / fp32 */
    int32_t value_dtype; /* dtype of the optional value output, 0 if none is produced */
    int32_t index_dtype; /* THOR_B200_UINT32 or THOR_B200_UINT64 */
    uint64_t outer, reduction, inner;
} thor_b200_argreduce_desc;

typedef struct thor_b200_argreduce_plan thor_b200_argreduce_plan;

/* Arg reductions: values are compared in fp32; NaN beats every number; among equal candidates
 * (NaNs included) the lowest index wins; the index is the position inside the reduction domain
 * (CubArgReductionOperation.cuh:31-73,127-151; CubReduction.h:405-411). */
THOR_B200_API int thor_b200_argreduce_plan_create(const thor_b200_argreduce_desc* desc, thor_b200_argreduce_plan** out_plan, size_t* workspace_bytes);
THOR_B200_API int thor_b200_argreduce_launch(const thor_b200_argreduce_plan* plan, const void* input, void* value_output, void* index_output,
                                             void* workspace, size_t workspace_bytes, void* stream);
THOR_B200_API void thor_b200_argreduce_plan_destroy(thor_b200_argreduce_plan* plan);

/* ---------------------------------------------------------------------------------------------
 * Reductions over axes that are not adjacent (the reference's StridedFixedSegment path:
 * CubReductionOperation.cuh:2946-2958, 3038-3050; index map CubReductionIndexing.cuh:33-53;
 * arg variant CubArgReductionOperation.cuh:1119-1178).  input is a dense row-major tensor of
 * `rank` dims or, with has_strides, any strided view of storage (permuted, gapped, broadcast: the
 * reference never materialises a view to regain a dense path, CubReduction.cpp:903-907); output is
 * dense over the kept axes in their order.  Stateless: no plan, no
 * workspace, one kernel, the same numeric rules as the planned reductions (fp32 accumulation in
 * a fixed order, NaN-propagating min / max; arg: NaN wins, lowest flattened index of the reduced
 * axes in row-major order among equals).  Geometries that reduce one adjacent block of axes are
 * accepted too, but the planned reductions above are the fast path for those.
 * ------------------------------------------------------------------------------------------- */
typedef struct thor_b200_strided_reduce_desc {
    int32_t op;           /* thor_b200_reduce_op; ignored for arg reductions */
    int32_t arg_op;       /* -1: value reduction, 0: argmin, 1: argmax */
    int32_t input_dtype;  /* fp8 / fp16 / bf16 / fp32 */
    int32_t output_dtype; /* value reductions: fp8 / fp16 / bf16 / fp32; arg reductions: uint32 or uint64 */
    uint32_t rank;        /* 1..8 */
    uint32_t has_strides; /* 0: the input is dense row-major; 1: `strides` describes a view (Tensor::aliasView, Tensor.h:146-152) */
    uint64_t dims[THOR_B200_MAX_RANK];
    uint8_t reduced[THOR_B200_MAX_RANK]; /* 1 = the axis is reduced */
    uint64_t strides[THOR_B200_MAX_RANK]; /* element strides of the view: any values, 0 (broadcast) and overlapping included;
                                           * `input` points at the view's first element */
} thor_b200_strided_reduce_desc;

THOR_B200_API int thor_b200_strided_reduce_launch(const thor_b200_strided_reduce_desc* desc, const void* input, void* output, float output_scale,
                                                  void* stream);

/* ---------------------------------------------------------------------------------------------
 * Backward of a dense min / max reduction.
 * Replaces the three steps the reference stamps for it (StampedEquation.h:1143-1179): zero-fill of
 * the input gradient, the arg reduction that finds each segment's winner, and
 * launchReduceMinMaxBackwardScatter (Utilities/Expression/ReduceMinMaxBackwardKernel.h:28-34).
 * input is [outer, reduction, inner] dense, grad_output [outer, inner], grad_input
 * [outer, reduction, inner]: the winner of every (outer, inner) segment -- arg-reduction rule: NaN
 * beats numbers, lowest index among equals -- receives the segment's gradient (converted through
 * fp32), every other element exactly zero.  Two kernels: the arg reduction (reads input once) and a
 * streaming route kernel (writes grad_input once, reading only winners and gradients).
 * workspace_bytes covers the arg reduction's workspace plus outer * inner uint32 winners.
 * ------------------------------------------------------------------------------------------- */
typedef struct thor_b200_minmax_backward_desc {
    int32_t is_max;            /* 0 = backward of a min reduction, 1 = of a max reduction */
    int32_t input_dtype;       /* fp8 / fp16 / bf16 / fp32: dtype of the forward input */
    int32_t grad_output_dtype; /* fp16 / bf16 / fp32 */
    int32_t grad_input_dtype;  /* fp16 / bf16 / fp32 */
    uint64_t outer, reduction, inner;
    int32_t grad_mode;         /* 0: grad_output holds outer * inner values; 1: one value for every segment; 2: no tensor, grad_value is used */
    float grad_value;          /* grad_mode 2: the gradient of every segment (the default seed 1 of a backward pass) */
} thor_b200_minmax_backward_desc;

typedef struct thor_b200_minmax_backward_plan thor_b200_minmax_backward_plan;

THOR_B200_API int thor_b200_minmax_backward_plan_create(const thor_b200_minmax_backward_desc* desc, thor_b200_minmax_backward_plan** out_plan,
                                                        size_t* workspace_bytes);
THOR_B200_API int thor_b200_minmax_backward_launch(const thor_b200_minmax_backward_plan* plan, const void* input, const void* grad_output,
                                                   void* grad_input, void* workspace, size_t workspace_bytes, void* stream);
THOR_B200_API void thor_b200_minmax_backward_plan_destroy(thor_b200_minmax_backward_plan* plan);

/* ---------------------------------------------------------------------------------------------
 * Flat scatter-add without atomics (the step behind arg scans in scan min / max backward)
 * Replaces prepareFlatScatterAdd / runFlatScatterAdd (Utilities/Expression/FlatScatterAddKernel.h:16-74; caller
 * StampedScanMinMaxBackward::runOn, Utilities/Expression/StampedEquation.cpp:3134-3137).
 *   output[:] = 0;  for i in [0, num_updates): dst = indices[i];
 *                   if dst != 0xFFFFFFFF and dst < output_numel: output[dst] += updates[i]
 * THOR_B200_SCATTER_CANONICALIZE (CanonicalizeDuplicatesAndSkipInvalid): duplicate destinations are summed and invalid
 * ones skipped; the sum of a destination's updates is taken in the order of their positions i, so the result equals the
 * sequential loop above bit for bit and is the same on every run (no atomics).  THOR_B200_SCATTER_UNIQUE_VALID
 * (IndicesAreUniqueAndValid): the caller guarantees in-range, non-sentinel, pairwise different destinations; no
 * workspace is used.  fp32 updates and output, uint32 indices (what the reference supports); num_updates < 2^31.
 * The workspace size depends on num_updates only; launch() allocates nothing and does not synchronise.
 * ------------------------------------------------------------------------------------------- */
enum { THOR_B200_SCATTER_CANONICALIZE = 0, THOR_B200_SCATTER_UNIQUE_VALID = 1 };

typedef struct thor_b200_scatter_add_desc {
    int32_t value_dtype;  /* THOR_B200_FP32 */
    int32_t index_policy; /* THOR_B200_SCATTER_* */
    uint64_t num_updates;
    uint64_t output_numel;
} thor_b200_scatter_add_desc;

THOR_B200_API int thor_b200_scatter_add_workspace_bytes(const thor_b200_scatter_add_desc* desc, size_t* bytes);
THOR_B200_API int thor_b200_scatter_add_launch(const thor_b200_scatter_add_desc* desc, const void* updates, const void* indices, void* output,
                                               void* workspace, size_t workspace_bytes, void* stream);
/* Kernels one launch() issues (the zero fill is a memset, not a kernel). */
THOR_B200_API int thor_b200_scatter_add_launch_count(const thor_b200_scatter_add_desc* desc);

/* ---------------------------------------------------------------------------------------------
 * Row programs: "elementwise -> row reduction -> elementwise" chains as ONE single-pass kernel.
 * No counterpart in the reference, which makes every reduction a stage boundary
 * (EquationCompiler.cpp:684-688) and therefore runs a composed softmax as 4 kernels and a composed
 * LayerNorm through materialised fp32 temporaries.  A row program takes the same SSA node list as
 * thor_b200_expr_compile, extended with REDUCE_* nodes, over tensors that are [rows, cols] (FULL),
 * [rows, 1] (ROW), [cols] (COL) or one element (SCALAR):
 *   - REDUCE_{SUM,AVG,MIN,MAX,PROD,NORM1,NORM2} with input_slot = 0 reduces along the columns of a FULL
 *     value and yields a ROW value that later nodes may consume (softmax max / sum, mean, variance);
 *   - REDUCE_{SUM,AVG} with input_slot = 1 reduces along the rows of a FULL value and yields a COL value
 *     that must be an output (LayerNorm dgamma / dbeta): persistent CTAs keep per-column fp32
 *     partials in registers, write them to the workspace and a second kernel folds them in order;
 *   - REDUCE_* with input_slot = 2 reduces over ALL rows * cols elements and must be an output; a program
 *     made only of such reductions (e.g. sum, sum of squares and max of one tensor) reads its inputs
 *     once for all of them: the single-pass replacement of several DeviceTransformReduce calls plus
 *     the materialised elementwise stages in front of them.
 * One CTA (or one warp for short rows) owns a row, keeps it in registers, and every node keeps the
 * per-node dtype rule of the fused stages; reductions convert to fp32, accumulate in fp32 and
 * round once to the node's output dtype, like the reduction seam.
 * ------------------------------------------------------------------------------------------- */
typedef enum thor_b200_row_shape {
    THOR_B200_SHAPE_FULL = 0, THOR_B200_SHAPE_ROW = 1, THOR_B200_SHAPE_COL = 2, THOR_B200_SHAPE_SCALAR = 3
} thor_b200_row_shape;

/* How a persistent row program (per-column operands or column reductions) moves its rows.  All zero = the measured
 * defaults; every combination computes the same values (the layouts differ in how operands reach the registers and
 * in which barriers are shared, not in the arithmetic), which the tests use to compare them bit for bit. */
typedef struct thor_b200_rowprog_tuning {
    int32_t ring_buffers;        /* rows arrive by bulk copies in a ring of shared-memory buffers: 0 = default, -1 = off
                                  * (register double buffer), -2 = as many as fit, n >= 3 = at most n buffers */
    int32_t pipeline_round_one;  /* round 1 of the next row shares the last round of the current row: 0 = default, 1 = on, -1 = off */
    int32_t copy_warpgroup;      /* ring mode: the copies are requested by a warpgroup of their own instead of a team thread: 0 = default, 1 = on, -1 = off */
    int32_t keep_values;         /* transcendental element values needed by several loops stay in registers: 0 = default (on), -1 = off */
    int32_t reciprocal_division; /* x / row value as x * (1 / row value): 0 = default (only with use_fast_math), 1 = on, -1 = off */
    int32_t wait_limit_ms;       /* time limit of a wait on a ring buffer's barrier; 0 = two seconds */
    int32_t test_skip_fill;      /* tests of the bounded waits only: n > 0 makes CTA 0's code lack the copy request of loop
                                  * iteration n, so the wait for that buffer runs out; 0 = none */
    int32_t reserve_sms;         /* persistent programs leave this many SMs without a CTA, for a kernel that has to run beside
                                  * them (the allreduce of the previous step's partials on another stream): 0 = none */
} thor_b200_rowprog_tuning;

typedef struct thor_b200_rowprog_desc {
    const thor_b200_expr_node* nodes;
    uint32_t n_nodes;
    const thor_b200_expr_input* inputs;
    const int32_t* input_shapes; /* thor_b200_row_shape per input (ignored for fp32 runtime scalars) */
    uint32_t n_inputs;
    const thor_b200_expr_output* outputs;
    uint32_t n_outputs;
    uint64_t rows, cols;
    thor_b200_expr_options options;
    thor_b200_rowprog_tuning tuning;
} thor_b200_rowprog_desc;

typedef struct thor_b200_rowprog thor_b200_rowprog;

/* Returns THOR_B200_UNSUPPORTED (and leaves *out_prog NULL) when the node list is valid but does not
 * fit a row program (row too long for one CTA, a ROW value reduced again, ...): the caller then runs
 * its ordinary stage list. */
THOR_B200_API int thor_b200_rowprog_compile(const thor_b200_rowprog_desc* desc, thor_b200_rowprog** out_prog, size_t* workspace_bytes);
THOR_B200_API int thor_b200_rowprog_launch(thor_b200_rowprog* prog, const void* const* input_ptrs, const float* runtime_scalars,
                                           void* const* output_ptrs, void* workspace, size_t workspace_bytes, void* stream);
/* The same launch for a caller that holds only a SHARD of the rows (rows split across GPUs): column_sums_f32, when not
 * NULL, receives the program's column reductions unrounded, fp32 [number of column reductions][cols] in the order of the
 * program's outputs, next to the rounded outputs.  The caller adds the shards' sums (thor_b200_comm_allreduce_f32) and
 * rounds once, instead of adding values that were already rounded to a 16-bit output dtype.  A mean over rows divides
 * by this program's own row count.  No counterpart in the reference, which is single-GPU on this path. */
THOR_B200_API int thor_b200_rowprog_launch_sharded(thor_b200_rowprog* prog, const void* const* input_ptrs, const float* runtime_scalars,
                                                   void* const* output_ptrs, void* workspace, size_t workspace_bytes, void* column_sums_f32,
                                                   void* stream);
THOR_B200_API const char* thor_b200_rowprog_source(const thor_b200_rowprog* prog);
/* Kernels one launch of the program runs (1, or 2 when column reductions need the fold kernel). */
THOR_B200_API uint32_t thor_b200_rowprog_launch_count(const thor_b200_rowprog* prog);
/* Programs whose rows arrive by bulk copies wait on shared-memory barriers; every such wait has a time limit, and a
 * wait that ran out is counted on the device instead of hanging the kernel.  Synchronises with the device and
 * stores the count since the program was loaded (0 for programs without such waits, or never launched); a
 * non-zero count means the outputs of the launches so far are not to be trusted, and once this call has reported one
 * the handle refuses further launches (THOR_B200_CUDA_ERROR): find the cause and compile the program again. */
THOR_B200_API int thor_b200_rowprog_waits_expired(thor_b200_rowprog* prog, uint32_t* count);
THOR_B200_API void thor_b200_rowprog_destroy(thor_b200_rowprog* prog);

/* ---------------------------------------------------------------------------------------------
 * Full reduction for callers that cannot allocate.  It has no counterpart in the reference, whose
 * reductions always stamp a workspace first (CubReduction::stampValidated).
 *
 * Reduces the n elements of `input` (one dense vector) to a single value in `output`, with the same
 * arithmetic as thor_b200_reduce_launch for outer = inner = 1.  The scratch the two-phase reduction
 * needs is a fixed 256 KiB array inside the library instead of a caller workspace, so the call
 * performs no cudaMalloc / cudaFree and uses no allocating library routine.  It exists for callers
 * that have no point at which they could allocate: a process that distributed all of its device memory
 * at start-up, a plug-in whose host application forbids it the allocator, a latency-critical loop that
 * must not hit cudaMalloc's device-wide synchronisation.
 *
 * Limit: at most 65536 partials, i.e. n <= 65536 * 4096 * (16 / element size) elements (2^30 for fp32,
 * 2^31 for fp16 / bf16, 2^32 for fp8); larger inputs are rejected with THOR_B200_INVALID_ARGUMENT.
 * The first call on each device looks up the array's device address; make that first call before
 * any stream capture begins, and do not use the entry point on a device after cudaDeviceReset.  All calls on a device share the one array: two calls whose kernels can
 * overlap on the GPU (different streams, no dependency) race on it and must be ordered by the caller.
 * ------------------------------------------------------------------------------------------- */
THOR_B200_API int thor_b200_reduce_full_noalloc(int op, const void* input, int input_dtype, uint64_t n, void* output, int output_dtype,
                                                float output_scale, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Multi-GPU: the one collective of the path.  Rows / flat ranges shard across GPUs without any
 * communication; only values reduced over the sharded dimension (full reductions, LayerNorm
 * dgamma / dbeta column sums) are combined, with one in-place fp32 allreduce of the per-GPU
 * partials over NCCL (one process per GPU).  No counterpart in the reference, which is single-GPU
 * on this path.  NCCL is loaded at run time (libnccl.so.2, or $THOR_B200_NCCL_LIB); rank 0 obtains
 * the 128-byte id and hands it to the other ranks by any host channel.
 * ------------------------------------------------------------------------------------------- */
typedef struct thor_b200_comm thor_b200_comm;
THOR_B200_API int thor_b200_comm_unique_id(void* out_id_128_bytes);
THOR_B200_API int thor_b200_comm_init(int nranks, int rank, const void* unique_id_128_bytes, thor_b200_comm** out_comm);
/* op: 0 = sum, 1 = max, 2 = min (NCCL's floating-point min / max: what they return when a shard holds a NaN is not
 * specified -- use thor_b200_comm_allreduce_stats_f32 for extremes).  Asynchronous on `stream`; every rank must make the
 * same calls in the same order. */
THOR_B200_API int thor_b200_comm_allreduce_f32(thor_b200_comm* comm, void* buffer, uint64_t count, int op, void* stream);
/* The statistics of one sharded reduction step in ONE NCCL group (ncclGroupStart / ncclGroupEnd): `sums` (n_sums fp32:
 * sum, sum of squares, column sums ...) combined with +, `maxima` with max, `minima` with min, each in place; a count of 0
 * skips that part.  Minima and maxima follow the reduction seam's rule that a NaN in any shard is the result (NCCL's own
 * floating-point min / max leave that open): they cross the ranks as order-preserving integer keys in which NaN wins.
 * Asynchronous on `stream`; every rank makes the same call. */
THOR_B200_API int thor_b200_comm_allreduce_stats_f32(thor_b200_comm* comm, void* sums, uint64_t n_sums, void* maxima, uint64_t n_maxima, void* minima,
                                                     uint64_t n_minima, void* stream);
/* Overlapped combine for a stepping job: the statistics of step i cross the ranks on a high-priority stream of the
 * combiner's own while the kernel of step i + 1 runs.  The caller keeps `slots` copies of its partial buffers and uses
 * slot i % slots in step i:
 *     thor_b200_combiner_wait(c, slot, stream);      -- the kernel may overwrite the slot's partials only after their last combine
 *     ... launch the step's kernels on `stream` ...
 *     thor_b200_combiner_submit(c, slot, stream, sums, n_sums, maxima, n_maxima, minima, n_minima, rounded_sums, dtype);
 * submit orders the combine behind everything `stream` holds so far, runs thor_b200_comm_allreduce_stats_f32 and then,
 * when rounded_sums is not NULL, converts the combined fp32 sums to `rounded_dtype` there (the single rounding of a
 * sharded column sum).  thor_b200_combiner_drain makes `stream` wait for every combine submitted so far.  No call
 * blocks the host or allocates after create. */
typedef struct thor_b200_combiner thor_b200_combiner;
THOR_B200_API int thor_b200_combiner_create(thor_b200_comm* comm, int slots, thor_b200_combiner** out_combiner);
THOR_B200_API int thor_b200_combiner_wait(thor_b200_combiner* combiner, int slot, void* stream);
THOR_B200_API int thor_b200_combiner_submit(thor_b200_combiner* combiner, int slot, void* producer_stream, void* sums, uint64_t n_sums, void* maxima,
                                            uint64_t n_maxima, void* minima, uint64_t n_minima, void* rounded_sums, int rounded_dtype);
THOR_B200_API int thor_b200_combiner_drain(thor_b200_combiner* combiner, void* stream);
/* The combiner's own stream (cudaStream_t), e.g. to time the collective alone. */
THOR_B200_API void* thor_b200_combiner_stream(thor_b200_combiner* combiner);
THOR_B200_API void thor_b200_combiner_destroy(thor_b200_combiner* combiner);
THOR_B200_API void thor_b200_comm_destroy(thor_b200_comm* comm);

#ifdef __cplusplus
}
#endif

#endif /* THOR_B200_H */
