// FusedEquation / StampedExecutionPlan with the reference's call surface
// (Utilities/Expression/FusedEquation.cpp:7014-7043 compile, :8885 stamp, :10760-10902 run;
// Utilities/Expression/StampedEquation.h:1549-1777 plan).  compile() records the outputs; the
// first stamp() with real tensors resolves dtypes, splits the DAG into stages at reduction
// boundaries (EquationCompiler.cpp:684-688, 6572), compiles the fused stages through the C ABI,
// allocates intermediates and outputs, and returns a plan whose run() launches without allocating.
#pragma once

#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "Expression.h"
#include "Tensor.h"

struct thor_b200_expr;
struct thor_b200_reduce_plan;
struct thor_b200_argreduce_plan;

namespace ThorB200 {

// A bound runtime value: a tensor, or an fp32 scalar passed by value (Expression::runtimeScalar).
struct RuntimeInputValue {
    Tensor tensor;
    float scalar = 0.0f;
    bool is_scalar = false;
    RuntimeInputValue() = default;
    RuntimeInputValue(const Tensor& t) : tensor(t) {}                // NOLINT
    RuntimeInputValue(float v) : scalar(v), is_scalar(true) {}       // NOLINT
    RuntimeInputValue(double v) : scalar(static_cast<float>(v)), is_scalar(true) {}  // NOLINT
};

enum class StageKind { FusedKernel, Reduction, ArgMinMax, View, FusedRows, ReduceMinMaxBackward };

// Layout choices of persistent row programs (thor_b200_rowprog_tuning of the C ABI, field for field); all zero = the
// measured defaults.  Every combination computes the same values.
struct RowProgramTuning {
    int ring_buffers = 0;
    int pipeline_round_one = 0;
    int copy_warpgroup = 0;
    int keep_values = 0;
    int reciprocal_division = 0;
    int wait_limit_ms = 0;
    int test_skip_fill = 0;
    int reserve_sms = 0;
};

struct FusedEquationOptions {
    bool use_fast_math = false;
    RowProgramTuning row_program;
    // For callers that hold one SHARD of the rows (rows split across GPUs): a row program with column reductions (LayerNorm
    // dgamma / dbeta) also delivers those sums unrounded, as the fp32 output "__column_sums" of shape [reductions, cols]
    // in the order of columnSumNames(), so that the shards' sums can be added before the single rounding to the gradient's
    // dtype.  The reference is single-GPU on this path and has no counterpart.
    bool unrounded_column_sums = false;
    // Stages that do not depend on each other run on helper streams joined by events, like the reference's stamped plans.
    bool branch_streams = true;
    // Joining lanes costs a few event records and waits per run (about 4 us measured), which only pays when the stages
    // are long: plans whose tensor inputs hold fewer bytes than this run on the caller's stream alone.  0 = always
    // use the lanes.  The lane assignment itself (stageLanes()) does not depend on it.
    uint64_t branch_streams_min_input_bytes = 64ull << 20;
    // Execute "elementwise -> row reduction -> elementwise" chains over the innermost axis (softmax,
    // LayerNorm forward / backward) as one single-pass kernel instead of the reference's stage list.
    // The logical stage list is still reported by stageKindNames().
    bool fuse_row_reductions = true;
};

class StampedExecutionPlan {
   public:
    struct Impl;
    StampedExecutionPlan() = default;
    explicit StampedExecutionPlan(std::shared_ptr<Impl> impl) : impl_(std::move(impl)) {}

    // Launches every stage on the stamped stream.  No allocation, no planning, no compilation.
    void run();
    void runOn(const Stream& stream);
    Tensor getOutput(const std::string& name) const;
    std::vector<std::string> getOutputNames() const;
    void setRuntimeScalar(const std::string& name, float value);

    // Logical stage list in execution order: "FusedKernel", "Reduction", "ArgMinMax", "View"
    // (StampedExecutionPlan::stageKindNames, StampedEquation.h:1683-1711).
    std::vector<std::string> stageKindNames() const;
    // What actually launches: kernel shape per physical stage ("bcast_tiled_v2", "rows_cta", "softmax_rows" ...).
    std::vector<std::string> physicalStageNames() const;
    // Emitted CUDA source of the fused stages (empty string for library stages).
    std::vector<std::string> stageSources() const;
    uint64_t intermediateBytes() const;
    uint64_t kernelLaunchesPerRun() const;
    // Kernels that wait on device-side barriers bound every wait in time; this is how many such waits ran out in the
    // launches so far (synchronises with the device).  Anything but 0 means the outputs are not to be trusted.
    uint64_t waitsExpired() const;
    // Names of the outputs whose unrounded sums the rows of "__column_sums" hold (empty unless the equation was compiled
    // with unrounded_column_sums and runs as a row program with column reductions).
    std::vector<std::string> columnSumNames() const;
    // Lane of every physical stage: 0 = the caller's stream, 1.. = helper streams for branches that do not depend on
    // each other (StampedExecutionPlan::runOn, StampedEquation.cpp:4057-4205; lane policy StampedEquation.h:1634-1646).
    std::vector<uint32_t> stageLanes() const;

   private:
    std::shared_ptr<Impl> impl_;
};

class FusedEquation {
   public:
    static FusedEquation compile(const Outputs& outputs, int device_num = 0, FusedEquationOptions options = {});
    static FusedEquation compile(const Expression& expr, int device_num = 0, FusedEquationOptions options = {});

    // Binds inputs (by name), plans, compiles and allocates.  `preallocated_outputs` adopts caller
    // tensors for the named outputs (their dtype and shape must match what the plan produces).
    StampedExecutionPlan stamp(const std::unordered_map<std::string, RuntimeInputValue>& inputs, const Stream& stream,
                               const std::unordered_map<std::string, Tensor>& preallocated_outputs = {});

    // Convenience path: single fused stage only (multi-stage reduction expressions are rejected, like
    // FusedEquation::run in the reference, FusedEquation.cpp:10760-10902).
    void run(const std::unordered_map<std::string, RuntimeInputValue>& inputs, const std::unordered_map<std::string, Tensor>& outputs,
             const Stream& stream);

    // Reverse-mode graph transform (FusedEquation::compileBackward, FusedEquation.cpp:7093-7135): returns
    // an equation whose outputs are "<wrt>_grad" for every requested input, taking the forward inputs
    // plus the upstream gradient(s) "<upstream_prefix><output name>" (one output: just upstream_prefix).
    FusedEquation compileBackward(const std::vector<std::string>& wrt_names, const std::string& upstream_prefix = "__grad_output") const;

    // The dtype-resolved SSA graph this equation evaluates for the given tensor shapes and dtypes, as JSON text: inputs by
    // slot, named outputs, and every node with its ExprOp integer, parents, literal, axes lists and resolved output /
    // compute dtypes.  For a backward equation this is the graph that stamp() differentiates for those shapes.  No GPU.
    std::string describeGraph(const std::unordered_map<std::string, std::vector<uint64_t>>& input_dims,
                              const std::unordered_map<std::string, DataType>& input_dtypes) const;

    const Outputs& outputs() const { return outputs_; }
    int deviceNum() const { return device_num_; }
    const FusedEquationOptions& options() const { return options_; }

   private:
    Outputs outputs_;
    int device_num_ = 0;
    FusedEquationOptions options_;
    // shape needed by compileBackward's sum-to-shape is bound at stamp time; backward equations keep
    // the forward graph so that the upstream/unbroadcast reductions are planned with real shapes
    struct Deferred;
    std::shared_ptr<Deferred> deferred_backward_;
    friend struct BackwardBuilder;
};

// Shape of every node for concrete input shapes (numpy-style right-aligned broadcasting; reductions
// keep reduced axes as 1 then apply squeeze_axes; StampedEquation.cpp:4308-4363).
std::vector<std::vector<uint64_t>> inferNodeShapes(const PhysicalExpression& expr, const std::vector<std::vector<uint64_t>>& input_dims);

}  // namespace ThorB200
