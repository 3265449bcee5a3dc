// Lazy tensor-expression DAG with the reference's public surface
// (Utilities/Expression/Expression.h:231-407, 516-1075): Expression::input / runtimeScalar /
// operators / math methods / reductions / Expression::outputs.  Only the ops that belong to the
// elementwise + reduction + cast hot path exist here; matmul, attention, convolution, scans and
// ragged ops stay with the reference.
#pragma once

#include <cstdint>
#include <memory>
#include <optional>
#include <string>
#include <utility>
#include <vector>

#include "DataType.h"

namespace ThorB200 {

// Integer values equal ThorImplementation::ExprOp (Expression.h:32-148).
enum class ExprOp : uint16_t {
    INPUT = 3, RUNTIME_SCALAR, TENSOR_RUNTIME_SCALAR, SCALAR_FP, ADD, SUB, MUL, DIV, POW, EQUAL, NOT_EQUAL, LESS, LESS_EQUAL, GREATER,
    GREATER_EQUAL, LOGICAL_AND, LOGICAL_OR, LOGICAL_NOT, CAST, WHERE, NEG, ABS, CEIL, FLOOR, ROUND, TRUNC, SIN, COS, TAN, ASIN, ACOS, ATAN,
    SINH, COSH, ASINH, ACOSH, ATANH, ERF, ERFC, ERFCX, ERFINV, ERFCINV, TGAMMA, LGAMMA, DIGAMMA, EXP, EXPM1, EXP2, EXP10, LN, LOG1P, LOG2,
    LOG10, SQRT, TANH, NORMCDF,
    SOFTMAX = 60,  // never stored in a graph: Expression::softmax / logSoftmax build the composite directly
    RESHAPE = 62, UNSQUEEZE = 65, SQUEEZE = 66,
    MIN = 69, MAX, MIN_GRAD_LEFT, MIN_GRAD_RIGHT, MAX_GRAD_LEFT, MAX_GRAD_RIGHT,
    REDUCE_SUM = 83, REDUCE_PROD, REDUCE_MIN, REDUCE_MAX, REDUCE_ARGMIN, REDUCE_ARGMAX,
    REDUCE_MIN_BACKWARD = 89, REDUCE_MAX_BACKWARD = 90,  // lhs = forward input, rhs = gradient of the reduced value
    REDUCE_AVG = 95, REDUCE_NORM1, REDUCE_NORM2,
};

inline bool isValueReductionOp(ExprOp op) {
    return op == ExprOp::REDUCE_SUM || op == ExprOp::REDUCE_PROD || op == ExprOp::REDUCE_MIN || op == ExprOp::REDUCE_MAX ||
           op == ExprOp::REDUCE_AVG || op == ExprOp::REDUCE_NORM1 || op == ExprOp::REDUCE_NORM2;
}
inline bool isArgReductionOp(ExprOp op) { return op == ExprOp::REDUCE_ARGMIN || op == ExprOp::REDUCE_ARGMAX; }
inline bool isReductionOp(ExprOp op) { return isValueReductionOp(op) || isArgReductionOp(op); }
inline bool isMinMaxBackwardOp(ExprOp op) { return op == ExprOp::REDUCE_MIN_BACKWARD || op == ExprOp::REDUCE_MAX_BACKWARD; }
inline bool isViewOp(ExprOp op) { return op == ExprOp::RESHAPE || op == ExprOp::UNSQUEEZE || op == ExprOp::SQUEEZE; }
inline bool isScalarLeafOp(ExprOp op) { return op == ExprOp::SCALAR_FP || op == ExprOp::RUNTIME_SCALAR || op == ExprOp::TENSOR_RUNTIME_SCALAR; }
inline bool isLeafOp(ExprOp op) { return op == ExprOp::INPUT || isScalarLeafOp(op); }
inline bool isComparisonOp(ExprOp op) { return op >= ExprOp::EQUAL && op <= ExprOp::GREATER_EQUAL; }
inline bool isLogicalOp(ExprOp op) { return op == ExprOp::LOGICAL_AND || op == ExprOp::LOGICAL_OR || op == ExprOp::LOGICAL_NOT; }
inline bool isBinaryOp(ExprOp op) {
    return (op >= ExprOp::ADD && op <= ExprOp::LOGICAL_OR) || (op >= ExprOp::MIN && op <= ExprOp::MAX_GRAD_RIGHT);
}
const char* opName(ExprOp op);

// Sentinel reduction-axis list {kAxesFromOne}: every axis except the first (the "instance" mode of
// the softmax op, whose rank is known only when shapes are bound).
constexpr uint64_t kAxesFromOne = UINT64_MAX - 1;

// Sentinel squeeze list meaning "squeeze every singleton axis" (StampedEquation.cpp:4308-4363).
constexpr uint64_t kSqueezeAll = UINT64_MAX;

struct ExprNode {
    ExprOp op = ExprOp::INPUT;
    uint32_t lhs = UINT32_MAX;
    uint32_t rhs = UINT32_MAX;
    uint32_t aux = UINT32_MAX;  // WHERE: false branch.  CAST before dtype resolution: node whose output dtype the cast takes
    uint32_t input_slot = UINT32_MAX;
    double scalar_fp = 0.0;
    std::optional<DataType> input_tensor_dtype;  // INPUT / *_RUNTIME_SCALAR: dtype of the bound value (filled at resolution)
    std::optional<DataType> output_dtype;
    std::optional<DataType> compute_dtype;
    std::vector<uint64_t> reduction_axes;  // empty = all axes
    std::vector<uint64_t> squeeze_axes;    // reductions / SQUEEZE
    std::vector<uint64_t> unsqueeze_axes;  // UNSQUEEZE
    std::vector<uint64_t> reshape_dims;    // RESHAPE
    bool stop_gradient = false;            // autodiff treats the node as a constant (the shift term of softmax)
};

// Which axes of a rank-`rank` operand the reduction node reduces (empty list = all axes).
std::vector<bool> reducedAxesMask(const ExprNode& reduction, size_t rank);

// cudnnSoftmaxAlgorithm_t / cudnnSoftmaxMode_t values, which the reference's softmax op takes (Expression.h:736-738).
enum class SoftmaxAlgorithm : int { FAST = 0, ACCURATE = 1, LOG = 2 };
enum class SoftmaxMode : int { INSTANCE = 0, CHANNEL = 1 };

struct NamedInput {
    enum class Kind : uint8_t { Tensor, RuntimeScalarFp32, TensorRuntimeScalar };
    std::string name;
    uint32_t slot = 0;
    Kind kind = Kind::Tensor;
};

struct NamedOutput {
    std::string name;
    uint32_t node_idx = 0;
};

struct PhysicalExpression {
    std::vector<ExprNode> nodes;
    std::vector<NamedInput> inputs;
};

struct PhysicalOutputs {
    std::shared_ptr<PhysicalExpression> expr;
    std::vector<NamedOutput> outputs;
};

class Outputs;

class Expression {
   public:
    Expression(double value);  // NOLINT: scalar literals convert implicitly, as in the reference

    static Expression input(const std::string& name, std::optional<DataType> compute_dtype = std::nullopt,
                            std::optional<DataType> output_dtype = std::nullopt);
    static Expression runtimeScalar(const std::string& name, std::optional<DataType> compute_dtype = std::nullopt,
                                    std::optional<DataType> output_dtype = std::nullopt);
    static Expression tensorRuntimeScalar(const std::string& name, std::optional<DataType> compute_dtype = std::nullopt,
                                          std::optional<DataType> output_dtype = std::nullopt);
    static Expression constantScalar(double value) { return Expression(value); }
    static Outputs outputs(const std::vector<std::pair<std::string, Expression>>& named_exprs);

    Expression operator+(const Expression& o) const { return binary(ExprOp::ADD, o); }
    Expression operator-(const Expression& o) const { return binary(ExprOp::SUB, o); }
    Expression operator*(const Expression& o) const { return binary(ExprOp::MUL, o); }
    Expression operator/(const Expression& o) const { return binary(ExprOp::DIV, o); }
    Expression operator-() const { return unary(ExprOp::NEG); }
    Expression operator!() const { return unary(ExprOp::LOGICAL_NOT); }
    Expression operator==(const Expression& o) const { return binary(ExprOp::EQUAL, o); }
    Expression operator!=(const Expression& o) const { return binary(ExprOp::NOT_EQUAL, o); }
    Expression operator<(const Expression& o) const { return binary(ExprOp::LESS, o); }
    Expression operator<=(const Expression& o) const { return binary(ExprOp::LESS_EQUAL, o); }
    Expression operator>(const Expression& o) const { return binary(ExprOp::GREATER, o); }
    Expression operator>=(const Expression& o) const { return binary(ExprOp::GREATER_EQUAL, o); }
    Expression logicalAnd(const Expression& o) const { return binary(ExprOp::LOGICAL_AND, o); }
    Expression logicalOr(const Expression& o) const { return binary(ExprOp::LOGICAL_OR, o); }
    Expression logicalNot() const { return unary(ExprOp::LOGICAL_NOT); }
    Expression cast(DataType output_dtype) const;
    static Expression where(const Expression& condition, const Expression& true_value, const Expression& false_value);

    Expression pow(const Expression& e) const { return binary(ExprOp::POW, e); }
    Expression min(const Expression& o) const { return binary(ExprOp::MIN, o); }
    Expression max(const Expression& o) const { return binary(ExprOp::MAX, o); }
    Expression abs() const { return unary(ExprOp::ABS); }
    Expression ceil() const { return unary(ExprOp::CEIL); }
    Expression floor() const { return unary(ExprOp::FLOOR); }
    Expression round() const { return unary(ExprOp::ROUND); }
    Expression trunc() const { return unary(ExprOp::TRUNC); }
    Expression sin() const { return unary(ExprOp::SIN); }
    Expression cos() const { return unary(ExprOp::COS); }
    Expression tan() const { return unary(ExprOp::TAN); }
    Expression asin() const { return unary(ExprOp::ASIN); }
    Expression acos() const { return unary(ExprOp::ACOS); }
    Expression atan() const { return unary(ExprOp::ATAN); }
    Expression sinh() const { return unary(ExprOp::SINH); }
    Expression cosh() const { return unary(ExprOp::COSH); }
    Expression asinh() const { return unary(ExprOp::ASINH); }
    Expression acosh() const { return unary(ExprOp::ACOSH); }
    Expression atanh() const { return unary(ExprOp::ATANH); }
    Expression erf() const { return unary(ExprOp::ERF); }
    Expression erfc() const { return unary(ExprOp::ERFC); }
    Expression erfcx() const { return unary(ExprOp::ERFCX); }
    Expression erfinv() const { return unary(ExprOp::ERFINV); }
    Expression erfcinv() const { return unary(ExprOp::ERFCINV); }
    Expression tgamma() const { return unary(ExprOp::TGAMMA); }
    Expression lgamma() const { return unary(ExprOp::LGAMMA); }
    Expression digamma() const { return unary(ExprOp::DIGAMMA); }
    Expression exp() const { return unary(ExprOp::EXP); }
    Expression expm1() const { return unary(ExprOp::EXPM1); }
    Expression exp2() const { return unary(ExprOp::EXP2); }
    Expression exp10() const { return unary(ExprOp::EXP10); }
    Expression ln() const { return unary(ExprOp::LN); }
    Expression log1p() const { return unary(ExprOp::LOG1P); }
    Expression log2() const { return unary(ExprOp::LOG2); }
    Expression log10() const { return unary(ExprOp::LOG10); }
    Expression sqrt() const { return unary(ExprOp::SQRT); }
    Expression tanh() const { return unary(ExprOp::TANH); }
    Expression normcdf() const { return unary(ExprOp::NORMCDF); }

    // Stable composites, spelled exactly as the reference spells them (Expression.h:1077-1115).
    Expression sigmoid() const;
    Expression softplus() const;
    Expression elu(double alpha = 1.0) const;
    Expression selu() const;
    Expression gelu() const;
    Expression swish() const;
    Expression relu() const { return max(Expression(0.0)); }  // DeepLearning/Api/Layers/Activations/Relu.h:21-22
    Expression relu6() const;
    Expression hardTanh(double min_value = -1.0, double max_value = 1.0) const;
    Expression clamp(double lower_bound, double upper_bound) const;

    // Softmax over axis 1 (CHANNEL) or over every axis but the first (INSTANCE), computed in fp32 and stored in
    // the operand's dtype (Expression.cpp:3724-3748).  The reference hands this op to cuDNN as a stage of its own;
    // here it is the composite max / exp / sum / divide, which the planner runs as one row program.
    Expression softmax(SoftmaxAlgorithm algorithm = SoftmaxAlgorithm::ACCURATE, SoftmaxMode mode = SoftmaxMode::CHANNEL) const;
    Expression logSoftmax(SoftmaxMode mode = SoftmaxMode::CHANNEL) const;

    Expression reshape(const std::vector<uint64_t>& new_dims) const;
    Expression unsqueeze(const std::vector<uint64_t>& axes) const;
    Expression squeeze(const std::vector<uint64_t>& axes) const;

    Expression reduction(ExprOp op, const std::vector<uint64_t>& reduction_axes, const std::vector<uint64_t>& squeeze_axes,
                         std::optional<DataType> compute_dtype) const;
#define THOR_B200_REDUCTION(NAME, OP)                                                                                       \
    Expression NAME(const std::vector<uint64_t>& reduction_axes = {}, const std::vector<uint64_t>& squeeze_axes = {},      \
                    std::optional<DataType> compute_dtype = std::nullopt) const {                                          \
        return reduction(ExprOp::OP, reduction_axes, squeeze_axes, compute_dtype);                                         \
    }
    THOR_B200_REDUCTION(reduce_sum, REDUCE_SUM)
    THOR_B200_REDUCTION(reduce_prod, REDUCE_PROD)
    THOR_B200_REDUCTION(reduce_min, REDUCE_MIN)
    THOR_B200_REDUCTION(reduce_max, REDUCE_MAX)
    THOR_B200_REDUCTION(reduce_mean, REDUCE_AVG)
    THOR_B200_REDUCTION(reduce_norm1, REDUCE_NORM1)
    THOR_B200_REDUCTION(reduce_norm2, REDUCE_NORM2)
    THOR_B200_REDUCTION(argmin, REDUCE_ARGMIN)
    THOR_B200_REDUCTION(argmax, REDUCE_ARGMAX)
#undef THOR_B200_REDUCTION
    // Gradient of a min / max reduction with respect to its input: the winner of every reduced segment (arg-reduction
    // rule) receives that segment's gradient, everything else zero (AutoDiff.cpp:5036-5050).  `forward_input` is the
    // tensor that was reduced, `grad` has the shape of the reduction's result.
    static Expression reduceMinMaxBackward(ExprOp op, const Expression& forward_input, const Expression& grad, const std::vector<uint64_t>& reduction_axes,
                                           const std::vector<uint64_t>& squeeze_axes);
    // Request a storage dtype for this node's value (reductions default to FP32, ExpressionDTypeResolution.cpp:777-791).
    Expression withOutputDType(DataType dtype) const;

    const std::shared_ptr<PhysicalExpression>& graph() const { return expr_; }
    uint32_t nodeIndex() const { return node_; }
    static Expression fromPhysicalNode(std::shared_ptr<PhysicalExpression> expr, uint32_t node) { return Expression(std::move(expr), node); }

   private:
    Expression(std::shared_ptr<PhysicalExpression> e, uint32_t n) : expr_(std::move(e)), node_(n) {}
    Expression unary(ExprOp op) const;
    Expression binary(ExprOp op, const Expression& other) const;

    std::shared_ptr<PhysicalExpression> expr_;
    uint32_t node_ = 0;
};

inline Expression operator+(double a, const Expression& b) { return Expression(a) + b; }
inline Expression operator-(double a, const Expression& b) { return Expression(a) - b; }
inline Expression operator*(double a, const Expression& b) { return Expression(a) * b; }
inline Expression operator/(double a, const Expression& b) { return Expression(a) / b; }

class Outputs {
   public:
    Outputs() = default;
    Outputs(std::shared_ptr<PhysicalExpression> expr, std::vector<NamedOutput> outputs) : expr_(std::move(expr)), outputs_(std::move(outputs)) {}
    const std::shared_ptr<PhysicalExpression>& expression() const { return expr_; }
    const std::vector<NamedOutput>& namedOutputs() const { return outputs_; }
    PhysicalOutputs physicalOutputs() const { return PhysicalOutputs{expr_, outputs_}; }

   private:
    std::shared_ptr<PhysicalExpression> expr_;
    std::vector<NamedOutput> outputs_;
};

// Appends `src` node `node` (with its ancestors) to `dst`, sharing structurally identical nodes and
// inputs of the same name; returns the index in dst.
uint32_t mergeInto(PhysicalExpression& dst, const PhysicalExpression& src, uint32_t node);

// Per-node output / compute dtype assignment for concrete input dtypes (indexed by input slot),
// following ExpressionDTypeResolution.cpp:1012-1148; materialized_output_nodes seed the backward
// compute-dtype propagation (:885-1010).
void resolveOutputsDTypesInPlace(PhysicalOutputs& outputs, const std::vector<DataType>& root_input_dtypes);
DataType promoteTensorValueDTypes(DataType a, DataType b);
DataType toSupportedComputeDType(ExprOp op, DataType requested);

}  // namespace ThorB200
