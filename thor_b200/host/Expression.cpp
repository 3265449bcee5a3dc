// Expression DAG builder and per-node dtype resolution of the host layer.
#include "Expression.h"

#include <algorithm>
#include <stdexcept>
#include <unordered_map>

namespace ThorB200 {

const char* opName(ExprOp op) {
    switch (op) {
        case ExprOp::INPUT: return "input"; case ExprOp::RUNTIME_SCALAR: return "runtime_scalar";
        case ExprOp::TENSOR_RUNTIME_SCALAR: return "tensor_runtime_scalar"; case ExprOp::SCALAR_FP: return "scalar";
        case ExprOp::ADD: return "add"; case ExprOp::SUB: return "sub"; case ExprOp::MUL: return "mul"; case ExprOp::DIV: return "div";
        case ExprOp::POW: return "pow"; case ExprOp::EQUAL: return "eq"; case ExprOp::NOT_EQUAL: return "ne"; case ExprOp::LESS: return "lt";
        case ExprOp::LESS_EQUAL: return "le"; case ExprOp::GREATER: return "gt"; case ExprOp::GREATER_EQUAL: return "ge";
        case ExprOp::LOGICAL_AND: return "and"; case ExprOp::LOGICAL_OR: return "or"; case ExprOp::LOGICAL_NOT: return "not";
        case ExprOp::REDUCE_MIN_BACKWARD: return "reduce_min_backward"; case ExprOp::REDUCE_MAX_BACKWARD: return "reduce_max_backward";
        case ExprOp::CAST: return "cast"; case ExprOp::WHERE: return "where"; case ExprOp::NEG: return "neg"; case ExprOp::ABS: return "abs";
        case ExprOp::EXP: return "exp"; case ExprOp::LN: return "ln"; case ExprOp::SQRT: return "sqrt"; case ExprOp::TANH: return "tanh";
        case ExprOp::MIN: return "min"; case ExprOp::MAX: return "max"; case ExprOp::RESHAPE: return "reshape";
        case ExprOp::UNSQUEEZE: return "unsqueeze"; case ExprOp::SQUEEZE: return "squeeze";
        case ExprOp::REDUCE_SUM: return "reduce_sum"; case ExprOp::REDUCE_PROD: return "reduce_prod"; case ExprOp::REDUCE_MIN: return "reduce_min";
        case ExprOp::REDUCE_MAX: return "reduce_max"; case ExprOp::REDUCE_ARGMIN: return "argmin"; case ExprOp::REDUCE_ARGMAX: return "argmax";
        case ExprOp::REDUCE_AVG: return "reduce_mean"; case ExprOp::REDUCE_NORM1: return "reduce_norm1"; case ExprOp::REDUCE_NORM2: return "reduce_norm2";
        default: return "op";
    }
}

namespace {

bool sameNode(const ExprNode& a, const ExprNode& b) {
    return a.op == b.op && a.lhs == b.lhs && a.rhs == b.rhs && a.aux == b.aux && a.input_slot == b.input_slot &&
           ((a.scalar_fp == b.scalar_fp) || (a.scalar_fp != a.scalar_fp && b.scalar_fp != b.scalar_fp)) && a.output_dtype == b.output_dtype &&
           a.compute_dtype == b.compute_dtype && a.reduction_axes == b.reduction_axes && a.squeeze_axes == b.squeeze_axes &&
           a.unsqueeze_axes == b.unsqueeze_axes && a.reshape_dims == b.reshape_dims && a.stop_gradient == b.stop_gradient;
}

// Appends a node unless a structurally identical one exists already (common sub-expressions are
// shared, so the graph stays a DAG however the user combined the pieces).
uint32_t appendShared(PhysicalExpression& g, const ExprNode& n) {
    for (uint32_t i = 0; i < g.nodes.size(); ++i)
        if (sameNode(g.nodes[i], n)) return i;
    g.nodes.push_back(n);
    return static_cast<uint32_t>(g.nodes.size() - 1);
}

uint32_t inputSlot(PhysicalExpression& g, const std::string& name, NamedInput::Kind kind) {
    for (const auto& in : g.inputs) {
        if (in.name == name) {
            if (in.kind != kind) throw std::invalid_argument("Expression: input '" + name + "' is used with two different kinds");
            return in.slot;
        }
    }
    const uint32_t slot = static_cast<uint32_t>(g.inputs.size());
    g.inputs.push_back(NamedInput{name, slot, kind});
    return slot;
}

Expression makeLeaf(ExprOp op, const std::string& name, NamedInput::Kind kind, std::optional<DataType> compute_dtype, std::optional<DataType> output_dtype) {
    auto g = std::make_shared<PhysicalExpression>();
    ExprNode n;
    n.op = op;
    n.input_slot = inputSlot(*g, name, kind);
    n.compute_dtype = compute_dtype;
    n.output_dtype = output_dtype;
    g->nodes.push_back(n);
    return Expression::fromPhysicalNode(g, 0);
}

}  // namespace

uint32_t mergeInto(PhysicalExpression& dst, const PhysicalExpression& src, uint32_t node) {
    std::unordered_map<uint32_t, uint32_t> remap;
    // nodes are topologically ordered, so one forward sweep over the ancestors of `node` suffices
    std::vector<bool> needed(src.nodes.size(), false);
    needed[node] = true;
    for (uint32_t k = node + 1; k-- > 0;) {
        if (!needed[k]) continue;
        for (uint32_t p : {src.nodes[k].lhs, src.nodes[k].rhs, src.nodes[k].aux})
            if (p != UINT32_MAX) needed[p] = true;
    }
    for (uint32_t k = 0; k <= node; ++k) {
        if (!needed[k]) continue;
        ExprNode n = src.nodes[k];
        if (n.lhs != UINT32_MAX) n.lhs = remap.at(n.lhs);
        if (n.rhs != UINT32_MAX) n.rhs = remap.at(n.rhs);
        if (n.aux != UINT32_MAX) n.aux = remap.at(n.aux);
        if (n.op == ExprOp::INPUT || n.op == ExprOp::RUNTIME_SCALAR || n.op == ExprOp::TENSOR_RUNTIME_SCALAR) {
            const NamedInput& in = src.inputs.at(n.input_slot);
            n.input_slot = inputSlot(dst, in.name, in.kind);
        }
        remap[k] = appendShared(dst, n);
    }
    return remap.at(node);
}

Expression::Expression(double value) {
    expr_ = std::make_shared<PhysicalExpression>();
    ExprNode n;
    n.op = ExprOp::SCALAR_FP;
    n.scalar_fp = value;
    expr_->nodes.push_back(n);
    node_ = 0;
}

Expression Expression::input(const std::string& name, std::optional<DataType> compute_dtype, std::optional<DataType> output_dtype) {
    return makeLeaf(ExprOp::INPUT, name, NamedInput::Kind::Tensor, compute_dtype, output_dtype);
}
Expression Expression::runtimeScalar(const std::string& name, std::optional<DataType> compute_dtype, std::optional<DataType> output_dtype) {
    return makeLeaf(ExprOp::RUNTIME_SCALAR, name, NamedInput::Kind::RuntimeScalarFp32, compute_dtype, output_dtype);
}
Expression Expression::tensorRuntimeScalar(const std::string& name, std::optional<DataType> compute_dtype, std::optional<DataType> output_dtype) {
    return makeLeaf(ExprOp::TENSOR_RUNTIME_SCALAR, name, NamedInput::Kind::TensorRuntimeScalar, compute_dtype, output_dtype);
}

Expression Expression::unary(ExprOp op) const {
    auto g = std::make_shared<PhysicalExpression>(*expr_);
    ExprNode n;
    n.op = op;
    n.lhs = node_;
    return Expression(g, appendShared(*g, n));
}

Expression Expression::binary(ExprOp op, const Expression& other) const {
    auto g = std::make_shared<PhysicalExpression>(*expr_);
    ExprNode n;
    n.op = op;
    n.lhs = node_;
    n.rhs = mergeInto(*g, *other.expr_, other.node_);
    return Expression(g, appendShared(*g, n));
}

Expression Expression::cast(DataType output_dtype) const {
    auto g = std::make_shared<PhysicalExpression>(*expr_);
    ExprNode n;
    n.op = ExprOp::CAST;
    n.lhs = node_;
    n.output_dtype = output_dtype;
    return Expression(g, appendShared(*g, n));
}

Expression Expression::withOutputDType(DataType dtype) const {
    auto g = std::make_shared<PhysicalExpression>(*expr_);
    ExprNode n = g->nodes[node_];
    n.output_dtype = dtype;
    return Expression(g, appendShared(*g, n));
}

Expression Expression::where(const Expression& condition, const Expression& true_value, const Expression& false_value) {
    auto g = std::make_shared<PhysicalExpression>(*condition.expr_);
    ExprNode n;
    n.op = ExprOp::WHERE;
    n.lhs = condition.node_;
    n.rhs = mergeInto(*g, *true_value.expr_, true_value.node_);
    n.aux = mergeInto(*g, *false_value.expr_, false_value.node_);
    return Expression(g, appendShared(*g, n));
}

Expression Expression::sigmoid() const {
    const Expression zero(0.0), one(1.0);
    const Expression neg = -*this;
    const Expression numerator = (-neg.max(zero)).exp();
    const Expression denominator = one + (-this->abs()).exp();
    return numerator / denominator;
}
Expression Expression::softplus() const { return this->max(Expression(0.0)) + (-this->abs()).exp().log1p(); }
Expression Expression::elu(double alpha) const { return this->max(Expression(0.0)) + (this->min(Expression(0.0)).expm1() * Expression(alpha)); }
Expression Expression::selu() const {
    return (this->max(Expression(0.0)) * Expression(1.05070098)) + (this->min(Expression(0.0)).expm1() * Expression(1.758099326));
}
Expression Expression::gelu() const { return *this * this->normcdf(); }
Expression Expression::swish() const { return *this * this->sigmoid(); }
Expression Expression::relu6() const { return this->max(Expression(0.0)).min(Expression(6.0)); }
Expression Expression::hardTanh(double min_value, double max_value) const {
    if (min_value > max_value) throw std::invalid_argument("Expression::hardTanh requires min_value <= max_value.");
    return this->max(Expression(min_value)).min(Expression(max_value));
}
Expression Expression::clamp(double lower_bound, double upper_bound) const {
    if (lower_bound > upper_bound) throw std::invalid_argument("Expression::clamp requires lower_bound <= upper_bound.");
    return this->max(Expression(lower_bound)).min(Expression(upper_bound));
}

Expression Expression::reshape(const std::vector<uint64_t>& new_dims) const {
    auto g = std::make_shared<PhysicalExpression>(*expr_);
    ExprNode n;
    n.op = ExprOp::RESHAPE;
    n.lhs = node_;
    n.reshape_dims = new_dims;
    return Expression(g, appendShared(*g, n));
}
Expression Expression::unsqueeze(const std::vector<uint64_t>& axes) const {
    auto g = std::make_shared<PhysicalExpression>(*expr_);
    ExprNode n;
    n.op = ExprOp::UNSQUEEZE;
    n.lhs = node_;
    n.unsqueeze_axes = axes;
    return Expression(g, appendShared(*g, n));
}
Expression Expression::squeeze(const std::vector<uint64_t>& axes) const {
    auto g = std::make_shared<PhysicalExpression>(*expr_);
    ExprNode n;
    n.op = ExprOp::SQUEEZE;
    n.lhs = node_;
    n.squeeze_axes = axes;
    return Expression(g, appendShared(*g, n));
}

Expression Expression::reduction(ExprOp op, const std::vector<uint64_t>& reduction_axes, const std::vector<uint64_t>& squeeze_axes,
                                 std::optional<DataType> compute_dtype) const {
    if (!isReductionOp(op)) throw std::invalid_argument("Expression::reduction requires a reduction op");
    std::vector<uint64_t> axes = reduction_axes;
    std::sort(axes.begin(), axes.end());
    if (axes.size() > 1 && axes.back() == kAxesFromOne) throw std::invalid_argument("Expression::reduction: the all-but-first sentinel stands alone");
    if (std::adjacent_find(axes.begin(), axes.end()) != axes.end()) throw std::invalid_argument("Expression::reduction axes must be unique");
    auto g = std::make_shared<PhysicalExpression>(*expr_);
    ExprNode n;
    n.op = op;
    n.lhs = node_;
    n.reduction_axes = axes;
    n.squeeze_axes = squeeze_axes;
    n.compute_dtype = compute_dtype;
    return Expression(g, appendShared(*g, n));
}

std::vector<bool> reducedAxesMask(const ExprNode& reduction, size_t rank) {
    const auto& axes = reduction.reduction_axes;
    if (axes.size() == 1 && axes[0] == kAxesFromOne) {
        std::vector<bool> mask(rank, true);
        if (rank > 0) mask[0] = false;
        return mask;
    }
    std::vector<bool> mask(rank, axes.empty());
    for (uint64_t ax : axes) {
        if (ax >= rank) throw std::logic_error("reduction axis out of range");
        mask[ax] = true;
    }
    return mask;
}

namespace {
Expression softmaxComposite(const Expression& x, SoftmaxAlgorithm algorithm, SoftmaxMode mode) {
    const std::vector<uint64_t> axes = mode == SoftmaxMode::CHANNEL ? std::vector<uint64_t>{1} : std::vector<uint64_t>{kAxesFromOne};
    const Expression xf = x.cast(DataType::FP32);
    Expression y = xf;
    if (algorithm == SoftmaxAlgorithm::FAST) {
        const Expression e = xf.exp();
        y = e / e.reduce_sum(axes);
    } else {
        // softmax is invariant to the shift, so the row maximum carries no gradient
        auto gm = std::make_shared<PhysicalExpression>(*xf.graph());
        ExprNode mx;
        mx.op = ExprOp::REDUCE_MAX;
        mx.lhs = xf.nodeIndex();
        mx.reduction_axes = axes;
        mx.stop_gradient = true;
        gm->nodes.push_back(mx);
        const Expression row_max = Expression::fromPhysicalNode(gm, static_cast<uint32_t>(gm->nodes.size() - 1));
        const Expression d = xf - row_max;
        const Expression e = d.exp();
        y = algorithm == SoftmaxAlgorithm::LOG ? d - e.reduce_sum(axes).ln() : e / e.reduce_sum(axes);
    }
    // store in the operand's dtype: a cast whose target is read from the operand when dtypes are resolved
    auto g = std::make_shared<PhysicalExpression>(*y.graph());
    ExprNode n;
    n.op = ExprOp::CAST;
    n.lhs = y.nodeIndex();
    n.aux = mergeInto(*g, *x.graph(), x.nodeIndex());
    g->nodes.push_back(n);
    return Expression::fromPhysicalNode(g, static_cast<uint32_t>(g->nodes.size() - 1));
}
}  // namespace

Expression Expression::softmax(SoftmaxAlgorithm algorithm, SoftmaxMode mode) const {
    if (algorithm == SoftmaxAlgorithm::LOG)
        throw std::invalid_argument("Expression::softmax computes ordinary softmax; use Expression::logSoftmax for the log algorithm.");
    if (algorithm != SoftmaxAlgorithm::FAST && algorithm != SoftmaxAlgorithm::ACCURATE)
        throw std::invalid_argument("Expression::softmax received an unsupported algorithm.");
    if (mode != SoftmaxMode::CHANNEL && mode != SoftmaxMode::INSTANCE) throw std::invalid_argument("Expression::softmax received an unsupported mode.");
    return softmaxComposite(*this, algorithm, mode);
}

Expression Expression::logSoftmax(SoftmaxMode mode) const {
    if (mode != SoftmaxMode::CHANNEL && mode != SoftmaxMode::INSTANCE) throw std::invalid_argument("Expression::logSoftmax received an unsupported mode.");
    return softmaxComposite(*this, SoftmaxAlgorithm::LOG, mode);
}

Expression Expression::reduceMinMaxBackward(ExprOp op, const Expression& forward_input, const Expression& grad, const std::vector<uint64_t>& reduction_axes,
                                             const std::vector<uint64_t>& squeeze_axes) {
    if (!isMinMaxBackwardOp(op)) throw std::invalid_argument("Expression::reduceMinMaxBackward requires REDUCE_MIN_BACKWARD or REDUCE_MAX_BACKWARD");
    auto g = std::make_shared<PhysicalExpression>(*forward_input.expr_);
    ExprNode n;
    n.op = op;
    n.lhs = forward_input.node_;
    n.rhs = mergeInto(*g, *grad.expr_, grad.node_);
    n.reduction_axes = reduction_axes;
    n.squeeze_axes = squeeze_axes;
    return Expression(g, appendShared(*g, n));
}

Outputs Expression::outputs(const std::vector<std::pair<std::string, Expression>>& named_exprs) {
    if (named_exprs.empty()) throw std::invalid_argument("Expression::outputs requires at least one output");
    auto g = std::make_shared<PhysicalExpression>();
    std::vector<NamedOutput> outs;
    for (const auto& [name, e] : named_exprs) {
        for (const auto& o : outs)
            if (o.name == name) throw std::invalid_argument("Expression::outputs: duplicate output name '" + name + "'");
        outs.push_back(NamedOutput{name, mergeInto(*g, *e.graph(), e.nodeIndex())});
    }
    return Outputs(g, outs);
}

// ---- dtype resolution ---------------------------------------------------------------------------

DataType promoteTensorValueDTypes(DataType a, DataType b) {
    if (a == b) return a;
    if (!isFusionFloat(a) || !isFusionFloat(b)) throw std::runtime_error("Unsupported dtype in promoteTensorValueDTypes.");
    if ((a == DataType::FP16 && b == DataType::BF16) || (a == DataType::BF16 && b == DataType::FP16)) return DataType::FP32;
    if (a == DataType::FP32 || b == DataType::FP32) return DataType::FP32;
    if (a == DataType::BF16 || b == DataType::BF16) return DataType::BF16;
    if (a == DataType::FP16 || b == DataType::FP16) return DataType::FP16;
    return DataType::FP16;  // fp8 with fp8
}

DataType toSupportedComputeDType(ExprOp op, DataType requested) {
    if (isComparisonOp(op) || isLogicalOp(op) || op == ExprOp::WHERE) {
        if (requested == DataType::BOOLEAN || requested == DataType::UINT8) return DataType::BOOLEAN;
        if (isFusionFloat(requested)) return toSupportedComputeDType(ExprOp::ADD, requested);
        throw std::runtime_error("Unsupported boolean/comparison/where dtype in toSupportedComputeDType.");
    }
    if (op == ExprOp::CAST || isViewOp(op)) return requested;
    if (!isFusionFloat(requested)) throw std::runtime_error(std::string("Unsupported dtype in toSupportedComputeDType: ") + dataTypeName(requested));
    if (isReductionOp(op) || isMinMaxBackwardOp(op)) return DataType::FP32;
    switch (requested) {
        case DataType::BF16: return DataType::BF16;
        case DataType::FP32: return DataType::FP32;
        default: return DataType::FP16;  // fp16 and both fp8 formats compute in fp16
    }
}

namespace {

bool isBooleanOutputOp(ExprOp op) { return isComparisonOp(op) || isLogicalOp(op); }

DataType resolveNodeOutputDType(const ExprNode& node, const std::vector<ExprNode>& nodes, const std::vector<DataType>& resolved) {
    if (isArgReductionOp(node.op)) return node.output_dtype.value_or(DataType::UINT32);
    if (isValueReductionOp(node.op)) {
        const DataType out = node.output_dtype.value_or(DataType::FP32);
        if (!isFusionFloat(out)) throw std::runtime_error("Dense floating-point reduction requested unsupported output dtype");
        return out;
    }
    if (isBooleanOutputOp(node.op)) return node.output_dtype.value_or(DataType::BOOLEAN);
    if (isMinMaxBackwardOp(node.op)) {
        const DataType in = resolved[node.lhs];
        const bool storable = in == DataType::FP32 || in == DataType::FP16 || in == DataType::BF16;
        return node.output_dtype.value_or(storable ? in : DataType::FP32);
    }
    auto isScalarParent = [&](uint32_t p) { return isScalarLeafOp(nodes[p].op); };
    if (node.op == ExprOp::WHERE) {
        if (resolved[node.lhs] != DataType::BOOLEAN) throw std::runtime_error("Where condition must have BOOLEAN dtype");
        std::vector<DataType> branches;
        if (!isScalarParent(node.rhs)) branches.push_back(resolved[node.rhs]);
        if (!isScalarParent(node.aux)) branches.push_back(resolved[node.aux]);
        DataType def = DataType::FP32;
        if (!branches.empty()) {
            def = branches.front();
            for (DataType b : branches)
                if (b != def) def = promoteTensorValueDTypes(def, b);
        }
        return node.output_dtype.value_or(def);
    }
    std::vector<DataType> parents;
    for (uint32_t p : {node.lhs, node.rhs, node.aux})
        if (p != UINT32_MAX && !isScalarParent(p)) parents.push_back(resolved[p]);
    DataType def = DataType::FP32;
    if (!parents.empty()) {
        def = parents.front();
        for (size_t i = 1; i < parents.size(); ++i) def = promoteTensorValueDTypes(def, parents[i]);
    }
    return node.output_dtype.value_or(def);
}

DataType resolveLogicalInputDType(const ExprNode& node, const std::vector<ExprNode>& nodes, const std::vector<DataType>& resolved) {
    if (node.op == ExprOp::SCALAR_FP) return node.output_dtype.value_or(DataType::FP32);
    if (node.op == ExprOp::CAST || isViewOp(node.op) || isReductionOp(node.op)) return resolved[node.lhs];
    std::vector<DataType> parents;
    for (uint32_t p : {node.lhs, node.rhs, node.aux})
        if (p != UINT32_MAX && !isScalarLeafOp(nodes[p].op)) {
            if (node.op == ExprOp::WHERE && p == node.lhs) continue;
            parents.push_back(resolved[p]);
        }
    if (parents.empty()) return DataType::FP32;
    DataType d = parents.front();
    for (size_t i = 1; i < parents.size(); ++i) {
        if (d == parents[i]) continue;
        if (isFusionFloat(d) && isFusionFloat(parents[i])) d = promoteTensorValueDTypes(d, parents[i]);
        else if (!isFusionFloat(d)) d = parents[i];
    }
    return d;
}

void seedRequired(std::optional<DataType>& slot, DataType dt) {
    if (!isFusionFloat(dt)) return;
    slot = slot.has_value() ? promoteTensorValueDTypes(*slot, dt) : dt;
}

DataType promoteRequiredComputeDType(ExprOp op, DataType current, DataType propagated) {
    if (op == ExprOp::CAST) return toSupportedComputeDType(op, current);
    if (isComparisonOp(op) || isLogicalOp(op) || op == ExprOp::WHERE) {
        if (isFusionFloat(current) && isFusionFloat(propagated)) return toSupportedComputeDType(op, promoteTensorValueDTypes(current, propagated));
        if (isFusionFloat(propagated)) return toSupportedComputeDType(op, propagated);
        return toSupportedComputeDType(op, current);
    }
    if (!isFusionFloat(current)) return current;
    return toSupportedComputeDType(op, promoteTensorValueDTypes(current, propagated));
}

}  // namespace

void resolveOutputsDTypesInPlace(PhysicalOutputs& outputs, const std::vector<DataType>& root_input_dtypes) {
    if (!outputs.expr) throw std::runtime_error("resolveOutputsDTypesInPlace requires non-null outputs.expr.");
    PhysicalExpression& expr = *outputs.expr;
    const size_t n = expr.nodes.size();
    std::vector<DataType> resolved(n, DataType::FP32);
    std::vector<uint8_t> explicit_compute(n, 0);
    for (size_t i = 0; i < n; ++i) explicit_compute[i] = expr.nodes[i].compute_dtype.has_value();

    for (size_t i = 0; i < n; ++i) {
        ExprNode& node = expr.nodes[i];
        if (node.op == ExprOp::INPUT || node.op == ExprOp::RUNTIME_SCALAR || node.op == ExprOp::TENSOR_RUNTIME_SCALAR) {
            if (node.input_slot >= root_input_dtypes.size()) throw std::runtime_error("Input slot out of range in resolveExpressionDTypesInPlace.");
            const DataType actual = root_input_dtypes[node.input_slot];
            node.input_tensor_dtype = actual;
            const DataType out = node.output_dtype.value_or(actual);
            DataType compute = out;
            if (isFusionFloat(actual) && isFusionFloat(out))
                compute = toSupportedComputeDType(node.op, node.compute_dtype.value_or(promoteTensorValueDTypes(actual, out)));
            else if (node.compute_dtype.has_value())
                compute = *node.compute_dtype;
            node.output_dtype = out;
            node.compute_dtype = compute;
            resolved[i] = out;
            continue;
        }
        if (node.op == ExprOp::CAST && node.aux != UINT32_MAX) {
            // "store like that node": the target dtype becomes explicit and the reference to the node is dropped
            if (!node.output_dtype.has_value()) node.output_dtype = resolved[node.aux];
            node.aux = UINT32_MAX;
        }
        const DataType out = resolveNodeOutputDType(node, expr.nodes, resolved);
        const DataType logical_in = resolveLogicalInputDType(node, expr.nodes, resolved);
        DataType requested;
        if (node.op == ExprOp::CAST || isViewOp(node.op)) {
            requested = out;
        } else if (isArgReductionOp(node.op) || isMinMaxBackwardOp(node.op)) {
            requested = DataType::FP32;
        } else if (isComparisonOp(node.op)) {
            if (node.compute_dtype.has_value()) requested = *node.compute_dtype;
            else if (logical_in == DataType::BOOLEAN || logical_in == DataType::UINT8) requested = DataType::BOOLEAN;
            else if (isFusionFloat(logical_in)) requested = toSupportedComputeDType(ExprOp::ADD, logical_in);
            else requested = DataType::FP32;
        } else if (isLogicalOp(node.op) || node.op == ExprOp::WHERE) {
            requested = node.compute_dtype.value_or(logical_in);
        } else {
            if (node.compute_dtype.has_value()) requested = *node.compute_dtype;
            else if (isFusionFloat(logical_in) && isFusionFloat(out)) requested = promoteTensorValueDTypes(logical_in, out);
            else requested = DataType::FP32;
        }
        node.output_dtype = out;
        node.compute_dtype = toSupportedComputeDType(node.op, requested);
        resolved[i] = out;
    }

    // Backward propagation of compute-dtype requirements from the materialized outputs
    // (ExpressionDTypeResolution.cpp:885-1010): a consumer that computes in a wider type widens
    // the compute dtype of its non-explicit ancestors, except across casts and reductions.
    std::vector<std::optional<DataType>> required(n);
    for (const auto& o : outputs.outputs) {
        const ExprNode& on = expr.nodes.at(o.node_idx);
        if (on.compute_dtype.has_value()) seedRequired(required[o.node_idx], *on.compute_dtype);
        else if (on.output_dtype.has_value()) seedRequired(required[o.node_idx], *on.output_dtype);
    }
    for (size_t i = n; i-- > 0;) {
        if (!required[i].has_value()) continue;
        ExprNode& node = expr.nodes[i];
        DataType propagated = *required[i];
        if (!isLeafOp(node.op) && node.compute_dtype.has_value()) {
            if (!explicit_compute[i]) node.compute_dtype = promoteRequiredComputeDType(node.op, *node.compute_dtype, propagated);
            propagated = *node.compute_dtype;
        }
        if (node.op == ExprOp::CAST || isMinMaxBackwardOp(node.op)) continue;
        if (isReductionOp(node.op)) {
            const ExprNode& producer = expr.nodes[node.lhs];
            if (producer.compute_dtype.has_value()) seedRequired(required[node.lhs], *producer.compute_dtype);
            else if (producer.output_dtype.has_value()) seedRequired(required[node.lhs], *producer.output_dtype);
            continue;
        }
        if (node.op == ExprOp::WHERE) {
            for (uint32_t p : {node.rhs, node.aux})
                if (expr.nodes[p].output_dtype.has_value() && isFusionFloat(*expr.nodes[p].output_dtype)) seedRequired(required[p], propagated);
            continue;
        }
        if (isLeafOp(node.op)) continue;
        for (uint32_t p : {node.lhs, node.rhs, node.aux})
            if (p != UINT32_MAX) seedRequired(required[p], propagated);
    }
}

}  // namespace ThorB200
