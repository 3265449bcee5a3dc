// Reverse-mode graph transform for the host layer's op set.  The backward pass is an ordinary
// Expression DAG (it recomputes the forward sub-expressions it needs), so it runs through the same
// planner, fused stages, reductions and row programs as any forward expression.
#include "AutoDiff.h"

#include <algorithm>
#include <map>
#include <stdexcept>

#include "FusedEquation.h"

namespace ThorB200 {

namespace {

uint64_t numelOf(const std::vector<uint64_t>& d) {
    uint64_t n = 1;
    for (uint64_t v : d) n *= v;
    return n;
}

struct Builder {
    std::shared_ptr<PhysicalExpression> fwd;                       // forward graph (shared by every forward handle)
    std::vector<std::vector<uint64_t>> fwd_shape;                  // per forward node
    std::unordered_map<std::string, std::vector<uint64_t>> dims;   // by input name (forward inputs + upstream grads)

    Expression forward(uint32_t node) const { return Expression::fromPhysicalNode(fwd, node); }

    // Shape of an arbitrary expression built from forward nodes and upstream-gradient inputs.
    std::vector<uint64_t> shapeOf(const Expression& e) const {
        const PhysicalExpression& g = *e.graph();
        std::vector<std::vector<uint64_t>> in(g.inputs.size());
        for (const NamedInput& ni : g.inputs) {
            if (ni.kind != NamedInput::Kind::Tensor) continue;
            auto it = dims.find(ni.name);
            if (it == dims.end()) throw std::logic_error("buildBackwardOutputs: no shape for input '" + ni.name + "'");
            in[ni.slot] = it->second;
        }
        return inferNodeShapes(g, in)[e.nodeIndex()];
    }

    // Un-broadcast: sum `grad` over the axes along which `target` was broadcast (AutoDiff.cpp:3403-3560).
    Expression sumToShape(const Expression& grad, const std::vector<uint64_t>& target) const {
        const std::vector<uint64_t> gs = shapeOf(grad);
        if (gs == target || numelOf(gs) <= numelOf(target)) return grad;
        if (target.empty()) return grad;  // scalar operands take no gradient here
        const size_t pad = gs.size() - target.size();
        std::vector<uint64_t> axes, squeeze;
        for (size_t i = 0; i < gs.size(); ++i) {
            const uint64_t t = i < pad ? 1 : target[i - pad];
            if (t == 1 && gs[i] != 1) axes.push_back(i);
            if (i < pad) {
                if (gs[i] != 1 && std::find(axes.begin(), axes.end(), i) == axes.end()) axes.push_back(i);
                squeeze.push_back(i);
            }
        }
        if (axes.empty() && squeeze.empty()) return grad;
        if (axes.empty()) return grad.squeeze(squeeze);
        return grad.reduce_sum(axes, squeeze);
    }
};

}  // namespace

Outputs buildBackwardOutputs(const Outputs& forward, const std::vector<std::string>& wrt_names, const std::string& upstream_prefix,
                             const std::unordered_map<std::string, std::vector<uint64_t>>& input_dims,
                             const std::unordered_map<std::string, DataType>& input_dtypes) {
    if (!forward.expression()) throw std::logic_error("buildBackwardOutputs requires forward outputs");
    Builder b;
    b.fwd = std::make_shared<PhysicalExpression>(*forward.expression());
    b.dims = input_dims;
    const PhysicalExpression& g = *b.fwd;
    std::vector<std::vector<uint64_t>> in_dims(g.inputs.size());
    for (const NamedInput& ni : g.inputs) {
        if (ni.kind == NamedInput::Kind::Tensor) {
            auto it = input_dims.find(ni.name);
            if (it == input_dims.end()) throw std::logic_error("buildBackwardOutputs: forward input '" + ni.name + "' is not bound");
            in_dims[ni.slot] = it->second;
        }
    }
    b.fwd_shape = inferNodeShapes(g, in_dims);
    // resolved dtypes of the forward nodes (queried by the CAST rule); the cloned forward nodes stay unresolved
    PhysicalOutputs resolved = forward.physicalOutputs();
    resolved.expr = std::make_shared<PhysicalExpression>(g);
    {
        std::vector<DataType> dts(g.inputs.size(), DataType::FP32);
        for (const NamedInput& ni : g.inputs) {
            auto it = input_dtypes.find(ni.name);
            if (it != input_dtypes.end()) dts[ni.slot] = it->second;
        }
        resolveOutputsDTypesInPlace(resolved, dts);
    }

    // seed: upstream gradient inputs
    std::map<uint32_t, Expression> grad;
    auto accumulate = [&](uint32_t node, const Expression& contribution) {
        const Expression c = b.sumToShape(contribution, b.fwd_shape[node]);
        auto it = grad.find(node);
        if (it == grad.end()) grad.emplace(node, c);
        else it->second = it->second + c;
    };
    const auto& outs = forward.namedOutputs();
    for (const NamedOutput& o : outs) {
        const std::string name = outs.size() == 1 ? upstream_prefix : upstream_prefix + "_" + o.name;
        // an upstream gradient that is not bound seeds the output with 1, the reference's default seed (AutoDiff.cpp:3819)
        if (!input_dims.count(name)) grad.emplace(o.node_idx, Expression(1.0));
        else accumulate(o.node_idx, Expression::input(name));
    }
    // which nodes reach a requested input
    std::vector<bool> reaches(g.nodes.size(), false);
    for (uint32_t k = 0; k < g.nodes.size(); ++k) {
        const ExprNode& nd = g.nodes[k];
        if (nd.op == ExprOp::INPUT) {
            reaches[k] = std::find(wrt_names.begin(), wrt_names.end(), g.inputs[nd.input_slot].name) != wrt_names.end();
            continue;
        }
        if (nd.stop_gradient) continue;
        for (uint32_t p : {nd.lhs, nd.rhs, nd.aux})
            if (p != UINT32_MAX && reaches[p]) reaches[k] = true;
    }

    for (uint32_t k = static_cast<uint32_t>(g.nodes.size()); k-- > 0;) {
        auto it = grad.find(k);
        if (it == grad.end() || !reaches[k]) continue;
        const Expression G = it->second;
        const ExprNode& nd = g.nodes[k];
        auto wants = [&](uint32_t p) { return p != UINT32_MAX && reaches[p]; };
        switch (nd.op) {
            case ExprOp::INPUT: case ExprOp::RUNTIME_SCALAR: case ExprOp::TENSOR_RUNTIME_SCALAR: case ExprOp::SCALAR_FP: break;
            case ExprOp::ADD:
                if (wants(nd.lhs)) accumulate(nd.lhs, G);
                if (wants(nd.rhs)) accumulate(nd.rhs, G);
                break;
            case ExprOp::SUB:
                if (wants(nd.lhs)) accumulate(nd.lhs, G);
                if (wants(nd.rhs)) accumulate(nd.rhs, -G);
                break;
            case ExprOp::MUL:
                if (wants(nd.lhs)) accumulate(nd.lhs, G * b.forward(nd.rhs));
                if (wants(nd.rhs)) accumulate(nd.rhs, G * b.forward(nd.lhs));
                break;
            case ExprOp::DIV:
                if (wants(nd.lhs)) accumulate(nd.lhs, G / b.forward(nd.rhs));
                if (wants(nd.rhs)) {
                    const Expression rhs = b.forward(nd.rhs);
                    accumulate(nd.rhs, -((G * b.forward(nd.lhs)) / (rhs * rhs)));
                }
                break;
            case ExprOp::NEG:
                if (wants(nd.lhs)) accumulate(nd.lhs, -G);
                break;
            case ExprOp::ABS:
                if (wants(nd.lhs)) {
                    // sign(x) with 0 at 0: MAX_GRAD_LEFT(x, -x) - MAX_GRAD_RIGHT(x, -x) (AutoDiff.cpp, ABS rule)
                    const Expression x = b.forward(nd.lhs);
                    const Expression nx = -x;
                    // the grad-mask ops are reachable through max(): d max(x,-x)/dx = left - right
                    const Expression left = Expression::where(x > nx, Expression(1.0), Expression::where(x < nx, Expression(0.0), Expression(0.5)));
                    const Expression right = Expression::where(x < nx, Expression(1.0), Expression::where(x > nx, Expression(0.0), Expression(0.5)));
                    accumulate(nd.lhs, G * (left - right));
                }
                break;
            case ExprOp::EXP:
                if (wants(nd.lhs)) accumulate(nd.lhs, G * b.forward(k));
                break;
            case ExprOp::LN:
                if (wants(nd.lhs)) accumulate(nd.lhs, G / b.forward(nd.lhs));
                break;
            case ExprOp::SQRT:
                if (wants(nd.lhs)) accumulate(nd.lhs, G / (Expression(2.0) * b.forward(k)));
                break;
            case ExprOp::TANH:
                if (wants(nd.lhs)) {
                    const Expression out = b.forward(k);
                    accumulate(nd.lhs, G * (Expression(1.0) - out * out));
                }
                break;
            case ExprOp::EXPM1:
                if (wants(nd.lhs)) accumulate(nd.lhs, G * b.forward(nd.lhs).exp());
                break;
            case ExprOp::LOG1P:
                if (wants(nd.lhs)) accumulate(nd.lhs, G / (Expression(1.0) + b.forward(nd.lhs)));
                break;
            case ExprOp::SIN:
                if (wants(nd.lhs)) accumulate(nd.lhs, G * b.forward(nd.lhs).cos());
                break;
            case ExprOp::COS:
                if (wants(nd.lhs)) accumulate(nd.lhs, -(G * b.forward(nd.lhs).sin()));
                break;
            case ExprOp::POW:
                if (wants(nd.lhs)) {
                    const Expression base = b.forward(nd.lhs), ex = b.forward(nd.rhs);
                    accumulate(nd.lhs, G * ex * base.pow(ex - Expression(1.0)));
                }
                if (wants(nd.rhs)) accumulate(nd.rhs, G * b.forward(k) * b.forward(nd.lhs).ln());
                break;
            case ExprOp::MAX: case ExprOp::MIN: {
                // 1 / 0 masks with 0.5 on ties (MAX_GRAD_LEFT / RIGHT, CudaSourceEmitter.cpp:1940-1954)
                const Expression l = b.forward(nd.lhs), r = b.forward(nd.rhs);
                const bool is_max = nd.op == ExprOp::MAX;
                const Expression l_wins = is_max ? (l > r) : (l < r);
                const Expression r_wins = is_max ? (l < r) : (l > r);
                if (wants(nd.lhs)) accumulate(nd.lhs, G * Expression::where(l_wins, Expression(1.0), Expression::where(r_wins, Expression(0.0), Expression(0.5))));
                if (wants(nd.rhs)) accumulate(nd.rhs, G * Expression::where(r_wins, Expression(1.0), Expression::where(l_wins, Expression(0.0), Expression(0.5))));
                break;
            }
            case ExprOp::WHERE: {
                const Expression cond = b.forward(nd.lhs);
                if (wants(nd.rhs)) accumulate(nd.rhs, Expression::where(cond, G, Expression(0.0)));
                if (wants(nd.aux)) accumulate(nd.aux, Expression::where(cond, Expression(0.0), G));
                break;
            }
            case ExprOp::CAST:
                // straight-through: the gradient is converted back to the source dtype (AutoDiff.cpp, CAST rule)
                if (wants(nd.lhs)) {
                    const std::optional<DataType> src = resolved.expr->nodes[nd.lhs].output_dtype;
                    accumulate(nd.lhs, src.has_value() ? G.cast(*src) : G);
                }
                break;
            case ExprOp::RESHAPE: case ExprOp::UNSQUEEZE: case ExprOp::SQUEEZE:
                // a gradient with fewer elements than the view (a broadcast seed) passes through unchanged
                if (wants(nd.lhs)) accumulate(nd.lhs, numelOf(b.shapeOf(G)) == numelOf(b.fwd_shape[nd.lhs]) ? G.reshape(b.fwd_shape[nd.lhs]) : G);
                break;
            case ExprOp::REDUCE_SUM: case ExprOp::REDUCE_AVG: {
                if (!wants(nd.lhs)) break;
                // unsqueeze the gradient back to keep-dims form; elementwise consumers broadcast it
                const std::vector<uint64_t>& in_shape = b.fwd_shape[nd.lhs];
                std::vector<uint64_t> keep(in_shape);
                const std::vector<bool> reduced = reducedAxesMask(nd, in_shape.size());
                uint64_t count = 1;
                for (size_t i = 0; i < in_shape.size(); ++i)
                    if (reduced[i]) {
                        count *= in_shape[i];
                        keep[i] = 1;
                    }
                const std::vector<uint64_t> gs = b.shapeOf(G);
                Expression Gk = (gs == keep || numelOf(gs) != numelOf(keep)) ? G : G.reshape(keep);
                if (nd.op == ExprOp::REDUCE_AVG) Gk = Gk / Expression(static_cast<double>(count));
                accumulate(nd.lhs, Gk);
                break;
            }
            case ExprOp::REDUCE_MIN: case ExprOp::REDUCE_MAX: {
                if (!wants(nd.lhs)) break;
                // the whole gradient of a segment goes to its winner (AutoDiff.cpp:5036-5050)
                if (numelOf(b.shapeOf(G)) != numelOf(b.fwd_shape[k]) && numelOf(b.shapeOf(G)) != 1)
                    throw std::runtime_error("Thor expressions autodiff: min/max reduction backward needs one gradient value per reduced segment, or one for all.");
                accumulate(nd.lhs, Expression::reduceMinMaxBackward(nd.op == ExprOp::REDUCE_MIN ? ExprOp::REDUCE_MIN_BACKWARD : ExprOp::REDUCE_MAX_BACKWARD,
                                                                   b.forward(nd.lhs), G, nd.reduction_axes, nd.squeeze_axes));
                break;
            }
            default:
                throw std::runtime_error(std::string("Thor expressions autodiff does not support backward for op ") + opName(nd.op) + ".");
        }
    }

    std::vector<std::pair<std::string, Expression>> named;
    for (const std::string& w : wrt_names) {
        bool found = false;
        for (uint32_t k = 0; k < g.nodes.size(); ++k) {
            const ExprNode& nd = g.nodes[k];
            if (nd.op != ExprOp::INPUT || g.inputs[nd.input_slot].name != w) continue;
            found = true;
            auto it = grad.find(k);
            if (it == grad.end()) throw std::logic_error("buildBackwardOutputs: no gradient reaches input '" + w + "'");
            Expression e = it->second;
            const std::vector<uint64_t> es = b.shapeOf(e);
            if (es != b.fwd_shape[k]) {
                if (numelOf(es) == numelOf(b.fwd_shape[k])) {
                    e = e.reshape(b.fwd_shape[k]);
                } else {
                    // explicit broadcast to the input's shape: a select whose condition is constantly true takes its
                    // shape from both branches and its value from the first; the generated kernel never reads the second
                    e = Expression::where(Expression(1.0) > Expression(0.0), e, b.forward(k));
                }
            }
            // terminal dtype = dtype of the forward input; a terminal reduction stores it directly
            auto dt = input_dtypes.find(w);
            if (dt != input_dtypes.end() && isFusionFloat(dt->second)) {
                const ExprNode& term = e.graph()->nodes[e.nodeIndex()];
                e = (isValueReductionOp(term.op) || isMinMaxBackwardOp(term.op)) ? e.withOutputDType(dt->second) : e.cast(dt->second);
            }
            named.emplace_back(w + "_grad", e);
            break;
        }
        if (!found) throw std::logic_error("buildBackwardOutputs: '" + w + "' is not an input of the forward expression");
    }
    return Expression::outputs(named);
}

}  // namespace ThorB200
