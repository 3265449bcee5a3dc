// Planner + stamper of the host layer: DAG -> stages -> C-ABI handles -> launch list.
#include "FusedEquation.h"

#include <algorithm>
#include <cstring>
#include <functional>
#include <set>
#include <sstream>
#include <stdexcept>

#include "AutoDiff.h"
#include "RowFusion.h"
#include "Schedule.h"
#include "thor_b200.h"

namespace ThorB200 {

namespace {

[[noreturn]] void throwFromStatus(int status, const char* what) {
    const std::string msg = std::string(what) + ": " + thor_b200_last_error();
    if (status == THOR_B200_INVALID_ARGUMENT || status == THOR_B200_UNSUPPORTED) throw std::logic_error(msg);
    throw std::runtime_error(msg);
}
void check(int status, const char* what) {
    if (status != THOR_B200_OK) throwFromStatus(status, what);
}

uint64_t numelOf(const std::vector<uint64_t>& dims) {
    uint64_t n = 1;
    for (uint64_t d : dims) n *= d;
    return n;
}

std::vector<uint64_t> broadcastDims(const std::vector<uint64_t>& a, const std::vector<uint64_t>& b) {
    const size_t r = std::max(a.size(), b.size());
    std::vector<uint64_t> out(r, 1);
    for (size_t i = 0; i < r; ++i) {
        const uint64_t da = i < r - a.size() ? 1 : a[i - (r - a.size())];
        const uint64_t db = i < r - b.size() ? 1 : b[i - (r - b.size())];
        if (da != db && da != 1 && db != 1) throw std::logic_error("Expression: operand shapes do not broadcast");
        out[i] = da == 1 ? db : da;
    }
    return out;
}

int reduceOpFor(ExprOp op) {
    switch (op) {
        case ExprOp::REDUCE_SUM: return THOR_B200_REDUCE_SUM;
        case ExprOp::REDUCE_PROD: return THOR_B200_REDUCE_PRODUCT;
        case ExprOp::REDUCE_MIN: return THOR_B200_REDUCE_MIN;
        case ExprOp::REDUCE_MAX: return THOR_B200_REDUCE_MAX;
        case ExprOp::REDUCE_AVG: return THOR_B200_REDUCE_MEAN;
        case ExprOp::REDUCE_NORM1: return THOR_B200_REDUCE_L1NORM;
        case ExprOp::REDUCE_NORM2: return THOR_B200_REDUCE_L2NORM;
        default: throw std::logic_error("not a value reduction");
    }
}

struct ExprHandle {
    thor_b200_expr* h = nullptr;
    ~ExprHandle() { thor_b200_expr_destroy(h); }
};
struct ReducePlanHandle {
    thor_b200_reduce_plan* h = nullptr;
    ~ReducePlanHandle() { thor_b200_reduce_plan_destroy(h); }
};
struct MinMaxBackwardPlanHandle {
    thor_b200_minmax_backward_plan* h = nullptr;
    ~MinMaxBackwardPlanHandle() { thor_b200_minmax_backward_plan_destroy(h); }
};
struct ArgReducePlanHandle {
    thor_b200_argreduce_plan* h = nullptr;
    ~ArgReducePlanHandle() { thor_b200_argreduce_plan_destroy(h); }
};

}  // namespace

std::vector<std::vector<uint64_t>> inferNodeShapes(const PhysicalExpression& expr, const std::vector<std::vector<uint64_t>>& input_dims) {
    std::vector<std::vector<uint64_t>> shape(expr.nodes.size());
    for (size_t k = 0; k < expr.nodes.size(); ++k) {
        const ExprNode& n = expr.nodes[k];
        if (n.op == ExprOp::INPUT) {
            shape[k] = input_dims.at(n.input_slot);
        } else if (isScalarLeafOp(n.op)) {
            shape[k] = {};
        } else if (isReductionOp(n.op)) {
            const auto& in = shape[n.lhs];
            const std::vector<bool> reduced = reducedAxesMask(n, in.size());
            std::vector<uint64_t> kept(in);
            for (size_t i = 0; i < in.size(); ++i)
                if (reduced[i]) kept[i] = 1;
            std::vector<uint64_t> out;
            const bool squeeze_all = n.squeeze_axes.size() == 1 && n.squeeze_axes[0] == kSqueezeAll;
            for (size_t i = 0; i < kept.size(); ++i) {
                bool drop = squeeze_all ? kept[i] == 1 : std::find(n.squeeze_axes.begin(), n.squeeze_axes.end(), i) != n.squeeze_axes.end();
                if (drop && kept[i] != 1) throw std::logic_error("squeeze axis is not a singleton");
                if (!drop) out.push_back(kept[i]);
            }
            if (out.empty()) out.push_back(1);
            shape[k] = out;
        } else if (isMinMaxBackwardOp(n.op)) {
            shape[k] = shape[n.lhs];
        } else if (n.op == ExprOp::RESHAPE) {
            if (numelOf(n.reshape_dims) != numelOf(shape[n.lhs])) throw std::logic_error("reshape changes the element count");
            shape[k] = n.reshape_dims;
        } else if (n.op == ExprOp::UNSQUEEZE) {
            std::vector<uint64_t> out = shape[n.lhs];
            std::vector<uint64_t> axes = n.unsqueeze_axes;
            std::sort(axes.begin(), axes.end());
            for (uint64_t ax : axes) {
                if (ax > out.size()) throw std::logic_error("unsqueeze axis out of range");
                out.insert(out.begin() + static_cast<long>(ax), 1);
            }
            shape[k] = out;
        } else if (n.op == ExprOp::SQUEEZE) {
            std::vector<uint64_t> out;
            const auto& in = shape[n.lhs];
            const bool squeeze_all = n.squeeze_axes.size() == 1 && n.squeeze_axes[0] == kSqueezeAll;
            for (size_t i = 0; i < in.size(); ++i) {
                const bool drop = squeeze_all ? in[i] == 1 : std::find(n.squeeze_axes.begin(), n.squeeze_axes.end(), i) != n.squeeze_axes.end();
                if (drop && in[i] != 1) throw std::logic_error("squeeze axis is not a singleton");
                if (!drop) out.push_back(in[i]);
            }
            if (out.empty()) out.push_back(1);
            shape[k] = out;
        } else {
            std::vector<uint64_t> out;
            for (uint32_t p : {n.lhs, n.rhs, n.aux})
                if (p != UINT32_MAX) out = broadcastDims(out, shape[p]);
            shape[k] = out;
        }
    }
    return shape;
}

// ---- stamped plan ---------------------------------------------------------------------------------

struct PhysicalStage {
    StageKind kind = StageKind::FusedKernel;
    std::string physical_name;
    std::string source;
    // FusedKernel
    std::shared_ptr<ExprHandle> expr;
    std::vector<const void*> input_ptrs;
    std::vector<float> scalars;
    std::vector<std::string> scalar_names;  // per slot, "" for tensors
    std::vector<void*> output_ptrs;
    uint64_t numel = 0;
    // Reduction / ArgMinMax
    std::shared_ptr<ReducePlanHandle> reduce;
    std::shared_ptr<ArgReducePlanHandle> argreduce;
    std::shared_ptr<MinMaxBackwardPlanHandle> minmax_backward;
    const void* in2 = nullptr;  // ReduceMinMaxBackward: gradient of the reduced value
    const void* in = nullptr;
    void* out = nullptr;
    Tensor workspace;
    size_t workspace_bytes = 0;
    // FusedRows
    std::function<void(void* stream)> custom_launch;
    std::shared_ptr<std::vector<float>> shared_scalars;  // FusedRows: runtime scalars the launch closure reads
    std::function<uint32_t()> waits_expired;             // FusedRows: bounded device-side waits that ran out
    uint64_t launches = 1;
    // device buffers the stage reads and writes: what orders it against the other stages of the plan
    std::vector<const void*> reads;
    std::vector<const void*> writes;
};

// Streams and events of a plan whose stages occupy more than one lane; owned by the plan, reused by every run.
struct LaneResources {
    std::vector<void*> lane_streams;   // [lane], entry 0 unused (the caller's stream)
    std::vector<void*> done_events;    // [scheduled stage], null where no other lane waits for the stage
    std::vector<void*> lane_end;       // [lane], recorded behind a helper lane's last stage of a run
    void* caller_ready = nullptr;
    ~LaneResources() {
        for (void* s : lane_streams) thor_b200_stream_destroy(s);
        for (void* e : done_events) thor_b200_event_destroy(e);
        for (void* e : lane_end) thor_b200_event_destroy(e);
        thor_b200_event_destroy(caller_ready);
    }
};

struct StampedExecutionPlan::Impl {
    Stream stream;
    std::vector<PhysicalStage> stages;
    std::vector<std::string> logical_stage_names;
    std::map<std::string, Tensor> outputs;
    std::vector<Tensor> keep_alive;
    uint64_t intermediate_bytes = 0;
    std::vector<std::string> column_sum_names;
    // branch scheduling (StampedEquation.cpp:4057-4205): stages that launch something, their dependencies and lanes
    std::vector<uint32_t> scheduled;  // indices into `stages` (views launch nothing and are left out)
    std::vector<std::vector<uint32_t>> dependencies;
    StampedExecutionSchedule schedule;
    std::shared_ptr<LaneResources> lanes;  // null: everything runs on the caller's stream
    bool plan_only = false;  // stamped with placeholder memory: describes the plan, cannot run
};

void StampedExecutionPlan::run() { runOn(impl_->stream); }

namespace {
void launchStage(PhysicalStage& s, void* stream) {
    switch (s.kind) {
        case StageKind::FusedKernel:
            check(thor_b200_expr_launch(s.expr->h, s.input_ptrs.data(), s.scalars.data(), s.output_ptrs.data(), s.numel, stream), "StampedExecutionPlan::run fused stage");
            break;
        case StageKind::Reduction:
            if (s.custom_launch) {
                s.custom_launch(stream);
                break;
            }
            check(thor_b200_reduce_launch(s.reduce->h, s.in, s.out, s.workspace.getMemPtr(), s.workspace_bytes, 1.0f, stream), "StampedExecutionPlan::run reduction");
            break;
        case StageKind::ArgMinMax:
            if (s.custom_launch) {
                s.custom_launch(stream);
                break;
            }
            check(thor_b200_argreduce_launch(s.argreduce->h, s.in, nullptr, s.out, s.workspace.getMemPtr(), s.workspace_bytes, stream),
                  "StampedExecutionPlan::run arg reduction");
            break;
        case StageKind::ReduceMinMaxBackward:
            check(thor_b200_minmax_backward_launch(s.minmax_backward->h, s.in, s.in2, s.out, s.workspace.getMemPtr(), s.workspace_bytes, stream),
                  "StampedExecutionPlan::run min/max backward");
            break;
        case StageKind::FusedRows: s.custom_launch(stream); break;
        case StageKind::View: break;
    }
}
}  // namespace

void StampedExecutionPlan::runOn(const Stream& stream) {
    if (!impl_) throw std::logic_error("StampedExecutionPlan is empty");
    if (impl_->plan_only) throw std::logic_error("StampedExecutionPlan was stamped in plan-only mode and cannot run");
    if (!impl_->lanes) {
        for (PhysicalStage& s : impl_->stages) launchStage(s, stream.handle);
        return;
    }
    // Independent branches run on helper streams beside the caller's: a stage waits for the events of the stages it
    // consumes that ran on other lanes, a helper lane's first stage without dependencies waits for the caller's stream as
    // it stood at the start of the run, and the caller's stream waits for every helper lane at the end.
    LaneResources& lr = *impl_->lanes;
    const StampedExecutionSchedule& sch = impl_->schedule;
    if (sch.needs_caller_ready_event) check(thor_b200_event_record(lr.caller_ready, stream.handle), "StampedExecutionPlan::run event");
    std::vector<bool> lane_used(lr.lane_streams.size(), false);
    for (size_t k = 0; k < impl_->scheduled.size(); ++k) {
        const uint32_t lane = sch.stage_lane_indices[k];
        void* lane_stream = lane == 0 ? stream.handle : lr.lane_streams[lane];
        if (lane != 0 && impl_->dependencies[k].empty()) check(thor_b200_stream_wait_event(lane_stream, lr.caller_ready), "StampedExecutionPlan::run wait");
        for (uint32_t dep : impl_->dependencies[k])
            if (sch.stage_lane_indices[dep] != lane) check(thor_b200_stream_wait_event(lane_stream, lr.done_events[dep]), "StampedExecutionPlan::run wait");
        launchStage(impl_->stages[impl_->scheduled[k]], lane_stream);
        if (lr.done_events[k]) check(thor_b200_event_record(lr.done_events[k], lane_stream), "StampedExecutionPlan::run event");
        lane_used[lane] = true;
    }
    for (size_t lane = 1; lane < lr.lane_streams.size(); ++lane)
        if (lane_used[lane]) {
            check(thor_b200_event_record(lr.lane_end[lane], lr.lane_streams[lane]), "StampedExecutionPlan::run event");
            check(thor_b200_stream_wait_event(stream.handle, lr.lane_end[lane]), "StampedExecutionPlan::run wait");
        }
}

std::vector<uint32_t> StampedExecutionPlan::stageLanes() const {
    std::vector<uint32_t> lanes(impl_->stages.size(), 0);
    for (size_t k = 0; k < impl_->scheduled.size(); ++k) lanes[impl_->scheduled[k]] = impl_->schedule.stage_lane_indices.empty() ? 0 : impl_->schedule.stage_lane_indices[k];
    return lanes;
}

Tensor StampedExecutionPlan::getOutput(const std::string& name) const {
    auto it = impl_->outputs.find(name);
    if (it == impl_->outputs.end()) throw std::logic_error("StampedExecutionPlan has no output named '" + name + "'");
    return it->second;
}
std::vector<std::string> StampedExecutionPlan::getOutputNames() const {
    std::vector<std::string> names;
    for (const auto& kv : impl_->outputs) names.push_back(kv.first);
    return names;
}
void StampedExecutionPlan::setRuntimeScalar(const std::string& name, float value) {
    bool found = false;
    for (PhysicalStage& s : impl_->stages)
        for (size_t i = 0; i < s.scalar_names.size(); ++i)
            if (s.scalar_names[i] == name) {
                s.scalars[i] = value;
                if (s.shared_scalars) (*s.shared_scalars)[i] = value;
                found = true;
            }
    if (!found) throw std::logic_error("StampedExecutionPlan has no runtime scalar named '" + name + "'");
}
std::vector<std::string> StampedExecutionPlan::stageKindNames() const { return impl_->logical_stage_names; }
std::vector<std::string> StampedExecutionPlan::physicalStageNames() const {
    std::vector<std::string> out;
    for (const auto& s : impl_->stages) out.push_back(s.physical_name);
    return out;
}
std::vector<std::string> StampedExecutionPlan::stageSources() const {
    std::vector<std::string> out;
    for (const auto& s : impl_->stages) out.push_back(s.source);
    return out;
}
uint64_t StampedExecutionPlan::intermediateBytes() const { return impl_->intermediate_bytes; }
uint64_t StampedExecutionPlan::waitsExpired() const {
    uint64_t n = 0;
    for (const auto& s : impl_->stages)
        if (s.waits_expired) n += s.waits_expired();
    return n;
}
std::vector<std::string> StampedExecutionPlan::columnSumNames() const { return impl_->column_sum_names; }
uint64_t StampedExecutionPlan::kernelLaunchesPerRun() const {
    uint64_t n = 0;
    for (const auto& s : impl_->stages)
        if (s.kind != StageKind::View) n += s.launches;
    return n;
}

// ---- FusedEquation ----------------------------------------------------------------------------------

struct FusedEquation::Deferred {
    Outputs forward;
    std::vector<std::string> wrt;
    std::string upstream_prefix;
};

FusedEquation FusedEquation::compile(const Outputs& outputs, int device_num, FusedEquationOptions options) {
    if (!outputs.expression()) throw std::logic_error("FusedEquation::compile requires outputs");
    FusedEquation eq;
    eq.outputs_ = outputs;
    eq.device_num_ = device_num;
    eq.options_ = options;
    return eq;
}

FusedEquation FusedEquation::compile(const Expression& expr, int device_num, FusedEquationOptions options) {
    return compile(Expression::outputs({{"output", expr}}), device_num, options);
}

FusedEquation FusedEquation::compileBackward(const std::vector<std::string>& wrt_names, const std::string& upstream_prefix) const {
    FusedEquation eq;
    eq.device_num_ = device_num_;
    eq.options_ = options_;
    eq.deferred_backward_ = std::make_shared<Deferred>(Deferred{outputs_, wrt_names, upstream_prefix});
    return eq;
}

namespace {

struct Planner {
    const PhysicalExpression& g;
    const std::vector<NamedOutput>& outs;
    const std::vector<std::vector<uint64_t>>& shape;
    std::vector<int> level;          // stage level at which the node's value exists
    std::vector<bool> materialize;   // elementwise nodes that must be written to memory
    std::vector<bool> needed;        // reachable from the outputs

    Planner(const PhysicalExpression& graph, const std::vector<NamedOutput>& outputs, const std::vector<std::vector<uint64_t>>& shapes)
        : g(graph), outs(outputs), shape(shapes) {
        const size_t n = g.nodes.size();
        needed.assign(n, false);
        for (const auto& o : outs) needed[o.node_idx] = true;
        for (size_t k = n; k-- > 0;) {
            if (!needed[k]) continue;
            for (uint32_t p : {g.nodes[k].lhs, g.nodes[k].rhs, g.nodes[k].aux})
                if (p != UINT32_MAX) needed[p] = true;
        }
        level.assign(n, 0);
        materialize.assign(n, false);
        for (size_t k = 0; k < n; ++k) {
            if (!needed[k]) continue;
            const ExprNode& nd = g.nodes[k];
            int lv = 0;
            for (uint32_t p : {nd.lhs, nd.rhs, nd.aux})
                if (p != UINT32_MAX) lv = std::max(lv, level[p]);
            if (isBoundary(k)) {
                lv += 1;  // a boundary op consumes a tensor that exists after level lv's fused stages
                if (isElementwise(nd.lhs)) materialize[nd.lhs] = true;
                if (isMinMaxBackwardOp(nd.op) && isElementwise(nd.rhs)) materialize[nd.rhs] = true;
            }
            level[k] = lv;
        }
        for (const auto& o : outs)
            if (isElementwise(o.node_idx)) materialize[o.node_idx] = true;
    }
    bool isBoundary(size_t k) const { return isReductionOp(g.nodes[k].op) || isViewOp(g.nodes[k].op) || isMinMaxBackwardOp(g.nodes[k].op); }
    bool isElementwise(size_t k) const { return !isBoundary(k) && !isLeafOp(g.nodes[k].op); }
};

}  // namespace

std::string FusedEquation::describeGraph(const std::unordered_map<std::string, std::vector<uint64_t>>& input_dims,
                                         const std::unordered_map<std::string, DataType>& input_dtypes) const {
    Outputs outputs = outputs_;
    if (deferred_backward_) outputs = buildBackwardOutputs(deferred_backward_->forward, deferred_backward_->wrt, deferred_backward_->upstream_prefix, input_dims, input_dtypes);
    PhysicalOutputs phys = outputs.physicalOutputs();
    phys.expr = std::make_shared<PhysicalExpression>(*phys.expr);
    std::vector<DataType> slot_dtypes(phys.expr->inputs.size(), DataType::FP32);
    for (const NamedInput& in : phys.expr->inputs) {
        if (in.kind == NamedInput::Kind::RuntimeScalarFp32) continue;
        auto it = input_dtypes.find(in.name);
        if (it == input_dtypes.end()) throw std::invalid_argument("describeGraph: no dtype given for input '" + in.name + "'");
        slot_dtypes[in.slot] = it->second;
    }
    resolveOutputsDTypesInPlace(phys, slot_dtypes);
    std::ostringstream os;
    os.precision(17);
    auto list = [&](const char* key, const std::vector<uint64_t>& v) {
        os << ",\"" << key << "\":[";
        for (size_t i = 0; i < v.size(); ++i) os << (i ? "," : "") << v[i];
        os << "]";
    };
    auto parent = [](uint32_t p) { return p == UINT32_MAX ? -1ll : static_cast<long long>(p); };
    os << "{\"inputs\":[";
    for (size_t i = 0; i < phys.expr->inputs.size(); ++i) {
        const NamedInput& in = phys.expr->inputs[i];
        os << (i ? "," : "") << "{\"name\":\"" << in.name << "\",\"slot\":" << in.slot << ",\"kind\":" << static_cast<int>(in.kind) << "}";
    }
    os << "],\"outputs\":[";
    for (size_t i = 0; i < phys.outputs.size(); ++i) os << (i ? "," : "") << "{\"name\":\"" << phys.outputs[i].name << "\",\"node\":" << phys.outputs[i].node_idx << "}";
    os << "],\"nodes\":[";
    for (size_t k = 0; k < phys.expr->nodes.size(); ++k) {
        const ExprNode& n = phys.expr->nodes[k];
        os << (k ? "," : "") << "{\"op\":" << static_cast<int>(n.op) << ",\"lhs\":" << parent(n.lhs) << ",\"rhs\":" << parent(n.rhs) << ",\"aux\":" << parent(n.aux)
           << ",\"slot\":" << parent(n.input_slot) << ",\"scalar\":" << n.scalar_fp << ",\"out\":" << (n.output_dtype ? static_cast<int>(*n.output_dtype) : 0)
           << ",\"compute\":" << (n.compute_dtype ? static_cast<int>(*n.compute_dtype) : 0);
        list("reduction_axes", n.reduction_axes);
        list("squeeze_axes", n.squeeze_axes);
        list("unsqueeze_axes", n.unsqueeze_axes);
        list("reshape_dims", n.reshape_dims);
        os << "}";
    }
    os << "]}";
    return os.str();
}

StampedExecutionPlan FusedEquation::stamp(const std::unordered_map<std::string, RuntimeInputValue>& inputs, const Stream& stream,
                                          const std::unordered_map<std::string, Tensor>& preallocated_outputs) {
    Outputs outputs = outputs_;
    if (deferred_backward_) {
        // shapes are known only now: build the backward DAG for these forward shapes
        std::unordered_map<std::string, std::vector<uint64_t>> dims;
        std::unordered_map<std::string, DataType> dtypes;
        for (const auto& kv : inputs)
            if (!kv.second.is_scalar) {
                dims[kv.first] = kv.second.tensor.getDimensions();
                dtypes[kv.first] = kv.second.tensor.getDataType();
            }
        outputs = buildBackwardOutputs(deferred_backward_->forward, deferred_backward_->wrt, deferred_backward_->upstream_prefix, dims, dtypes);
    }
    PhysicalOutputs phys = outputs.physicalOutputs();
    // private copy: dtype resolution writes into the graph
    phys.expr = std::make_shared<PhysicalExpression>(*phys.expr);
    PhysicalExpression& g = *phys.expr;

    // bind inputs
    std::vector<DataType> in_dtypes(g.inputs.size(), DataType::FP32);
    std::vector<std::vector<uint64_t>> in_dims(g.inputs.size());
    std::vector<RuntimeInputValue> bound(g.inputs.size());
    for (const NamedInput& in : g.inputs) {
        auto it = inputs.find(in.name);
        if (it == inputs.end()) throw std::logic_error("FusedEquation::stamp: missing input '" + in.name + "'");
        const RuntimeInputValue& v = it->second;
        if (in.kind == NamedInput::Kind::RuntimeScalarFp32) {
            if (!v.is_scalar) throw std::logic_error("FusedEquation::stamp: input '" + in.name + "' must be an fp32 scalar value");
            in_dtypes[in.slot] = DataType::FP32;
        } else {
            if (v.is_scalar || !v.tensor.isInitialized()) throw std::logic_error("FusedEquation::stamp: input '" + in.name + "' must be a tensor");
            if (v.tensor.getGpuNum() != device_num_) throw std::logic_error("FusedEquation::stamp: input '" + in.name + "' lives on another device");
            in_dtypes[in.slot] = v.tensor.getDataType();
            in_dims[in.slot] = v.tensor.getDimensions();
            if (in.kind == NamedInput::Kind::TensorRuntimeScalar && v.tensor.getTotalNumElements() != 1)
                throw std::logic_error("FusedEquation::stamp: tensor runtime scalar '" + in.name + "' must hold one element");
        }
        bound[in.slot] = v;
    }
    resolveOutputsDTypesInPlace(phys, in_dtypes);
    std::vector<std::vector<uint64_t>> shape_inputs = in_dims;
    for (const NamedInput& in : g.inputs)
        if (in.kind == NamedInput::Kind::TensorRuntimeScalar) shape_inputs[in.slot] = {};
    const auto shape = inferNodeShapes(g, shape_inputs);
    // tensor-runtime-scalar leaves are rank-0 in shape inference (handled by isScalarLeafOp)

    Planner plan(g, phys.outputs, shape);
    auto impl = std::make_shared<StampedExecutionPlan::Impl>();
    impl->stream = stream;
    impl->plan_only = Tensor::planOnly();

    // tensor that holds each materialised node (inputs, boundary outputs, materialised elementwise nodes)
    std::vector<Tensor> node_tensor(g.nodes.size());
    for (size_t k = 0; k < g.nodes.size(); ++k)
        if (g.nodes[k].op == ExprOp::INPUT || g.nodes[k].op == ExprOp::TENSOR_RUNTIME_SCALAR) {
            if (g.nodes[k].output_dtype != g.nodes[k].input_tensor_dtype)
                continue;  // an input with an output-dtype override is converted inside the consuming fused stage
            node_tensor[k] = bound[g.nodes[k].input_slot].tensor;
        }
    std::map<uint32_t, std::string> output_name_of;
    for (const auto& o : phys.outputs) output_name_of[o.node_idx] = o.name;

    auto allocateFor = [&](uint32_t node, bool is_output) -> Tensor {
        const DataType dt = *g.nodes[node].output_dtype;
        if (is_output) {
            auto it = preallocated_outputs.find(output_name_of.at(node));
            if (it != preallocated_outputs.end()) {
                if (it->second.getDataType() != dt) throw std::logic_error("FusedEquation::stamp: preallocated output '" + it->first + "' has the wrong dtype");
                if (it->second.getTotalNumElements() != numelOf(shape[node])) throw std::logic_error("FusedEquation::stamp: preallocated output '" + it->first + "' has the wrong size");
                return it->second;
            }
        }
        Tensor t = Tensor::allocate(dt, shape[node], device_num_);
        if (!is_output) impl->intermediate_bytes += t.getArraySizeInBytes();
        return t;
    };

    int max_level = 0;
    for (size_t k = 0; k < g.nodes.size(); ++k)
        if (plan.needed[k]) max_level = std::max(max_level, plan.level[k]);

    // Logical stage list first (what the reference's planner would run); the row-fusion pass may then
    // replace runs of logical stages by one physical super-stage.
    struct LogicalStage {
        StageKind kind;
        std::vector<uint32_t> nodes;  // FusedKernel: materialised nodes it produces; others: the boundary node
    };
    std::vector<LogicalStage> logical;
    for (int lv = 0; lv <= max_level; ++lv) {
        // fused groups of this level, grouped by output shape
        std::vector<std::pair<std::vector<uint64_t>, std::vector<uint32_t>>> groups;
        for (uint32_t k = 0; k < g.nodes.size(); ++k) {
            if (!plan.needed[k] || !plan.materialize[k] || plan.level[k] != lv) continue;
            bool placed = false;
            for (auto& grp : groups)
                if (grp.first == shape[k]) {
                    grp.second.push_back(k);
                    placed = true;
                    break;
                }
            if (!placed) groups.push_back({shape[k], {k}});
        }
        for (auto& grp : groups) logical.push_back({StageKind::FusedKernel, grp.second});
        for (uint32_t k = 0; k < g.nodes.size(); ++k) {
            if (!plan.needed[k] || !plan.isBoundary(k) || plan.level[k] != lv + 1) continue;
            const ExprOp op = g.nodes[k].op;
            logical.push_back({isViewOp(op) ? StageKind::View
                               : isArgReductionOp(op) ? StageKind::ArgMinMax
                               : isMinMaxBackwardOp(op) ? StageKind::ReduceMinMaxBackward : StageKind::Reduction,
                               {k}});
        }
    }
    for (const auto& ls : logical) {
        impl->logical_stage_names.push_back(ls.kind == StageKind::FusedKernel ? "FusedKernel" : ls.kind == StageKind::Reduction ? "Reduction"
                                            : ls.kind == StageKind::ArgMinMax ? "ArgMinMax"
                                            : ls.kind == StageKind::ReduceMinMaxBackward ? "ReduceMinMaxBackward" : "View");
    }

    // Optional physical fusion of row-reduction chains (softmax / LayerNorm class).
    std::vector<bool> covered(g.nodes.size(), false);  // nodes whose values a super-stage already produced or made unnecessary
    if (options_.fuse_row_reductions) {
        RowFusionContext ctx{g, phys.outputs, shape, bound, device_num_, options_.use_fast_math, options_.row_program, options_.unrounded_column_sums};
        std::vector<RowFusionMatch> matches = matchRowFusions(ctx);
        for (RowFusionMatch& m : matches) {
            PhysicalStage st;
            st.kind = StageKind::FusedRows;
            st.physical_name = m.name;
            st.source = m.source;
            st.launches = m.launches;
            st.scalar_names = m.scalar_names;
            st.shared_scalars = m.scalars;
            st.scalars = *m.scalars;
            for (auto& [node, is_out] : m.produced) {
                Tensor t = allocateFor(node, is_out);
                node_tensor[node] = t;
                if (is_out) impl->outputs[output_name_of.at(node)] = t;
                covered[node] = true;
            }
            for (uint32_t node : m.absorbed) covered[node] = true;
            for (auto& [node, is_out] : m.produced) st.writes.push_back(node_tensor[node].getMemPtr());
            for (const RuntimeInputValue& v : bound)
                if (!v.is_scalar && v.tensor.isInitialized()) st.reads.push_back(v.tensor.getMemPtr());
            st.custom_launch = m.bind(node_tensor, impl->keep_alive, impl->intermediate_bytes);
            if (m.column_sums) {
                impl->outputs["__column_sums"] = *m.column_sums;
                impl->column_sum_names = m.column_sum_names;
            }
            st.waits_expired = m.waits_expired;
            impl->stages.push_back(std::move(st));
        }
    }

    auto needsRun = [&](const LogicalStage& ls) {
        for (uint32_t k : ls.nodes)
            if (!covered[k]) return true;
        return false;
    };

    for (const LogicalStage& ls : logical) {
        if (!needsRun(ls)) continue;
        if (ls.kind == StageKind::View) {
            const uint32_t k = ls.nodes[0];
            const Tensor& src = node_tensor[g.nodes[k].lhs];
            if (!src.isInitialized()) throw std::logic_error("FusedEquation::stamp: view of a value that is not materialised");
            node_tensor[k] = Tensor::wrap(src.getMemPtr(), src.getDataType(), shape[k], device_num_);
            impl->keep_alive.push_back(src);
            PhysicalStage st;
            st.kind = StageKind::View;
            st.physical_name = "view";
            impl->stages.push_back(std::move(st));
            if (output_name_of.count(k)) impl->outputs[output_name_of[k]] = node_tensor[k];
            continue;
        }
        if (ls.kind == StageKind::Reduction || ls.kind == StageKind::ArgMinMax || ls.kind == StageKind::ReduceMinMaxBackward) {
            const uint32_t k = ls.nodes[0];
            const ExprNode& nd = g.nodes[k];
            const Tensor& src = node_tensor[nd.lhs];
            if (!src.isInitialized()) throw std::logic_error("FusedEquation::stamp: reduction input is not materialised");
            const auto& in_shape = shape[nd.lhs];
            const std::vector<bool> reduced = reducedAxesMask(nd, in_shape.size());
            // [outer, reduction, inner] needs the non-singleton reduced axes to form one contiguous block;
            // anything else takes the strided kernels (the reference's StridedFixedSegment path)
            uint64_t outer = 1, red = 1, inner = 1;
            int phase = 0;
            bool strided = false;
            for (size_t i = 0; i < in_shape.size(); ++i) {
                if (in_shape[i] == 1) continue;
                if (reduced[i]) {
                    if (phase == 2) strided = true;
                    phase = 1;
                    red *= in_shape[i];
                } else if (phase == 0) {
                    outer *= in_shape[i];
                } else {
                    phase = 2;
                    inner *= in_shape[i];
                }
            }
            if (strided) {
                if (ls.kind == StageKind::ReduceMinMaxBackward) throw std::logic_error("FusedEquation::stamp: min/max backward over non-adjacent axes is not provided");
                if (in_shape.size() > THOR_B200_MAX_RANK) throw std::logic_error("FusedEquation::stamp: reductions over non-adjacent axes support rank <= 8");
                const bool is_out_s = output_name_of.count(k) != 0;
                Tensor dst_s = allocateFor(k, is_out_s);
                node_tensor[k] = dst_s;
                if (is_out_s) impl->outputs[output_name_of[k]] = dst_s;
                auto d = std::make_shared<thor_b200_strided_reduce_desc>();
                d->op = ls.kind == StageKind::Reduction ? reduceOpFor(nd.op) : 0;
                d->arg_op = ls.kind == StageKind::ArgMinMax ? (nd.op == ExprOp::REDUCE_ARGMAX ? 1 : 0) : -1;
                d->input_dtype = static_cast<int>(src.getDataType());
                d->output_dtype = static_cast<int>(*nd.output_dtype);
                d->rank = static_cast<uint32_t>(in_shape.size());
                for (size_t i = 0; i < in_shape.size(); ++i) {
                    d->dims[i] = in_shape[i];
                    d->reduced[i] = reduced[i] ? 1 : 0;
                }
                PhysicalStage st;
                st.kind = ls.kind;
                st.physical_name = ls.kind == StageKind::Reduction ? "strided" : "arg_strided";
                const void* in_ptr = src.getMemPtr();
                void* out_ptr = dst_s.getMemPtr();
                st.custom_launch = [d, in_ptr, out_ptr](void* stream) {
                    check(thor_b200_strided_reduce_launch(d.get(), in_ptr, out_ptr, 1.0f, stream), "StampedExecutionPlan::run strided reduction");
                };
                impl->keep_alive.push_back(src);
                st.reads.push_back(in_ptr);
                st.writes.push_back(out_ptr);
                impl->stages.push_back(std::move(st));
                continue;
            }
            const bool is_out = output_name_of.count(k) != 0;
            Tensor dst = allocateFor(k, is_out);
            node_tensor[k] = dst;
            if (is_out) impl->outputs[output_name_of[k]] = dst;
            PhysicalStage st;
            st.kind = ls.kind;
            st.in = src.getMemPtr();
            st.out = dst.getMemPtr();
            impl->keep_alive.push_back(src);
            size_t ws = 1;
            if (ls.kind == StageKind::ReduceMinMaxBackward) {
                thor_b200_minmax_backward_desc d{};
                d.is_max = nd.op == ExprOp::REDUCE_MAX_BACKWARD ? 1 : 0;
                d.input_dtype = static_cast<int>(src.getDataType());
                d.grad_input_dtype = static_cast<int>(*nd.output_dtype);
                d.outer = outer;
                d.reduction = red;
                d.inner = inner;
                if (g.nodes[nd.rhs].op == ExprOp::SCALAR_FP) {
                    // a literal gradient (the default seed 1 of a backward pass) needs no tensor
                    d.grad_mode = 2;
                    d.grad_value = static_cast<float>(g.nodes[nd.rhs].scalar_fp);
                    d.grad_output_dtype = static_cast<int>(DataType::FP32);
                } else {
                    const Tensor& grad = node_tensor[nd.rhs];
                    if (!grad.isInitialized()) throw std::logic_error("FusedEquation::stamp: min/max backward gradient is not materialised");
                    if (grad.getTotalNumElements() == outer * inner) d.grad_mode = 0;
                    else if (grad.getTotalNumElements() == 1) d.grad_mode = 1;
                    else throw std::logic_error("FusedEquation::stamp: min/max backward needs one gradient value per reduced segment, or one for all");
                    d.grad_output_dtype = static_cast<int>(grad.getDataType());
                    st.in2 = grad.getMemPtr();
                    impl->keep_alive.push_back(grad);
                }
                st.minmax_backward = std::make_shared<MinMaxBackwardPlanHandle>();
                check(thor_b200_minmax_backward_plan_create(&d, &st.minmax_backward->h, &ws), "FusedEquation::stamp min/max backward plan");
                st.physical_name = "minmax_backward";
                st.launches = 2;
            } else if (ls.kind == StageKind::Reduction) {
                thor_b200_reduce_desc d{};
                d.op = reduceOpFor(nd.op);
                d.input_dtype = static_cast<int>(src.getDataType());
                d.output_dtype = static_cast<int>(*nd.output_dtype);
                d.outer = outer;
                d.reduction = red;
                d.inner = inner;
                st.reduce = std::make_shared<ReducePlanHandle>();
                check(thor_b200_reduce_plan_create(&d, &st.reduce->h, &ws), "FusedEquation::stamp reduction plan");
                st.physical_name = thor_b200_reduce_plan_kind(st.reduce->h);
                st.launches = st.physical_name.find("split") != std::string::npos || st.physical_name == "full" ? 2 : 1;
            } else {
                thor_b200_argreduce_desc d{};
                d.op = nd.op == ExprOp::REDUCE_ARGMAX ? 1 : 0;
                d.input_dtype = static_cast<int>(src.getDataType());
                d.value_dtype = 0;
                d.index_dtype = static_cast<int>(*nd.output_dtype);
                d.outer = outer;
                d.reduction = red;
                d.inner = inner;
                st.argreduce = std::make_shared<ArgReducePlanHandle>();
                check(thor_b200_argreduce_plan_create(&d, &st.argreduce->h, &ws), "FusedEquation::stamp arg-reduction plan");
                st.physical_name = "arg_reduce";
            }
            st.workspace_bytes = ws;
            st.workspace = Tensor::allocate(DataType::UINT8, {static_cast<uint64_t>(ws)}, device_num_);
            if (ws > 1) impl->intermediate_bytes += ws;
            st.reads.push_back(st.in);
            if (st.in2) st.reads.push_back(st.in2);
            st.writes.push_back(st.out);
            impl->stages.push_back(std::move(st));
            continue;
        }

        // ---- fused elementwise / broadcast stage -------------------------------------------------
        std::vector<uint32_t> stage_outputs;
        for (uint32_t k : ls.nodes)
            if (!covered[k]) stage_outputs.push_back(k);
        // ancestors back to materialised roots
        std::vector<bool> in_stage(g.nodes.size(), false);
        std::vector<uint32_t> stack(stage_outputs.begin(), stage_outputs.end());
        while (!stack.empty()) {
            const uint32_t k = stack.back();
            stack.pop_back();
            if (in_stage[k]) continue;
            in_stage[k] = true;
            const bool root = node_tensor[k].isInitialized() || isLeafOp(g.nodes[k].op);
            if (root) continue;
            for (uint32_t p : {g.nodes[k].lhs, g.nodes[k].rhs, g.nodes[k].aux})
                if (p != UINT32_MAX) stack.push_back(p);
        }
        std::vector<thor_b200_expr_node> nodes;
        std::vector<thor_b200_expr_input> ins;
        std::vector<const void*> in_ptrs;
        std::vector<float> scalars;
        std::vector<std::string> scalar_names;
        std::vector<std::vector<uint64_t>> in_shapes;
        std::map<uint32_t, uint32_t> remap;
        std::map<const void*, uint32_t> slot_of_ptr;
        std::map<std::string, uint32_t> slot_of_scalar;
        const std::vector<uint64_t>& out_dims = shape[stage_outputs[0]];
        for (uint32_t k = 0; k < g.nodes.size(); ++k) {
            if (!in_stage[k]) continue;
            const ExprNode& nd = g.nodes[k];
            thor_b200_expr_node cn{};
            cn.lhs = cn.rhs = cn.aux = THOR_B200_NO_NODE;
            cn.input_slot = THOR_B200_NO_NODE;
            cn.output_dtype = static_cast<uint16_t>(*nd.output_dtype);
            cn.compute_dtype = static_cast<uint16_t>(nd.compute_dtype.value_or(*nd.output_dtype));
            const bool is_stage_output = std::find(stage_outputs.begin(), stage_outputs.end(), k) != stage_outputs.end();
            if (node_tensor[k].isInitialized() && !(is_stage_output && plan.isElementwise(k))) {
                // materialised tensor (external input, reduction result, view): a stage input
                const Tensor& t = node_tensor[k];
                const bool one_elem_scalar = nd.op == ExprOp::TENSOR_RUNTIME_SCALAR;
                uint32_t slot;
                auto it = slot_of_ptr.find(t.getMemPtr());
                if (it != slot_of_ptr.end() && static_cast<int>(t.getDataType()) == ins[it->second].dtype) {
                    slot = it->second;
                } else {
                    slot = static_cast<uint32_t>(ins.size());
                    ins.push_back({one_elem_scalar ? THOR_B200_INPUT_TENSOR_RUNTIME_SCALAR : THOR_B200_INPUT_TENSOR, static_cast<int>(t.getDataType())});
                    in_ptrs.push_back(t.getMemPtr());
                    scalars.push_back(0.0f);
                    scalar_names.push_back("");
                    in_shapes.push_back(one_elem_scalar ? std::vector<uint64_t>{} : shape[k]);
                    slot_of_ptr[t.getMemPtr()] = slot;
                    impl->keep_alive.push_back(t);
                }
                cn.op = one_elem_scalar ? THOR_B200_OP_TENSOR_RUNTIME_SCALAR : THOR_B200_OP_INPUT;
                cn.input_slot = slot;
                cn.input_dtype = static_cast<uint16_t>(t.getDataType());
                // a materialised value is read back in its storage dtype
                cn.output_dtype = static_cast<uint16_t>(nd.op == ExprOp::INPUT || one_elem_scalar ? *nd.output_dtype : t.getDataType());
            } else if (nd.op == ExprOp::INPUT || nd.op == ExprOp::TENSOR_RUNTIME_SCALAR) {
                // input whose output dtype differs from its storage dtype: converted on load
                const Tensor& t = bound[nd.input_slot].tensor;
                const bool one_elem_scalar = nd.op == ExprOp::TENSOR_RUNTIME_SCALAR;
                const uint32_t slot = static_cast<uint32_t>(ins.size());
                ins.push_back({one_elem_scalar ? THOR_B200_INPUT_TENSOR_RUNTIME_SCALAR : THOR_B200_INPUT_TENSOR, static_cast<int>(t.getDataType())});
                in_ptrs.push_back(t.getMemPtr());
                scalars.push_back(0.0f);
                scalar_names.push_back("");
                in_shapes.push_back(one_elem_scalar ? std::vector<uint64_t>{} : shape[k]);
                impl->keep_alive.push_back(t);
                cn.op = one_elem_scalar ? THOR_B200_OP_TENSOR_RUNTIME_SCALAR : THOR_B200_OP_INPUT;
                cn.input_slot = slot;
                cn.input_dtype = static_cast<uint16_t>(t.getDataType());
            } else if (nd.op == ExprOp::RUNTIME_SCALAR) {
                const std::string& name = g.inputs[nd.input_slot].name;
                uint32_t slot;
                auto it = slot_of_scalar.find(name);
                if (it != slot_of_scalar.end()) {
                    slot = it->second;
                } else {
                    slot = static_cast<uint32_t>(ins.size());
                    ins.push_back({THOR_B200_INPUT_RUNTIME_SCALAR_FP32, THOR_B200_FP32});
                    in_ptrs.push_back(nullptr);
                    scalars.push_back(bound[nd.input_slot].scalar);
                    scalar_names.push_back(name);
                    in_shapes.push_back({});
                    slot_of_scalar[name] = slot;
                }
                cn.op = THOR_B200_OP_RUNTIME_SCALAR;
                cn.input_slot = slot;
                cn.input_dtype = THOR_B200_FP32;
            } else if (nd.op == ExprOp::SCALAR_FP) {
                cn.op = THOR_B200_OP_SCALAR_FP;
                cn.scalar_fp = nd.scalar_fp;
            } else {
                cn.op = static_cast<uint16_t>(nd.op);
                if (nd.lhs != UINT32_MAX) cn.lhs = remap.at(nd.lhs);
                if (nd.rhs != UINT32_MAX) cn.rhs = remap.at(nd.rhs);
                if (nd.aux != UINT32_MAX) cn.aux = remap.at(nd.aux);
            }
            remap[k] = static_cast<uint32_t>(nodes.size());
            nodes.push_back(cn);
        }
        std::vector<thor_b200_expr_output> outs;
        std::vector<void*> out_ptrs;
        for (uint32_t k : stage_outputs) {
            const bool is_out = output_name_of.count(k) != 0;
            Tensor dst = allocateFor(k, is_out);
            node_tensor[k] = dst;
            if (is_out) impl->outputs[output_name_of[k]] = dst;
            outs.push_back({remap.at(k), static_cast<int>(*g.nodes[k].output_dtype)});
            out_ptrs.push_back(dst.getMemPtr());
        }
        // broadcast geometry: flat when every tensor input covers the whole output
        const uint64_t out_numel = numelOf(out_dims);
        bool flat = true;
        for (size_t s = 0; s < ins.size(); ++s)
            if (ins[s].kind == THOR_B200_INPUT_TENSOR && numelOf(in_shapes[s]) != out_numel) flat = false;
        thor_b200_expr_broadcast bc{};
        std::vector<int64_t> strides(ins.size() * THOR_B200_MAX_RANK, 0);
        if (!flat) {
            if (out_dims.size() > THOR_B200_MAX_RANK) throw std::logic_error("FusedEquation::stamp: broadcast rank above 8");
            bc.rank = static_cast<uint32_t>(out_dims.size());
            for (size_t d = 0; d < out_dims.size(); ++d) bc.dims[d] = out_dims[d];
            for (size_t s = 0; s < ins.size(); ++s) {
                if (ins[s].kind != THOR_B200_INPUT_TENSOR) continue;
                const auto& d = in_shapes[s];
                const size_t pad = out_dims.size() - d.size();
                int64_t stride = 1;
                for (size_t i = d.size(); i-- > 0;) {
                    strides[s * THOR_B200_MAX_RANK + pad + i] = (d[i] == 1 && out_dims[pad + i] != 1) ? 0 : (d[i] == 1 ? 0 : stride);
                    stride *= static_cast<int64_t>(d[i]);
                }
            }
            bc.input_strides = strides.data();
        }
        thor_b200_expr_options opt{};
        opt.use_fast_math = options_.use_fast_math;
        opt.compile_only = Tensor::planOnly() ? 1 : 0;
        PhysicalStage st;
        st.kind = StageKind::FusedKernel;
        st.expr = std::make_shared<ExprHandle>();
        check(thor_b200_expr_compile(nodes.data(), static_cast<uint32_t>(nodes.size()), ins.data(), static_cast<uint32_t>(ins.size()), outs.data(),
                                     static_cast<uint32_t>(outs.size()), flat ? nullptr : &bc, &opt, &st.expr->h),
              "FusedEquation::stamp fused stage");
        st.physical_name = thor_b200_expr_launch_kind(st.expr->h);
        st.source = thor_b200_expr_source(st.expr->h);
        st.input_ptrs = in_ptrs;
        st.scalars = scalars;
        st.scalar_names = scalar_names;
        st.output_ptrs = out_ptrs;
        st.numel = out_numel;
        for (const void* q : in_ptrs)
            if (q) st.reads.push_back(q);
        for (void* q : out_ptrs) st.writes.push_back(q);
        impl->stages.push_back(std::move(st));
    }

    // outputs that are plain inputs or were produced by boundary stages
    for (const auto& o : phys.outputs) {
        if (impl->outputs.count(o.name)) continue;
        if (!node_tensor[o.node_idx].isInitialized()) throw std::logic_error("FusedEquation::stamp: output '" + o.name + "' was not produced");
        impl->outputs[o.name] = node_tensor[o.node_idx];
    }
    for (auto& t : node_tensor)
        if (t.isInitialized()) impl->keep_alive.push_back(t);

    // Lanes: a stage depends on the earlier stages that wrote what it reads (and on those that read or wrote what it
    // writes); stages that share no such edge run on different streams.  Views launch nothing and are left out.
    for (uint32_t i = 0; i < impl->stages.size(); ++i)
        if (impl->stages[i].kind != StageKind::View) impl->scheduled.push_back(i);
    auto overlap = [](const std::vector<const void*>& a, const std::vector<const void*>& b) {
        for (const void* x : a)
            for (const void* y : b)
                if (x == y) return true;
        return false;
    };
    impl->dependencies.assign(impl->scheduled.size(), {});
    for (uint32_t k = 0; k < impl->scheduled.size(); ++k) {
        const PhysicalStage& later = impl->stages[impl->scheduled[k]];
        for (uint32_t e = 0; e < k; ++e) {
            const PhysicalStage& earlier = impl->stages[impl->scheduled[e]];
            if (overlap(later.reads, earlier.writes) || overlap(later.writes, earlier.writes) || overlap(later.writes, earlier.reads)) impl->dependencies[k].push_back(e);
        }
    }
    impl->schedule = buildStampedExecutionSchedule(impl->dependencies, static_cast<uint32_t>(device_num_));
    uint64_t input_bytes = 0;
    for (const auto& kv : inputs)
        if (!kv.second.is_scalar && kv.second.tensor.isInitialized()) input_bytes += kv.second.tensor.getArraySizeInBytes();
    if (options_.branch_streams && !Tensor::planOnly() && impl->schedule.lane_gpu_nums.size() > 1 && input_bytes >= options_.branch_streams_min_input_bytes) {
        auto lr = std::make_shared<LaneResources>();
        lr->lane_streams.assign(impl->schedule.lane_gpu_nums.size(), nullptr);
        lr->lane_end.assign(impl->schedule.lane_gpu_nums.size(), nullptr);
        lr->done_events.assign(impl->scheduled.size(), nullptr);
        for (size_t lane = 1; lane < lr->lane_streams.size(); ++lane) {
            check(thor_b200_stream_create(&lr->lane_streams[lane]), "FusedEquation::stamp helper stream");
            check(thor_b200_event_create(&lr->lane_end[lane]), "FusedEquation::stamp event");
        }
        for (size_t k = 0; k < impl->scheduled.size(); ++k)
            if (impl->schedule.stage_needs_completion_event[k]) check(thor_b200_event_create(&lr->done_events[k]), "FusedEquation::stamp event");
        check(thor_b200_event_create(&lr->caller_ready), "FusedEquation::stamp event");
        impl->lanes = lr;
    }
    return StampedExecutionPlan(impl);
}

void FusedEquation::run(const std::unordered_map<std::string, RuntimeInputValue>& inputs, const std::unordered_map<std::string, Tensor>& outputs,
                        const Stream& stream) {
    StampedExecutionPlan plan = stamp(inputs, stream, outputs);
    const auto kinds = plan.stageKindNames();
    if (kinds.size() != 1 || kinds[0] != "FusedKernel")
        throw std::logic_error("FusedEquation::run supports single fused-stage expressions only; use stamp() for staged reductions");
    plan.run();
}

}  // namespace ThorB200
