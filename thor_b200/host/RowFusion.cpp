#include "RowFusion.h"

#include <algorithm>
#include <map>
#include <stdexcept>

#include "thor_b200.h"

namespace ThorB200 {

namespace {

uint64_t numelOf(const std::vector<uint64_t>& d) {
    uint64_t n = 1;
    for (uint64_t v : d) n *= v;
    return n;
}

struct ProgHandle {
    thor_b200_rowprog* h = nullptr;
    ~ProgHandle() { thor_b200_rowprog_destroy(h); }
};

}  // namespace

namespace {
std::vector<RowFusionMatch> matchOutputs(const RowFusionContext& ctx);
}

// The whole equation is tried as one row program first (three full reductions of one tensor share a
// single pass that way).  If it does not fit, the outputs are split into groups that share computed
// nodes (sharing only inputs does not tie two outputs together); every group is tried as a row program
// of its own, and groups that do not fit run through the ordinary stage list.
// {"y": softmax(x), "idx": argmax(x)} therefore still gets its single-pass softmax.
std::vector<RowFusionMatch> matchRowFusions(const RowFusionContext& ctx) {
    {
        std::vector<RowFusionMatch> whole = matchOutputs(ctx);
        if (!whole.empty() || ctx.outputs.size() < 2) return whole;
    }
    const PhysicalExpression& g = ctx.graph;
    const size_t n = g.nodes.size();
    const size_t n_out = ctx.outputs.size();
    std::vector<std::vector<bool>> reach(n_out, std::vector<bool>(n, false));
    for (size_t o = 0; o < n_out; ++o) {
        reach[o][ctx.outputs[o].node_idx] = true;
        for (size_t k = n; k-- > 0;) {
            if (!reach[o][k]) continue;
            for (uint32_t p : {g.nodes[k].lhs, g.nodes[k].rhs, g.nodes[k].aux})
                if (p != UINT32_MAX) reach[o][p] = true;
        }
    }
    std::vector<int> group(n_out, -1);
    int n_groups = 0;
    for (size_t o = 0; o < n_out; ++o) {
        if (group[o] >= 0) continue;
        group[o] = n_groups;
        bool grew = true;
        while (grew) {
            grew = false;
            for (size_t a = 0; a < n_out; ++a) {
                if (group[a] != n_groups) continue;
                for (size_t b = 0; b < n_out; ++b) {
                    if (group[b] >= 0) continue;
                    bool shared = false;
                    for (size_t k = 0; k < n && !shared; ++k) shared = reach[a][k] && reach[b][k] && !isLeafOp(g.nodes[k].op);
                    if (shared) {
                        group[b] = n_groups;
                        grew = true;
                    }
                }
            }
        }
        ++n_groups;
    }
    std::vector<RowFusionMatch> all;
    for (int gi = 0; gi < n_groups; ++gi) {
        std::vector<NamedOutput> subset;
        for (size_t o = 0; o < n_out; ++o)
            if (group[o] == gi) subset.push_back(ctx.outputs[o]);
        RowFusionContext sub{ctx.graph, subset, ctx.shape, ctx.bound, ctx.device_num, ctx.use_fast_math};
        for (RowFusionMatch& m : matchOutputs(sub)) all.push_back(std::move(m));
    }
    return all;
}

namespace {

std::vector<RowFusionMatch> matchOutputs(const RowFusionContext& ctx) {
    const PhysicalExpression& g = ctx.graph;
    const size_t n = g.nodes.size();
    std::vector<bool> needed(n, false);
    for (const auto& o : ctx.outputs) needed[o.node_idx] = true;
    for (size_t k = n; k-- > 0;) {
        if (!needed[k]) continue;
        for (uint32_t p : {g.nodes[k].lhs, g.nodes[k].rhs, g.nodes[k].aux})
            if (p != UINT32_MAX) needed[p] = true;
    }
    // The [rows, cols] frame: the shape of the first reduction's argument, cut at `split` into leading axes
    // (rows) and trailing axes (cols).  The cut comes from the first reduction that reduces exactly a
    // trailing block of axes (row statistics: softmax over the last axis, instance softmax, LayerNorm over
    // the last two axes ...) or exactly a leading block (column sums); the last axis otherwise.
    std::vector<uint64_t> frame;
    for (size_t k = 0; k < n && frame.empty(); ++k)
        if (needed[k] && isReductionOp(g.nodes[k].op)) frame = ctx.shape[g.nodes[k].lhs];
    if (frame.empty()) return {};
    size_t split = frame.size() - 1;
    for (size_t k = 0; k < n; ++k) {
        if (!needed[k] || !isValueReductionOp(g.nodes[k].op) || ctx.shape[g.nodes[k].lhs] != frame) continue;
        const std::vector<bool> reduced = reducedAxesMask(g.nodes[k], frame.size());
        size_t first_red = frame.size(), last_red = 0, first_keep = frame.size(), last_keep = 0;
        bool any_red = false, any_keep = false;
        for (size_t i = 0; i < frame.size(); ++i) {
            if (frame[i] == 1) continue;
            if (reduced[i]) {
                if (!any_red) first_red = i;
                last_red = i;
                any_red = true;
            } else {
                if (!any_keep) first_keep = i;
                last_keep = i;
                any_keep = true;
            }
        }
        if (!any_red || !any_keep) continue;  // reduces everything or nothing: tells nothing about the cut
        if (last_keep < first_red) {
            split = first_red;
            break;
        }
        if (last_red < first_keep) {
            split = first_keep;
            break;
        }
        return {};  // interleaved reduced and kept axes
    }
    uint64_t cols = 1;
    for (size_t i = split; i < frame.size(); ++i) cols *= frame[i];
    const uint64_t total = numelOf(frame);
    const uint64_t rows = total / cols;

    auto classify = [&](const std::vector<uint64_t>& d) -> int {
        const uint64_t ne = numelOf(d);
        if (ne == 1) return THOR_B200_SHAPE_SCALAR;
        if (d.size() > frame.size()) return -1;
        const size_t pad = frame.size() - d.size();
        bool full = true, row = true, col = true;
        for (size_t i = 0; i < frame.size(); ++i) {
            const uint64_t v = i < pad ? 1 : d[i - pad];
            const bool trailing = i >= split;
            if (v != frame[i]) full = false;
            if (trailing ? v != 1 : v != frame[i]) row = false;
            if (trailing ? v != frame[i] : v != 1) col = false;
        }
        if (full) return THOR_B200_SHAPE_FULL;
        if (row) return THOR_B200_SHAPE_ROW;
        if (col) return THOR_B200_SHAPE_COL;
        return -1;
    };

    std::vector<thor_b200_expr_node> nodes;
    std::vector<thor_b200_expr_input> inputs;
    std::vector<int32_t> input_shapes;
    std::vector<std::string> scalar_names;
    auto scalars = std::make_shared<std::vector<float>>();
    std::vector<uint32_t> input_graph_slot;  // program slot -> graph input slot
    std::map<uint32_t, uint32_t> remap;      // graph node -> program node
    std::map<uint32_t, uint32_t> slot_of_graph_input;
    for (uint32_t k = 0; k < n; ++k) {
        if (!needed[k]) continue;
        const ExprNode& nd = g.nodes[k];
        if (isMinMaxBackwardOp(nd.op)) return {};
        if (isArgReductionOp(nd.op) && *nd.output_dtype != DataType::UINT32) return {};
        if (isViewOp(nd.op)) {
            // squeeze / unsqueeze / reshape of a value whose class does not change is an alias
            const int a = classify(ctx.shape[nd.lhs]), b = classify(ctx.shape[k]);
            if (a < 0 || a != b) {
                // [1, C] column sums squeezed to [C] keep class COL; anything else is not a row program
                return {};
            }
            remap[k] = remap.at(nd.lhs);
            continue;
        }
        thor_b200_expr_node cn{};
        cn.lhs = cn.rhs = cn.aux = THOR_B200_NO_NODE;
        cn.input_slot = THOR_B200_NO_NODE;
        cn.output_dtype = static_cast<uint16_t>(*nd.output_dtype);
        cn.compute_dtype = static_cast<uint16_t>(nd.compute_dtype.value_or(*nd.output_dtype));
        if (nd.op == ExprOp::INPUT || nd.op == ExprOp::TENSOR_RUNTIME_SCALAR || nd.op == ExprOp::RUNTIME_SCALAR) {
            uint32_t slot;
            auto it = slot_of_graph_input.find(nd.input_slot);
            if (it != slot_of_graph_input.end()) {
                slot = it->second;
            } else {
                slot = static_cast<uint32_t>(inputs.size());
                slot_of_graph_input[nd.input_slot] = slot;
                input_graph_slot.push_back(nd.input_slot);
                if (nd.op == ExprOp::RUNTIME_SCALAR) {
                    inputs.push_back({THOR_B200_INPUT_RUNTIME_SCALAR_FP32, THOR_B200_FP32});
                    input_shapes.push_back(THOR_B200_SHAPE_SCALAR);
                    scalar_names.push_back(g.inputs[nd.input_slot].name);
                    scalars->push_back(ctx.bound[nd.input_slot].scalar);
                } else {
                    const Tensor& t = ctx.bound[nd.input_slot].tensor;
                    const int cls = nd.op == ExprOp::TENSOR_RUNTIME_SCALAR ? THOR_B200_SHAPE_SCALAR : classify(t.getDimensions());
                    if (cls < 0) return {};
                    inputs.push_back({nd.op == ExprOp::TENSOR_RUNTIME_SCALAR ? THOR_B200_INPUT_TENSOR_RUNTIME_SCALAR : THOR_B200_INPUT_TENSOR,
                                      static_cast<int>(t.getDataType())});
                    input_shapes.push_back(cls);
                    scalar_names.push_back("");
                    scalars->push_back(0.0f);
                }
            }
            cn.op = static_cast<uint16_t>(nd.op);
            cn.input_slot = slot;
            cn.input_dtype = static_cast<uint16_t>(inputs[slot].dtype);
        } else if (nd.op == ExprOp::SCALAR_FP) {
            cn.op = THOR_B200_OP_SCALAR_FP;
            cn.scalar_fp = nd.scalar_fp;
        } else if (isReductionOp(nd.op)) {
            const auto& in_shape = ctx.shape[nd.lhs];
            if (classify(in_shape) != THOR_B200_SHAPE_FULL) return {};
            const size_t pad = frame.size() - in_shape.size();
            if (pad != 0) return {};
            const std::vector<bool> reduced = reducedAxesMask(nd, in_shape.size());
            bool only_last = true, all_but_last = true, all = true;
            for (size_t i = 0; i < in_shape.size(); ++i) {
                if (in_shape[i] == 1) continue;
                const bool last = i >= split;  // trailing block = the columns of the frame
                if (last ? !reduced[i] : reduced[i]) only_last = false;
                if (last ? reduced[i] : !reduced[i]) all_but_last = false;
                if (!reduced[i]) all = false;
            }
            if (!only_last && !all_but_last && !all) return {};
            if (isArgReductionOp(nd.op) && !only_last) return {};  // arg reductions are fused along the columns only
            cn.op = static_cast<uint16_t>(nd.op);
            cn.lhs = remap.at(nd.lhs);
            cn.input_slot = all ? 2u : (only_last ? 0u : 1u);
        } else {
            if (classify(ctx.shape[k]) < 0) return {};
            cn.op = static_cast<uint16_t>(nd.op);
            if (nd.lhs != UINT32_MAX) cn.lhs = remap.at(nd.lhs);
            if (nd.rhs != UINT32_MAX) cn.rhs = remap.at(nd.rhs);
            if (nd.aux != UINT32_MAX) cn.aux = remap.at(nd.aux);
        }
        remap[k] = static_cast<uint32_t>(nodes.size());
        nodes.push_back(cn);
    }
    // an equation whose only reductions are arg reductions keeps the dedicated arg-reduction kernels
    {
        bool any_value_reduction = false;
        for (uint32_t k = 0; k < n; ++k) any_value_reduction = any_value_reduction || (needed[k] && isValueReductionOp(g.nodes[k].op));
        if (!any_value_reduction) return {};
    }
    std::vector<thor_b200_expr_output> outs;
    for (const auto& o : ctx.outputs) {
        const ExprNode& on = g.nodes[o.node_idx];
        if (isLeafOp(on.op)) return {};
        outs.push_back({remap.at(o.node_idx), static_cast<int>(*on.output_dtype)});
    }
    // two outputs that alias one program node (e.g. a value and its squeezed view) are not handled here
    for (size_t i = 0; i < outs.size(); ++i)
        for (size_t j = i + 1; j < outs.size(); ++j)
            if (outs[i].node == outs[j].node) return {};

    thor_b200_rowprog_desc d{};
    d.nodes = nodes.data();
    d.n_nodes = static_cast<uint32_t>(nodes.size());
    d.inputs = inputs.data();
    d.input_shapes = input_shapes.data();
    d.n_inputs = static_cast<uint32_t>(inputs.size());
    d.outputs = outs.data();
    d.n_outputs = static_cast<uint32_t>(outs.size());
    d.rows = rows;
    d.cols = cols;
    d.options.use_fast_math = ctx.use_fast_math;
    d.options.compile_only = Tensor::planOnly() ? 1 : 0;
    d.tuning.ring_buffers = ctx.tuning.ring_buffers;
    d.tuning.pipeline_round_one = ctx.tuning.pipeline_round_one;
    d.tuning.copy_warpgroup = ctx.tuning.copy_warpgroup;
    d.tuning.keep_values = ctx.tuning.keep_values;
    d.tuning.reciprocal_division = ctx.tuning.reciprocal_division;
    d.tuning.wait_limit_ms = ctx.tuning.wait_limit_ms;
    d.tuning.test_skip_fill = ctx.tuning.test_skip_fill;
    d.tuning.reserve_sms = ctx.tuning.reserve_sms;
    auto prog = std::make_shared<ProgHandle>();
    size_t ws_bytes = 1;
    const int status = thor_b200_rowprog_compile(&d, &prog->h, &ws_bytes);
    if (status == THOR_B200_UNSUPPORTED) return {};
    if (status != THOR_B200_OK) throw std::runtime_error(std::string("row program: ") + thor_b200_last_error());

    RowFusionMatch m;
    m.name = "row_program";
    m.source = thor_b200_rowprog_source(prog->h);
    m.launches = thor_b200_rowprog_launch_count(prog->h);
    m.scalar_names = scalar_names;
    m.scalars = scalars;
    m.waits_expired = [prog]() {
        uint32_t count = 0;
        if (thor_b200_rowprog_waits_expired(prog->h, &count) != THOR_B200_OK) throw std::runtime_error(std::string("row program: ") + thor_b200_last_error());
        return count;
    };
    std::vector<uint32_t> out_nodes;
    for (const auto& o : ctx.outputs) {
        m.produced.push_back({o.node_idx, true});
        out_nodes.push_back(o.node_idx);
        const thor_b200_expr_node& pn = nodes[remap.at(o.node_idx)];
        const bool column_reduction = (pn.op == THOR_B200_OP_REDUCE_SUM || pn.op == THOR_B200_OP_REDUCE_AVG) && pn.input_slot == 1;
        if (ctx.unrounded_column_sums && column_reduction) m.column_sum_names.push_back(o.name);
    }
    if (!m.column_sum_names.empty()) m.column_sums = std::make_shared<Tensor>();
    const std::shared_ptr<Tensor> column_sums = m.column_sums;
    const uint64_t n_column_sums = m.column_sum_names.size(), n_cols = cols;
    for (uint32_t k = 0; k < n; ++k)
        if (needed[k] && !isLeafOp(g.nodes[k].op)) m.absorbed.push_back(k);
    const int device = ctx.device_num;
    std::vector<Tensor> in_tensors;
    for (uint32_t gs : input_graph_slot) in_tensors.push_back(ctx.bound[gs].tensor);
    m.bind = [prog, ws_bytes, out_nodes, in_tensors, scalars, device, column_sums, n_column_sums, n_cols](std::vector<Tensor>& node_tensor, std::vector<Tensor>& keep_alive,
                                                                       uint64_t& intermediate_bytes) -> std::function<void(void*)> {
        Tensor ws = Tensor::allocate(DataType::UINT8, {static_cast<uint64_t>(ws_bytes)}, device);
        if (ws_bytes > 1) intermediate_bytes += ws_bytes;
        std::vector<const void*> in_ptrs;
        for (const Tensor& t : in_tensors) {
            in_ptrs.push_back(t.isInitialized() ? t.getMemPtr() : nullptr);
            if (t.isInitialized()) keep_alive.push_back(t);
        }
        std::vector<void*> out_ptrs;
        for (uint32_t k : out_nodes) out_ptrs.push_back(node_tensor[k].getMemPtr());
        keep_alive.push_back(ws);
        void* sums_ptr = nullptr;
        if (column_sums) {
            *column_sums = Tensor::allocate(DataType::FP32, {n_column_sums, n_cols}, device);
            sums_ptr = column_sums->getMemPtr();
        }
        return [prog, in_ptrs, out_ptrs, ws, ws_bytes, scalars, sums_ptr](void* stream) {
            const int st = thor_b200_rowprog_launch_sharded(prog->h, in_ptrs.data(), scalars->data(), out_ptrs.data(), ws.getMemPtr(), ws_bytes, sums_ptr, stream);
            if (st != THOR_B200_OK) throw std::runtime_error(std::string("row program launch: ") + thor_b200_last_error());
        };
    };
    std::vector<RowFusionMatch> out;
    out.push_back(std::move(m));
    return out;
}

}  // namespace

}  // namespace ThorB200
