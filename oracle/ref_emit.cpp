// Source dumper for the REFERENCE's own flat fused-kernel emitter.
//
// TEST AND BASELINE INFRASTRUCTURE ONLY (never shipped, never linked by the product).  No reference
// source is copied here: the build compiles the reference's Expression.cpp,
// ExpressionDTypeResolution.cpp and CudaSourceEmitter.cpp where they lie and links them with this
// file, which builds an expression through the reference's public Expression API from a small
// postfix description, resolves dtypes with resolveOutputsDTypesInPlace and returns what
// CudaSourceEmitter::emitFlat generates (Utilities/Expression/CudaSourceEmitter.h:21-22,
// CudaSourceEmitter.cpp:6727-6859) plus CudaSourceEmitter::flatElementsPerThread for the launch grid.
// The tests compile that source with NVRTC and run it beside our kernel on the same device buffers.
//
// Only the entry point below is exported; the link drops every function it cannot reach
// (--gc-sections) and -z defs proves that what remains needs nothing else of the reference.
#include <algorithm>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "Utilities/Expression/CudaSourceEmitter.h"
#include "Utilities/Expression/EquationCompiler.h"
#include "Utilities/Expression/ExpressionDTypeResolution.h"
#include "ref_postfix.h"

using namespace ThorImplementation;

namespace {

thread_local std::string g_text;
using thor_ref_dump::buildFromPostfix;

}  // namespace

namespace {

uint64_t product(const std::vector<uint64_t>& d) {
    uint64_t n = 1;
    for (uint64_t v : d) n *= v;
    return n;
}
std::vector<uint64_t> broadcastOf(const std::vector<uint64_t>& a, const std::vector<uint64_t>& b) {
    const size_t r = std::max(a.size(), b.size());
    std::vector<uint64_t> out(r, 1);
    for (size_t i = 0; i < r; ++i) {
        const uint64_t x = i < r - a.size() ? 1 : a[i - (r - a.size())];
        const uint64_t y = i < r - b.size() ? 1 : b[i - (r - b.size())];
        if (x != y && x != 1 && y != 1) throw std::invalid_argument("inputs do not broadcast");
        out[i] = std::max(x, y);
    }
    return out;
}
// Packed strides of an input of dims `in` inside the output domain `out` (right aligned, 0 along broadcast axes).
std::vector<uint64_t> broadcastStrides(const std::vector<uint64_t>& in, const std::vector<uint64_t>& out) {
    std::vector<uint64_t> strides(out.size(), 0);
    uint64_t s = 1;
    for (size_t i = in.size(); i-- > 0;) {
        const size_t o = out.size() - in.size() + i;
        strides[o] = in[i] == 1 ? 0 : s;
        s *= in[i];
    }
    return strides;
}

}  // namespace

// Emits the reference's SPECIALIZED BROADCAST kernel for `program` with concrete input dims.  The group descriptor that
// the reference's stamp would build from live tensors (FusedEquation.cpp:5802-6020: every referenced input slot is used
// and offset-indexed; packed right-aligned broadcast strides; pair-vector loads for inputs whose innermost stride is 1
// when the innermost output extent is even; one active axis per non-singleton output axis that some input walks) is
// reconstructed here from those rules for dense inputs and a single output.  input_dims holds, per input, its rank
// followed by its dims (rank 0 for runtime scalars).  elements_per_thread and the u64 numel argument follow
// EquationCompiler.cpp:8090-8110 and EquationRunner.cpp:262-289.
extern "C" __attribute__((visibility("default"))) int thor_ref_emit_broadcast(const char* program, const char* const* input_names, const int* input_dtypes,
                                                                              const unsigned long long* input_dims, int n_inputs, const char** source,
                                                                              unsigned* elements_per_thread, int* input_order, int* output_dtype,
                                                                              unsigned long long* out_numel) {
    try {
        Expression e = buildFromPostfix(program);
        PhysicalOutputs outputs = Expression::outputs({{"output", e}}).physicalOutputs();
        const size_t n_slots = outputs.expr->inputs.size();
        std::vector<DataType> dtypes(n_slots, DataType::FP32);
        std::vector<std::vector<uint64_t>> slot_dims(n_slots);
        std::vector<std::vector<uint64_t>> given(n_inputs);
        {
            const unsigned long long* p = input_dims;
            for (int i = 0; i < n_inputs; ++i) {
                const unsigned long long rank = *p++;
                given[i].assign(p, p + rank);
                p += rank;
            }
        }
        for (const NamedInput& in : outputs.expr->inputs) {
            int found = -1;
            for (int i = 0; i < n_inputs; ++i)
                if (in.name == input_names[i]) found = i;
            if (found < 0) throw std::invalid_argument("no dtype given for input '" + in.name + "'");
            dtypes[in.slot] = static_cast<DataType>(input_dtypes[found]);
            slot_dims[in.slot] = given[found];
            if (input_order) input_order[in.slot] = found;
        }
        resolveOutputsDTypesInPlace(outputs, dtypes);
        PhysicalExpression expr = *outputs.expr;
        expr.output_node = outputs.outputs.front().node_idx;

        // dims of every local node
        std::vector<std::vector<uint64_t>> node_dims(expr.nodes.size());
        for (size_t k = 0; k < expr.nodes.size(); ++k) {
            const ExprNode& n = expr.nodes[k];
            if (n.op == ExprOp::INPUT || n.op == ExprOp::RUNTIME_SCALAR || n.op == ExprOp::TENSOR_RUNTIME_SCALAR) {
                node_dims[k] = slot_dims[n.input_slot];
                continue;
            }
            if (Expression::isLeafOp(n.op)) continue;
            std::vector<uint64_t> d;
            for (uint32_t par : {n.lhs, n.rhs, n.aux})
                if (par != UINT32_MAX) d = broadcastOf(d, node_dims[par]);
            node_dims[k] = d;
        }
        const std::vector<uint64_t> out_dims = node_dims[expr.output_node];

        std::vector<uint32_t> value_ids(n_slots);
        for (uint32_t i = 0; i < n_slots; ++i) value_ids[i] = i;
        CompiledExecutionStage stage(expr, std::shared_ptr<CompiledEquation>{}, value_ids,
                                     {CompiledStageOutput{.name = "output", .local_node_idx = expr.output_node, .value_id = static_cast<uint32_t>(n_slots)}});

        SpecializedBroadcastGroup group;
        group.numel = product(out_dims);
        group.output_dims = out_dims;
        group.node_dims = node_dims;
        group.output_indices = {0u};
        std::vector<std::vector<uint64_t>> strides_by_used;
        for (uint32_t slot = 0; slot < n_slots; ++slot) {
            group.used_input_slots.push_back(slot);
            group.used_input_broadcast_offset_required.push_back(true);
            group.used_input_visible_dims.push_back(slot_dims[slot]);
            group.used_input_visible_strides.push_back(broadcastStrides(slot_dims[slot], slot_dims[slot]));
            strides_by_used.push_back(broadcastStrides(slot_dims[slot], out_dims));
        }
        group.used_input_load_kinds.assign(n_slots, SpecializedInputLoadKind::ScalarPack);
        if (!out_dims.empty() && out_dims.back() % 2ULL == 0ULL)
            for (size_t u = 0; u < n_slots; ++u)
                if (strides_by_used[u][out_dims.size() - 1] == 1ULL) group.used_input_load_kinds[u] = SpecializedInputLoadKind::NativeVector;
        std::vector<uint64_t> out_strides(out_dims.size(), 1);
        for (size_t i = out_dims.size(); i-- > 1;) out_strides[i - 1] = out_strides[i] * out_dims[i];
        for (size_t axis = 0; axis < out_dims.size(); ++axis) {
            if (out_dims[axis] == 1ULL) continue;
            SpecializedBroadcastAxis ad;
            ad.dim = out_dims[axis];
            ad.output_stride = out_strides[axis];
            bool any = false;
            for (size_t u = 0; u < n_slots; ++u) {
                ad.input_strides.push_back(strides_by_used[u][axis]);
                any = any || strides_by_used[u][axis] != 0ULL;
            }
            if (any) group.active_axes.push_back(std::move(ad));
        }

        g_text = CudaSourceEmitter::emitSpecializedBroadcast(stage, {group}, "fused_kernel");
        *source = g_text.c_str();
        if (elements_per_thread) *elements_per_thread = CudaSourceEmitter::getVectorizedStageStorageDType(stage).has_value() ? 2u : 1u;
        if (output_dtype) *output_dtype = static_cast<int>(expr.nodes[expr.output_node].output_dtype.value());
        if (out_numel) *out_numel = group.numel;
        return 0;
    } catch (const std::exception& ex) {
        g_text = ex.what();
        *source = g_text.c_str();
        return 1;
    }
}

// Runs the reference's dtype resolution on `program` and returns (op, output dtype, compute dtype) of every node of the
// reference's graph, three ints per node, in its node order.  Returns the number of nodes, or -1 on error.
extern "C" __attribute__((visibility("default"))) int thor_ref_resolve_dtypes(const char* program, const char* const* input_names, const int* input_dtypes,
                                                                              int n_inputs, int* triplets, int capacity_nodes) {
    try {
        Expression e = buildFromPostfix(program);
        PhysicalOutputs outputs = Expression::outputs({{"output", e}}).physicalOutputs();
        std::vector<DataType> dtypes(outputs.expr->inputs.size(), DataType::FP32);
        for (const NamedInput& in : outputs.expr->inputs) {
            int found = -1;
            for (int i = 0; i < n_inputs; ++i)
                if (in.name == input_names[i]) found = i;
            if (found < 0) throw std::invalid_argument("no dtype given for input '" + in.name + "'");
            dtypes[in.slot] = static_cast<DataType>(input_dtypes[found]);
        }
        resolveOutputsDTypesInPlace(outputs, dtypes);
        const auto& nodes = outputs.expr->nodes;
        if (static_cast<int>(nodes.size()) > capacity_nodes) return -1;
        for (size_t k = 0; k < nodes.size(); ++k) {
            triplets[3 * k + 0] = static_cast<int>(nodes[k].op);
            triplets[3 * k + 1] = nodes[k].output_dtype.has_value() ? static_cast<int>(nodes[k].output_dtype.value()) : 0;
            triplets[3 * k + 2] = nodes[k].compute_dtype.has_value() ? static_cast<int>(nodes[k].compute_dtype.value()) : 0;
        }
        return static_cast<int>(nodes.size());
    } catch (const std::exception& ex) {
        g_text = ex.what();
        return -1;
    }
}

// Emits the flat fused kernel "fused_kernel" for `program`.  input_names / input_dtypes give the dtype of every
// tensor input and fp32 runtime scalar by name.  On success returns 0, *source points at the generated CUDA source
// (valid until the next call on this thread), *elements_per_thread is the reference's launch geometry
// (grid = ceil(numel / elements_per_thread / 256), 256 threads; EquationRunner.cpp:274-289), and input_order (if given) receives
// the slot order of the kernel's input parameters as indices into input_names.
extern "C" __attribute__((visibility("default"))) int thor_ref_emit_flat(const char* program, const char* const* input_names, const int* input_dtypes,
                                                                         int n_inputs, const char** source, unsigned* elements_per_thread, int* input_order,
                                                                         int* output_dtype) {
    try {
        Expression e = buildFromPostfix(program);
        PhysicalOutputs outputs = Expression::outputs({{"output", e}}).physicalOutputs();
        std::vector<DataType> dtypes(outputs.expr->inputs.size(), DataType::FP32);
        for (const NamedInput& in : outputs.expr->inputs) {
            int found = -1;
            for (int i = 0; i < n_inputs; ++i)
                if (in.name == input_names[i]) found = i;
            if (found < 0) throw std::invalid_argument("no dtype given for input '" + in.name + "'");
            dtypes[in.slot] = static_cast<DataType>(input_dtypes[found]);
            if (input_order) input_order[in.slot] = found;
        }
        resolveOutputsDTypesInPlace(outputs, dtypes);
        PhysicalExpression expr = *outputs.expr;
        expr.output_node = outputs.outputs.front().node_idx;
        PhysicalExecutionStage stage{
            .kind = PhysicalExecutionStage::Kind::FusedKernel,
            .expr = expr,
            .input_value_ids = {},
            .outputs = {CompiledStageOutput{.name = "output", .local_node_idx = expr.output_node, .value_id = 0}},
        };
        g_text = CudaSourceEmitter::emitFlat(stage, "fused_kernel", true);
        *source = g_text.c_str();
        if (elements_per_thread) *elements_per_thread = CudaSourceEmitter::flatElementsPerThread(stage);
        if (output_dtype) *output_dtype = static_cast<int>(expr.nodes[expr.output_node].output_dtype.value());
        return 0;
    } catch (const std::exception& ex) {
        g_text = ex.what();
        *source = g_text.c_str();
        return 1;
    }
}
