// Graph dumper for the REFERENCE's own reverse-mode differentiation.
//
// TEST INFRASTRUCTURE ONLY (never shipped, never linked by the product).  No reference source is copied here: the build
// compiles the reference's Expression.cpp, ExpressionDTypeResolution.cpp and AutoDiff.cpp where they lie and links them
// with this file.  The entry point builds a forward expression through the reference's public Expression API from a
// postfix description (ref_postfix.h), resolves its dtypes against the given input dtypes, calls the reference's
// buildBackwardOutputs with concrete forward input dims -- the sequence of FusedEquation::buildShapeSpecializedOutputs
// (Utilities/Expression/FusedEquation.cpp:6701-6796; AutoDiff.h:16-63; AutoDiff.cpp:6210-6290) -- resolves the dtypes
// of the backward graph the same way, and returns that graph as JSON text: every node with its op integer, parents,
// scalar, reduction / squeeze / reshape / unsqueeze / fill dims and resolved output / compute dtypes, the inputs by
// slot, and the named gradient outputs.  The tests compare the host layer's backward graph with it and evaluate it
// with the numpy oracle as a second reference for the gradients.
//
// AutoDiff.cpp also names three functions whose translation units pull in the reference's whole runtime
// (StampedEquation.cpp, CudaKernelExpression.cpp).  They are defined at the end of this file: the two custom-kernel
// queries refuse (no expression built here holds a custom kernel), and the shape of a reduction's result -- reduced
// axes become 1, then the listed axes are squeezed, UINT64_MAX meaning every singleton -- is computed by this file's
// own few lines, so a difference from StampedEquation.cpp:4308-4363 would show as a shape mismatch in the tests.
#include <sstream>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "Utilities/Expression/AutoDiff.h"
#include "Utilities/Expression/CudaKernelExpression.h"
#include "Utilities/Expression/StampedEquation.h"
#include "Utilities/Expression/ExpressionDTypeResolution.h"
#include "ref_postfix.h"

using namespace ThorImplementation;

namespace {

thread_local std::string g_text;

void list(std::ostringstream& os, const char* key, const std::vector<uint64_t>& v) {
    os << ",\"" << key << "\":[";
    for (size_t i = 0; i < v.size(); ++i) os << (i ? "," : "") << v[i];
    os << "]";
}
long long parent(uint32_t p) { return p == UINT32_MAX ? -1 : static_cast<long long>(p); }
int dtypeOrZero(const std::optional<DataType>& d) { return d.has_value() ? static_cast<int>(d.value()) : 0; }

}  // namespace

// input_dims holds, per named input, its rank followed by its dims (rank 0 for runtime scalars).  upstream_dtype is the
// dtype of the gradient that arrives for the single forward output ("output"), bound under the reference's default name.
// Returns 0 and the JSON text, or 1 and the exception message.
extern "C" __attribute__((visibility("default"))) int thor_ref_backward_graph(const char* program, const char* const* input_names, const int* input_dtypes,
                                                                              const unsigned long long* input_dims, int n_inputs, const char* const* wrt_names,
                                                                              int n_wrt, int upstream_dtype, const char** text) {
    try {
        Expression e = thor_ref_dump::buildFromPostfix(program);
        PhysicalOutputs forward = Expression::outputs({{"output", e}}).physicalOutputs();
        forward.expr = std::make_shared<PhysicalExpression>(*forward.expr);
        std::vector<DataType> forward_dtypes(forward.expr->inputs.size(), DataType::FP32);
        std::unordered_map<std::string, std::vector<uint64_t>> forward_dims;
        std::unordered_map<std::string, DataType> dtype_by_name;
        {
            const unsigned long long* p = input_dims;
            for (int i = 0; i < n_inputs; ++i) {
                const unsigned long long rank = *p++;
                forward_dims[input_names[i]] = std::vector<uint64_t>(p, p + rank);
                dtype_by_name[input_names[i]] = static_cast<DataType>(input_dtypes[i]);
                p += rank;
            }
        }
        for (const NamedInput& in : forward.expr->inputs) {
            auto it = dtype_by_name.find(in.name);
            if (it == dtype_by_name.end()) throw std::invalid_argument("no dtype given for input '" + in.name + "'");
            forward_dtypes[in.slot] = it->second;
        }
        resolveOutputsDTypesInPlace(forward, forward_dtypes);

        const std::string upstream = DEFAULT_BACKWARD_UPSTREAM_INPUT_NAME;
        std::vector<std::string> wrt(wrt_names, wrt_names + n_wrt);
        PhysicalOutputs backward = buildBackwardOutputs(forward, wrt, std::unordered_map<std::string, std::string>{{"output", upstream}},
                                                        std::unordered_map<std::string, DataType>{{"output", static_cast<DataType>(upstream_dtype)}},
                                                        std::optional<std::unordered_map<std::string, std::vector<uint64_t>>>(forward_dims), false);
        dtype_by_name[upstream] = static_cast<DataType>(upstream_dtype);
        std::vector<DataType> backward_dtypes(backward.expr->inputs.size(), DataType::FP32);
        for (const NamedInput& in : backward.expr->inputs) {
            auto it = dtype_by_name.find(in.name);
            if (it == dtype_by_name.end()) throw std::invalid_argument("backward graph reads an input without a dtype: '" + in.name + "'");
            backward_dtypes[in.slot] = it->second;
        }
        resolveOutputsDTypesInPlace(backward, backward_dtypes);

        std::ostringstream os;
        os.precision(17);
        os << "{\"inputs\":[";
        for (size_t i = 0; i < backward.expr->inputs.size(); ++i) {
            const NamedInput& in = backward.expr->inputs[i];
            os << (i ? "," : "") << "{\"name\":\"" << in.name << "\",\"slot\":" << in.slot << ",\"kind\":" << static_cast<int>(in.kind) << "}";
        }
        os << "],\"outputs\":[";
        for (size_t i = 0; i < backward.outputs.size(); ++i)
            os << (i ? "," : "") << "{\"name\":\"" << backward.outputs[i].name << "\",\"node\":" << backward.outputs[i].node_idx << "}";
        os << "],\"nodes\":[";
        for (size_t k = 0; k < backward.expr->nodes.size(); ++k) {
            const ExprNode& n = backward.expr->nodes[k];
            os << (k ? "," : "") << "{\"op\":" << static_cast<int>(n.op) << ",\"lhs\":" << parent(n.lhs) << ",\"rhs\":" << parent(n.rhs) << ",\"aux\":" << parent(n.aux)
               << ",\"slot\":" << parent(n.input_slot) << ",\"scalar\":" << n.scalar_fp << ",\"out\":" << dtypeOrZero(n.output_dtype) << ",\"compute\":"
               << dtypeOrZero(n.compute_dtype);
            list(os, "reduction_axes", n.reduction_axes);
            list(os, "squeeze_axes", n.squeeze_axes);
            list(os, "unsqueeze_axes", n.unsqueeze_axes);
            list(os, "reshape_dims", n.reshape_dims);
            list(os, "fill_dims", n.fill_dims);
            os << "}";
        }
        os << "]}";
        g_text = os.str();
        *text = g_text.c_str();
        return 0;
    } catch (const std::exception& ex) {
        g_text = ex.what();
        *text = g_text.c_str();
        return 1;
    }
}

namespace ThorImplementation {

const CudaKernelExpression::BackwardSpec* CudaKernelExpression::backwardSpecForOutput(const std::string&) const {
    throw std::logic_error("custom CUDA kernel expressions are outside what this dumper builds");
}
std::vector<std::vector<uint64_t>> CudaKernelExpression::inferOutputShapesFromInputShapes(const std::unordered_map<std::string, std::vector<uint64_t>>&) const {
    throw std::logic_error("custom CUDA kernel expressions are outside what this dumper builds");
}
std::vector<uint64_t> StampedEquation::computeReductionOutputDims(const std::vector<uint64_t>& input_dims, const std::vector<uint64_t>& reduction_axes,
                                                                  const std::vector<uint64_t>& squeeze_axes) {
    std::vector<uint64_t> kept = input_dims;
    for (uint64_t axis : reduction_axes) {
        if (axis >= kept.size()) throw std::runtime_error("reduction axis out of range");
        kept[axis] = 1;
    }
    if (squeeze_axes.empty()) return kept;
    const bool all_singletons = squeeze_axes.size() == 1 && squeeze_axes[0] == UINT64_MAX;
    std::vector<uint64_t> out;
    for (size_t axis = 0; axis < kept.size(); ++axis) {
        bool squeezed = all_singletons ? kept[axis] == 1 : false;
        if (!all_singletons)
            for (uint64_t s : squeeze_axes) squeezed = squeezed || s == axis;
        if (squeezed && kept[axis] != 1) throw std::runtime_error("only axes of size 1 can be squeezed");
        if (!squeezed) out.push_back(kept[axis]);
    }
    if (out.empty()) out.push_back(1);
    return out;
}

}  // namespace ThorImplementation
