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
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "Utilities/Expression/CudaSourceEmitter.h"
#include "Utilities/Expression/EquationCompiler.h"
#include "Utilities/Expression/ExpressionDTypeResolution.h"

using namespace ThorImplementation;

namespace {

thread_local std::string g_text;

Expression unaryByName(const Expression& x, const std::string& op) {
#define TB_U(NAME) if (op == #NAME) return x.NAME();
    TB_U(abs) TB_U(ceil) TB_U(floor) TB_U(round) TB_U(trunc) TB_U(sin) TB_U(cos) TB_U(tan) TB_U(asin) TB_U(acos) TB_U(atan) TB_U(sinh) TB_U(cosh)
    TB_U(asinh) TB_U(acosh) TB_U(atanh) TB_U(erf) TB_U(erfc) TB_U(erfcx) TB_U(erfinv) TB_U(erfcinv) TB_U(tgamma) TB_U(lgamma) TB_U(digamma) TB_U(ln)
    TB_U(log1p) TB_U(log2) TB_U(log10) TB_U(exp) TB_U(expm1) TB_U(exp2) TB_U(exp10) TB_U(sqrt) TB_U(normcdf) TB_U(sigmoid) TB_U(tanh) TB_U(softplus)
    TB_U(selu) TB_U(gelu) TB_U(relu6) TB_U(swish)
#undef TB_U
    if (op == "neg") return -x;
    if (op == "relu") return x.max(Expression(0.0));
    throw std::invalid_argument("unknown unary op '" + op + "'");
}

// Postfix program, tokens separated by blanks: in:<name>  rs:<name> (fp32 runtime scalar)  lit:<value>  cast:<dtype int>
// binary: add sub mul div pow min max   unary: see above.
Expression buildFromPostfix(const std::string& program) {
    std::vector<Expression> stack;
    std::istringstream is(program);
    std::string tok;
    auto pop = [&]() {
        if (stack.empty()) throw std::invalid_argument("postfix program pops an empty stack");
        Expression e = stack.back();
        stack.pop_back();
        return e;
    };
    while (is >> tok) {
        if (tok.rfind("in:", 0) == 0) stack.push_back(Expression::input(tok.substr(3)));
        else if (tok.rfind("rs:", 0) == 0) stack.push_back(Expression::runtimeScalar(tok.substr(3)));
        else if (tok.rfind("lit:", 0) == 0) stack.push_back(Expression(std::stod(tok.substr(4))));
        else if (tok.rfind("cast:", 0) == 0) {
            Expression a = pop();
            stack.push_back(a.cast(static_cast<DataType>(std::stoi(tok.substr(5)))));
        } else if (tok == "add" || tok == "sub" || tok == "mul" || tok == "div" || tok == "pow" || tok == "min" || tok == "max") {
            Expression b = pop();
            Expression a = pop();
            stack.push_back(tok == "add" ? a + b : tok == "sub" ? a - b : tok == "mul" ? a * b : tok == "div" ? a / b : tok == "pow" ? a.pow(b)
                            : tok == "min" ? a.min(b) : a.max(b));
        } else {
            Expression a = pop();
            stack.push_back(unaryByName(a, tok));
        }
    }
    if (stack.size() != 1) throw std::invalid_argument("postfix program must leave exactly one value");
    return stack.back();
}

}  // namespace

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
