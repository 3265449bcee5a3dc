// Flat C surface over the C++ host layer, for the ctypes binding (the role nanobind plays in the
// reference's bindings/python/src/core/physical/expression.cpp).  Every function catches C++
// exceptions: logic errors return 1, runtime errors 2, and thb_last_error() holds the message.
#include <sstream>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "CubReduction.h"
#include "FusedEquation.h"
#include "Schedule.h"

using namespace ThorB200;

#define THB_API extern "C" __attribute__((visibility("default")))

namespace {
thread_local std::string g_error;

template <class F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::logic_error& e) {
        g_error = e.what();
        return 1;
    } catch (const std::exception& e) {
        g_error = e.what();
        return 2;
    }
}

struct Plan {
    StampedExecutionPlan plan;
    std::vector<std::string> strings;  // storage for returned C strings
};
}  // namespace

THB_API const char* thb_last_error() { return g_error.c_str(); }

// ---- expressions ------------------------------------------------------------------------------------
THB_API int thb_input(const char* name, int kind, int compute_dtype, int output_dtype, Expression** out) {
    return guarded([&] {
        std::optional<DataType> c = compute_dtype ? std::optional<DataType>(static_cast<DataType>(compute_dtype)) : std::nullopt;
        std::optional<DataType> o = output_dtype ? std::optional<DataType>(static_cast<DataType>(output_dtype)) : std::nullopt;
        Expression e = kind == 0 ? Expression::input(name, c, o) : (kind == 1 ? Expression::runtimeScalar(name, c, o) : Expression::tensorRuntimeScalar(name, c, o));
        *out = new Expression(e);
    });
}
THB_API int thb_scalar(double value, Expression** out) {
    return guarded([&] { *out = new Expression(value); });
}
THB_API void thb_expr_free(Expression* e) { delete e; }

THB_API int thb_unary(int op, const Expression* a, Expression** out) {
    return guarded([&] {
        const ExprOp o = static_cast<ExprOp>(op);
        Expression r = *a;
        switch (o) {
            case ExprOp::NEG: r = -*a; break;
            case ExprOp::LOGICAL_NOT: r = a->logicalNot(); break;
            case ExprOp::ABS: r = a->abs(); break;
            case ExprOp::CEIL: r = a->ceil(); break;
            case ExprOp::FLOOR: r = a->floor(); break;
            case ExprOp::ROUND: r = a->round(); break;
            case ExprOp::TRUNC: r = a->trunc(); break;
            case ExprOp::SIN: r = a->sin(); break;
            case ExprOp::COS: r = a->cos(); break;
            case ExprOp::TAN: r = a->tan(); break;
            case ExprOp::ASIN: r = a->asin(); break;
            case ExprOp::ACOS: r = a->acos(); break;
            case ExprOp::ATAN: r = a->atan(); break;
            case ExprOp::SINH: r = a->sinh(); break;
            case ExprOp::COSH: r = a->cosh(); break;
            case ExprOp::ASINH: r = a->asinh(); break;
            case ExprOp::ACOSH: r = a->acosh(); break;
            case ExprOp::ATANH: r = a->atanh(); break;
            case ExprOp::ERF: r = a->erf(); break;
            case ExprOp::ERFC: r = a->erfc(); break;
            case ExprOp::ERFCX: r = a->erfcx(); break;
            case ExprOp::ERFINV: r = a->erfinv(); break;
            case ExprOp::ERFCINV: r = a->erfcinv(); break;
            case ExprOp::TGAMMA: r = a->tgamma(); break;
            case ExprOp::LGAMMA: r = a->lgamma(); break;
            case ExprOp::DIGAMMA: r = a->digamma(); break;
            case ExprOp::EXP: r = a->exp(); break;
            case ExprOp::EXPM1: r = a->expm1(); break;
            case ExprOp::EXP2: r = a->exp2(); break;
            case ExprOp::EXP10: r = a->exp10(); break;
            case ExprOp::LN: r = a->ln(); break;
            case ExprOp::LOG1P: r = a->log1p(); break;
            case ExprOp::LOG2: r = a->log2(); break;
            case ExprOp::LOG10: r = a->log10(); break;
            case ExprOp::SQRT: r = a->sqrt(); break;
            case ExprOp::TANH: r = a->tanh(); break;
            case ExprOp::NORMCDF: r = a->normcdf(); break;
            default: throw std::invalid_argument("thb_unary: not a unary op");
        }
        *out = new Expression(r);
    });
}

THB_API int thb_binary(int op, const Expression* a, const Expression* b, Expression** out) {
    return guarded([&] {
        Expression r = *a;
        switch (static_cast<ExprOp>(op)) {
            case ExprOp::ADD: r = *a + *b; break;
            case ExprOp::SUB: r = *a - *b; break;
            case ExprOp::MUL: r = *a * *b; break;
            case ExprOp::DIV: r = *a / *b; break;
            case ExprOp::POW: r = a->pow(*b); break;
            case ExprOp::MIN: r = a->min(*b); break;
            case ExprOp::MAX: r = a->max(*b); break;
            case ExprOp::EQUAL: r = *a == *b; break;
            case ExprOp::NOT_EQUAL: r = *a != *b; break;
            case ExprOp::LESS: r = *a < *b; break;
            case ExprOp::LESS_EQUAL: r = *a <= *b; break;
            case ExprOp::GREATER: r = *a > *b; break;
            case ExprOp::GREATER_EQUAL: r = *a >= *b; break;
            case ExprOp::LOGICAL_AND: r = a->logicalAnd(*b); break;
            case ExprOp::LOGICAL_OR: r = a->logicalOr(*b); break;
            default: throw std::invalid_argument("thb_binary: not a binary op");
        }
        *out = new Expression(r);
    });
}

THB_API int thb_where(const Expression* c, const Expression* t, const Expression* f, Expression** out) {
    return guarded([&] { *out = new Expression(Expression::where(*c, *t, *f)); });
}
THB_API int thb_cast(const Expression* a, int dtype, Expression** out) {
    return guarded([&] { *out = new Expression(a->cast(static_cast<DataType>(dtype))); });
}
THB_API int thb_with_output_dtype(const Expression* a, int dtype, Expression** out) {
    return guarded([&] { *out = new Expression(a->withOutputDType(static_cast<DataType>(dtype))); });
}
THB_API int thb_composite(const char* name, const Expression* a, double p0, double p1, Expression** out) {
    return guarded([&] {
        const std::string n(name);
        Expression r = *a;
        if (n == "sigmoid") r = a->sigmoid();
        else if (n == "softplus") r = a->softplus();
        else if (n == "elu") r = a->elu(p0);
        else if (n == "selu") r = a->selu();
        else if (n == "gelu") r = a->gelu();
        else if (n == "swish") r = a->swish();
        else if (n == "relu") r = a->relu();
        else if (n == "relu6") r = a->relu6();
        else if (n == "hard_tanh") r = a->hardTanh(p0, p1);
        else if (n == "clamp") r = a->clamp(p0, p1);
        else if (n == "softmax") r = a->softmax(static_cast<SoftmaxAlgorithm>(static_cast<int>(p0)), static_cast<SoftmaxMode>(static_cast<int>(p1)));
        else if (n == "log_softmax") r = a->logSoftmax(static_cast<SoftmaxMode>(static_cast<int>(p1)));
        else throw std::invalid_argument("thb_composite: unknown composite '" + n + "'");
        *out = new Expression(r);
    });
}
THB_API int thb_reduce(const Expression* a, int op, const uint64_t* axes, uint32_t n_axes, const uint64_t* squeeze, uint32_t n_squeeze,
                       int compute_dtype, Expression** out) {
    return guarded([&] {
        std::optional<DataType> c = compute_dtype ? std::optional<DataType>(static_cast<DataType>(compute_dtype)) : std::nullopt;
        *out = new Expression(a->reduction(static_cast<ExprOp>(op), std::vector<uint64_t>(axes, axes + n_axes), std::vector<uint64_t>(squeeze, squeeze + n_squeeze), c));
    });
}
THB_API int thb_shape_op(const Expression* a, int op, const uint64_t* values, uint32_t n, Expression** out) {
    return guarded([&] {
        const std::vector<uint64_t> v(values, values + n);
        switch (static_cast<ExprOp>(op)) {
            case ExprOp::RESHAPE: *out = new Expression(a->reshape(v)); break;
            case ExprOp::UNSQUEEZE: *out = new Expression(a->unsqueeze(v)); break;
            case ExprOp::SQUEEZE: *out = new Expression(a->squeeze(v)); break;
            default: throw std::invalid_argument("thb_shape_op: not a shape op");
        }
    });
}
THB_API uint32_t thb_expr_node_count(const Expression* a) { return static_cast<uint32_t>(a->graph()->nodes.size()); }

// ---- equations --------------------------------------------------------------------------------------
// row_tuning: NULL or the eight RowProgramTuning fields in declaration order
THB_API int thb_compile(const char* const* names, Expression* const* exprs, uint32_t n, int device, int fast_math, int fuse_rows, const int32_t* row_tuning,
                        int unrounded_column_sums, int branch_streams, FusedEquation** out) {
    return guarded([&] {
        std::vector<std::pair<std::string, Expression>> named;
        for (uint32_t i = 0; i < n; ++i) named.emplace_back(names[i], *exprs[i]);
        FusedEquationOptions opt;
        opt.use_fast_math = fast_math != 0;
        opt.fuse_row_reductions = fuse_rows != 0;
        opt.unrounded_column_sums = unrounded_column_sums != 0;
        opt.branch_streams = branch_streams != 0;  // 0 = off, 1 = on for plans above the default size, 2 = on for every plan
        if (branch_streams == 2) opt.branch_streams_min_input_bytes = 0;
        if (row_tuning != nullptr)
            opt.row_program = RowProgramTuning{row_tuning[0], row_tuning[1], row_tuning[2], row_tuning[3], row_tuning[4], row_tuning[5], row_tuning[6], row_tuning[7]};
        *out = new FusedEquation(FusedEquation::compile(Expression::outputs(named), device, opt));
    });
}
THB_API int thb_compile_backward(const FusedEquation* eq, const char* const* wrt, uint32_t n, const char* upstream_prefix, FusedEquation** out) {
    return guarded([&] {
        std::vector<std::string> names(wrt, wrt + n);
        *out = new FusedEquation(eq->compileBackward(names, upstream_prefix));
    });
}
THB_API void thb_equation_free(FusedEquation* eq) { delete eq; }

struct thb_binding {
    const char* name;
    void* ptr;           // device pointer (tensors)
    int32_t dtype;       // DataType (tensors)
    uint32_t rank;
    uint64_t dims[8];
    int32_t is_scalar;   // 1: fp32 runtime scalar passed in `scalar`
    float scalar;
};

THB_API int thb_stamp(FusedEquation* eq, const thb_binding* inputs, uint32_t n_inputs, const thb_binding* outputs, uint32_t n_outputs, void* stream,
                      Plan** out) {
    return guarded([&] {
        std::unordered_map<std::string, RuntimeInputValue> in;
        for (uint32_t i = 0; i < n_inputs; ++i) {
            const thb_binding& b = inputs[i];
            if (b.is_scalar) in[b.name] = RuntimeInputValue(b.scalar);
            else in[b.name] = RuntimeInputValue(Tensor::wrap(b.ptr, static_cast<DataType>(b.dtype), std::vector<uint64_t>(b.dims, b.dims + b.rank), eq->deviceNum()));
        }
        std::unordered_map<std::string, Tensor> pre;
        for (uint32_t i = 0; i < n_outputs; ++i) {
            const thb_binding& b = outputs[i];
            pre[b.name] = Tensor::wrap(b.ptr, static_cast<DataType>(b.dtype), std::vector<uint64_t>(b.dims, b.dims + b.rank), eq->deviceNum());
        }
        auto p = new Plan();
        try {
            p->plan = eq->stamp(in, Stream(stream, eq->deviceNum()), pre);
        } catch (...) {
            delete p;
            throw;
        }
        *out = p;
    });
}
// JSON description of the dtype-resolved graph the equation evaluates for the bound shapes and dtypes (ptr ignored).
// The text lives until the next call on the calling thread.
THB_API int thb_equation_graph(FusedEquation* eq, const thb_binding* inputs, uint32_t n_inputs, const char** text) {
    static thread_local std::string g_graph;
    return guarded([&] {
        std::unordered_map<std::string, std::vector<uint64_t>> dims;
        std::unordered_map<std::string, DataType> dtypes;
        for (uint32_t i = 0; i < n_inputs; ++i) {
            if (inputs[i].is_scalar) continue;
            dims[inputs[i].name] = std::vector<uint64_t>(inputs[i].dims, inputs[i].dims + inputs[i].rank);
            dtypes[inputs[i].name] = static_cast<DataType>(inputs[i].dtype);
        }
        g_graph = eq->describeGraph(dims, dtypes);
        *text = g_graph.c_str();
    });
}
// Same as thb_stamp, but nothing touches a GPU: bindings carry shapes and dtypes only (their ptr is
// ignored), outputs and intermediates get placeholder addresses and kernels are compiled, not loaded.
THB_API int thb_stamp_plan_only(FusedEquation* eq, const thb_binding* inputs, uint32_t n_inputs, Plan** out) {
    std::vector<thb_binding> in(inputs, inputs + n_inputs);
    uint64_t placeholder = 0x200000000000ull;
    for (auto& b : in) {
        if (b.is_scalar) continue;
        uint64_t bytes = dataTypeSize(static_cast<DataType>(b.dtype));
        for (uint32_t i = 0; i < b.rank; ++i) bytes *= b.dims[i];
        b.ptr = reinterpret_cast<void*>(placeholder);
        placeholder += (bytes + 511) / 256 * 256;
    }
    Tensor::setPlanOnly(true);
    const int status = thb_stamp(eq, in.data(), n_inputs, nullptr, 0, nullptr, out);
    Tensor::setPlanOnly(false);
    return status;
}
THB_API void thb_plan_free(Plan* p) { delete p; }
THB_API int thb_plan_run(Plan* p, void* stream) {
    return guarded([&] {
        if (stream) p->plan.runOn(Stream(stream, 0));
        else p->plan.run();
    });
}
THB_API int thb_plan_set_scalar(Plan* p, const char* name, float value) {
    return guarded([&] { p->plan.setRuntimeScalar(name, value); });
}
THB_API int thb_plan_output(Plan* p, const char* name, thb_binding* out) {
    return guarded([&] {
        Tensor t = p->plan.getOutput(name);
        out->ptr = t.getMemPtr();
        out->dtype = static_cast<int32_t>(t.getDataType());
        out->rank = static_cast<uint32_t>(t.getDimensions().size());
        if (out->rank > 8) throw std::logic_error("output rank above 8");
        for (uint32_t i = 0; i < out->rank; ++i) out->dims[i] = t.getDimensions()[i];
        out->is_scalar = 0;
    });
}
// kind: 0 logical stage names, 1 physical stage names, 2 stage sources, 3 output names, 4 column-sum names; items are joined by '\x1e'
THB_API const char* thb_plan_strings(Plan* p, int kind) {
    std::vector<std::string> items;
    try {
        items = kind == 0 ? p->plan.stageKindNames() : kind == 1 ? p->plan.physicalStageNames() : kind == 2 ? p->plan.stageSources() : kind == 4 ? p->plan.columnSumNames() : p->plan.getOutputNames();
    } catch (...) {
    }
    std::string joined;
    for (size_t i = 0; i < items.size(); ++i) {
        if (i) joined += '\x1e';
        joined += items[i];
    }
    p->strings.push_back(joined);
    return p->strings.back().c_str();
}
// Lane of every physical stage of the plan (0 = the caller's stream); returns the number written.
THB_API uint32_t thb_plan_stage_lanes(Plan* p, uint32_t* lanes, uint32_t capacity) {
    const std::vector<uint32_t> v = p->plan.stageLanes();
    for (size_t i = 0; i < v.size() && i < capacity; ++i) lanes[i] = v[i];
    return static_cast<uint32_t>(v.size());
}
// The pure lane-assignment function: deps is a flat list, stage s consuming deps[offsets[s] .. offsets[s + 1]).
THB_API int thb_build_schedule(const uint32_t* deps, const uint32_t* offsets, uint32_t n_stages, uint32_t* lanes, uint8_t* completion_event, uint32_t* n_lanes,
                               int32_t* needs_caller_ready) {
    return guarded([&] {
        std::vector<std::vector<uint32_t>> d(n_stages);
        for (uint32_t s = 0; s < n_stages; ++s) d[s].assign(deps + offsets[s], deps + offsets[s + 1]);
        StampedExecutionSchedule sch;
        try {
            sch = buildStampedExecutionSchedule(d, 0);
        } catch (const std::runtime_error& e) {
            throw std::logic_error(e.what());
        }
        for (uint32_t s = 0; s < n_stages; ++s) {
            lanes[s] = sch.stage_lane_indices[s];
            completion_event[s] = sch.stage_needs_completion_event[s] ? 1 : 0;
        }
        *n_lanes = static_cast<uint32_t>(sch.lane_gpu_nums.size());
        *needs_caller_ready = sch.needs_caller_ready_event ? 1 : 0;
    });
}
THB_API uint64_t thb_plan_intermediate_bytes(Plan* p) { return p->plan.intermediateBytes(); }
THB_API uint64_t thb_plan_launches(Plan* p) { return p->plan.kernelLaunchesPerRun(); }
THB_API int thb_plan_waits_expired(Plan* p, uint64_t* count) {
    return guarded([&] { *count = p->plan.waitsExpired(); });
}

// ---- dtype resolution probe (no GPU needed) ---------------------------------------------------------
// Resolves dtypes for the given input dtypes and writes (op, output_dtype, compute_dtype) triples of every node.
THB_API int thb_resolve_dtypes(const char* const* names, Expression* const* exprs, uint32_t n, const char* const* input_names, const int32_t* input_dtypes,
                               uint32_t n_inputs, int32_t* triples, uint32_t capacity, uint32_t* n_nodes) {
    return guarded([&] {
        std::vector<std::pair<std::string, Expression>> named;
        for (uint32_t i = 0; i < n; ++i) named.emplace_back(names[i], *exprs[i]);
        Outputs outs = Expression::outputs(named);
        PhysicalOutputs phys = outs.physicalOutputs();
        phys.expr = std::make_shared<PhysicalExpression>(*phys.expr);
        std::vector<DataType> dts(phys.expr->inputs.size(), DataType::FP32);
        for (const auto& in : phys.expr->inputs) {
            bool found = false;
            for (uint32_t i = 0; i < n_inputs; ++i)
                if (in.name == input_names[i]) {
                    dts[in.slot] = static_cast<DataType>(input_dtypes[i]);
                    found = true;
                }
            if (!found) throw std::logic_error("thb_resolve_dtypes: missing dtype for input '" + in.name + "'");
        }
        resolveOutputsDTypesInPlace(phys, dts);
        *n_nodes = static_cast<uint32_t>(phys.expr->nodes.size());
        if (*n_nodes > capacity) throw std::logic_error("thb_resolve_dtypes: buffer too small");
        for (uint32_t k = 0; k < *n_nodes; ++k) {
            triples[3 * k] = static_cast<int32_t>(phys.expr->nodes[k].op);
            triples[3 * k + 1] = static_cast<int32_t>(*phys.expr->nodes[k].output_dtype);
            triples[3 * k + 2] = static_cast<int32_t>(phys.expr->nodes[k].compute_dtype.value_or(*phys.expr->nodes[k].output_dtype));
        }
    });
}

// ---- CubReduction / CubArgReduction -----------------------------------------------------------------
THB_API int thb_reduction_geometry(const uint64_t* dims, uint32_t rank, const uint32_t* axes, uint32_t n_axes, uint64_t* outer_red_inner, int32_t* path) {
    return guarded([&] {
        const CubReductionGeometry g = CubReduction::analyzeGeometry(std::vector<uint64_t>(dims, dims + rank), std::vector<uint32_t>(axes, axes + n_axes));
        outer_red_inner[0] = g.outer_size;
        outer_red_inner[1] = g.reduction_size;
        outer_red_inner[2] = g.inner_size;
        *path = static_cast<int32_t>(g.path);
    });
}

// Every field of CubReduction::analyzeGeometry for a (possibly strided) view, as JSON text; strides may be NULL (dense).
THB_API int thb_reduction_geometry_json(const uint64_t* dims, const uint64_t* strides, uint32_t rank, const uint32_t* axes, uint32_t n_axes, const char** text) {
    static thread_local std::string g_text;
    return guarded([&] {
        const std::vector<uint64_t> d(dims, dims + rank);
        const std::vector<uint32_t> a(axes, axes + n_axes);
        const CubReductionGeometry g = strides ? CubReduction::analyzeGeometry(d, std::vector<uint64_t>(strides, strides + rank), a) : CubReduction::analyzeGeometry(d, a);
        std::ostringstream os;
        auto list = [&](const char* key, const auto& v) {
            os << "\"" << key << "\":[";
            for (size_t i = 0; i < v.size(); ++i) os << (i ? "," : "") << v[i];
            os << "],";
        };
        os << "{\"path\":" << static_cast<int>(g.path) << ",\"rank\":" << g.rank << ",\"reduced_axes_are_contiguous\":" << (g.reduced_axes_are_contiguous ? 1 : 0)
           << ",\"outer_size\":" << g.outer_size << ",\"reduction_size\":" << g.reduction_size << ",\"inner_size\":" << g.inner_size << ",\"input_elements\":"
           << g.input_elements << ",\"output_elements\":" << g.output_elements << ",";
        list("output_dimensions", g.output_dimensions);
        list("squeezed_output_dimensions", g.squeezed_output_dimensions);
        list("input_strides", g.indexing.input_strides);
        list("reduced_axes", g.indexing.reduced_axes);
        list("physical_non_singleton_axis_order", g.physical_non_singleton_axis_order);
        os << "\"physical_layout_is_dense_permutation\":" << (g.physical_layout_is_dense_permutation ? 1 : 0) << ",\"tiled_output_permuted\":" << (g.tiled_output_permuted ? 1 : 0)
           << ",\"tiled_output_shared_transpose\":" << (g.tiled_output_shared_transpose ? 1 : 0) << ",\"tiled_output_outer_stride\":" << g.tiled_output_outer_stride
           << ",\"tiled_output_inner_stride\":" << g.tiled_output_inner_stride << ",\"device_transform_uses_affine_stride\":" << (g.device_transform_uses_affine_stride ? 1 : 0)
           << ",\"affine_input_stride\":" << g.affine_input_stride << ",\"permutation_aware_tiled_geometry\":";
        if (g.permutation_aware_tiled_geometry) {
            const auto& c = *g.permutation_aware_tiled_geometry;
            os << "{";
            list("physical_outer_axes", c.physical_outer_axes);
            list("physical_reduction_axes", c.physical_reduction_axes);
            list("physical_inner_axes", c.physical_inner_axes);
            list("logical_non_singleton_retained_axes", c.logical_non_singleton_retained_axes);
            os << "\"outer_size\":" << c.outer_size << ",\"reduction_size\":" << c.reduction_size << ",\"inner_size\":" << c.inner_size << ",\"retained_output_order\":"
               << static_cast<int>(c.retained_output_order) << "}";
        } else {
            os << "null";
        }
        os << "}";
        g_text = os.str();
        *text = g_text.c_str();
    });
}
THB_API int thb_reduction_map_index(const uint64_t* dims, const uint64_t* strides, uint32_t rank, const uint32_t* axes, uint32_t n_axes, uint64_t output_index,
                                    uint64_t reduction_index, uint64_t* physical) {
    return guarded([&] {
        const std::vector<uint64_t> d(dims, dims + rank);
        const std::vector<uint32_t> a(axes, axes + n_axes);
        const CubReductionGeometry g = strides ? CubReduction::analyzeGeometry(d, std::vector<uint64_t>(strides, strides + rank), a) : CubReduction::analyzeGeometry(d, a);
        *physical = CubReduction::mapLogicalReductionIndexToPhysicalIndex(g, output_index, reduction_index);
    });
}
// Stamp on a strided VIEW: `input` binds the view's first element and dims, view_strides its element strides.
THB_API int thb_cub_reduction_stamp_view(int op, const uint32_t* axes, uint32_t n_axes, int output_dtype, float output_scale, const thb_binding* input,
                                         const uint64_t* view_strides, const thb_binding* output, void* stream, int device, StampedCubReduction** out) {
    return guarded([&] {
        std::optional<DataType> od = output_dtype ? std::optional<DataType>(static_cast<DataType>(output_dtype)) : std::nullopt;
        CubReduction r(static_cast<CubReductionOp>(op), std::vector<uint32_t>(axes, axes + n_axes), od, output_scale);
        const std::vector<uint64_t> dims(input->dims, input->dims + input->rank), strides(view_strides, view_strides + input->rank);
        uint64_t extent = 1;
        for (size_t i = 0; i < dims.size(); ++i) extent += (dims[i] - 1) * strides[i];
        Tensor storage = Tensor::wrap(input->ptr, static_cast<DataType>(input->dtype), {extent}, device);
        Tensor in = storage.aliasView(dims, strides, 0);
        Tensor o = Tensor::wrap(output->ptr, static_cast<DataType>(output->dtype), std::vector<uint64_t>(output->dims, output->dims + output->rank), device);
        *out = new StampedCubReduction(r.stamp(in, o, Stream(stream, device)));
    });
}
THB_API int thb_cub_reduction_stamp(int op, const uint32_t* axes, uint32_t n_axes, int output_dtype, float output_scale, const thb_binding* input,
                                    const thb_binding* output, void* stream, int device, StampedCubReduction** out) {
    return guarded([&] {
        std::optional<DataType> od = output_dtype ? std::optional<DataType>(static_cast<DataType>(output_dtype)) : std::nullopt;
        CubReduction r(static_cast<CubReductionOp>(op), std::vector<uint32_t>(axes, axes + n_axes), od, output_scale);
        Tensor in = Tensor::wrap(input->ptr, static_cast<DataType>(input->dtype), std::vector<uint64_t>(input->dims, input->dims + input->rank), device);
        Tensor o = Tensor::wrap(output->ptr, static_cast<DataType>(output->dtype), std::vector<uint64_t>(output->dims, output->dims + output->rank), device);
        *out = new StampedCubReduction(r.stamp(in, o, Stream(stream, device)));
    });
}
THB_API int thb_cub_reduction_run(StampedCubReduction* s) {
    return guarded([&] { s->run(); });
}
THB_API const char* thb_cub_reduction_kind(StampedCubReduction* s) { return s->kernelKind(); }
THB_API uint64_t thb_cub_reduction_workspace_bytes(StampedCubReduction* s) { return s->workspaceBytes(); }
THB_API void thb_cub_reduction_free(StampedCubReduction* s) { delete s; }
THB_API float thb_cub_empty_value(int op) { return CubReduction::getFp32EmptyReductionValue(static_cast<CubReductionOp>(op)); }

// Tensor::copyFromAsync between two bound tensors; device -1 = pinned host memory.
THB_API int thb_tensor_copy_from(const thb_binding* dst, int dst_device, const thb_binding* src, int src_device, void* stream) {
    return guarded([&] {
        Tensor d = Tensor::wrap(dst->ptr, static_cast<DataType>(dst->dtype), std::vector<uint64_t>(dst->dims, dst->dims + dst->rank), dst_device);
        Tensor s = Tensor::wrap(src->ptr, static_cast<DataType>(src->dtype), std::vector<uint64_t>(src->dims, src->dims + src->rank), src_device);
        d.copyFromAsync(s, Stream(stream, dst_device >= 0 ? dst_device : src_device));
    });
}
THB_API int thb_type_convert(void* src, void* dst, int src_dtype, int dst_dtype, long n, void* stream, int device) {
    return guarded([&] { TypeConverter::convertType(src, dst, static_cast<DataType>(src_dtype), static_cast<DataType>(dst_dtype), n, Stream(stream, device)); });
}
