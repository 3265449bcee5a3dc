// Fused-stage emitter.
//
// The generated kernel is one pass over the output: every tensor input is read once with 16-byte
// packs, the whole DAG is evaluated in registers, every output is written once with 16-byte
// packs.  Three kernel shapes exist:
//   flat        all tensors share one element count; CTA b owns packs [b*256*U, (b+1)*256*U)
//   tiled       broadcast stage viewed as [rows, cols]; a thread owns ONE column pack and walks
//               U rows, so operands that are constant along rows (per-column vectors) are loaded
//               once per thread into registers, operands constant along columns (per-row scalars)
//               cost one warp-uniform load per row, and no per-element div/mod is executed
//   generic     one element per thread with baked div/mod index math; no alignment assumption
// Numerics follow the reference's per-node rule: a node computes in its compute dtype and its
// value is rounded to its output dtype (ExpressionDTypeResolution.cpp:1012-1128).  When every
// tensor and node of the stage is one 16-bit float type the body is emitted on half2/bfloat162
// pairs with the same intrinsics the reference's vector path uses (CudaSourceEmitter.cpp:4373-4435);
// otherwise on typed scalars with the scalar op table (CudaSourceEmitter.cpp:1749-1959).
#include "expr_emit.h"

#include <cmath>
#include <cstdio>
#include <algorithm>
#include <cstdlib>
#include <sstream>

#include "common.cuh"

namespace tb::expr {

namespace {

using Op = thor_b200_expr_op;

bool isScalarLeaf(uint16_t op) { return op == THOR_B200_OP_SCALAR_FP || op == THOR_B200_OP_RUNTIME_SCALAR || op == THOR_B200_OP_TENSOR_RUNTIME_SCALAR; }
bool isLeaf(uint16_t op) { return op == THOR_B200_OP_INPUT || isScalarLeaf(op); }
bool isComparison(uint16_t op) { return op >= THOR_B200_OP_EQUAL && op <= THOR_B200_OP_GREATER_EQUAL; }
bool isLogicalBinary(uint16_t op) { return op == THOR_B200_OP_LOGICAL_AND || op == THOR_B200_OP_LOGICAL_OR; }
bool isBinary(uint16_t op) {
    return (op >= THOR_B200_OP_ADD && op <= THOR_B200_OP_LOGICAL_OR) || (op >= THOR_B200_OP_MIN && op <= THOR_B200_OP_MAX_GRAD_RIGHT);
}
bool isUnary(uint16_t op) {
    return op == THOR_B200_OP_LOGICAL_NOT || op == THOR_B200_OP_CAST || (op >= THOR_B200_OP_NEG && op <= THOR_B200_OP_NORMCDF);
}
bool isKnownOp(uint16_t op) { return isLeaf(op) || isBinary(op) || isUnary(op) || op == THOR_B200_OP_WHERE; }

bool isIntegral(int dt) { return dt >= THOR_B200_INT8 && dt <= THOR_B200_UINT64; }
bool isStorable(int dt) { return dtypeSize(dt) != 0 && dt != THOR_B200_FP64; }
bool isArithCompute(int dt) { return dt == THOR_B200_FP32 || dt == THOR_B200_FP16 || dt == THOR_B200_BF16; }

const char* ctype(int dt) {
    switch (dt) {
        case THOR_B200_FP16: return "__half";
        case THOR_B200_BF16: return "__nv_bfloat16";
        case THOR_B200_FP32: return "float";
        case THOR_B200_INT8: return "signed char";
        case THOR_B200_INT16: return "short";
        case THOR_B200_INT32: return "int";
        case THOR_B200_INT64: return "long long";
        case THOR_B200_UINT8: return "unsigned char";
        case THOR_B200_UINT16: return "unsigned short";
        case THOR_B200_UINT32: return "unsigned int";
        case THOR_B200_UINT64: return "unsigned long long";
        case THOR_B200_BOOLEAN: return "bool";
        case THOR_B200_FP8_E4M3: return "__nv_fp8_e4m3";
        case THOR_B200_FP8_E5M2: return "__nv_fp8_e5m2";
        default: return "void";
    }
}

std::string floatLiteral(double v) {
    if (std::isnan(v)) return "__int_as_float(0x7fffffff)";
    if (std::isinf(v)) return v > 0 ? "__int_as_float(0x7f800000)" : "__int_as_float(0xff800000)";
    const float f = static_cast<float>(v);
    char buf[64];
    snprintf(buf, sizeof(buf), "%.9g", static_cast<double>(f));
    std::string s(buf);
    if (s.find('.') == std::string::npos && s.find('e') == std::string::npos && s.find("inf") == std::string::npos) s += ".0";
    return s + "f";
}

// Conversion of a typed scalar expression.  Everything goes through float except same-type and
// integer<->integer casts (CudaSourceEmitter.cpp:1610-1745).
std::string cvt(const std::string& e, int src, int dst) {
    if (src == dst) return e;
    if (dst == THOR_B200_FP32) {
        switch (src) {
            case THOR_B200_FP16: return "__half2float(" + e + ")";
            case THOR_B200_BF16: return "__bfloat162float(" + e + ")";
            case THOR_B200_BOOLEAN: return "(" + e + " ? 1.0f : 0.0f)";
            default: return "float(" + e + ")";
        }
    }
    if (dst == THOR_B200_BOOLEAN) return "(" + cvt(e, src, THOR_B200_FP32) + " != 0.0f)";
    if (isIntegral(dst)) {
        if (isIntegral(src)) return std::string("static_cast<") + ctype(dst) + ">(" + e + ")";
        if (src == THOR_B200_BOOLEAN) return std::string("static_cast<") + ctype(dst) + ">(" + e + " ? 1 : 0)";
        return std::string("static_cast<") + ctype(dst) + ">(" + cvt(e, src, THOR_B200_FP32) + ")";
    }
    const std::string f = cvt(e, src, THOR_B200_FP32);
    switch (dst) {
        case THOR_B200_FP16: return "__float2half_rn(" + f + ")";
        case THOR_B200_BF16: return "__float2bfloat16_rn(" + f + ")";
        case THOR_B200_FP8_E4M3: return "tb_to_e4m3(" + f + ")";
        case THOR_B200_FP8_E5M2: return "__nv_fp8_e5m2(" + f + ")";
        default: return f;
    }
}

const char* floatFunction(uint16_t op) {
    switch (op) {
        case THOR_B200_OP_ABS: return "fabsf";
        case THOR_B200_OP_CEIL: return "ceilf";
        case THOR_B200_OP_FLOOR: return "floorf";
        case THOR_B200_OP_ROUND: return "roundf";
        case THOR_B200_OP_TRUNC: return "truncf";
        case THOR_B200_OP_SIN: return "sinf";
        case THOR_B200_OP_COS: return "cosf";
        case THOR_B200_OP_TAN: return "tanf";
        case THOR_B200_OP_ASIN: return "asinf";
        case THOR_B200_OP_ACOS: return "acosf";
        case THOR_B200_OP_ATAN: return "atanf";
        case THOR_B200_OP_SINH: return "sinhf";
        case THOR_B200_OP_COSH: return "coshf";
        case THOR_B200_OP_ASINH: return "asinhf";
        case THOR_B200_OP_ACOSH: return "acoshf";
        case THOR_B200_OP_ATANH: return "atanhf";
        case THOR_B200_OP_ERF: return "erff";
        case THOR_B200_OP_ERFC: return "erfcf";
        case THOR_B200_OP_ERFCX: return "erfcxf";
        case THOR_B200_OP_ERFINV: return "erfinvf";
        case THOR_B200_OP_ERFCINV: return "erfcinvf";
        case THOR_B200_OP_TGAMMA: return "tgammaf";
        case THOR_B200_OP_LGAMMA: return "lgammaf";
        case THOR_B200_OP_DIGAMMA: return "tb_digammaf";
        case THOR_B200_OP_EXP: return "expf";
        case THOR_B200_OP_EXPM1: return "expm1f";
        case THOR_B200_OP_EXP2: return "exp2f";
        case THOR_B200_OP_EXP10: return "exp10f";
        case THOR_B200_OP_LN: return "logf";
        case THOR_B200_OP_LOG1P: return "log1pf";
        case THOR_B200_OP_LOG2: return "log2f";
        case THOR_B200_OP_LOG10: return "log10f";
        case THOR_B200_OP_SQRT: return "sqrtf";
        case THOR_B200_OP_TANH: return "tanhf";
        case THOR_B200_OP_NORMCDF: return "normcdff";
        default: return nullptr;
    }
}

std::string gradMask(uint16_t op, const std::string& a, const std::string& b) {
    // 1 / 0 / 0.5 on ties (CudaSourceEmitter.cpp:1940-1954)
    const char* first = (op == THOR_B200_OP_MIN_GRAD_LEFT || op == THOR_B200_OP_MAX_GRAD_RIGHT) ? " < " : " > ";
    const char* second = (op == THOR_B200_OP_MIN_GRAD_LEFT || op == THOR_B200_OP_MAX_GRAD_RIGHT) ? " > " : " < ";
    return "((" + a + first + b + ") ? 1.0f : ((" + a + second + b + ") ? 0.0f : 0.5f))";
}

struct Plan {
    const Stage& st;
    std::vector<bool> live;
    bool v2 = false;
    int v2_dtype = 0;
    // value-range facts used to pick cheaper bit-identical routines: "<= 0 or NaN" / ">= 0 or NaN"
    std::vector<bool> nonpos, nonneg;
    // half2 bodies: node k = exp(-max(-z, 0)) takes its value from node exp_twin[k] = exp(-|z|) of the same z (node
    // exp_twin_z[k]) where z < 0 and is 1 elsewhere; `order` is the emission order (such a node moves behind its twin)
    std::vector<int> exp_twin;
    std::vector<uint32_t> exp_twin_z;
    std::vector<uint32_t> order;
    explicit Plan(const Stage& s) : st(s) {}
};

void analyseSigns(Plan& p) {
    const auto& n = p.st.nodes;
    p.nonpos.assign(n.size(), false);
    p.nonneg.assign(n.size(), false);
    for (size_t k = 0; k < n.size(); ++k) {
        if (!p.live[k]) continue;
        const auto& nd = n[k];
        auto np = [&](uint32_t i) { return i != THOR_B200_NO_NODE && p.nonpos[i]; };
        auto nn = [&](uint32_t i) { return i != THOR_B200_NO_NODE && p.nonneg[i]; };
        switch (nd.op) {
            case THOR_B200_OP_SCALAR_FP: p.nonneg[k] = nd.scalar_fp >= 0.0; p.nonpos[k] = nd.scalar_fp <= 0.0; break;
            case THOR_B200_OP_ABS: case THOR_B200_OP_EXP: case THOR_B200_OP_EXP2: case THOR_B200_OP_EXP10: case THOR_B200_OP_SQRT: case THOR_B200_OP_COSH:
                p.nonneg[k] = true; break;
            case THOR_B200_OP_NEG: p.nonneg[k] = np(nd.lhs); p.nonpos[k] = nn(nd.lhs); break;
            case THOR_B200_OP_CAST: p.nonneg[k] = nn(nd.lhs); p.nonpos[k] = np(nd.lhs); break;
            case THOR_B200_OP_MAX: p.nonneg[k] = nn(nd.lhs) || nn(nd.rhs); p.nonpos[k] = np(nd.lhs) && np(nd.rhs); break;
            case THOR_B200_OP_MIN: p.nonpos[k] = np(nd.lhs) || np(nd.rhs); p.nonneg[k] = nn(nd.lhs) && nn(nd.rhs); break;
            case THOR_B200_OP_MUL: case THOR_B200_OP_DIV:
                p.nonneg[k] = (nn(nd.lhs) && nn(nd.rhs)) || (np(nd.lhs) && np(nd.rhs));
                p.nonpos[k] = (nn(nd.lhs) && np(nd.rhs)) || (np(nd.lhs) && nn(nd.rhs));
                break;
            case THOR_B200_OP_ADD: p.nonneg[k] = nn(nd.lhs) && nn(nd.rhs); p.nonpos[k] = np(nd.lhs) && np(nd.rhs); break;
            default: break;
        }
    }
}

void markLive(Plan& p) {
    const auto& n = p.st.nodes;
    p.live.assign(n.size(), false);
    for (const auto& o : p.st.outputs) p.live[o.node] = true;
    for (size_t k = n.size(); k-- > 0;) {
        if (!p.live[k]) continue;
        for (uint32_t parent : {n[k].lhs, n[k].rhs, n[k].aux})
            if (parent != THOR_B200_NO_NODE) p.live[parent] = true;
    }
}

// half2 / bfloat162 body eligibility: one 16-bit float type everywhere and only ops that the pair
// table covers.
void decideV2(Plan& p) {
    int d = 0;
    for (const auto& in : p.st.inputs) {
        if (in.kind == THOR_B200_INPUT_RUNTIME_SCALAR_FP32) continue;
        if (in.kind == THOR_B200_INPUT_TENSOR_RUNTIME_SCALAR) continue;
        if (d == 0) d = in.dtype;
        if (in.dtype != d) return;
    }
    for (const auto& o : p.st.outputs) {
        if (d == 0) d = o.dtype;
        if (o.dtype != d) return;
    }
    if (d != THOR_B200_FP16 && d != THOR_B200_BF16) return;
    for (size_t k = 0; k < p.st.nodes.size(); ++k) {
        if (!p.live[k]) continue;
        const auto& nd = p.st.nodes[k];
        if (isScalarLeaf(nd.op)) continue;
        if (nd.op == THOR_B200_OP_INPUT) {
            if (nd.output_dtype != d) return;
            continue;
        }
        if (nd.output_dtype != d || nd.compute_dtype != d) return;
        if (isComparison(nd.op) || isLogicalBinary(nd.op) || nd.op == THOR_B200_OP_LOGICAL_NOT || nd.op == THOR_B200_OP_WHERE) return;
    }
    p.v2 = true;
    p.v2_dtype = d;
}

std::string nodeVar(size_t k) { return "v" + std::to_string(k); }

// Type in which a node's value lives inside a kernel (CudaSourceEmitter.cpp:2077-2083): leaves and
// casts carry their output dtype; every other arithmetic node stays in its compute dtype and is
// rounded to its output dtype only where it is materialised -- when a stage stores it, or when a
// reduction consumes it.  fp16 / bf16 / fp32 graphs compute and store in one type, so this only shows
// in fp8 graphs (compute fp16, store fp8) and on nodes with an explicitly requested output dtype.
int valueDTypeImpl(const std::vector<thor_b200_expr_node>& nodes, size_t k) {
    const auto& nd = nodes[k];
    if (isLeaf(nd.op) || nd.op == THOR_B200_OP_CAST) return nd.output_dtype;
    if (isComparison(nd.op) || isLogicalBinary(nd.op) || nd.op == THOR_B200_OP_LOGICAL_NOT) return nd.output_dtype;
    if (!isKnownOp(nd.op)) return nd.output_dtype;  // reductions of row programs: their result is a stored value
    return isArithCompute(nd.compute_dtype) ? nd.compute_dtype : nd.output_dtype;
}

// ---- scalar body -------------------------------------------------------------------------------
std::string scalarNodeExprImpl(const std::vector<thor_b200_expr_node>& nodes, const std::vector<thor_b200_expr_input>& inputs, size_t k) {
    const auto& nd = nodes[k];
    const int C = nd.compute_dtype;
    const int O = valueDTypeImpl(nodes, k);  // the type the value is kept in
    auto parent = [&](uint32_t idx, int to) { return cvt(nodeVar(idx), valueDTypeImpl(nodes, idx), to); };
    switch (nd.op) {
        case THOR_B200_OP_INPUT: return cvt("x" + std::to_string(nd.input_slot), inputs[nd.input_slot].dtype, O);
        case THOR_B200_OP_RUNTIME_SCALAR: return cvt("s" + std::to_string(nd.input_slot), THOR_B200_FP32, O);
        case THOR_B200_OP_TENSOR_RUNTIME_SCALAR: return cvt("s" + std::to_string(nd.input_slot), inputs[nd.input_slot].dtype, O);
        case THOR_B200_OP_SCALAR_FP: return cvt(floatLiteral(nd.scalar_fp), THOR_B200_FP32, O);
        case THOR_B200_OP_CAST: return parent(nd.lhs, O);
        case THOR_B200_OP_WHERE:
            return cvt("(" + parent(nd.lhs, THOR_B200_BOOLEAN) + " ? " + parent(nd.rhs, C) + " : " + parent(nd.aux, C) + ")", C, O);
        default: break;
    }
    if (isComparison(nd.op)) {
        const std::string a = cvt(parent(nd.lhs, C), C, THOR_B200_FP32), b = cvt(parent(nd.rhs, C), C, THOR_B200_FP32);
        const char* sym = nd.op == THOR_B200_OP_EQUAL ? " == " : nd.op == THOR_B200_OP_NOT_EQUAL ? " != " : nd.op == THOR_B200_OP_LESS ? " < "
                        : nd.op == THOR_B200_OP_LESS_EQUAL ? " <= " : nd.op == THOR_B200_OP_GREATER ? " > " : " >= ";
        return cvt("(" + a + sym + b + ")", THOR_B200_BOOLEAN, O);
    }
    if (isLogicalBinary(nd.op)) {
        const char* sym = nd.op == THOR_B200_OP_LOGICAL_AND ? " && " : " || ";
        return cvt("(" + parent(nd.lhs, THOR_B200_BOOLEAN) + sym + parent(nd.rhs, THOR_B200_BOOLEAN) + ")", THOR_B200_BOOLEAN, O);
    }
    if (nd.op == THOR_B200_OP_LOGICAL_NOT) return cvt("(!" + parent(nd.lhs, THOR_B200_BOOLEAN) + ")", THOR_B200_BOOLEAN, O);

    // arithmetic: native in fp32 / fp16 / bf16 for + - * / and unary minus, through float otherwise
    const std::string a = parent(nd.lhs, C);
    const std::string af = cvt(a, C, THOR_B200_FP32);
    if (nd.op == THOR_B200_OP_NEG) {
        if (C == THOR_B200_FP32) return cvt("(-" + a + ")", C, O);
        return cvt("__hneg(" + a + ")", C, O);
    }
    if (nd.op == THOR_B200_OP_TANH && C == THOR_B200_FP16) return cvt("htanh(" + a + ")", C, O);
    if (const char* fn = floatFunction(nd.op)) return cvt(cvt(std::string(fn) + "(" + af + ")", THOR_B200_FP32, C), C, O);

    const std::string b = parent(nd.rhs, C);
    const std::string bf = cvt(b, C, THOR_B200_FP32);
    std::string r;
    switch (nd.op) {
        case THOR_B200_OP_ADD: r = C == THOR_B200_FP32 ? "(" + a + " + " + b + ")" : "__hadd(" + a + ", " + b + ")"; break;
        case THOR_B200_OP_SUB: r = C == THOR_B200_FP32 ? "(" + a + " - " + b + ")" : "__hsub(" + a + ", " + b + ")"; break;
        case THOR_B200_OP_MUL: r = C == THOR_B200_FP32 ? "(" + a + " * " + b + ")" : "__hmul(" + a + ", " + b + ")"; break;
        case THOR_B200_OP_DIV: r = C == THOR_B200_FP32 ? "(" + a + " / " + b + ")" : "__hdiv(" + a + ", " + b + ")"; break;
        case THOR_B200_OP_POW: r = cvt("powf(" + af + ", " + bf + ")", THOR_B200_FP32, C); break;
        case THOR_B200_OP_MIN: r = cvt("fminf(" + af + ", " + bf + ")", THOR_B200_FP32, C); break;
        case THOR_B200_OP_MAX: r = cvt("fmaxf(" + af + ", " + bf + ")", THOR_B200_FP32, C); break;
        default: r = cvt(gradMask(nd.op, af, bf), THOR_B200_FP32, C); break;
    }
    return cvt(r, C, O);
}

std::string scalarNodeExpr(const Plan& p, size_t k) { return scalarNodeExprImpl(p.st.nodes, p.st.inputs, k); }

// ---- half2 / bfloat162 body --------------------------------------------------------------------
// The reference's overflow-safe sigmoid (Expression.h:1077-1088) is exp(-max(-z, 0)) / (1 + exp(-|z|)).  For z < 0 both
// exponentials have the same argument (z itself); elsewhere (z >= 0, -0, NaN) the first is exp(-0) = 1.  So the first
// is a select of the second: one exponential per element instead of two, with identical bits.
void findExpTwins(Plan& p) {
    const auto& n = p.st.nodes;
    p.exp_twin.assign(n.size(), -1);
    p.exp_twin_z.assign(n.size(), THOR_B200_NO_NODE);
    p.order.clear();
    for (uint32_t k = 0; k < n.size(); ++k) p.order.push_back(k);
    // the same routine evaluates both exponentials, whichever it is, so equal arguments give equal bits; in scalar bodies
    // the nodes of both chains must also round alike (same compute and output dtype everywhere)
    auto sameDTypes = [&](uint32_t k, uint32_t m) {
        if (p.v2) return true;
        auto chainOk = [&](uint32_t e) {
            uint32_t i = e;
            for (int hops = 0; hops < 3 && i != THOR_B200_NO_NODE; ++hops) {  // exp, neg, max / abs
                if (n[i].op == THOR_B200_OP_CAST) return false;
                if (n[i].compute_dtype != n[e].compute_dtype || n[i].output_dtype != n[e].output_dtype) return false;
                i = n[i].lhs;
            }
            return true;
        };
        return chainOk(k) && chainOk(m) && n[k].compute_dtype == n[m].compute_dtype && n[k].output_dtype == n[m].output_dtype && isArithCompute(n[k].compute_dtype);
    };
    auto strip = [&](uint32_t i) {
        while (i != THOR_B200_NO_NODE && n[i].op == THOR_B200_OP_CAST) i = n[i].lhs;
        return i;
    };
    auto isZero = [&](uint32_t i) { return i != THOR_B200_NO_NODE && n[i].op == THOR_B200_OP_SCALAR_FP && n[i].scalar_fp == 0.0; };
    auto negOf = [&](uint32_t i) -> uint32_t {  // z when node i is -z
        i = strip(i);
        return i != THOR_B200_NO_NODE && n[i].op == THOR_B200_OP_NEG ? strip(n[i].lhs) : THOR_B200_NO_NODE;
    };
    auto clampedForm = [&](uint32_t i) -> uint32_t {  // z when node i is exp(-max(-z, 0))
        if (n[i].op != THOR_B200_OP_EXP) return THOR_B200_NO_NODE;
        const uint32_t m = negOf(n[i].lhs);
        if (m == THOR_B200_NO_NODE || n[m].op != THOR_B200_OP_MAX) return THOR_B200_NO_NODE;
        const uint32_t a = strip(n[m].lhs), b = strip(n[m].rhs);
        if (isZero(b)) return negOf(a);
        if (isZero(a)) return negOf(b);
        return THOR_B200_NO_NODE;
    };
    auto absForm = [&](uint32_t i) -> uint32_t {  // z when node i is exp(-|z|), |z| spelled abs(z) or max(z, -z)
        if (n[i].op != THOR_B200_OP_EXP) return THOR_B200_NO_NODE;
        const uint32_t m = negOf(n[i].lhs);
        if (m == THOR_B200_NO_NODE) return THOR_B200_NO_NODE;
        if (n[m].op == THOR_B200_OP_ABS) return strip(n[m].lhs);
        if (n[m].op != THOR_B200_OP_MAX) return THOR_B200_NO_NODE;
        const uint32_t a = strip(n[m].lhs), b = strip(n[m].rhs);
        if (a != THOR_B200_NO_NODE && negOf(b) == a) return a;
        if (b != THOR_B200_NO_NODE && negOf(a) == b) return b;
        return THOR_B200_NO_NODE;
    };
    for (uint32_t k = 0; k < n.size(); ++k) {
        if (!p.live[k]) continue;
        const uint32_t z = clampedForm(k);
        if (z == THOR_B200_NO_NODE) continue;
        for (uint32_t m = 0; m < n.size(); ++m) {
            if (m == k || !p.live[m] || p.exp_twin[m] >= 0 || absForm(m) != z || !sameDTypes(k, m)) continue;
            // k is emitted behind m: every consumer of k must come later still
            bool ok = true;
            for (uint32_t j = 0; j <= m && ok; ++j)
                for (uint32_t par : {n[j].lhs, n[j].rhs, n[j].aux}) ok = ok && !(par == k && p.live[j]);
            if (!ok) continue;
            p.exp_twin[k] = static_cast<int>(m);
            p.exp_twin_z[k] = z;
            if (m > k) {
                p.order.erase(std::find(p.order.begin(), p.order.end(), k));
                p.order.insert(std::find(p.order.begin(), p.order.end(), m) + 1, k);
            }
            break;
        }
    }
}

std::string v2NodeExpr(const Plan& p, size_t k) {
    const auto& nd = p.st.nodes[k];
    const int D = p.v2_dtype;
    const bool bf = D == THOR_B200_BF16;
    const std::string from2 = bf ? "__floats2bfloat162_rn" : "__floats2half2_rn";
    const std::string dup = bf ? "__bfloat162bfloat162" : "__half2half2";
    auto lo = [&](const std::string& v) { return "__low2float(" + v + ")"; };
    auto hi = [&](const std::string& v) { return "__high2float(" + v + ")"; };
    switch (nd.op) {
        case THOR_B200_OP_INPUT: return "x" + std::to_string(nd.input_slot);
        case THOR_B200_OP_RUNTIME_SCALAR:
            // fp32 value -> node output dtype -> pair compute dtype (CudaSourceEmitter.cpp:4348-4364)
            return dup + "(" + cvt(cvt("s" + std::to_string(nd.input_slot), THOR_B200_FP32, nd.output_dtype), nd.output_dtype, D) + ")";
        case THOR_B200_OP_TENSOR_RUNTIME_SCALAR:
            return dup + "(" + cvt(cvt("s" + std::to_string(nd.input_slot), p.st.inputs[nd.input_slot].dtype, nd.output_dtype), nd.output_dtype, D) + ")";
        case THOR_B200_OP_SCALAR_FP: return dup + "(" + cvt(cvt(floatLiteral(nd.scalar_fp), THOR_B200_FP32, nd.output_dtype), nd.output_dtype, D) + ")";
        case THOR_B200_OP_CAST: return nodeVar(nd.lhs);
        default: break;
    }
    if (!p.exp_twin.empty() && p.exp_twin[k] >= 0)
        return "tb_h2sel_neg(" + nodeVar(p.exp_twin_z[k]) + ", " + nodeVar(static_cast<size_t>(p.exp_twin[k])) + ", " + dup + "(" + cvt("1.0f", THOR_B200_FP32, D) + "))";
    const std::string a = nodeVar(nd.lhs);
    const std::string b = nd.rhs != THOR_B200_NO_NODE ? nodeVar(nd.rhs) : std::string();
    switch (nd.op) {
        case THOR_B200_OP_ADD: return "__hadd2(" + a + ", " + b + ")";
        case THOR_B200_OP_SUB: return "__hsub2(" + a + ", " + b + ")";
        case THOR_B200_OP_MUL: return "__hmul2(" + a + ", " + b + ")";
        case THOR_B200_OP_DIV: return (!bf ? "tb_h2div(" : "__h2div(") + a + ", " + b + ")";
        case THOR_B200_OP_NEG: return "__hneg2(" + a + ")";
        case THOR_B200_OP_ABS: return "__hmax2(" + a + ", __hneg2(" + a + "))";
        case THOR_B200_OP_EXP:
            if (!bf) return std::string(p.nonpos[nd.lhs] ? "tb_h2exp_nonpos(" : "tb_h2exp(") + a + ")";
            return "h2exp(" + a + ")";
        case THOR_B200_OP_EXP2: return "h2exp2(" + a + ")";
        case THOR_B200_OP_EXP10: return "h2exp10(" + a + ")";
        case THOR_B200_OP_LN: return "h2log(" + a + ")";
        case THOR_B200_OP_LOG2: return "h2log2(" + a + ")";
        case THOR_B200_OP_LOG10: return "h2log10(" + a + ")";
        case THOR_B200_OP_SQRT: return "h2sqrt(" + a + ")";
        case THOR_B200_OP_MIN: return "__hmin2(" + a + ", " + b + ")";
        case THOR_B200_OP_MAX: return "__hmax2(" + a + ", " + b + ")";
        case THOR_B200_OP_TANH:
            if (!bf) return "h2tanh(" + a + ")";
            break;
        case THOR_B200_OP_POW: return from2 + "(powf(" + lo(a) + ", " + lo(b) + "), powf(" + hi(a) + ", " + hi(b) + "))";
        case THOR_B200_OP_MIN_GRAD_LEFT: case THOR_B200_OP_MIN_GRAD_RIGHT: case THOR_B200_OP_MAX_GRAD_LEFT: case THOR_B200_OP_MAX_GRAD_RIGHT:
            return from2 + "(" + gradMask(nd.op, lo(a), lo(b)) + ", " + gradMask(nd.op, hi(a), hi(b)) + ")";
        default: break;
    }
    const char* fn = floatFunction(nd.op);
    return from2 + "(" + fn + "(" + lo(a) + "), " + fn + "(" + hi(a) + "))";
}

// Body function: tensor inputs (slot order) by value, scalars by value, outputs by reference.
void emitBody(const Plan& p, std::ostringstream& os) {
    const Stage& st = p.st;
    const std::string T2 = p.v2_dtype == THOR_B200_BF16 ? "__nv_bfloat162" : "__half2";
    os << "__device__ __forceinline__ void tb_body(";
    bool first = true;
    for (size_t s = 0; s < st.inputs.size(); ++s) {
        if (!first) os << ", ";
        first = false;
        const auto& in = st.inputs[s];
        if (in.kind == THOR_B200_INPUT_TENSOR) os << "const " << (p.v2 ? T2 : std::string(ctype(in.dtype))) << " x" << s;
        else if (in.kind == THOR_B200_INPUT_RUNTIME_SCALAR_FP32) os << "const float s" << s;
        else os << "const " << ctype(in.dtype) << " s" << s;
    }
    for (size_t o = 0; o < st.outputs.size(); ++o) {
        if (!first) os << ", ";
        first = false;
        os << (p.v2 ? T2 : std::string(ctype(st.outputs[o].dtype))) << "& y" << o;
    }
    os << ") {\n";
    for (size_t k : p.order) {
        if (!p.live[k]) continue;
        const std::string type = p.v2 ? T2 : std::string(ctype(valueDTypeImpl(st.nodes, k)));
        if (!p.v2 && !p.exp_twin.empty() && p.exp_twin[k] >= 0) {
            // exp(-max(-z, 0)) from its twin exp(-|z|): identical where z < 0, exactly 1 elsewhere
            const int V = valueDTypeImpl(st.nodes, k);
            os << "    const " << type << " " << nodeVar(k) << " = (" << cvt(nodeVar(p.exp_twin_z[k]), valueDTypeImpl(st.nodes, p.exp_twin_z[k]), THOR_B200_FP32) << " < 0.0f) ? "
               << nodeVar(static_cast<size_t>(p.exp_twin[k])) << " : " << cvt("1.0f", THOR_B200_FP32, V) << ";\n";
            continue;
        }
        os << "    const " << type << " " << nodeVar(k) << " = " << (p.v2 ? v2NodeExpr(p, k) : scalarNodeExpr(p, k)) << ";\n";
    }
    for (size_t o = 0; o < st.outputs.size(); ++o) {
        const uint32_t k = st.outputs[o].node;
        os << "    y" << o << " = " << (p.v2 ? nodeVar(k) : cvt(nodeVar(k), valueDTypeImpl(st.nodes, k), st.outputs[o].dtype)) << ";\n";
    }
    os << "}\n\n";
}

std::string kernelParams(const Stage& st, bool with_numel) {
    std::ostringstream os;
    bool first = true;
    for (size_t s = 0; s < st.inputs.size(); ++s) {
        if (!first) os << ", ";
        first = false;
        const auto& in = st.inputs[s];
        if (in.kind == THOR_B200_INPUT_RUNTIME_SCALAR_FP32) os << "const float s" << s;
        else os << "const " << ctype(in.dtype) << "* in" << s;
    }
    for (size_t o = 0; o < st.outputs.size(); ++o) {
        if (!first) os << ", ";
        first = false;
        os << ctype(st.outputs[o].dtype) << "* out" << o;
    }
    if (with_numel) os << (first ? "" : ", ") << "const tb_u64 numel";
    return os.str();
}

std::string launchBounds(const Stage& st) {
    if (st.min_ctas_per_sm > 0) return "__launch_bounds__(256, " + std::to_string(st.min_ctas_per_sm) + ")";
    return "__launch_bounds__(256)";
}

// Loads of one-element tensor scalars, once per thread.
void emitScalarLoads(const Stage& st, std::ostringstream& os) {
    for (size_t s = 0; s < st.inputs.size(); ++s)
        if (st.inputs[s].kind == THOR_B200_INPUT_TENSOR_RUNTIME_SCALAR) os << "    const " << ctype(st.inputs[s].dtype) << " s" << s << " = in" << s << "[0];\n";
}

// Call of tb_body on lane j of the packs: `inExpr(slot)` names the j-th element (or pair) of input slot.
template <class InFn, class OutFn>
std::string bodyCall(const Stage& st, InFn inExpr, OutFn outExpr) {
    std::ostringstream os;
    os << "tb_body(";
    bool first = true;
    for (size_t s = 0; s < st.inputs.size(); ++s) {
        if (!first) os << ", ";
        first = false;
        if (st.inputs[s].kind == THOR_B200_INPUT_TENSOR) os << inExpr(s);
        else os << "s" << s;
    }
    for (size_t o = 0; o < st.outputs.size(); ++o) {
        if (!first) os << ", ";
        first = false;
        os << outExpr(o);
    }
    os << ");";
    return os.str();
}

int chooseVec(const Plan& p) {
    if (p.v2) return 8;
    size_t mn = 8, mx = 1;
    auto upd = [&](int dt) { const size_t s = dtypeSize(dt); if (s < mn) mn = s; if (s > mx) mx = s; };
    for (const auto& in : p.st.inputs) if (in.kind == THOR_B200_INPUT_TENSOR) upd(in.dtype);
    for (const auto& o : p.st.outputs) upd(o.dtype);
    int vec = static_cast<int>(16 / mn);
    while (vec > 1 && static_cast<size_t>(vec) * mx > 64) vec /= 2;
    return vec;
}

int tensorInputCount(const Stage& st) {
    int c = 0;
    for (const auto& in : st.inputs) c += in.kind == THOR_B200_INPUT_TENSOR;
    return c;
}

std::string elemType(const Plan& p, int dt) { return p.v2 ? (p.v2_dtype == THOR_B200_BF16 ? "__nv_bfloat162" : "__half2") : std::string(ctype(dt)); }

// ---- flat kernel -------------------------------------------------------------------------------
void emitFlat(const Plan& p, Emitted* out, std::ostringstream& os) {
    const Stage& st = p.st;
    const int VEC = chooseVec(p);
    const int lanes = p.v2 ? VEC / 2 : VEC;
    size_t in_bytes = 0;
    for (const auto& in : st.inputs) if (in.kind == THOR_B200_INPUT_TENSOR) in_bytes += dtypeSize(in.dtype) * VEC;
    int U = in_bytes >= 48 ? 1 : 2;
    if (st.packs_per_thread == 1 || st.packs_per_thread == 2 || st.packs_per_thread == 4) U = st.packs_per_thread;
    out->kind = p.v2 ? Kind::FlatV2 : Kind::FlatScalar;
    out->vec = VEC;
    out->unroll = U;
    out->threads = 256;
    os << "extern \"C\" __global__ void " << launchBounds(st) << " fused_kernel(" << kernelParams(st, true) << ") {\n";
    os << "    tb_grid_wait();\n";
    os << "    constexpr int VEC = " << VEC << ", U = " << U << ";\n";
    os << "    const tb_u64 n_packs = numel / VEC;\n";
    os << "    const tb_u64 base = (tb_u64)blockIdx.x * (256 * U) + threadIdx.x;\n";
    emitScalarLoads(st, os);
    for (size_t s = 0; s < st.inputs.size(); ++s)
        if (st.inputs[s].kind == THOR_B200_INPUT_TENSOR) os << "    tb_pack<VEC * " << dtypeSize(st.inputs[s].dtype) << "> p" << s << "[U];\n";
    os << "#pragma unroll\n    for (int u = 0; u < U; ++u) {\n        const tb_u64 q = base + (tb_u64)u * 256;\n        if (q < n_packs) {\n";
    for (size_t s = 0; s < st.inputs.size(); ++s)
        if (st.inputs[s].kind == THOR_B200_INPUT_TENSOR) os << "            tb_load_stream(p" << s << "[u], in" << s << " + q * VEC);\n";
    os << "        }\n    }\n";
    os << "#pragma unroll\n    for (int u = 0; u < U; ++u) {\n        const tb_u64 q = base + (tb_u64)u * 256;\n        if (q < n_packs) {\n";
    for (size_t o = 0; o < st.outputs.size(); ++o) os << "            tb_pack<VEC * " << dtypeSize(st.outputs[o].dtype) << "> r" << o << ";\n";
    os << "#pragma unroll\n            for (int j = 0; j < " << lanes << "; ++j) {\n                "
       << bodyCall(st, [&](size_t s) { return "reinterpret_cast<const " + elemType(p, st.inputs[s].dtype) + "*>(&p" + std::to_string(s) + "[u])[j]"; },
                   [&](size_t o) { return "reinterpret_cast<" + elemType(p, st.outputs[o].dtype) + "*>(&r" + std::to_string(o) + ")[j]"; })
       << "\n            }\n";
    for (size_t o = 0; o < st.outputs.size(); ++o) os << "            tb_store_stream(out" << o << " + q * VEC, r" << o << ");\n";
    os << "        }\n    }\n";
    // ragged tail: numel % VEC elements, one per thread of the first CTA
    os << "    if (blockIdx.x == 0) {\n        const tb_u64 i = n_packs * VEC + threadIdx.x;\n        if (i < numel) {\n";
    if (p.v2) {
        const std::string dup = p.v2_dtype == THOR_B200_BF16 ? "__bfloat162bfloat162" : "__half2half2";
        for (size_t o = 0; o < st.outputs.size(); ++o) os << "            " << elemType(p, 0) << " t" << o << ";\n";
        os << "            " << bodyCall(st, [&](size_t s) { return dup + "(in" + std::to_string(s) + "[i])"; }, [&](size_t o) { return "t" + std::to_string(o); }) << "\n";
        for (size_t o = 0; o < st.outputs.size(); ++o) os << "            out" << o << "[i] = __low2" << (p.v2_dtype == THOR_B200_BF16 ? "bfloat16" : "half") << "(t" << o << ");\n";
    } else {
        for (size_t o = 0; o < st.outputs.size(); ++o) os << "            " << ctype(st.outputs[o].dtype) << " t" << o << ";\n";
        os << "            " << bodyCall(st, [&](size_t s) { return "in" + std::to_string(s) + "[i]"; }, [&](size_t o) { return "t" + std::to_string(o); }) << "\n";
        for (size_t o = 0; o < st.outputs.size(); ++o) os << "            out" << o << "[i] = t" << o << ";\n";
    }
    os << "        }\n    }\n}\n";
    out->input_align.assign(st.inputs.size(), 1);
    for (size_t s = 0; s < st.inputs.size(); ++s)
        if (st.inputs[s].kind == THOR_B200_INPUT_TENSOR) out->input_align[s] = static_cast<int>(std::min<size_t>(16, dtypeSize(st.inputs[s].dtype) * VEC));
    out->output_align.assign(st.outputs.size(), 1);
    for (size_t o = 0; o < st.outputs.size(); ++o) out->output_align[o] = static_cast<int>(std::min<size_t>(16, dtypeSize(st.outputs[o].dtype) * VEC));
}

// ---- broadcast geometry ------------------------------------------------------------------------
struct Collapsed {
    std::vector<uint64_t> dims;                 // outer -> inner
    std::vector<std::vector<int64_t>> strides;  // [slot][dim]
};

// Drops size-1 axes and merges neighbouring axes that every tensor input walks contiguously
// (stride[d] == stride[d+1] * dim[d+1], which also holds when both are 0).
Collapsed collapse(const Stage& st) {
    Collapsed c;
    const size_t n_in = st.inputs.size();
    c.strides.assign(n_in, {});
    for (uint32_t d = 0; d < st.rank; ++d) {
        if (st.dims[d] == 1) continue;
        c.dims.push_back(st.dims[d]);
        for (size_t s = 0; s < n_in; ++s) c.strides[s].push_back(st.inputs[s].kind == THOR_B200_INPUT_TENSOR ? st.strides[s][d] : 0);
    }
    if (c.dims.empty()) {
        c.dims.push_back(1);
        for (size_t s = 0; s < n_in; ++s) c.strides[s].push_back(st.inputs[s].kind == THOR_B200_INPUT_TENSOR ? 1 : 0);
        return c;
    }
    for (size_t d = c.dims.size() - 1; d-- > 0;) {
        bool ok = true;
        for (size_t s = 0; s < n_in && ok; ++s) {
            if (st.inputs[s].kind != THOR_B200_INPUT_TENSOR) continue;
            ok = c.strides[s][d] == c.strides[s][d + 1] * static_cast<int64_t>(c.dims[d + 1]);
        }
        if (!ok) continue;
        c.dims[d] *= c.dims[d + 1];
        c.dims.erase(c.dims.begin() + d + 1);
        for (size_t s = 0; s < n_in; ++s) {
            c.strides[s][d] = c.strides[s][d + 1];
            c.strides[s].erase(c.strides[s].begin() + d + 1);
        }
    }
    return c;
}

// Emits `const tb_u64 <name><slot> = <offset of row r of input slot>` for every tensor input, from
// the outer (all but last) collapsed axes.  Axis extents and strides are literals.
void emitRowOffsets(const Stage& st, const Collapsed& c, const std::string& r, const std::string& indent, const std::string& suffix, std::ostringstream& os) {
    const size_t outer = c.dims.size() - 1;
    if (outer > 1) {
        os << indent << "tb_u64 rem" << suffix << " = " << r << ";\n";
        for (size_t d = outer; d-- > 0;) {
            if (d == 0) os << indent << "const tb_u64 c" << suffix << "_" << d << " = rem" << suffix << ";\n";
            else os << indent << "const tb_u64 c" << suffix << "_" << d << " = rem" << suffix << " % " << c.dims[d] << "ull; rem" << suffix << " /= " << c.dims[d] << "ull;\n";
        }
    }
    for (size_t s = 0; s < st.inputs.size(); ++s) {
        if (st.inputs[s].kind != THOR_B200_INPUT_TENSOR) continue;
        os << indent << "const tb_u64 ro" << suffix << "_" << s << " = 0";
        for (size_t d = 0; d < outer; ++d) {
            if (c.strides[s][d] == 0) continue;
            os << " + " << (outer > 1 ? "c" + suffix + "_" + std::to_string(d) : r) << " * " << c.strides[s][d] << "ull";
        }
        os << ";\n";
    }
}

bool tiledEligible(const Plan& p, const Collapsed& c, int VEC) {
    const Stage& st = p.st;
    if (c.dims.size() < 2) return false;
    const uint64_t cols = c.dims.back();
    if (cols % VEC != 0) return false;
    const size_t last = c.dims.size() - 1;
    for (size_t s = 0; s < st.inputs.size(); ++s) {
        if (st.inputs[s].kind != THOR_B200_INPUT_TENSOR) continue;
        const int64_t inner = c.strides[s][last];
        if (inner != 0 && inner != 1) return false;
        for (size_t d = 0; d < last; ++d) {
            if (c.strides[s][d] < 0) return false;
            // packs of dense operands must stay aligned on every row
            if (inner == 1 && (c.strides[s][d] % VEC) != 0) return false;
        }
    }
    return true;
}

void emitTiled(const Plan& p, const Collapsed& c, Emitted* out, std::ostringstream& os) {
    const Stage& st = p.st;
    const int VEC = chooseVec(p);
    const int lanes = p.v2 ? VEC / 2 : VEC;
    const size_t last = c.dims.size() - 1;
    const uint64_t cols = c.dims.back();
    uint64_t rows = 1;
    for (size_t d = 0; d < last; ++d) rows *= c.dims[d];
    const uint64_t ppr = cols / VEC;
    int tx = 256;
    while (tx > 1 && static_cast<uint64_t>(tx / 2) >= ppr) tx /= 2;
    const int ty = 256 / tx;
    // operand classes
    enum Cls { Dense, ColVec, RowScalar, OneElem };
    std::vector<Cls> cls(st.inputs.size(), Dense);
    int dense = 0;
    for (size_t s = 0; s < st.inputs.size(); ++s) {
        if (st.inputs[s].kind != THOR_B200_INPUT_TENSOR) continue;
        bool outer_zero = true;
        for (size_t d = 0; d < last; ++d) outer_zero = outer_zero && c.strides[s][d] == 0;
        if (c.strides[s][last] == 1) cls[s] = outer_zero ? ColVec : Dense;
        else cls[s] = outer_zero ? OneElem : RowScalar;
        dense += cls[s] == Dense;
    }
    // rows per thread, measured on relu(a*x+b)*sigmoid(z) fp16 (two dense inputs) in the linear CTA order below, 1 / 2 / 4 rows:
    // [8192, 8192] 60.9 / 60.1 / 61.4 us, [4096, 8192] 31.6 / 31.7 / 32.7 us, [2048, 8192] 17.2 / 17.3 / 18.4 us, [1024, 8192]
    // 9.9 / 10.2 / 11.0 us: two rows once the grid is large, one row on smaller tensors, where fewer CTAs fill the last wave worse
    int U = dense <= 1 ? 4 : (rows * ((ppr + tx - 1) / tx) >= 32768 ? 2 : 1);
    if (st.rows_per_thread == 1 || st.rows_per_thread == 2 || st.rows_per_thread == 4 || st.rows_per_thread == 8) U = st.rows_per_thread;
    while (U > 1 && static_cast<uint64_t>(ty) * (U / 2) >= rows) U /= 2;
    out->kind = p.v2 ? Kind::TiledV2 : Kind::TiledScalar;
    out->vec = VEC;
    out->unroll = U;
    out->threads = 256;
    out->rows = rows;
    out->cols = cols;
    out->tx = tx;
    out->ty = ty;
    const std::string T2dup = p.v2_dtype == THOR_B200_BF16 ? "__bfloat162bfloat162" : "__half2half2";

    os << "// rows = " << rows << ", cols = " << cols << ", packs per row = " << ppr << ", CTA = " << tx << " x " << ty << " threads, " << U << " rows per thread\n";
    os << "extern \"C\" __global__ void " << launchBounds(st) << " fused_kernel(" << kernelParams(st, false) << ") {\n";
    os << "    tb_grid_wait();\n";
    os << "    constexpr int VEC = " << VEC << ", U = " << U << ", TX = " << tx << ", TY = " << ty << ";\n";
    os << "    constexpr tb_u64 ROWS = " << rows << "ull, COLS = " << cols << "ull, PPR = " << ppr << "ull;\n";
    os << "    const tb_u32 tx = threadIdx.x % TX, ty = threadIdx.x / TX;\n";
    const uint64_t gy = (ppr + tx - 1) / tx;
    // CTA order: the column chunks of a row block sit in consecutive CTAs of a one-dimensional grid, so the CTAs that
    // run at the same time stream one contiguous range of every dense tensor.  With the row block in blockIdx.x and the
    // chunk in blockIdx.y, neighbouring CTAs read pieces a whole row apart: relu(a*x+b)*sigmoid(z) fp16 [8192, 8192]
    // 65.3 us against 60.6 us in this order (0.944 -> 1.016 of the measured copy bandwidth), [4096, 8192] 34.1 -> 31.5 us.
    {
        const uint64_t rows_per_cta = static_cast<uint64_t>(ty) * U;
        const uint64_t gx = (rows + rows_per_cta - 1) / rows_per_cta;
        out->linear_grid = gx * gy <= 0x7FFFFFFFull;
    }
    if (out->linear_grid) {
        os << "    constexpr tb_u32 GY = " << gy << "u;\n";
        os << "    const tb_u32 by = blockIdx.x % GY, bx = blockIdx.x / GY;\n";
    } else {
        os << "    const tb_u32 by = blockIdx.y, bx = blockIdx.x;\n";
    }
    os << "    const tb_u64 cp = (tb_u64)by * TX + tx;\n";
    os << "    if (cp >= PPR) return;\n";
    os << "    const tb_u64 col = cp * VEC;\n";
    os << "    const tb_u64 row0 = (tb_u64)bx * (TY * U) + ty;\n";
    emitScalarLoads(st, os);
    for (size_t s = 0; s < st.inputs.size(); ++s) {
        if (st.inputs[s].kind != THOR_B200_INPUT_TENSOR) continue;
        if (cls[s] == ColVec) {
            os << "    tb_pack<VEC * " << dtypeSize(st.inputs[s].dtype) << "> k" << s << ";  // constant along rows: loaded once\n";
            os << "    tb_load_keep(k" << s << ", in" << s << " + col);\n";
        } else if (cls[s] == OneElem) {
            os << "    const " << ctype(st.inputs[s].dtype) << " e" << s << " = in" << s << "[0];\n";
        } else if (cls[s] == Dense) {
            os << "    tb_pack<VEC * " << dtypeSize(st.inputs[s].dtype) << "> p" << s << "[U];\n";
        } else {
            os << "    " << ctype(st.inputs[s].dtype) << " e" << s << "[U];  // constant along columns: one load per row\n";
        }
    }
    os << "#pragma unroll\n    for (int u = 0; u < U; ++u) {\n        const tb_u64 r = row0 + (tb_u64)u * TY;\n        if (r < ROWS) {\n";
    emitRowOffsets(st, c, "r", "            ", "", os);
    for (size_t s = 0; s < st.inputs.size(); ++s) {
        if (st.inputs[s].kind != THOR_B200_INPUT_TENSOR) continue;
        if (cls[s] == Dense) os << "            tb_load_stream(p" << s << "[u], in" << s << " + ro_" << s << " + col);\n";
        else if (cls[s] == RowScalar) os << "            e" << s << "[u] = in" << s << "[ro_" << s << "];\n";
    }
    os << "        }\n    }\n";
    os << "#pragma unroll\n    for (int u = 0; u < U; ++u) {\n        const tb_u64 r = row0 + (tb_u64)u * TY;\n        if (r < ROWS) {\n";
    for (size_t o = 0; o < st.outputs.size(); ++o) os << "            tb_pack<VEC * " << dtypeSize(st.outputs[o].dtype) << "> r" << o << ";\n";
    os << "#pragma unroll\n            for (int j = 0; j < " << lanes << "; ++j) {\n                "
       << bodyCall(st,
                   [&](size_t s) -> std::string {
                       const std::string et = elemType(p, st.inputs[s].dtype);
                       switch (cls[s]) {
                           case Dense: return "reinterpret_cast<const " + et + "*>(&p" + std::to_string(s) + "[u])[j]";
                           case ColVec: return "reinterpret_cast<const " + et + "*>(&k" + std::to_string(s) + ")[j]";
                           case RowScalar: return p.v2 ? T2dup + "(e" + std::to_string(s) + "[u])" : "e" + std::to_string(s) + "[u]";
                           default: return p.v2 ? T2dup + "(e" + std::to_string(s) + ")" : "e" + std::to_string(s);
                       }
                   },
                   [&](size_t o) { return "reinterpret_cast<" + elemType(p, st.outputs[o].dtype) + "*>(&r" + std::to_string(o) + ")[j]"; })
       << "\n            }\n";
    for (size_t o = 0; o < st.outputs.size(); ++o) os << "            tb_store_stream(out" << o << " + r * COLS + col, r" << o << ");\n";
    os << "        }\n    }\n}\n";

    out->input_align.assign(st.inputs.size(), 1);
    for (size_t s = 0; s < st.inputs.size(); ++s)
        if (st.inputs[s].kind == THOR_B200_INPUT_TENSOR && (cls[s] == Dense || cls[s] == ColVec))
            out->input_align[s] = static_cast<int>(std::min<size_t>(16, dtypeSize(st.inputs[s].dtype) * VEC));
    out->output_align.assign(st.outputs.size(), 1);
    for (size_t o = 0; o < st.outputs.size(); ++o) out->output_align[o] = static_cast<int>(std::min<size_t>(16, dtypeSize(st.outputs[o].dtype) * VEC));
}

// ---- generic kernel ----------------------------------------------------------------------------
void emitGeneric(const Plan& p, Emitted* out, std::ostringstream& os) {
    const Stage& st = p.st;
    out->kind = Kind::Generic;
    out->vec = 1;
    out->unroll = 1;
    out->threads = 256;
    const std::string T2dup = p.v2_dtype == THOR_B200_BF16 ? "__bfloat162bfloat162" : "__half2half2";
    const std::string low = p.v2_dtype == THOR_B200_BF16 ? "__low2bfloat16" : "__low2half";
    Collapsed c;
    uint64_t numel = 0;
    if (st.broadcast) {
        c = collapse(st);
        numel = 1;
        for (uint64_t d : c.dims) numel *= d;
        out->numel = numel;
    }
    os << "extern \"C\" __global__ void " << launchBounds(st) << " fused_kernel(" << kernelParams(st, !st.broadcast) << ") {\n";
    os << "    tb_grid_wait();\n";
    if (st.broadcast) os << "    constexpr tb_u64 numel = " << numel << "ull;\n";
    os << "    const tb_u64 i = (tb_u64)blockIdx.x * 256 + threadIdx.x;\n    if (i >= numel) return;\n";
    emitScalarLoads(st, os);
    if (st.broadcast) {
        // full coordinate decode, innermost axis included
        Collapsed full = c;
        full.dims.push_back(1);  // emitRowOffsets treats all but the last axis as "outer"
        for (auto& s : full.strides) s.push_back(0);
        emitRowOffsets(st, full, "i", "    ", "", os);
    }
    for (size_t o = 0; o < st.outputs.size(); ++o) os << "    " << elemType(p, st.outputs[o].dtype) << " t" << o << ";\n";
    os << "    "
       << bodyCall(st,
                   [&](size_t s) {
                       const std::string at = "in" + std::to_string(s) + "[" + (st.broadcast ? "ro_" + std::to_string(s) : std::string("i")) + "]";
                       return p.v2 ? T2dup + "(" + at + ")" : at;
                   },
                   [&](size_t o) { return "t" + std::to_string(o); })
       << "\n";
    for (size_t o = 0; o < st.outputs.size(); ++o) os << "    out" << o << "[i] = " << (p.v2 ? low + "(t" + std::to_string(o) + ")" : "t" + std::to_string(o)) << ";\n";
    os << "}\n";
    out->input_align.assign(st.inputs.size(), 1);
    out->output_align.assign(st.outputs.size(), 1);
}

}  // namespace

std::string scalarNodeExpression(const std::vector<thor_b200_expr_node>& nodes, const std::vector<thor_b200_expr_input>& inputs, size_t k) {
    return scalarNodeExprImpl(nodes, inputs, k);
}
const char* cTypeName(int dtype) { return ctype(dtype); }
int nodeValueDType(const std::vector<thor_b200_expr_node>& nodes, size_t k) { return valueDTypeImpl(nodes, k); }
std::string convertExpression(const std::string& e, int src, int dst) { return cvt(e, src, dst); }
bool isFusedStageOp(uint16_t op) { return isKnownOp(op); }

const char* kindName(Kind k) {
    switch (k) {
        case Kind::FlatV2: return "flat_v2";
        case Kind::FlatScalar: return "flat_scalar";
        case Kind::TiledV2: return "bcast_tiled_v2";
        case Kind::TiledScalar: return "bcast_tiled_scalar";
        default: return "bcast_generic";
    }
}

std::string validate(const Stage& st) {
    char buf[256];
    if (st.nodes.empty()) return "stage has no nodes";
    if (st.outputs.empty()) return "stage has no outputs";
    if (st.broadcast) {
        if (st.rank == 0 || st.rank > THOR_B200_MAX_RANK) return "broadcast rank must be 1..8";
        for (uint64_t d : st.dims) if (d == 0) return "zero-sized dimension";
    }
    for (size_t s = 0; s < st.inputs.size(); ++s) {
        const auto& in = st.inputs[s];
        if (in.kind < 0 || in.kind > 2) { snprintf(buf, sizeof(buf), "input %zu: unknown kind %d", s, in.kind); return buf; }
        if (in.kind == THOR_B200_INPUT_RUNTIME_SCALAR_FP32 && in.dtype != THOR_B200_FP32) { snprintf(buf, sizeof(buf), "input %zu: runtime scalars are fp32", s); return buf; }
        if (!isStorable(in.dtype)) { snprintf(buf, sizeof(buf), "input %zu: unsupported dtype %d", s, in.dtype); return buf; }
    }
    for (size_t k = 0; k < st.nodes.size(); ++k) {
        const auto& nd = st.nodes[k];
        if (!isKnownOp(nd.op)) { snprintf(buf, sizeof(buf), "node %zu: op %u is not a fused-stage op", k, nd.op); return buf; }
        if (!isStorable(nd.output_dtype)) { snprintf(buf, sizeof(buf), "node %zu: unsupported output dtype %u", k, nd.output_dtype); return buf; }
        auto parentOk = [&](uint32_t idx) { return idx != THOR_B200_NO_NODE && idx < k; };
        if (isLeaf(nd.op)) {
            if (nd.op != THOR_B200_OP_SCALAR_FP) {
                if (nd.input_slot >= st.inputs.size()) { snprintf(buf, sizeof(buf), "node %zu: input slot %u out of range", k, nd.input_slot); return buf; }
                const int kind = st.inputs[nd.input_slot].kind;
                const int want = nd.op == THOR_B200_OP_INPUT ? THOR_B200_INPUT_TENSOR
                                 : nd.op == THOR_B200_OP_RUNTIME_SCALAR ? THOR_B200_INPUT_RUNTIME_SCALAR_FP32 : THOR_B200_INPUT_TENSOR_RUNTIME_SCALAR;
                if (kind != want) { snprintf(buf, sizeof(buf), "node %zu: input slot %u has kind %d, node needs %d", k, nd.input_slot, kind, want); return buf; }
            }
            continue;
        }
        if (!parentOk(nd.lhs)) { snprintf(buf, sizeof(buf), "node %zu: lhs must name an earlier node", k); return buf; }
        if ((isBinary(nd.op) || nd.op == THOR_B200_OP_WHERE) && !parentOk(nd.rhs)) { snprintf(buf, sizeof(buf), "node %zu: rhs must name an earlier node", k); return buf; }
        if (nd.op == THOR_B200_OP_WHERE && !parentOk(nd.aux)) { snprintf(buf, sizeof(buf), "node %zu: aux must name an earlier node", k); return buf; }
        const bool logical = isLogicalBinary(nd.op) || nd.op == THOR_B200_OP_LOGICAL_NOT || nd.op == THOR_B200_OP_CAST;
        if (!logical && !isArithCompute(nd.compute_dtype)) { snprintf(buf, sizeof(buf), "node %zu: compute dtype %u must be fp32, fp16 or bf16", k, nd.compute_dtype); return buf; }
    }
    for (size_t o = 0; o < st.outputs.size(); ++o) {
        if (st.outputs[o].node >= st.nodes.size()) { snprintf(buf, sizeof(buf), "output %zu: node out of range", o); return buf; }
        if (st.outputs[o].dtype != st.nodes[st.outputs[o].node].output_dtype) { snprintf(buf, sizeof(buf), "output %zu: dtype differs from its node's output dtype", o); return buf; }
    }
    return "";
}

size_t foldConstantsAndIdentities(std::vector<thor_b200_expr_node>& nodes, const std::vector<uint32_t>& keep) {
    const size_t n = nodes.size();
    std::vector<bool> is_const(n, false), kept(n, false);
    std::vector<double> value(n, 0.0);
    for (uint32_t k : keep)
        if (k < n) kept[k] = true;
    size_t rewritten = 0;
    for (size_t k = 0; k < n; ++k) {
        thor_b200_expr_node& nd = nodes[k];
        auto constant = [&](uint32_t i) { return i != THOR_B200_NO_NODE && i < k && is_const[i]; };
        if (nd.op == THOR_B200_OP_SCALAR_FP) {
            is_const[k] = true;
            value[k] = nd.scalar_fp;
            continue;
        }
        const bool arith4 = nd.op == THOR_B200_OP_ADD || nd.op == THOR_B200_OP_SUB || nd.op == THOR_B200_OP_MUL || nd.op == THOR_B200_OP_DIV;
        // the dtype the node's value is held in: what the literal or the aliased value is converted to
        const uint16_t held = isArithCompute(nd.compute_dtype) ? nd.compute_dtype : nd.output_dtype;
        if ((nd.op == THOR_B200_OP_NEG && constant(nd.lhs)) || (arith4 && constant(nd.lhs) && constant(nd.rhs))) {
            const double a = value[nd.lhs], b = arith4 ? value[nd.rhs] : 0.0;
            is_const[k] = true;
            value[k] = nd.op == THOR_B200_OP_NEG ? -a : nd.op == THOR_B200_OP_ADD ? a + b : nd.op == THOR_B200_OP_SUB ? a - b : nd.op == THOR_B200_OP_MUL ? a * b : a / b;
            nd.op = THOR_B200_OP_SCALAR_FP;
            nd.scalar_fp = value[k];
            nd.lhs = nd.rhs = nd.aux = THOR_B200_NO_NODE;
            if (!kept[k]) nd.output_dtype = held;
            ++rewritten;
            continue;
        }
        if (!arith4) continue;
        uint32_t source = THOR_B200_NO_NODE;
        const bool lhs_zero = constant(nd.lhs) && value[nd.lhs] == 0.0, rhs_zero = constant(nd.rhs) && value[nd.rhs] == 0.0;
        const bool lhs_one = constant(nd.lhs) && value[nd.lhs] == 1.0, rhs_one = constant(nd.rhs) && value[nd.rhs] == 1.0;
        if (nd.op == THOR_B200_OP_ADD) source = lhs_zero ? nd.rhs : (rhs_zero ? nd.lhs : THOR_B200_NO_NODE);
        else if (nd.op == THOR_B200_OP_SUB) source = rhs_zero ? nd.lhs : THOR_B200_NO_NODE;
        else if (nd.op == THOR_B200_OP_MUL) source = lhs_one ? nd.rhs : (rhs_one ? nd.lhs : THOR_B200_NO_NODE);
        else source = rhs_one ? nd.lhs : THOR_B200_NO_NODE;
        if (source == THOR_B200_NO_NODE) continue;
        nd.op = THOR_B200_OP_CAST;  // a conversion of the source's value and nothing else
        nd.lhs = source;
        nd.rhs = nd.aux = THOR_B200_NO_NODE;
        if (!kept[k]) nd.output_dtype = held;
        ++rewritten;
    }
    return rewritten;
}

std::string emit(const Stage& original, bool force_generic, Emitted* out) {
    std::string why = validate(original);
    if (!why.empty()) return why;
    Stage st = original;
    {
        std::vector<uint32_t> keep;
        for (const auto& o : st.outputs) keep.push_back(o.node);
        foldConstantsAndIdentities(st.nodes, keep);
    }
    Plan p(st);
    markLive(p);
    decideV2(p);
    analyseSigns(p);
    findExpTwins(p);
    std::ostringstream os;
    os << "// generated by thor_b200: fused stage, " << st.nodes.size() << " nodes, " << st.inputs.size() << " inputs, " << st.outputs.size() << " outputs\n";
    os << "#include \"tb_prelude.cuh\"\n\n";
    emitBody(p, os);
    if (force_generic) {
        emitGeneric(p, out, os);
    } else if (!st.broadcast) {
        emitFlat(p, out, os);
    } else {
        Collapsed c = collapse(st);
        if (c.dims.size() == 1) {
            // a single collapsed axis is a one-row matrix for the tiled kernel
            c.dims.insert(c.dims.begin(), 1);
            for (auto& s : c.strides) s.insert(s.begin(), 0);
        }
        const int VEC = chooseVec(p);
        if (tiledEligible(p, c, VEC)) emitTiled(p, c, out, os);
        else emitGeneric(p, out, os);
    }
    out->source = os.str();
    return "";
}

}  // namespace tb::expr
