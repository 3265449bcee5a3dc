// Row programs: one single-pass kernel for "elementwise -> row reduction -> elementwise" chains.
//
// Kernel shape (generated source, NVRTC): a team of TEAM threads owns one row of `cols` elements
// and keeps every FULL input of that row in registers as 16-byte packs (pack q of the row belongs
// to thread q % TEAM).  Rounds alternate between
//   (a) an element loop over the thread's packs that recomputes the needed part of the DAG from
//       the registers and accumulates the arguments of the row reductions of this round in fp32,
//   (b) one team-wide combine (shuffle tree + one shared-memory exchange) after which every
//       thread holds the reduction results, and the ROW-class nodes that depend on them.
// The last element loop evaluates the FULL outputs and stores them with 16-byte packs.  Each
// input row is therefore read from HBM exactly once and each output row written exactly once.
// With per-column operands (gamma, beta) or column reductions (dgamma, dbeta) the CTAs are
// persistent: they walk rows r, r + grid, ..., keep the per-column operands in registers and
// accumulate per-column fp32 partials, which a small fold kernel sums in CTA order.
#include <algorithm>
#include <cctype>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <sstream>

#include "common.cuh"
#include "expr_emit.h"
#include "jit.h"

namespace tb::rowprog {

using tb::expr::cTypeName;
using tb::expr::convertExpression;
using tb::expr::scalarNodeExpression;

namespace {

enum Shape { FULL = THOR_B200_SHAPE_FULL, ROW = THOR_B200_SHAPE_ROW, COL = THOR_B200_SHAPE_COL, SCALAR = THOR_B200_SHAPE_SCALAR };

// value reductions and arg reductions (the latter only along the columns of a row program, as [rows] uint32 outputs)
bool isReduce(uint16_t op) {
    return (op >= THOR_B200_OP_REDUCE_SUM && op <= THOR_B200_OP_REDUCE_ARGMAX) || (op >= THOR_B200_OP_REDUCE_AVG && op <= THOR_B200_OP_REDUCE_NORM2) || op == 0xF001;
}
bool isArgReduce(uint16_t op) { return op == THOR_B200_OP_REDUCE_ARGMIN || op == THOR_B200_OP_REDUCE_ARGMAX; }
// Internal op: index of the first column whose value equals the row's min / max, which another node of the program
// (rhs) already computes.  An arg reduction that sits beside the matching value reduction is rewritten to this: the
// search costs a compare and an integer min per element and runs one round after the value reduction.
constexpr uint16_t kOpFirstMatch = 0xF001;
bool isIndexReduce(uint16_t op) { return isArgReduce(op) || op == kOpFirstMatch; }
bool isLeaf(uint16_t op) { return op >= THOR_B200_OP_INPUT && op <= THOR_B200_OP_SCALAR_FP; }

struct Program {
    std::vector<thor_b200_expr_node> nodes;
    std::vector<thor_b200_expr_input> inputs;
    std::vector<int> input_shape;
    std::vector<thor_b200_expr_output> outputs;
    uint64_t rows = 0, cols = 0;
    bool fast_math = false;
    // analysis
    std::vector<int> shape;   // per node
    std::vector<bool> live;
    std::vector<int> depth;   // number of row reductions below the node
    std::vector<uint32_t> row_reduces, col_reduces, all_reduces;
    // geometry
    int vec = 4, team = 256, cta = 256, vpt = 1;
    bool persistent = false;
    bool prefetch = false;  // persistent programs: load row r + stride while row r is being computed
    int min_ctas = 0;       // second __launch_bounds__ argument, 0 = none
    bool pairs = false;     // element loops handle two neighbouring elements per step; fp32 + - * map onto the packed f32x2 instructions
    int ring_stages = 0;  // persistent programs: > 0 = rows arrive by bulk copies in a ring of this many shared-memory buffers
    size_t ring_stage_bytes = 0;
    bool producer = false;  // ring mode: a warpgroup of its own requests the copies; the teams only wait, compute and release buffers
    std::vector<size_t> ring_offset;         // ring mode: byte offset of each [rows, cols] input inside a buffer, by input slot
    std::vector<uint8_t> cache_state;  // per node: 1 = its [rows, cols] fp32 value is kept in registers once computed, 2 = it has been
    bool cache_wanted = true;
    bool reciprocal_division = false;  // x / (row value) in fp32 becomes x * (1 / row value): one rounding more than the reference's division
    int wait_limit_ms = 0;         // ring mode: time limit of a barrier wait (0 = the prelude's default of two seconds)
    int drop_fill_iteration = -1;  // ring mode, tests only: CTA 0 never requests the rows of this iteration
    bool pipeline_wanted = true;
    bool pipelined = false;                  // ring mode: round 1 of the next row shares the last round of the current row
    bool elements_from_next_buffer = false;  // emission state: element operands come from the next ring buffer, not from registers
    size_t smem_bytes = 0;
    uint32_t grid = 0;
    std::string source;
};

const char* combineExpr(uint16_t op) {
    switch (op) {
        case THOR_B200_OP_REDUCE_PROD: return "tb_mul";
        case THOR_B200_OP_REDUCE_MIN: return "tb_nanmin";
        case THOR_B200_OP_REDUCE_MAX: return "tb_nanmax";
        default: return "tb_add";
    }
}
const char* identityExpr(uint16_t op) {
    switch (op) {
        case THOR_B200_OP_REDUCE_PROD: return "1.0f";
        case THOR_B200_OP_REDUCE_MIN: return "__int_as_float(0x7f800000)";
        case THOR_B200_OP_REDUCE_MAX: return "__int_as_float(0xff800000)";
        default: return "0.0f";
    }
}
std::string transformExpr(uint16_t op, const std::string& f) {
    if (op == THOR_B200_OP_REDUCE_NORM1) return "fabsf(" + f + ")";
    if (op == THOR_B200_OP_REDUCE_NORM2) return "(" + f + " * " + f + ")";
    return f;
}

// Structurally equal nodes become one (reverse-mode differentiation repeats sub-expressions, and a repeated row sum
// would otherwise cost an accumulator, a shuffle tree and an exchange slot of its own).  Duplicates stay in the list, dead.
void mergeDuplicates(Program& p) {
    const size_t n = p.nodes.size();
    std::vector<uint32_t> canon(n);
    auto same = [](const thor_b200_expr_node& a, const thor_b200_expr_node& b) {
        return a.op == b.op && a.output_dtype == b.output_dtype && a.compute_dtype == b.compute_dtype && a.input_dtype == b.input_dtype && a.lhs == b.lhs &&
               a.rhs == b.rhs && a.aux == b.aux && a.input_slot == b.input_slot && std::memcmp(&a.scalar_fp, &b.scalar_fp, sizeof(double)) == 0;
    };
    for (uint32_t k = 0; k < n; ++k) {
        auto& nd = p.nodes[k];
        const bool reduce = isReduce(nd.op);
        for (uint32_t* par : {&nd.lhs, &nd.rhs, &nd.aux})
            if (*par != THOR_B200_NO_NODE && *par < k && !(reduce && par != &nd.lhs && !(nd.op == kOpFirstMatch && par == &nd.rhs))) *par = canon[*par];
        canon[k] = k;
        for (uint32_t m = 0; m < k; ++m)
            if (canon[m] == m && same(p.nodes[m], nd)) {
                canon[k] = m;
                break;
            }
    }
    for (auto& o : p.outputs) o.node = canon[o.node];
}

std::string analyse(Program& p) {
    const size_t n = p.nodes.size();
    p.shape.assign(n, SCALAR);
    p.depth.assign(n, 0);
    p.live.assign(n, false);
    for (const auto& o : p.outputs) {
        if (o.node >= n) return "output node out of range";
        p.live[o.node] = true;
    }
    for (size_t k = n; k-- > 0;) {
        if (!p.live[k]) continue;
        for (uint32_t par : {p.nodes[k].lhs, p.nodes[k].rhs, p.nodes[k].aux})
            if (par != THOR_B200_NO_NODE && !(isReduce(p.nodes[k].op) && par != p.nodes[k].lhs && !(p.nodes[k].op == kOpFirstMatch && par == p.nodes[k].rhs))) {
                if (par >= k) return "nodes are not topologically ordered";
                p.live[par] = true;
            }
    }
    std::vector<int> consumers(n, 0);
    for (size_t k = 0; k < n; ++k) {
        if (!p.live[k]) continue;
        const auto& nd = p.nodes[k];
        if (isLeaf(nd.op)) {
            if (nd.op == THOR_B200_OP_INPUT) {
                if (nd.input_slot >= p.inputs.size() || p.inputs[nd.input_slot].kind != THOR_B200_INPUT_TENSOR) return "bad input slot";
                p.shape[k] = p.input_shape[nd.input_slot];
            } else if (nd.op != THOR_B200_OP_SCALAR_FP) {
                if (nd.input_slot >= p.inputs.size()) return "bad input slot";
            }
            continue;
        }
        if (isReduce(nd.op)) {
            const int ps = p.shape[nd.lhs];
            consumers[nd.lhs]++;
            if (isIndexReduce(nd.op) && (nd.input_slot != 0 || nd.output_dtype != THOR_B200_UINT32)) return "arg reductions of a row program run along the columns and yield uint32";
            if (nd.input_slot == 0) {
                if (ps != FULL) return "a row reduction needs a [rows, cols] argument";
                p.shape[k] = ROW;
                p.depth[k] = p.depth[nd.lhs] + 1;
                if (nd.op == kOpFirstMatch) {
                    consumers[nd.rhs]++;
                    p.depth[k] = std::max(p.depth[nd.lhs], p.depth[nd.rhs]) + 1;
                }
                p.row_reduces.push_back(static_cast<uint32_t>(k));
            } else if (nd.input_slot == 1) {
                if (ps != FULL) return "a column reduction needs a [rows, cols] argument";
                if (nd.op != THOR_B200_OP_REDUCE_SUM && nd.op != THOR_B200_OP_REDUCE_AVG) return "column reductions support sum and mean";
                p.shape[k] = COL;
                p.depth[k] = p.depth[nd.lhs];
                p.col_reduces.push_back(static_cast<uint32_t>(k));
            } else if (nd.input_slot == 2) {
                if (ps != FULL) return "a full reduction needs a full-shaped argument";
                p.shape[k] = SCALAR;
                p.depth[k] = p.depth[nd.lhs];
                p.all_reduces.push_back(static_cast<uint32_t>(k));
            } else {
                return "reduction axis selector must be 0 (columns), 1 (rows) or 2 (all elements)";
            }
            continue;
        }
        if (!tb::expr::isFusedStageOp(nd.op)) return "op is not supported in a row program";
        int sh = SCALAR, d = 0;
        for (uint32_t par : {nd.lhs, nd.rhs, nd.aux}) {
            if (par == THOR_B200_NO_NODE) continue;
            consumers[par]++;
            const int ps = p.shape[par];
            if (ps == SCALAR) {
            } else if (sh == SCALAR) sh = ps;
            else if (sh != ps) sh = FULL;
            d = std::max(d, p.depth[par]);
        }
        p.shape[k] = sh;
        p.depth[k] = d;
    }
    for (uint32_t k : p.col_reduces)
        if (consumers[k] != 0) return "a column reduction may only be an output";
    for (uint32_t k : p.row_reduces)
        if (isIndexReduce(p.nodes[k].op) && consumers[k] != 0) return "an arg reduction may only be an output";
    if (!p.all_reduces.empty()) {
        // flat reduce program: every output is a reduction over all elements of an elementwise expression
        if (!p.row_reduces.empty() || !p.col_reduces.empty()) return "full reductions cannot be mixed with row or column reductions";
        for (uint32_t k : p.all_reduces)
            if (consumers[k] != 0) return "a full reduction may only be an output";
        for (const auto& o : p.outputs) {
            if (std::find(p.all_reduces.begin(), p.all_reduces.end(), o.node) == p.all_reduces.end()) return "every output of a flat reduce program must be a full reduction";
            if (o.dtype != p.nodes[o.node].output_dtype) return "output dtype differs from its node's output dtype";
        }
        for (size_t s = 0; s < p.inputs.size(); ++s)
            if (p.inputs[s].kind == THOR_B200_INPUT_TENSOR && p.input_shape[s] != FULL && p.input_shape[s] != SCALAR) return "flat reduce programs take full-shaped or one-element tensors";
        return "";
    }
    bool any_full = false;
    for (const auto& o : p.outputs) {
        const int sh = p.shape[o.node];
        if (sh == SCALAR) return "scalar outputs are not produced by a row program";
        if (sh == COL && !isReduce(p.nodes[o.node].op)) return "per-column outputs must be column reductions";
        if (o.dtype != p.nodes[o.node].output_dtype) return "output dtype differs from its node's output dtype";
        any_full = any_full || sh == FULL || sh == ROW || sh == COL;
    }
    if (p.row_reduces.empty() && p.col_reduces.empty()) return "no reduction: an ordinary fused stage is the right kernel";
    return "";
}


// ---- linear hoisting of row sums -----------------------------------------------------------------
// sum_j (c * f_j) = c * sum_j f_j when c is constant along the row.  Reverse-mode graphs are full of
// such sums (every un-broadcast of a gradient that was scaled by a per-row statistic), and each
// one that depends on an earlier row statistic costs a whole extra pass over the row in registers.
// The rewrite expresses a SUM / AVG row reduction of a linear combination as the same combination of
// reductions of its row-varying factors, which usually have a smaller depth.  Only fp32 nodes are
// rewritten (in 16-bit graphs the per-element rounding of the products is part of the result), and
// only when the reduction's depth drops.  The value changes by fp32 re-association only.
struct LinearTerm {
    std::vector<std::pair<uint32_t, bool>> coeffs;  // row-constant factors (node, is divisor)
    uint32_t atom;                                  // row-varying factor; THOR_B200_NO_NODE: the constant 1
    bool negative;
};

bool isF32Node(const thor_b200_expr_node& n) { return n.output_dtype == THOR_B200_FP32 && n.compute_dtype == THOR_B200_FP32; }

void decomposeLinear(const Program& p, uint32_t k, std::vector<std::pair<uint32_t, bool>> coeffs, bool negative, std::vector<LinearTerm>& out) {
    const auto& nd = p.nodes[k];
    auto rowConst = [&](uint32_t i) { return p.shape[i] == ROW || p.shape[i] == SCALAR; };
    if (p.shape[k] == FULL && isF32Node(nd)) {
        if (nd.op == THOR_B200_OP_NEG) return decomposeLinear(p, nd.lhs, coeffs, !negative, out);
        if (nd.op == THOR_B200_OP_ADD || nd.op == THOR_B200_OP_SUB) {
            // a row-constant operand c contributes c once per column: a term whose row-varying factor is 1
            const bool rhs_negative = nd.op == THOR_B200_OP_SUB ? !negative : negative;
            for (int side = 0; side < 2; ++side) {
                const uint32_t operand = side == 0 ? nd.lhs : nd.rhs;
                const bool neg = side == 0 ? negative : rhs_negative;
                if (rowConst(operand)) {
                    auto with = coeffs;
                    with.push_back({operand, false});
                    out.push_back({with, THOR_B200_NO_NODE, neg});
                } else {
                    decomposeLinear(p, operand, coeffs, neg, out);
                }
            }
            return;
        }
        if (nd.op == THOR_B200_OP_MUL && (rowConst(nd.lhs) != rowConst(nd.rhs))) {
            const uint32_t c = rowConst(nd.lhs) ? nd.lhs : nd.rhs, f = rowConst(nd.lhs) ? nd.rhs : nd.lhs;
            coeffs.push_back({c, false});
            return decomposeLinear(p, f, coeffs, negative, out);
        }
        if (nd.op == THOR_B200_OP_DIV && rowConst(nd.rhs) && !rowConst(nd.lhs)) {
            coeffs.push_back({nd.rhs, true});
            return decomposeLinear(p, nd.lhs, coeffs, negative, out);
        }
    }
    out.push_back({coeffs, k, negative});
}

// Returns true when the program was rewritten (the caller re-runs analyse()).
bool hoistLinearRowSums(Program& p) {
    bool changed = false;
    std::vector<thor_b200_expr_node> out_nodes;
    std::vector<uint32_t> remap(p.nodes.size(), THOR_B200_NO_NODE);
    auto push = [&](thor_b200_expr_node n) {
        out_nodes.push_back(n);
        return static_cast<uint32_t>(out_nodes.size() - 1);
    };
    auto f32 = [&](uint16_t op, uint32_t lhs, uint32_t rhs) {
        thor_b200_expr_node n{};
        n.op = op;
        n.output_dtype = n.compute_dtype = THOR_B200_FP32;
        n.lhs = lhs;
        n.rhs = rhs;
        n.aux = THOR_B200_NO_NODE;
        n.input_slot = THOR_B200_NO_NODE;
        return n;
    };
    for (uint32_t k = 0; k < p.nodes.size(); ++k) {
        thor_b200_expr_node nd = p.nodes[k];
        const bool candidate = p.live[k] && isReduce(nd.op) && nd.input_slot == 0 && (nd.op == THOR_B200_OP_REDUCE_SUM || nd.op == THOR_B200_OP_REDUCE_AVG) &&
                               nd.output_dtype == THOR_B200_FP32;
        std::vector<LinearTerm> terms;
        if (candidate) decomposeLinear(p, nd.lhs, {}, false, terms);
        int new_depth = 0;
        bool any_coeff = false;
        for (const auto& t : terms) {
            if (t.atom != THOR_B200_NO_NODE) new_depth = std::max(new_depth, p.depth[t.atom] + 1);
            for (const auto& c : t.coeffs) {
                new_depth = std::max(new_depth, p.depth[c.first]);
                any_coeff = true;
            }
        }
        if (candidate && any_coeff && new_depth < p.depth[k]) {
            // value = sum over terms of (+-) reduce(atom) * c1 * c2 / d1 ...
            uint32_t total = THOR_B200_NO_NODE;
            std::vector<std::pair<uint32_t, uint32_t>> reduced;  // atom (new index) -> reduce node
            auto scalar = [&](double value) {
                thor_b200_expr_node sn = f32(THOR_B200_OP_SCALAR_FP, THOR_B200_NO_NODE, THOR_B200_NO_NODE);
                sn.scalar_fp = value;
                return push(sn);
            };
            const double n_cols = static_cast<double>(p.cols);
            for (const auto& t : terms) {
                uint32_t r = THOR_B200_NO_NODE;
                if (t.atom == THOR_B200_NO_NODE) {
                    // sum of the constant 1 over the row: cols for a sum, 1 for a mean
                    r = scalar(nd.op == THOR_B200_OP_REDUCE_SUM ? n_cols : 1.0);
                } else {
                    const uint32_t atom = remap[t.atom];
                    for (const auto& pr : reduced)
                        if (pr.first == atom) r = pr.second;
                    if (r == THOR_B200_NO_NODE) {
                        // a sum or a mean of the same values that the program already computes serves, scaled by the row length
                        for (uint32_t e = 0; e < out_nodes.size() && r == THOR_B200_NO_NODE; ++e) {
                            const auto& en = out_nodes[e];
                            if (!isReduce(en.op) || en.input_slot != 0 || en.lhs != atom || en.output_dtype != THOR_B200_FP32) continue;
                            if (en.op == nd.op) r = e;
                            else if (en.op == THOR_B200_OP_REDUCE_AVG && nd.op == THOR_B200_OP_REDUCE_SUM) r = push(f32(THOR_B200_OP_MUL, e, scalar(n_cols)));
                            else if (en.op == THOR_B200_OP_REDUCE_SUM && nd.op == THOR_B200_OP_REDUCE_AVG) r = push(f32(THOR_B200_OP_DIV, e, scalar(n_cols)));
                        }
                    }
                    if (r == THOR_B200_NO_NODE) {
                        thor_b200_expr_node rn = f32(nd.op, atom, THOR_B200_NO_NODE);
                        rn.input_slot = 0;
                        r = push(rn);
                    }
                    reduced.push_back({atom, r});
                }
                uint32_t v = r;
                for (const auto& c : t.coeffs) v = push(f32(c.second ? THOR_B200_OP_DIV : THOR_B200_OP_MUL, v, remap[c.first]));
                if (total == THOR_B200_NO_NODE) total = t.negative ? push(f32(THOR_B200_OP_NEG, v, THOR_B200_NO_NODE)) : v;
                else total = push(f32(t.negative ? THOR_B200_OP_SUB : THOR_B200_OP_ADD, total, v));
            }
            remap[k] = total;
            changed = true;
            continue;
        }
        for (uint32_t* par : {&nd.lhs, &nd.rhs, &nd.aux})
            if (*par != THOR_B200_NO_NODE && !(isReduce(nd.op) && par != &nd.lhs && !(nd.op == kOpFirstMatch && par == &nd.rhs)))
                *par = remap[*par] != THOR_B200_NO_NODE ? remap[*par] : *par;
        remap[k] = push(nd);
    }
    if (!changed) return false;
    for (auto& o : p.outputs) o.node = remap[o.node];
    p.nodes = out_nodes;
    p.row_reduces.clear();
    p.col_reduces.clear();
    p.all_reduces.clear();
    return true;
}

// dtype a node's value is held in inside the kernel, and the fp32 view a reduction takes of its argument:
// reductions consume materialised values, i.e. rounded to the argument node's output dtype first
int vdt(const Program& p, uint32_t k) { return tb::expr::nodeValueDType(p.nodes, k); }
std::string reduceArgF32(const Program& p, uint32_t a, const std::string& name) {
    return convertExpression(convertExpression(name, vdt(p, a), p.nodes[a].output_dtype), p.nodes[a].output_dtype, THOR_B200_FP32);
}

// Statements "const T vK = <expr>;" for the given nodes (already in topological order).
void emitStatements(const Program& p, const std::vector<uint32_t>& ids, const std::string& indent, std::ostringstream& os) {
    for (uint32_t k : ids) os << indent << "const " << cTypeName(vdt(p, k)) << " v" << k << " = " << scalarNodeExpression(p.nodes, p.inputs, k) << ";\n";
}

// ---- pair mode ---------------------------------------------------------------------------------
// Element loops of a pair-mode program advance two elements per step.  Every element-level node k
// is a two-lane value pK (float2, __half2, __nv_bfloat162 or tb_pr<T>); row-scope values keep their
// scalar names vK.  fp32 additions, subtractions and multiplications become one packed f32x2
// instruction per pair (a multiply feeding an add becomes a packed fma), 16-bit float conversions
// use the two-lane conversion instructions, and every other op is evaluated lane by lane from the
// scalar expression, so the value of each lane is the one the scalar body would compute up to the
// placement of fused multiply-adds.
std::string pairType(int d) {
    if (d == THOR_B200_FP32) return "float2";
    if (d == THOR_B200_FP16) return "__half2";
    if (d == THOR_B200_BF16) return "__nv_bfloat162";
    return std::string("tb_pr<") + cTypeName(d) + ">";
}
std::string makePair(int d, const std::string& x, const std::string& y) {
    if (d == THOR_B200_FP32) return "make_float2(" + x + ", " + y + ")";
    if (d == THOR_B200_FP16) return "__halves2half2(" + x + ", " + y + ")";
    if (d == THOR_B200_BF16) return "__halves2bfloat162(" + x + ", " + y + ")";
    return pairType(d) + "{" + x + ", " + y + "}";
}
// `e` must be a plain name: it may be evaluated once per lane.
std::string convertPair(const std::string& e, int src, int dst) {
    if (src == dst) return e;
    if (dst == THOR_B200_FP32 && src == THOR_B200_BF16) return "__bfloat1622float2(" + e + ")";
    if (dst == THOR_B200_FP32 && src == THOR_B200_FP16) return "__half22float2(" + e + ")";
    if (src == THOR_B200_FP32 && dst == THOR_B200_BF16) return "__float22bfloat162_rn(" + e + ")";
    if (src == THOR_B200_FP32 && dst == THOR_B200_FP16) return "__float22half2_rn(" + e + ")";
    return makePair(dst, convertExpression(e + ".x", src, dst), convertExpression(e + ".y", src, dst));
}
bool elementLevel(const Program& p, uint32_t k) { return p.shape[k] == FULL || p.shape[k] == COL; }

// float2 view of node `idx` for a packed fp32 instruction.
std::string pairAsFloat2(const Program& p, uint32_t idx) {
    const int d = vdt(p, idx);
    if (elementLevel(p, idx)) return convertPair("p" + std::to_string(idx), d, THOR_B200_FP32);
    return "tb_both(" + convertExpression("v" + std::to_string(idx), d, THOR_B200_FP32) + ")";
}
bool packedMul(const Program& p, uint32_t idx) {
    if (idx == THOR_B200_NO_NODE || !elementLevel(p, idx)) return false;
    const auto& m = p.nodes[idx];
    return m.op == THOR_B200_OP_MUL && m.compute_dtype == THOR_B200_FP32;
}
// fp32 value of node `idx` plus `addend` (a float2 expression), with the multiply folded into an fma when `idx` is one.
std::string pairPlus(const Program& p, uint32_t idx, const std::string& addend) {
    if (packedMul(p, idx)) return "__ffma2_rn(" + pairAsFloat2(p, p.nodes[idx].lhs) + ", " + pairAsFloat2(p, p.nodes[idx].rhs) + ", " + addend + ")";
    return "__fadd2_rn(" + pairAsFloat2(p, idx) + ", " + addend + ")";
}

// float2 expression of reduction argument `a` as the reduction sees it: rounded to the node's output dtype when that
// differs from the dtype the value is held in (emits the rounding as a statement of its own in that case).
std::string pairReduceArg(const Program& p, uint32_t a, const std::string& indent, std::ostringstream& os) {
    const int V = vdt(p, a), O = p.nodes[a].output_dtype;
    if (V == O || !elementLevel(p, a)) {
        if (!elementLevel(p, a)) return "tb_both(" + reduceArgF32(p, a, "v" + std::to_string(a)) + ")";
        return pairAsFloat2(p, a);
    }
    const std::string m = "m" + std::to_string(a);
    os << indent << "const " << pairType(O) << " " << m << " = " << convertPair("p" + std::to_string(a), V, O) << ";\n";
    return convertPair(m, O, THOR_B200_FP32);
}
bool storedAsHeld(const Program& p, uint32_t a) { return vdt(p, a) == static_cast<int>(p.nodes[a].output_dtype); }

void emitPairStatements(const Program& p, const std::vector<uint32_t>& ids, const std::string& indent, std::ostringstream& os) {
    for (uint32_t k : ids) {
        const auto& nd = p.nodes[k];
        const int O = vdt(p, k);
        const std::string name = "p" + std::to_string(k);
        std::string packed;  // float2 expression when the node has a packed form
        const uint8_t cached = p.cache_state.empty() ? 0 : p.cache_state[k];
        if (cached == 2) {
            os << indent << "const float2 " << name << " = h" << k << "[k][j >> 1];\n";
            continue;
        }
        if (nd.op == THOR_B200_OP_INPUT) {
            os << indent << "const " << pairType(O) << " " << name << " = " << convertPair("px" + std::to_string(nd.input_slot), p.inputs[nd.input_slot].dtype, O) << ";\n";
            continue;
        }
        if (nd.op == THOR_B200_OP_CAST && elementLevel(p, nd.lhs)) {
            os << indent << "const " << pairType(O) << " " << name << " = " << convertPair("p" + std::to_string(nd.lhs), vdt(p, nd.lhs), O) << ";\n";
            continue;
        }
        if (nd.compute_dtype == THOR_B200_FP32) {
            if (nd.op == THOR_B200_OP_ADD) {
                if (packedMul(p, nd.lhs)) packed = pairPlus(p, nd.lhs, pairAsFloat2(p, nd.rhs));
                else packed = pairPlus(p, nd.rhs, pairAsFloat2(p, nd.lhs));
            } else if (nd.op == THOR_B200_OP_SUB && !elementLevel(p, nd.rhs)) {
                // the negated row value is loop invariant
                packed = "__fadd2_rn(" + pairAsFloat2(p, nd.lhs) + ", tb_both(-" + convertExpression("v" + std::to_string(nd.rhs), vdt(p, nd.rhs), THOR_B200_FP32) + "))";
            } else if (nd.op == THOR_B200_OP_SUB) {
                packed = "__ffma2_rn(" + pairAsFloat2(p, nd.rhs) + ", tb_both(-1.0f), " + pairAsFloat2(p, nd.lhs) + ")";  // a - b, exact
            } else if (nd.op == THOR_B200_OP_MUL) {
                packed = "__fmul2_rn(" + pairAsFloat2(p, nd.lhs) + ", " + pairAsFloat2(p, nd.rhs) + ")";
            } else if (nd.op == THOR_B200_OP_DIV && p.reciprocal_division && elementLevel(p, nd.lhs) && !elementLevel(p, nd.rhs)) {
                // the reciprocal of the row value is loop invariant
                packed = "__fmul2_rn(" + pairAsFloat2(p, nd.lhs) + ", tb_both(__frcp_rn(" + convertExpression("v" + std::to_string(nd.rhs), vdt(p, nd.rhs), THOR_B200_FP32) + ")))";
            }
        }
        if (!packed.empty()) {
            if (O == THOR_B200_FP32) {
                os << indent << "const float2 " << name << " = " << packed << ";\n";
                if (cached == 1) os << indent << "h" << k << "[k][j >> 1] = " << name << ";\n";
            } else {
                os << indent << "const float2 t" << k << " = " << packed << ";\n";
                os << indent << "const " << pairType(O) << " " << name << " = " << convertPair("t" + std::to_string(k), THOR_B200_FP32, O) << ";\n";
            }
            continue;
        }
        // lane by lane from the scalar expression
        const std::string expr = scalarNodeExpression(p.nodes, p.inputs, k);
        os << indent << pairType(O) << " " << name << ";\n";
        for (const char* lane : {".x", ".y"}) {
            os << indent << "{ ";
            std::vector<uint32_t> seen;
            for (uint32_t par : {nd.lhs, nd.rhs, nd.aux}) {
                if (par == THOR_B200_NO_NODE || !elementLevel(p, par) || std::find(seen.begin(), seen.end(), par) != seen.end()) continue;
                seen.push_back(par);
                os << "const " << cTypeName(vdt(p, par)) << " v" << par << " = p" << par << lane << "; ";
            }
            os << name << lane << " = " << expr << "; }\n";
        }
        if (cached == 1) os << indent << "h" << k << "[k][j >> 1] = " << name << ";\n";
    }
}

// FULL / COL-class ancestors of `targets` (inclusive) that an element loop has to evaluate.
std::vector<uint32_t> elementClosure(const Program& p, const std::vector<uint32_t>& targets) {
    std::vector<bool> need(p.nodes.size(), false);
    std::vector<uint32_t> stack(targets.begin(), targets.end());
    while (!stack.empty()) {
        const uint32_t k = stack.back();
        stack.pop_back();
        if (need[k]) continue;
        const int sh = p.shape[k];
        if (sh == ROW || sh == SCALAR) continue;  // row-scope values: already computed, referenced by name
        need[k] = true;
        if (isLeaf(p.nodes[k].op) || isReduce(p.nodes[k].op)) continue;
        if (!p.cache_state.empty() && p.cache_state[k] == 2) continue;  // kept in registers by an earlier element loop
        for (uint32_t par : {p.nodes[k].lhs, p.nodes[k].rhs, p.nodes[k].aux})
            if (par != THOR_B200_NO_NODE) stack.push_back(par);
    }
    std::vector<uint32_t> out;
    for (uint32_t k = 0; k < p.nodes.size(); ++k)
        if (need[k]) out.push_back(k);
    return out;
}

std::string elemTypeOfInput(const Program& p, size_t slot) { return cTypeName(p.inputs[slot].dtype); }

// Declarations of the element values x<slot> that `ids` read, for lane j of pack k.
void emitElementInputs(const Program& p, const std::vector<uint32_t>& ids, const std::string& indent, std::ostringstream& os) {
    const bool staged = p.elements_from_next_buffer;
    std::vector<bool> done(p.inputs.size(), false);
    for (uint32_t k : ids) {
        const auto& nd = p.nodes[k];
        if (nd.op != THOR_B200_OP_INPUT || done[nd.input_slot]) continue;
        done[nd.input_slot] = true;
        const size_t s = nd.input_slot;
        const std::string T = elemTypeOfInput(p, s);
        if (p.pairs) {
            const std::string PT = pairType(p.inputs[s].dtype);
            const std::string src = p.input_shape[s] == FULL ? (staged ? "g" + std::to_string(s) : "f" + std::to_string(s) + "[k]") : "c" + std::to_string(s) + "[k]";
            os << indent << "const " << PT << " px" << s << " = reinterpret_cast<const " << PT << "*>(&" << src << ")[j >> 1];\n";
            continue;
        }
        if (p.input_shape[s] == FULL)
            os << indent << "const " << T << " x" << s << " = reinterpret_cast<const " << T << "*>(&" << (staged ? "g" + std::to_string(s) : "f" + std::to_string(s) + "[k]")
               << ")[j];\n";
        else os << indent << "const " << T << " x" << s << " = reinterpret_cast<const " << T << "*>(&c" << s << "[k])[j];\n";
    }
}

// Per-pack loads of COL inputs for non-persistent programs (L1/L2 resident, re-read each round).
void emitColumnPackLoads(const Program& p, const std::vector<uint32_t>& ids, const std::string& indent, std::ostringstream& os) {
    if (p.elements_from_next_buffer) {
        // this thread's pack k of the team's next row, from the ring buffer the bulk copy filled
        std::vector<bool> done(p.inputs.size(), false);
        for (uint32_t k : ids) {
            const auto& nd = p.nodes[k];
            if (nd.op != THOR_B200_OP_INPUT || p.input_shape[nd.input_slot] != FULL || done[nd.input_slot]) continue;
            done[nd.input_slot] = true;
            const size_t es = dtypeSize(p.inputs[nd.input_slot].dtype);
            os << indent << "const tb_pack<VEC * " << es << "> g" << nd.input_slot << " = *reinterpret_cast<const tb_pack<VEC * " << es << ">*>(tb_ring + nstage * STAGE_BYTES + "
               << p.ring_offset[nd.input_slot] << "u + ((tb_u32)team_id * (tb_u32)COLS + q * VEC) * " << es << "u);\n";
        }
        return;
    }
    if (p.persistent) return;
    std::vector<bool> done(p.inputs.size(), false);
    for (uint32_t k : ids) {
        const auto& nd = p.nodes[k];
        if (nd.op != THOR_B200_OP_INPUT || p.input_shape[nd.input_slot] != COL || done[nd.input_slot]) continue;
        done[nd.input_slot] = true;
        os << indent << "tb_load_keep(c" << nd.input_slot << "[k], in" << nd.input_slot << " + (tb_u64)q * VEC);\n";
    }
}

// Round 1 of a row can ride on the previous row's last round when there are at least two rounds, its operands are
// [rows, cols] / per-column / scalar values only, and it holds no index reductions.
bool canPipeline(const Program& p) {
    int max_depth = 0;
    bool any_first = false;
    for (uint32_t k : p.row_reduces) {
        max_depth = std::max(max_depth, p.depth[k]);
        if (p.depth[k] == 1) {
            any_first = true;
            if (isIndexReduce(p.nodes[k].op)) return false;
        }
    }
    for (size_t s = 0; s < p.inputs.size(); ++s)
        if (p.inputs[s].kind == THOR_B200_INPUT_TENSOR && p.input_shape[s] == ROW) return false;
    return any_first && max_depth >= 2;
}

std::string emit(Program& p) {
    std::ostringstream os;
    const int VEC = p.vec, TEAM = p.team, CTA = p.cta, VPT = p.vpt;
    const int teams_per_cta = CTA / TEAM;
    const uint64_t packs_per_row = p.cols / VEC;
    int max_depth = 0;
    for (uint32_t k : p.row_reduces) max_depth = std::max(max_depth, p.depth[k]);
    p.pipelined = p.persistent && p.ring_stages > 0 && p.pipeline_wanted && canPipeline(p);
    // Element loops recompute what they need from the row's registers.  A transcendental (or a division) that more than
    // one loop needs -- exp(x - max) of a softmax, needed by the sum and by the output -- is kept in registers instead
    // when the program is not already short of them: non-persistent programs, at most 32 floats per thread.
    p.cache_state.assign(p.nodes.size(), 0);
    if (!p.persistent && p.pairs && p.cache_wanted) {
        auto expensive = [](uint16_t op) {
            return op == THOR_B200_OP_DIV || op == THOR_B200_OP_POW || (op >= THOR_B200_OP_SIN && op <= THOR_B200_OP_NORMCDF);
        };
        std::vector<int> uses(p.nodes.size(), 0);
        auto count = [&](const std::vector<uint32_t>& targets) {
            if (targets.empty()) return;
            for (uint32_t k : elementClosure(p, targets)) ++uses[k];
        };
        for (int d = 1; d <= max_depth; ++d) {
            std::vector<uint32_t> args;
            for (uint32_t k : p.row_reduces)
                if (p.depth[k] == d) args.push_back(p.nodes[k].lhs);
            count(args);
        }
        std::vector<uint32_t> finals;
        for (const auto& o : p.outputs)
            if (p.shape[o.node] == FULL) finals.push_back(o.node);
        count(finals);
        int budget = 32;
        for (uint32_t k = static_cast<uint32_t>(p.nodes.size()); k-- > 0;) {
            if (uses[k] < 2 || p.shape[k] != FULL || !expensive(p.nodes[k].op) || vdt(p, k) != THOR_B200_FP32) continue;
            if (budget < VPT * VEC) break;
            budget -= VPT * VEC;
            p.cache_state[k] = 1;
        }
    }

    os << "// generated by thor_b200: row program, " << p.nodes.size() << " nodes, rows = " << p.rows << ", cols = " << p.cols << ", team = " << TEAM
       << " threads, " << VPT << " packs of " << VEC << " per thread" << (p.persistent ? ", persistent" : "") << "\n";
    if (p.ring_stages > 0) {
        os << "#define TB_BULK_RING 1\n";
        if (p.wait_limit_ms > 0) os << "#define TB_WAIT_LIMIT_NS " << static_cast<unsigned long long>(p.wait_limit_ms) * 1000000ull << "ull\n";
    }
    os << "#include \"tb_prelude.cuh\"\n#include \"tb_rowprog.cuh\"\n\n";
    // kernel signature
    os << "extern \"C\" __global__ void __launch_bounds__(" << (p.ring_stages > 0 && p.producer ? CTA + 128 : CTA)
       << (p.ring_stages > 0 && p.producer ? std::string(", 1") : (p.min_ctas > 0 ? ", " + std::to_string(p.min_ctas) : std::string()))
       << ") row_kernel(";
    bool first = true;
    for (size_t s = 0; s < p.inputs.size(); ++s) {
        os << (first ? "" : ", ");
        first = false;
        if (p.inputs[s].kind == THOR_B200_INPUT_RUNTIME_SCALAR_FP32) os << "const float s" << s;
        else os << "const " << cTypeName(p.inputs[s].dtype) << "* __restrict__ in" << s;
    }
    for (size_t o = 0; o < p.outputs.size(); ++o) {
        os << (first ? "" : ", ");
        first = false;
        os << cTypeName(p.outputs[o].dtype) << "* __restrict__ out" << o;
    }
    os << (first ? "" : ", ") << "float* __restrict__ ws) {\n    tb_grid_wait();\n";
    os << "    constexpr int VEC = " << VEC << ", TEAM = " << TEAM << ", VPT = " << VPT << ", TEAMS = " << teams_per_cta << ";\n";
    os << "    constexpr tb_u64 ROWS = " << p.rows << "ull, COLS = " << p.cols << "ull;\n";
    os << "    constexpr tb_u32 PPR = " << packs_per_row << "u;\n";
    // persistent programs alternate between two sets of exchange slots from row to row, so that a row's
    // slots are not rewritten before every thread has passed a barrier of the row in between
    os << "    __shared__ float red_smem_all[" << (p.persistent ? 2 : 1) << "][" << std::max<size_t>(1, p.row_reduces.size()) << "][TEAMS][TEAM > 32 ? TEAM / 32 : 1];\n";
    bool any_arg = false;
    for (uint32_t k : p.row_reduces) any_arg = any_arg || isIndexReduce(p.nodes[k].op);
    if (any_arg)
        os << "    __shared__ tb_u64 red_key_all[" << (p.persistent ? 2 : 1) << "][" << p.row_reduces.size() << "][TEAMS][TEAM > 32 ? TEAM / 32 : 1];\n";
    if (p.persistent) os << "    int red_set = 0;\n";
    else {
        os << "    float (*red_smem)[TEAMS][TEAM > 32 ? TEAM / 32 : 1] = red_smem_all[0];\n";
        if (any_arg) os << "    tb_u64 (*red_key)[TEAMS][TEAM > 32 ? TEAM / 32 : 1] = red_key_all[0];\n";
    }
    os << "    const int t = threadIdx.x % TEAM, team_id = threadIdx.x / TEAM;\n";
    for (size_t s = 0; s < p.inputs.size(); ++s)
        if (p.inputs[s].kind == THOR_B200_INPUT_TENSOR_RUNTIME_SCALAR || (p.inputs[s].kind == THOR_B200_INPUT_TENSOR && p.input_shape[s] == SCALAR))
            os << "    const " << cTypeName(p.inputs[s].dtype) << (p.inputs[s].kind == THOR_B200_INPUT_TENSOR ? " x" : " s") << s << " = in" << s << "[0];\n";
    // per-column operands and column accumulators live in registers for the whole kernel; in producer mode they are
    // declared after the copy warpgroup has left, so that they belong to the teams' enlarged register allowance
    auto emitColumnState = [&]() {
        // per-column operands: registers for the whole kernel when persistent
        for (size_t s = 0; s < p.inputs.size(); ++s)
            if (p.inputs[s].kind == THOR_B200_INPUT_TENSOR && p.input_shape[s] == COL) {
                os << "    tb_pack<VEC * " << dtypeSize(p.inputs[s].dtype) << "> c" << s << "[VPT];\n";
                if (p.persistent) {
                    os << "#pragma unroll\n    for (int k = 0; k < VPT; ++k) {\n        const tb_u32 q = t + k * TEAM;\n        if (q < PPR) tb_load_keep(c" << s
                       << "[k], in" << s << " + (tb_u64)q * VEC);\n    }\n";
                }
            }
        // column-reduction accumulators
        for (uint32_t k : p.col_reduces) {
            if (p.pairs)
                os << "    float2 acc" << k << "[VPT][VEC / 2];\n#pragma unroll\n    for (int k = 0; k < VPT; ++k)\n#pragma unroll\n        for (int j = 0; j < VEC / 2; ++j) acc" << k
                   << "[k][j] = make_float2(0.0f, 0.0f);\n";
            else
                os << "    float acc" << k << "[VPT][VEC];\n#pragma unroll\n    for (int k = 0; k < VPT; ++k)\n#pragma unroll\n        for (int j = 0; j < VEC; ++j) acc" << k
                   << "[k][j] = 0.0f;\n";
        }
    };
    if (!(p.ring_stages > 0 && p.producer)) emitColumnState();
    // row loop
    const std::string I = "        ";
    auto declareFull = [&](const std::string& prefix, const std::string& indent) {
        for (size_t s = 0; s < p.inputs.size(); ++s)
            if (p.inputs[s].kind == THOR_B200_INPUT_TENSOR && p.input_shape[s] == FULL)
                os << indent << "tb_pack<VEC * " << dtypeSize(p.inputs[s].dtype) << "> " << prefix << s << "[VPT];\n";
    };
    auto loadFull = [&](const std::string& prefix, const std::string& row, const std::string& cond, const std::string& indent) {
        os << "#pragma unroll\n" << indent << "for (int k = 0; k < VPT; ++k) {\n" << indent << "    const tb_u32 q = t + k * TEAM;\n" << indent << "    if (" << cond << ") {\n";
        for (size_t s = 0; s < p.inputs.size(); ++s)
            if (p.inputs[s].kind == THOR_B200_INPUT_TENSOR && p.input_shape[s] == FULL)
                os << indent << "        tb_load_stream(" << prefix << s << "[k], in" << s << " + (" << row << ") * COLS + (tb_u64)q * VEC);\n";
        os << indent << "    }\n" << indent << "}\n";
    };
    const std::string guard = "row_ok && q < PPR";
    // the barrier of a reduction round: the whole CTA, or -- with a copy warpgroup beside the teams -- the team threads only
    const std::string team_sync = p.ring_stages > 0 && p.producer ? "if (TEAM > 32) tb_named_barrier<1, CONSUMERS>();\n" : "if (TEAM > 32) __syncthreads();\n";
    std::string ring_refill;  // ring mode: statements that refill the consumed buffer, emitted after the first barrier of the iteration
    if (p.persistent && p.ring_stages > 0) {
        // Rows of all [rows, cols] inputs arrive by bulk copies (one per input and iteration, covering the CTA's TEAMS
        // consecutive rows) in a ring of STAGES buffers; a buffer is copied to registers, then refilled for the
        // iteration STAGES ahead, so STAGES iterations of traffic are in flight per SM at no register cost.
        // Who requests the copies: thread 0 of the CTA after the first barrier of an iteration, or -- producer mode -- one
        // thread of a warpgroup that does nothing else.  Issuing a bulk copy stalls its thread for a few hundred cycles;
        // in a CTA whose warps all wait for each other twice per row that stall is on every row's critical path, so
        // programs that run one CTA per SM give the copies a warpgroup of their own: it hands its registers to the teams
        // (setmaxnreg) and waits on per-buffer "empty" barriers on which every team thread arrives once it holds its packs.
        os << "    constexpr int STAGES = " << p.ring_stages << ";\n    constexpr tb_u32 STAGE_BYTES = " << p.ring_stage_bytes << "u;\n";
        os << "    extern __shared__ __align__(128) unsigned char tb_ring[];  // [STAGES][full input][TEAMS][COLS]\n";
        os << "    __shared__ tb_u64 tb_full[STAGES];\n    __shared__ int tb_gave_up;\n";
        if (p.producer) os << "    __shared__ tb_u64 tb_empty[STAGES];\n    constexpr int CONSUMERS = TEAM * TEAMS;  // threads " << CTA << " and up are the copy warpgroup\n";
        os << "    const tb_u64 row_stride = (tb_u64)gridDim.x * TEAMS;\n";
        std::ostringstream fill;  // body of: refill buffer `stage` with the rows from `r0`
        {
            size_t off = 0;
            p.ring_offset.assign(p.inputs.size(), 0);
            std::string total;
            for (size_t s = 0; s < p.inputs.size(); ++s)
                if (p.inputs[s].kind == THOR_B200_INPUT_TENSOR && p.input_shape[s] == FULL) total += (total.empty() ? "" : " + ") + std::to_string(p.cols * dtypeSize(p.inputs[s].dtype)) + "u";
            fill << "const tb_u32 rows_here = ROWS - r0 < TEAMS ? (tb_u32)(ROWS - r0) : (tb_u32)TEAMS;\n";
            fill << "tb_mbar_expect(&tb_full[stage], rows_here * (" << total << "));\n";
            for (size_t s = 0; s < p.inputs.size(); ++s)
                if (p.inputs[s].kind == THOR_B200_INPUT_TENSOR && p.input_shape[s] == FULL) {
                    const size_t row_bytes = p.cols * dtypeSize(p.inputs[s].dtype);
                    fill << "tb_bulk_load(tb_ring + stage * STAGE_BYTES + " << off << "u, in" << s << " + r0 * COLS, rows_here * " << row_bytes << "u, &tb_full[stage]);\n";
                    p.ring_offset[s] = off;
                    off += row_bytes * teams_per_cta;
                }
        }
        auto emitFill = [&](const std::string& indent, std::ostringstream& to) {
            std::istringstream lines(fill.str());
            std::string line;
            while (std::getline(lines, line)) to << indent << line << "\n";
        };
        os << "    if (threadIdx.x == 0) {\n#pragma unroll\n        for (int s = 0; s < STAGES; ++s) {\n            tb_mbar_init(&tb_full[s], 1);\n";
        if (p.producer) os << "            tb_mbar_init(&tb_empty[s], CONSUMERS);\n";
        os << "        }\n        tb_gave_up = 0;\n        tb_mbar_init_fence();\n    }\n";
        os << "    __syncthreads();\n";
        if (p.producer) {
            // host-side fault injection for the tests of the bounded waits: the generated kernel simply lacks one copy
            // request (CTA 0, one iteration), so that the wait on that buffer's barrier runs out and the counter is raised
            os << "    if (threadIdx.x >= CONSUMERS) {\n        tb_release_registers();\n        if (threadIdx.x == CONSUMERS) {\n            tb_u32 stage = 0, it = 0;\n"
               << "            for (tb_u64 r0 = (tb_u64)blockIdx.x * TEAMS; r0 < ROWS; r0 += row_stride, ++it) {\n"
               << "                // the buffer is free once every team thread holds its packs of the iteration that used it last\n"
               << "                if (it >= STAGES) tb_mbar_wait(&tb_empty[stage], ((it / STAGES) + 1u) & 1u, &tb_gave_up);\n";
            if (p.drop_fill_iteration >= 0) os << "                if (!(blockIdx.x == 0 && it == " << p.drop_fill_iteration << "u)) {\n";
            else os << "                {\n";
            emitFill("                    ", os);
            os << "                }\n                if (++stage == STAGES) stage = 0;\n            }\n        }\n        return;\n    }\n    tb_claim_registers();\n";
            emitColumnState();
        } else {
            os << "    if (threadIdx.x == 0) {\n        for (int stage = 0; stage < STAGES; ++stage) {\n            const tb_u64 r0 = (tb_u64)blockIdx.x * TEAMS + stage * row_stride;\n"
               << "            if (r0 < ROWS) {\n";
            emitFill("                ", os);
            os << "            }\n        }\n    }\n";
        }
        declareFull("f", "    ");
        os << "    tb_u32 stage = 0, parity = 0;\n";
        if (p.pipelined) {
            for (uint32_t k : p.row_reduces)
                if (p.depth[k] == 1) os << "    " << cTypeName(p.nodes[k].output_dtype) << " cr" << k << ";  // round 1 of the row the next iteration works on\n";
            os << "    /*@row-loop*/\n";
        }
        os << "    for (tb_u64 row0 = (tb_u64)blockIdx.x * TEAMS; row0 < ROWS; row0 += row_stride) {  // same trip count for every team of the CTA\n";
        os << I << "const tb_u64 row = row0 + team_id;\n" << I << "const bool row_ok = " << (teams_per_cta == 1 ? "true" : "row < ROWS") << ";\n";
        if (!p.pipelined) os << I << "tb_mbar_wait(&tb_full[stage], parity, &tb_gave_up);\n";
        else os << I << "// this row's buffer was waited for when round 1 of the row ran\n";
        os << "#pragma unroll\n" << I << "for (int k = 0; k < VPT; ++k) {\n" << I << "    const tb_u32 q = t + k * TEAM;\n" << I << "    if (q < PPR) {\n";
        {
            size_t off = 0;
            for (size_t s = 0; s < p.inputs.size(); ++s)
                if (p.inputs[s].kind == THOR_B200_INPUT_TENSOR && p.input_shape[s] == FULL) {
                    const size_t es = dtypeSize(p.inputs[s].dtype);
                    os << I << "        f" << s << "[k] = *reinterpret_cast<const tb_pack<VEC * " << es << ">*>(tb_ring + stage * STAGE_BYTES + " << off << "u + ((tb_u32)team_id * (tb_u32)COLS + q * VEC) * "
                       << es << "u);\n";
                    off += p.cols * es * teams_per_cta;
                }
        }
        os << I << "    }\n" << I << "}\n";
        if (p.producer) {
            os << I << "tb_mbar_arrive(&tb_empty[stage]);  // this thread is done with the buffer\n";
        } else {
            // the buffer can take the rows of the iteration STAGES ahead once every thread holds its packs: after the
            // barrier of the first reduction round when the program has one, after a barrier of its own otherwise
            std::ostringstream refill;
            refill << I << "if (threadIdx.x == 0) {\n" << I << "    const tb_u64 r0 = row0 + STAGES * row_stride;\n";
            if (p.drop_fill_iteration >= 0)
                refill << I << "    if (r0 < ROWS && !(blockIdx.x == 0 && r0 == (tb_u64)" << p.drop_fill_iteration << " * row_stride)) {\n";
            else refill << I << "    if (r0 < ROWS) {\n";
            emitFill(I + "        ", refill);
            refill << I << "    }\n" << I << "}\n";
            if (TEAM > 32 && max_depth >= (p.pipelined ? 2 : 1)) ring_refill = refill.str();
            else os << I << "__syncthreads();\n" << refill.str();
        }
    } else if (p.persistent && p.prefetch) {
        os << "    const tb_u64 row_first = (tb_u64)blockIdx.x * TEAMS + team_id, row_stride = (tb_u64)gridDim.x * TEAMS;\n";
        declareFull("f", "    ");
        declareFull("n", "    ");
        loadFull("f", "row_first", "row_first < ROWS && q < PPR", "    ");
        os << "    for (tb_u64 row0 = (tb_u64)blockIdx.x * TEAMS; row0 < ROWS; row0 += row_stride) {  // same trip count for every team of the CTA\n";
        os << I << "const tb_u64 row = row0 + team_id;\n" << I << "const bool row_ok = " << (teams_per_cta == 1 ? "true" : "row < ROWS") << ";\n";
        os << I << "// the next row of this team is requested before the current one is touched\n";
        loadFull("n", "row + row_stride", "row + row_stride < ROWS && q < PPR", I);
    } else if (p.persistent) {
        os << "    for (tb_u64 row0 = (tb_u64)blockIdx.x * TEAMS; row0 < ROWS; row0 += (tb_u64)gridDim.x * TEAMS) {  // same trip count for every team of the CTA\n";
        os << I << "const tb_u64 row = row0 + team_id;\n" << I << "const bool row_ok = " << (teams_per_cta == 1 ? "true" : "row < ROWS") << ";\n";
        declareFull("f", I);
        loadFull("f", "row", guard, I);
    } else {
        os << "    {\n        const tb_u64 row = (tb_u64)blockIdx.x * TEAMS + team_id;\n        const bool row_ok = row < ROWS;\n";
        declareFull("f", I);
        loadFull("f", "row", guard, I);
    }
    if (p.persistent) {
        os << I << "float (*red_smem)[TEAMS][TEAM > 32 ? TEAM / 32 : 1] = red_smem_all[red_set];\n";
        if (any_arg) os << I << "tb_u64 (*red_key)[TEAMS][TEAM > 32 ? TEAM / 32 : 1] = red_key_all[red_set];\n";
    }
    // ROW inputs
    for (size_t s = 0; s < p.inputs.size(); ++s)
        if (p.inputs[s].kind == THOR_B200_INPUT_TENSOR && p.input_shape[s] == ROW)
            os << I << "const " << cTypeName(p.inputs[s].dtype) << " x" << s << " = row_ok ? in" << s << "[row] : " << cTypeName(p.inputs[s].dtype) << "();\n";

    for (uint32_t k = 0; k < p.nodes.size(); ++k)
        if (p.cache_state[k] == 1) os << I << "float2 h" << k << "[VPT][VEC / 2];  // kept from the first element loop that computes it\n";
    // row-scope nodes are emitted as soon as their depth is reached
    std::vector<bool> emitted(p.nodes.size(), false);
    auto emitRowScope = [&](int d) {
        std::vector<uint32_t> ids;
        for (uint32_t k = 0; k < p.nodes.size(); ++k) {
            if (!p.live[k] || emitted[k] || isReduce(p.nodes[k].op)) continue;
            if ((p.shape[k] == ROW || p.shape[k] == SCALAR) && p.depth[k] <= d) {
                ids.push_back(k);
                emitted[k] = true;
            }
        }
        emitStatements(p, ids, I, os);
    };
    emitRowScope(0);
    auto isMinMax = [&](uint32_t k) { return p.nodes[k].op == THOR_B200_OP_REDUCE_MIN || p.nodes[k].op == THOR_B200_OP_REDUCE_MAX; };
    // the pieces of one reduction round: accumulators, element loop, fold of the two lanes, the exchange before and after the barrier
    auto roundAccumulators = [&](const std::vector<uint32_t>& round) {
        for (uint32_t k : round) {
            if (p.nodes[k].op == kOpFirstMatch) {
                const uint32_t m = p.nodes[k].rhs;
                os << I << "tb_u32 i" << k << " = 0xffffffffu;\n" << I << "const float m" << k << " = " << convertExpression("v" + std::to_string(m), p.nodes[m].output_dtype, THOR_B200_FP32)
                   << ";\n" << I << "const bool mnan" << k << " = m" << k << " != m" << k << ";  // a NaN extreme matches the first NaN\n";
                continue;
            }
            if (isArgReduce(p.nodes[k].op)) {
                os << I << "float r" << k << " = " << (p.nodes[k].op == THOR_B200_OP_REDUCE_ARGMAX ? "__int_as_float(0xff800000)" : "__int_as_float(0x7f800000)") << ";\n"
                   << I << "tb_u32 i" << k << " = 0xffffffffu, n" << "an_i" << k << " = 0xffffffffu;  // no candidate, no NaN yet\n";
                continue;
            }
            if (p.pairs) os << I << "float2 q" << k << " = tb_both(" << identityExpr(p.nodes[k].op) << ");  // one partial per lane\n";
            else os << I << "float r" << k << " = " << identityExpr(p.nodes[k].op) << ";\n";
        }
    };
    auto roundElementLoop = [&](const std::vector<uint32_t>& round, const std::vector<uint32_t>& closure, const std::string& guard_expr) {
        os << "#pragma unroll\n" << I << "for (int k = 0; k < VPT; ++k) {\n" << I << "    const tb_u32 q = t + k * TEAM;\n" << I << "    if (" << guard_expr << ") {\n";
        emitColumnPackLoads(p, closure, I + "        ", os);
        // "first column equal to the row extreme": the element loop only ORs one compare per element into a per-pack flag;
        // the index arithmetic runs after the loop, for the few packs that hold a match (every pack of a row whose extreme is
        // NaN, where the first NaN is what is looked for)
        if (p.pairs)
            for (uint32_t k : round)
                if (p.nodes[k].op == kOpFirstMatch) os << I << "        bool hit" << k << " = mnan" << k << ";\n";
        os << "#pragma unroll\n" << I << "        for (int j = 0; j < VEC; " << (p.pairs ? "j += 2" : "++j") << ") {\n";
        emitElementInputs(p, closure, I + "            ", os);
        if (p.pairs) {
            emitPairStatements(p, closure, I + "            ", os);
            for (uint32_t k : round) {
                const uint32_t a = p.nodes[k].lhs;
                const uint16_t op = p.nodes[k].op;
                const std::string acc = "q" + std::to_string(k);
                const std::string II = I + "            ";
                if (op == kOpFirstMatch) {
                    const std::string arg = pairReduceArg(p, a, II, os);
                    os << II << "{ const float2 a" << k << " = " << arg << "; hit" << k << " = hit" << k << " | (a" << k << ".x == m" << k << ") | (a" << k << ".y == m" << k << "); }\n";
                    continue;
                }
                if (isArgReduce(op)) {
                    const std::string arg = pairReduceArg(p, a, II, os);
                    const char* mx = op == THOR_B200_OP_REDUCE_ARGMAX ? "true" : "false";
                    os << II << "{ const float2 a" << k << " = " << arg << "; tb_arg_scan<" << mx << ">(r" << k << ", i" << k << ", nan_i" << k << ", a" << k
                       << ".x, q * VEC + j); tb_arg_scan<" << mx << ">(r" << k << ", i" << k << ", nan_i" << k << ", a" << k << ".y, q * VEC + j + 1); }\n";
                    continue;
                }
                if ((op == THOR_B200_OP_REDUCE_SUM || op == THOR_B200_OP_REDUCE_AVG) && storedAsHeld(p, a) && elementLevel(p, a)) {
                    os << II << acc << " = " << pairPlus(p, a, acc) << ";\n";
                } else if (op == THOR_B200_OP_REDUCE_SUM || op == THOR_B200_OP_REDUCE_AVG) {
                    const std::string arg = pairReduceArg(p, a, II, os);
                    os << II << acc << " = __fadd2_rn(" << arg << ", " << acc << ");\n";
                } else if (op == THOR_B200_OP_REDUCE_NORM2) {
                    const std::string arg = pairReduceArg(p, a, II, os);
                    os << I << "            { const float2 a" << k << " = " << arg << "; " << acc << " = __ffma2_rn(a" << k << ", a" << k << ", " << acc << "); }\n";
                } else if (isMinMax(k)) {
                    // both elements of the pair with the NaN-propagating max / min of the hardware, two instructions
                    // (fmaxf per lane plus a sticky NaN predicate took five); only the .x lane of the partial is used
                    const char* fn = op == THOR_B200_OP_REDUCE_MAX ? "tb_max3_nan" : "tb_min3_nan";
                    const std::string arg = pairReduceArg(p, a, II, os);
                    os << I << "            { const float2 a" << k << " = " << arg << "; " << acc << ".x = " << fn << "(" << acc << ".x, a" << k << ".x, a" << k << ".y); }\n";
                } else {
                    const std::string arg = pairReduceArg(p, a, II, os);
                    os << I << "            { const float2 a" << k << " = " << arg << "; " << acc << ".x = " << combineExpr(op) << "(" << acc << ".x, "
                       << transformExpr(op, "a" + std::to_string(k) + ".x") << "); " << acc << ".y = " << combineExpr(op) << "(" << acc << ".y, "
                       << transformExpr(op, "a" + std::to_string(k) + ".y") << "); }\n";
                }
            }
        } else {
            emitStatements(p, closure, I + "            ", os);
            for (uint32_t k : round) {
                const uint32_t a = p.nodes[k].lhs;
                const std::string f = reduceArgF32(p, a, "v" + std::to_string(a));
                if (p.nodes[k].op == kOpFirstMatch)
                    os << I << "            { const float a" << k << " = " << f << "; i" << k << " = min(i" << k << ", (a" << k << " == m" << k << " || (mnan" << k << " && a" << k << " != a" << k
                       << ")) ? (tb_u32)(q * VEC + j) : 0xffffffffu); }\n";
                else if (isArgReduce(p.nodes[k].op))
                    os << I << "            tb_arg_scan<" << (p.nodes[k].op == THOR_B200_OP_REDUCE_ARGMAX ? "true" : "false") << ">(r" << k << ", i" << k << ", nan_i" << k << ", " << f
                       << ", q * VEC + j);\n";
                else if (isMinMax(k))
                    os << I << "            r" << k << " = " << (p.nodes[k].op == THOR_B200_OP_REDUCE_MAX ? "tb_max_nan" : "tb_min_nan") << "(r" << k << ", " << f << ");\n";
                else
                    os << I << "            r" << k << " = " << combineExpr(p.nodes[k].op) << "(r" << k << ", " << transformExpr(p.nodes[k].op, f) << ");\n";
            }
        }
        os << I << "        }\n";
        if (p.pairs)
            for (uint32_t k : round) {
                if (p.nodes[k].op != kOpFirstMatch) continue;
                const uint32_t a = p.nodes[k].lhs;
                const std::vector<uint32_t> arg_closure = elementClosure(p, std::vector<uint32_t>{a});
                const std::string II = I + "                ";
                os << I << "        if (hit" << k << ") {\n#pragma unroll\n" << I << "            for (int j = 0; j < VEC; j += 2) {\n";
                emitElementInputs(p, arg_closure, II, os);
                emitPairStatements(p, arg_closure, II, os);
                const std::string arg = pairReduceArg(p, a, II, os);
                os << II << "const float2 a" << k << " = " << arg << ";\n"
                   << II << "i" << k << " = min(i" << k << ", (a" << k << ".x == m" << k << " || (mnan" << k << " && a" << k << ".x != a" << k << ".x)) ? (tb_u32)(q * VEC + j) : 0xffffffffu);\n"
                   << II << "i" << k << " = min(i" << k << ", (a" << k << ".y == m" << k << " || (mnan" << k << " && a" << k << ".y != a" << k << ".y)) ? (tb_u32)(q * VEC + j + 1) : 0xffffffffu);\n";
                os << I << "            }\n" << I << "        }\n";
            }
        os << I << "    }\n" << I << "}\n";
        for (uint32_t k : closure)
            if (p.cache_state[k] == 1) p.cache_state[k] = 2;  // later loops read the registers
    };
    auto roundLaneFold = [&](const std::vector<uint32_t>& round) {
        if (p.pairs)
            for (uint32_t k : round) {
                if (isIndexReduce(p.nodes[k].op)) continue;
                const bool mm = isMinMax(k);
                os << I << "float r" << k << " = " << (mm ? (p.nodes[k].op == THOR_B200_OP_REDUCE_MAX ? "tb_max_nan" : "tb_min_nan") : combineExpr(p.nodes[k].op)) << "(q" << k << ".x, q" << k << ".y);\n";
            }
    };
    auto roundBeforeBarrier = [&](const std::vector<uint32_t>& round) {
        size_t slot = 0;
        for (uint32_t k : round) {
            const size_t idx = std::find(p.row_reduces.begin(), p.row_reduces.end(), k) - p.row_reduces.begin();
            if (p.nodes[k].op == kOpFirstMatch)
                os << I << "tb_u64 key" << k << " = tb_team_arg_stage1<TEAM>((tb_u64)(tb_u32)~i" << k << ", red_key[" << idx << "][team_id]);  // max of ~index = lowest index\n";
            else if (isArgReduce(p.nodes[k].op))
                os << I << "tb_arg_scan_finish<" << (p.nodes[k].op == THOR_B200_OP_REDUCE_ARGMAX ? "true" : "false") << ">(r" << k << ", i" << k << ", nan_i" << k
                   << ", row_ok && (tb_u32)t < PPR, (tb_u32)t * VEC);\n"
                   << I << "tb_u64 key" << k << " = tb_team_arg_stage1<TEAM>(tb_arg_key<" << (p.nodes[k].op == THOR_B200_OP_REDUCE_ARGMAX ? "true" : "false") << ">(r" << k
                   << ", i" << k << "), red_key[" << idx << "][team_id]);\n";
            else
                os << I << "r" << k << " = tb_team_reduce_stage1<TEAM, " << combineExpr(p.nodes[k].op) << ">(r" << k << ", red_smem[" << idx << "][team_id]);\n";
            ++slot;
        }
    };
    auto roundAfterBarrier = [&](const std::vector<uint32_t>& round, bool carry) {
        for (uint32_t k : round) {
            const size_t idx = std::find(p.row_reduces.begin(), p.row_reduces.end(), k) - p.row_reduces.begin();
            const auto& nd = p.nodes[k];
            if (isIndexReduce(nd.op)) {
                // only the team's first thread stores the index, so only it folds the warp keys
                os << I << "tb_u32 v" << k << " = 0u;\n" << I << "if (t == 0) v" << k << " = tb_team_arg_stage2<TEAM>(key" << k << ", red_key[" << idx << "][team_id]);\n";
                emitted[k] = true;
                continue;
            }
            os << I << "r" << k << " = tb_team_reduce_stage2<TEAM, " << combineExpr(nd.op) << ">(r" << k << ", red_smem[" << idx << "][team_id]);\n";
            std::string fin = "r" + std::to_string(k);
            if (nd.op == THOR_B200_OP_REDUCE_AVG) fin = "(" + fin + " / " + std::to_string(p.cols) + ".0f)";
            if (nd.op == THOR_B200_OP_REDUCE_NORM2) fin = "sqrtf(" + fin + ")";
            if (carry) {
                os << I << "cr" << k << " = " << convertExpression(fin, THOR_B200_FP32, nd.output_dtype) << ";\n";
                continue;
            }
            os << I << "const " << cTypeName(nd.output_dtype) << " v" << k << " = " << convertExpression(fin, THOR_B200_FP32, nd.output_dtype) << ";\n";
            emitted[k] = true;
        }
    };
    auto roundOfDepth = [&](int d) {
        std::vector<uint32_t> round;
        for (uint32_t k : p.row_reduces)
            if (p.depth[k] == d) round.push_back(k);
        return round;
    };
    auto closureOfRound = [&](const std::vector<uint32_t>& round) {
        std::vector<uint32_t> args;
        for (uint32_t k : round) args.push_back(p.nodes[k].lhs);
        return elementClosure(p, args);
    };
    int last_round = 0;
    for (int d = 1; d <= max_depth; ++d)
        if (!roundOfDepth(d).empty()) last_round = d;
    const std::vector<uint32_t> first_round = roundOfDepth(1);
    if (p.pipelined) {
        // Round 1 of the team's NEXT row rides on the last round of the current row: its operands come straight from the
        // next ring buffer, its partial sums share that round's exchange and barrier, and its results are carried into
        // the next iteration.  One exchange less per row, and the element work of the next row overlaps the shuffle chain.
        std::ostringstream pro;
        std::swap(pro, os);  // the prologue (round 1 of the CTA's first rows) is written first and spliced in before the loop
        os << "    {\n" << I << "float (*red_smem)[TEAMS][TEAM > 32 ? TEAM / 32 : 1] = red_smem_all[1];  // iteration 0 exchanges through set 0\n";
        os << I << "const bool next_ok = (tb_u64)blockIdx.x * TEAMS + team_id < ROWS;\n" << I << "const tb_u32 nstage = 0;\n";
        os << I << "tb_mbar_wait(&tb_full[0], 0, &tb_gave_up);\n";
        {
            std::vector<uint32_t> ids;
            for (uint32_t k = 0; k < p.nodes.size(); ++k)
                if (p.live[k] && !isReduce(p.nodes[k].op) && (p.shape[k] == ROW || p.shape[k] == SCALAR) && p.depth[k] == 0) ids.push_back(k);
            emitStatements(p, ids, I, os);
        }
        const std::vector<uint32_t> closure = closureOfRound(first_round);
        roundAccumulators(first_round);
        p.elements_from_next_buffer = true;
        roundElementLoop(first_round, closure, "next_ok && q < PPR");
        p.elements_from_next_buffer = false;
        roundLaneFold(first_round);
        roundBeforeBarrier(first_round);
        os << I << team_sync;
        roundAfterBarrier(first_round, true);
        os << "    }\n";
        std::swap(pro, os);
        const std::string marker = "    /*@row-loop*/\n";
        std::string text = os.str();
        const size_t at = text.find(marker);
        text.replace(at, marker.size(), pro.str());
        os.str(text);
        os.seekp(0, std::ios_base::end);
    }
    for (int d = 1; d <= max_depth; ++d) {
        const std::vector<uint32_t> round = roundOfDepth(d);
        if (round.empty()) continue;
        if (p.pipelined && d == 1) {
            os << I << "// round 1 of this row ran with the previous row\n";
            for (uint32_t k : round) {
                os << I << "const " << cTypeName(p.nodes[k].output_dtype) << " v" << k << " = cr" << k << ";\n";
                emitted[k] = true;
            }
            emitRowScope(d);
            continue;
        }
        const std::vector<uint32_t> closure = closureOfRound(round);
        os << I << "// round " << d << ": " << round.size() << " row reduction(s)\n";
        roundAccumulators(round);
        roundElementLoop(round, closure, guard);
        const bool carries_next = p.pipelined && d == last_round;
        if (carries_next) {
            os << I << "// ... and round 1 of the next row, read from its ring buffer\n";
            os << I << "const bool next_ok = row + row_stride < ROWS;\n";
            os << I << "const tb_u32 nstage = stage + 1 == STAGES ? 0u : stage + 1;\n";
            os << I << "if (row0 + row_stride < ROWS) tb_mbar_wait(&tb_full[nstage], nstage == 0 ? parity ^ 1u : parity, &tb_gave_up);\n";
            roundAccumulators(first_round);
            p.elements_from_next_buffer = true;
            roundElementLoop(first_round, closureOfRound(first_round), "next_ok && q < PPR");
            p.elements_from_next_buffer = false;
        }
        roundLaneFold(round);
        if (carries_next) roundLaneFold(first_round);
        // team combine: all reductions of the round share one shared-memory exchange
        roundBeforeBarrier(round);
        if (carries_next) roundBeforeBarrier(first_round);
        os << I << team_sync;
        if (!ring_refill.empty()) {
            os << ring_refill;
            ring_refill.clear();
        }
        roundAfterBarrier(round, false);
        if (carries_next) roundAfterBarrier(first_round, true);
        emitRowScope(d);
    }
    // final element loop: FULL outputs and column-reduction arguments
    std::vector<uint32_t> finals;
    for (const auto& o : p.outputs)
        if (p.shape[o.node] == FULL) finals.push_back(o.node);
    for (uint32_t k : p.col_reduces) finals.push_back(p.nodes[k].lhs);
    if (!finals.empty()) {
        const std::vector<uint32_t> closure = elementClosure(p, finals);
        os << I << "// outputs\n#pragma unroll\n" << I << "for (int k = 0; k < VPT; ++k) {\n" << I << "    const tb_u32 q = t + k * TEAM;\n" << I << "    if (" << guard << ") {\n";
        emitColumnPackLoads(p, closure, I + "        ", os);
        for (size_t o = 0; o < p.outputs.size(); ++o)
            if (p.shape[p.outputs[o].node] == FULL) os << I << "        tb_pack<VEC * " << dtypeSize(p.outputs[o].dtype) << "> w" << o << ";\n";
        os << "#pragma unroll\n" << I << "        for (int j = 0; j < VEC; " << (p.pairs ? "j += 2" : "++j") << ") {\n";
        emitElementInputs(p, closure, I + "            ", os);
        if (p.pairs) {
            emitPairStatements(p, closure, I + "            ", os);
            for (size_t o = 0; o < p.outputs.size(); ++o)
                if (p.shape[p.outputs[o].node] == FULL)
                    os << I << "            reinterpret_cast<" << pairType(p.outputs[o].dtype) << "*>(&w" << o << ")[j >> 1] = "
                       << convertPair("p" + std::to_string(p.outputs[o].node), vdt(p, p.outputs[o].node), p.outputs[o].dtype) << ";\n";
            for (uint32_t k : p.col_reduces) {
                const uint32_t a = p.nodes[k].lhs;
                const std::string slot = "acc" + std::to_string(k) + "[k][j >> 1]";
                if (storedAsHeld(p, a) && elementLevel(p, a)) os << I << "            " << slot << " = " << pairPlus(p, a, slot) << ";\n";
                else os << I << "            " << slot << " = __fadd2_rn(" << pairReduceArg(p, a, I + "            ", os) << ", " << slot << ");\n";
            }
        } else {
            emitStatements(p, closure, I + "            ", os);
            for (size_t o = 0; o < p.outputs.size(); ++o)
                if (p.shape[p.outputs[o].node] == FULL)
                    os << I << "            reinterpret_cast<" << cTypeName(p.outputs[o].dtype) << "*>(&w" << o << ")[j] = "
                       << convertExpression("v" + std::to_string(p.outputs[o].node), vdt(p, p.outputs[o].node), p.outputs[o].dtype) << ";\n";
            for (uint32_t k : p.col_reduces) {
                const uint32_t a = p.nodes[k].lhs;
                os << I << "            acc" << k << "[k][j] += " << reduceArgF32(p, a, "v" + std::to_string(a)) << ";\n";
            }
        }
        os << I << "        }\n";
        for (size_t o = 0; o < p.outputs.size(); ++o)
            if (p.shape[p.outputs[o].node] == FULL) os << I << "        tb_store_stream(out" << o << " + row * COLS + (tb_u64)q * VEC, w" << o << ");\n";
        os << I << "    }\n" << I << "}\n";
    }
    // ROW outputs
    for (size_t o = 0; o < p.outputs.size(); ++o)
        if (p.shape[p.outputs[o].node] == ROW) os << I << "if (t == 0 && row_ok) out" << o << "[row] = "
                                                      << convertExpression("v" + std::to_string(p.outputs[o].node), vdt(p, p.outputs[o].node), p.outputs[o].dtype) << ";\n";
    if (p.persistent) os << I << "red_set ^= 1;\n";
    if (p.persistent && p.ring_stages > 0) {
        os << I << "if (++stage == STAGES) {\n" << I << "    stage = 0;\n" << I << "    parity ^= 1;\n" << I << "}\n";
    } else if (p.persistent && p.prefetch) {
        os << "#pragma unroll\n" << I << "for (int k = 0; k < VPT; ++k) {\n";
        for (size_t s = 0; s < p.inputs.size(); ++s)
            if (p.inputs[s].kind == THOR_B200_INPUT_TENSOR && p.input_shape[s] == FULL) os << I << "    f" << s << "[k] = n" << s << "[k];\n";
        os << I << "}\n";
    }
    os << "    }\n";
    // column partials: ws[c][cta*TEAMS + team][COLS]
    size_t ci = 0;
    for (uint32_t k : p.col_reduces) {
        os << "    {\n        float* part = ws + ((tb_u64)" << ci << " * gridDim.x * TEAMS + (tb_u64)blockIdx.x * TEAMS + team_id) * COLS;\n";
        os << "#pragma unroll\n        for (int k = 0; k < VPT; ++k) {\n            const tb_u32 q = t + k * TEAM;\n            if (q < PPR) {\n";
        if (p.pairs)
            os << "#pragma unroll\n                for (int j = 0; j < VEC; j += 4) *reinterpret_cast<float4*>(part + (tb_u64)q * VEC + j) = make_float4(acc" << k << "[k][j >> 1].x, acc"
               << k << "[k][j >> 1].y, acc" << k << "[k][(j >> 1) + 1].x, acc" << k << "[k][(j >> 1) + 1].y);\n";
        else
            os << "#pragma unroll\n                for (int j = 0; j < VEC; j += 4) *reinterpret_cast<float4*>(part + (tb_u64)q * VEC + j) = make_float4(acc" << k << "[k][j], acc" << k
               << "[k][j + 1], acc" << k << "[k][j + 2], acc" << k << "[k][j + 3]);\n";
        os << "            }\n        }\n    }\n";
        ++ci;
    }
    os << "}\n";
    p.source = os.str();
    return "";
}

// Flat reduce program: rows * cols elements viewed as one vector.  CTA b streams packs
// [b * CHUNK, (b + 1) * CHUNK) with 4 independent 16-byte loads in flight per thread and tensor,
// evaluates the elementwise DAG per element, keeps one fp32 accumulator per requested reduction
// and writes one partial per reduction; foldFullPartials then combines the partials in CTA order.
std::string emitFlat(Program& p) {
    std::ostringstream os;
    const int VEC = p.vec;
    const uint64_t numel = p.rows * p.cols;
    os << "// generated by thor_b200: flat reduce program, " << p.nodes.size() << " nodes, " << numel << " elements, " << p.all_reduces.size() << " reduction(s)\n";
    os << "#include \"tb_prelude.cuh\"\n#include \"tb_rowprog.cuh\"\n\n";
    os << "extern \"C\" __global__ void __launch_bounds__(256) row_kernel(";
    bool first = true;
    for (size_t s = 0; s < p.inputs.size(); ++s) {
        os << (first ? "" : ", ");
        first = false;
        if (p.inputs[s].kind == THOR_B200_INPUT_RUNTIME_SCALAR_FP32) os << "const float s" << s;
        else os << "const " << cTypeName(p.inputs[s].dtype) << "* __restrict__ in" << s;
    }
    for (size_t o = 0; o < p.outputs.size(); ++o) {
        os << (first ? "" : ", ");
        first = false;
        os << cTypeName(p.outputs[o].dtype) << "* __restrict__ out" << o;
    }
    os << (first ? "" : ", ") << "float* __restrict__ ws) {\n    tb_grid_wait();\n";
    os << "    constexpr int VEC = " << VEC << ", U = 4, ITERS = " << p.vpt << ";\n";
    os << "    constexpr tb_u64 NUMEL = " << numel << "ull, NPACKS = NUMEL / VEC, CHUNK = 256ull * U * ITERS;\n";
    os << "    __shared__ float red_smem[" << p.all_reduces.size() << "][1][8];\n";
    os << "    const int t = threadIdx.x;\n";
    for (size_t s = 0; s < p.inputs.size(); ++s)
        if (p.inputs[s].kind == THOR_B200_INPUT_TENSOR_RUNTIME_SCALAR || (p.inputs[s].kind == THOR_B200_INPUT_TENSOR && p.input_shape[s] == SCALAR))
            os << "    const " << cTypeName(p.inputs[s].dtype) << (p.inputs[s].kind == THOR_B200_INPUT_TENSOR ? " x" : " s") << s << " = in" << s << "[0];\n";
    // scalar-class nodes
    std::vector<uint32_t> scalars_first;
    for (uint32_t k = 0; k < p.nodes.size(); ++k)
        if (p.live[k] && p.shape[k] == SCALAR && !isReduce(p.nodes[k].op)) scalars_first.push_back(k);
    emitStatements(p, scalars_first, "    ", os);
    auto isMinMax = [&](uint32_t k) { return p.nodes[k].op == THOR_B200_OP_REDUCE_MIN || p.nodes[k].op == THOR_B200_OP_REDUCE_MAX; };
    for (uint32_t k : p.all_reduces) {
        os << "    float r" << k << " = " << identityExpr(p.nodes[k].op) << ";\n";
        // min / max: the per-element step is ONE instruction, the NaN-propagating min.NaN / max.NaN of the hardware
        // (fminf / fmaxf plus a sticky "saw a NaN" predicate took three)
    }
    std::vector<uint32_t> args;
    for (uint32_t k : p.all_reduces) args.push_back(p.nodes[k].lhs);
    const std::vector<uint32_t> closure = elementClosure(p, args);
    auto emitAccumulate = [&](const std::string& indent) {
        emitStatements(p, closure, indent, os);
        for (uint32_t k : p.all_reduces) {
            const uint32_t a = p.nodes[k].lhs;
            const std::string f = reduceArgF32(p, a, "v" + std::to_string(a));
            if (isMinMax(k)) {
                os << indent << "r" << k << " = " << (p.nodes[k].op == THOR_B200_OP_REDUCE_MAX ? "tb_max_nan" : "tb_min_nan") << "(r" << k << ", " << f << ");\n";
            } else {
                os << indent << "r" << k << " = " << combineExpr(p.nodes[k].op) << "(r" << k << ", " << transformExpr(p.nodes[k].op, f) << ");\n";
            }
        }
    };
    os << "    const tb_u64 chunk0 = (tb_u64)blockIdx.x * CHUNK;\n";
    os << "#pragma unroll 1\n    for (int it = 0; it < ITERS; ++it) {\n";
    for (size_t s = 0; s < p.inputs.size(); ++s)
        if (p.inputs[s].kind == THOR_B200_INPUT_TENSOR && p.input_shape[s] == FULL) os << "        tb_pack<VEC * " << dtypeSize(p.inputs[s].dtype) << "> f" << s << "[U];\n";
    os << "#pragma unroll\n        for (int k = 0; k < U; ++k) {\n            const tb_u64 q = chunk0 + (tb_u64)(it * U + k) * 256 + t;\n            if (q < NPACKS) {\n";
    for (size_t s = 0; s < p.inputs.size(); ++s)
        if (p.inputs[s].kind == THOR_B200_INPUT_TENSOR && p.input_shape[s] == FULL) os << "                tb_load_stream(f" << s << "[k], in" << s << " + q * VEC);\n";
    os << "            }\n        }\n";
    os << "#pragma unroll\n        for (int k = 0; k < U; ++k) {\n            const tb_u64 q = chunk0 + (tb_u64)(it * U + k) * 256 + t;\n            if (q < NPACKS) {\n";
    os << "#pragma unroll\n                for (int j = 0; j < VEC; ++j) {\n";
    emitElementInputs(p, closure, "                    ", os);
    emitAccumulate("                    ");
    os << "                }\n            }\n        }\n    }\n";
    // ragged tail: NUMEL % VEC elements, one per thread of CTA 0
    os << "    if (blockIdx.x == 0) {\n        const tb_u64 i = NPACKS * VEC + t;\n        if (i < NUMEL) {\n";
    {
        std::vector<bool> done(p.inputs.size(), false);
        for (uint32_t k : closure) {
            const auto& nd = p.nodes[k];
            if (nd.op != THOR_B200_OP_INPUT || done[nd.input_slot] || p.input_shape[nd.input_slot] != FULL) continue;
            done[nd.input_slot] = true;
            os << "            const " << cTypeName(p.inputs[nd.input_slot].dtype) << " x" << nd.input_slot << " = in" << nd.input_slot << "[i];\n";
        }
    }
    emitAccumulate("            ");
    os << "        }\n    }\n";
    size_t idx = 0;
    for (uint32_t k : p.all_reduces) {
        os << "    r" << k << " = tb_team_reduce_stage1<256, " << combineExpr(p.nodes[k].op) << ">(r" << k << ", red_smem[" << idx << "][0]);\n";
        ++idx;
    }
    os << "    __syncthreads();\n";
    idx = 0;
    for (uint32_t k : p.all_reduces) {
        os << "    r" << k << " = tb_team_reduce_stage2<256, " << combineExpr(p.nodes[k].op) << ">(r" << k << ", red_smem[" << idx << "][0]);\n";
        os << "    if (t == 0) ws[(tb_u64)" << idx << " * gridDim.x + blockIdx.x] = r" << k << ";\n";
        ++idx;
    }
    os << "}\n";
    p.source = os.str();
    return "";
}

// Combine step of the folds below.
template <int OP>
__device__ __forceinline__ float foldCombine(float a, float b) {
    if (OP == 1) return a * b;
    if (OP == 2) return a != a ? a : (b != b ? b : fminf(a, b));
    if (OP == 3) return a != a ? a : (b != b ? b : fmaxf(a, b));
    return a + b;
}
// One launch folds every full reduction of a program: CTA i owns reduction i (thread t takes partials t, t + 1024, ...,
// then a fixed shuffle / warp-order combine, so the result does not depend on timing).
constexpr int kMaxFullFolds = 8;
struct FullFoldArgs {
    void* out[kMaxFullFolds];
    int out_dtype[kMaxFullFolds];
    float divisor[kMaxFullFolds];
    int op[kMaxFullFolds];  // 0 sum, 1 product, 2 min, 3 max
    int take_sqrt[kMaxFullFolds];
};
__device__ __forceinline__ float foldCombineAny(int op, float a, float b) {
    switch (op) {
        case 1: return foldCombine<1>(a, b);
        case 2: return foldCombine<2>(a, b);
        case 3: return foldCombine<3>(a, b);
        default: return foldCombine<0>(a, b);
    }
}
__global__ void __launch_bounds__(1024) foldFullPartials(const float* __restrict__ ws_all, uint32_t parts, FullFoldArgs a) {
    gridDependencyWait();
    gridLaunchDependents();
    __shared__ float sm[32];
    const int which = blockIdx.x, op = a.op[which];
    const float* ws = ws_all + static_cast<size_t>(which) * parts;
    const float identity = op == 1 ? 1.0f : (op == 2 ? __int_as_float(0x7f800000) : (op == 3 ? __int_as_float(0xff800000) : 0.0f));
    float v = identity;
    for (uint32_t s = threadIdx.x; s < parts; s += 1024) v = foldCombineAny(op, v, ws[s]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = foldCombineAny(op, v, __shfl_xor_sync(0xffffffffu, v, off));
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        float r = sm[0];
        for (int w = 1; w < 32; ++w) r = foldCombineAny(op, r, sm[w]);
        if (a.divisor[which] != 1.0f) r = r / a.divisor[which];
        if (a.take_sqrt[which]) r = sqrtf(r);
        void* out = a.out[which];
        switch (a.out_dtype[which]) {
            case THOR_B200_FP32: static_cast<float*>(out)[0] = r; break;
            case THOR_B200_FP16: static_cast<__half*>(out)[0] = __float2half_rn(r); break;
            case THOR_B200_BF16: static_cast<__nv_bfloat16*>(out)[0] = __float2bfloat16_rn(r); break;
            case THOR_B200_FP8_E4M3: static_cast<__nv_fp8_storage_t*>(out)[0] = __nv_cvt_float_to_fp8(r, __NV_SATFINITE, __NV_E4M3); break;
            case THOR_B200_FP8_E5M2: static_cast<__nv_fp8_storage_t*>(out)[0] = __nv_cvt_float_to_fp8(r, __NV_SATFINITE, __NV_E5M2); break;
            default: break;
        }
    }
}

// Folds the column partials of every column reduction of a program in ONE launch.  ws holds [reduction][parts][cols]
// fp32.  A CTA of 8 warps owns 32 * VEC neighbouring columns of one reduction: warp w adds parts w, w + 8, ... (coalesced
// VEC-wide loads, all of a thread's loads independent), the eight warp sums meet in shared memory and are added in warp
// order, so the result does not depend on timing.  The value is divided (means), optionally written unrounded to
// sums_f32[reduction][cols] -- what a caller that combines several GPUs' shards adds up before rounding once -- and
// stored in the output's dtype.
constexpr int kMaxColumnFolds = 8;
struct ColumnFoldArgs {
    void* out[kMaxColumnFolds];
    int out_dtype[kMaxColumnFolds];
    float divisor[kMaxColumnFolds];
};

__device__ __forceinline__ void storeAs(void* out, uint64_t i, int dtype, float v) {
    switch (dtype) {
        case THOR_B200_FP32: static_cast<float*>(out)[i] = v; break;
        case THOR_B200_FP16: static_cast<__half*>(out)[i] = __float2half_rn(v); break;
        case THOR_B200_BF16: static_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v); break;
        case THOR_B200_FP8_E4M3: static_cast<__nv_fp8_storage_t*>(out)[i] = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3); break;
        case THOR_B200_FP8_E5M2: static_cast<__nv_fp8_storage_t*>(out)[i] = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E5M2); break;
        default: break;
    }
}

template <int VEC>
__global__ void __launch_bounds__(256) foldColumnPartials(const float* __restrict__ ws, uint32_t parts, uint64_t cols, ColumnFoldArgs args, float* __restrict__ sums_f32) {
    gridDependencyWait();
    gridLaunchDependents();
    __shared__ float sm[8][32 * VEC];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, r = blockIdx.y;
    const uint64_t c0 = (static_cast<uint64_t>(blockIdx.x) * 32 + lane) * VEC;
    const float* base = ws + static_cast<uint64_t>(r) * parts * cols;
    float acc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = 0.0f;
    if (c0 < cols) {
        for (uint32_t s = warp; s < parts; s += 8) {
            if (VEC == 4) {
                const float4 v = *reinterpret_cast<const float4*>(base + static_cast<uint64_t>(s) * cols + c0);
                acc[0] += v.x;
                acc[1 % VEC] += v.y;
                acc[2 % VEC] += v.z;
                acc[3 % VEC] += v.w;
            } else {
                acc[0] += base[static_cast<uint64_t>(s) * cols + c0];
            }
        }
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) sm[warp][lane * VEC + j] = acc[j];
    __syncthreads();
    // thread t of the CTA finishes column t of the CTA's 32 * VEC (VEC = 4: the first 128 threads)
    if (threadIdx.x < 32 * VEC) {
        const uint64_t c = static_cast<uint64_t>(blockIdx.x) * 32 * VEC + threadIdx.x;
        if (c < cols) {
            float v = sm[0][threadIdx.x];
#pragma unroll
            for (int w = 1; w < 8; ++w) v += sm[w][threadIdx.x];
            if (args.divisor[r] != 1.0f) v = v / args.divisor[r];
            if (sums_f32 != nullptr) sums_f32[static_cast<uint64_t>(r) * cols + c] = v;
            storeAs(args.out[r], c, args.out_dtype[r], v);
        }
    }
}

}  // namespace
}  // namespace tb::rowprog

struct thor_b200_rowprog {
    tb::rowprog::Program prog;
    std::shared_ptr<tb::jit::Module> module;
    size_t workspace_bytes = 1;
    bool compile_only = false;
    bool smem_opted_in[64] = {};
    std::atomic<uint32_t> expired_seen{0};  // what thor_b200_rowprog_waits_expired last reported
};

extern "C" {

int thor_b200_rowprog_compile(const thor_b200_rowprog_desc* d, thor_b200_rowprog** out_prog, size_t* workspace_bytes) {
    using namespace tb;
    using namespace tb::rowprog;
    TB_REQUIRE(d != nullptr && out_prog != nullptr && workspace_bytes != nullptr, "rowprog_compile: null argument");
    *out_prog = nullptr;
    TB_REQUIRE(d->nodes != nullptr && d->n_nodes > 0 && d->outputs != nullptr && d->n_outputs > 0, "rowprog_compile: empty program");
    TB_REQUIRE(d->rows > 0 && d->cols > 0, "rowprog_compile: zero-sized dimension");
    TB_REQUIRE(d->n_inputs == 0 || (d->inputs != nullptr && d->input_shapes != nullptr), "rowprog_compile: inputs missing");
    auto h = std::make_unique<thor_b200_rowprog>();
    Program& p = h->prog;
    p.nodes.assign(d->nodes, d->nodes + d->n_nodes);
    p.inputs.assign(d->inputs, d->inputs + d->n_inputs);
    p.input_shape.assign(d->input_shapes, d->input_shapes + d->n_inputs);
    p.outputs.assign(d->outputs, d->outputs + d->n_outputs);
    p.rows = d->rows;
    p.cols = d->cols;
    p.fast_math = d->options.use_fast_math != 0;
    h->compile_only = d->options.compile_only != 0;
    for (size_t s = 0; s < p.inputs.size(); ++s) {
        TB_REQUIRE(p.inputs[s].kind >= 0 && p.inputs[s].kind <= 2, "rowprog_compile: input %zu has an unknown kind", s);
        TB_REQUIRE(dtypeSize(p.inputs[s].dtype) != 0 && p.inputs[s].dtype != THOR_B200_FP64, "rowprog_compile: input %zu has an unsupported dtype", s);
        if (p.inputs[s].kind == THOR_B200_INPUT_TENSOR) TB_REQUIRE(p.input_shape[s] >= 0 && p.input_shape[s] <= 3, "rowprog_compile: input %zu has an unknown shape class", s);
    }
    // an arg reduction beside the min / max of the same values becomes "first column that equals that min / max"
    for (size_t k = 0; k < p.nodes.size(); ++k) {
        auto& nd = p.nodes[k];
        if (!isArgReduce(nd.op) || nd.input_slot != 0) continue;
        const uint16_t value_op = nd.op == THOR_B200_OP_REDUCE_ARGMAX ? THOR_B200_OP_REDUCE_MAX : THOR_B200_OP_REDUCE_MIN;
        for (size_t m = 0; m < k; ++m) {
            const auto& vm = p.nodes[m];
            if (vm.op == value_op && vm.input_slot == 0 && vm.lhs == nd.lhs && vm.output_dtype == THOR_B200_FP32) {
                nd.op = kOpFirstMatch;
                nd.rhs = static_cast<uint32_t>(m);
                break;
            }
        }
    }
    {
        // constants and identities first, as in the fused stages (the reference's emitter rule)
        std::vector<uint32_t> keep;
        for (const auto& o : p.outputs) keep.push_back(o.node);
        tb::expr::foldConstantsAndIdentities(p.nodes, keep);
    }
    mergeDuplicates(p);
    std::string why = analyse(p);
    if (!why.empty()) return fail(THOR_B200_UNSUPPORTED, "rowprog_compile: %s", why.c_str());
    for (int pass = 0; pass < 4 && hoistLinearRowSums(p); ++pass) {
        mergeDuplicates(p);
        why = analyse(p);
        if (!why.empty()) return fail(THOR_B200_UNSUPPORTED, "rowprog_compile: %s", why.c_str());
    }

    // geometry: pack width from the narrowest FULL / COL tensor, team size from the row length
    size_t mn = 8, mx = 1;
    for (size_t s = 0; s < p.inputs.size(); ++s)
        if (p.inputs[s].kind == THOR_B200_INPUT_TENSOR && (p.input_shape[s] == FULL || p.input_shape[s] == COL)) {
            mn = std::min(mn, dtypeSize(p.inputs[s].dtype));
            mx = std::max(mx, dtypeSize(p.inputs[s].dtype));
        }
    for (const auto& o : p.outputs)
        if (p.shape[o.node] == FULL) {
            mn = std::min(mn, dtypeSize(o.dtype));
            mx = std::max(mx, dtypeSize(o.dtype));
        }
    if (mn > mx) return fail(THOR_B200_UNSUPPORTED, "rowprog_compile: no [rows, cols] tensor in the program");
    if (!p.all_reduces.empty()) {
        // flat reduce program over rows * cols elements
        p.vec = static_cast<int>(16 / mn);
        p.team = p.cta = 256;
        const uint64_t numel = p.rows * p.cols;
        const uint64_t packs = numel / p.vec;
        p.vpt = 4;  // iterations of 4 packs per thread: one CTA streams 256 * 16 packs (64 KiB of the narrowest tensor)
        const uint64_t chunk = 256ull * 4 * p.vpt;
        const uint64_t blocks = std::max<uint64_t>(1, (packs + chunk - 1) / chunk);
        if (blocks > 0x7FFFFFFFull) return fail(THOR_B200_UNSUPPORTED, "rowprog_compile: too many elements for one grid");
        p.grid = static_cast<uint32_t>(blocks);
        p.persistent = false;
        const std::string ferr = emitFlat(p);
        if (!ferr.empty()) return fail(THOR_B200_UNSUPPORTED, "rowprog_compile: %s", ferr.c_str());
        h->workspace_bytes = p.all_reduces.size() * static_cast<size_t>(p.grid) * sizeof(float);
        if (int st = jit::compileSource(p.source, p.fast_math, "row_kernel", &h->module)) return st;
        if (!h->compile_only)
            if (int st = jit::ensureLoaded(*h->module)) return st;
        *workspace_bytes = h->workspace_bytes;
        *out_prog = h.release();
        return THOR_B200_OK;
    }
    int vec = static_cast<int>(16 / mn);
    if (vec < 4) vec = 4;
    while (vec > 4 && static_cast<size_t>(vec) * mx > 64) vec /= 2;
    if (p.cols % vec != 0) return fail(THOR_B200_UNSUPPORTED, "rowprog_compile: cols (%llu) is not a multiple of the pack width %d", static_cast<unsigned long long>(p.cols), vec);
    const uint64_t packs = p.cols / vec;
    if (packs > 1024ull * 8) return fail(THOR_B200_UNSUPPORTED, "rowprog_compile: rows of %llu elements do not fit one CTA's registers", static_cast<unsigned long long>(p.cols));
    const thor_b200_rowprog_tuning& tune = d->tuning;
    TB_REQUIRE(tune.reserve_sms >= 0 && tune.reserve_sms <= 64, "rowprog_compile: tuning.reserve_sms must be between 0 and 64");
    TB_REQUIRE(tune.ring_buffers >= -2 && tune.ring_buffers != 1 && tune.ring_buffers != 2, "rowprog_compile: tuning.ring_buffers must be 0, -1, -2 or at least 3");
    const int vpt_target = 4;  // measured: 4 packs per thread beat 2 even with column accumulators in registers
    int team = 32;
    while (team < 1024 && packs > static_cast<uint64_t>(team) * vpt_target) team *= 2;
    if (team == 64) team = 128;
    p.vec = vec;
    p.team = team;
    p.cta = team < 256 ? 256 : team;
    p.vpt = static_cast<int>((packs + team - 1) / team);
    bool has_col_input = false;
    for (size_t s = 0; s < p.inputs.size(); ++s) has_col_input = has_col_input || (p.inputs[s].kind == THOR_B200_INPUT_TENSOR && p.input_shape[s] == COL);
    p.persistent = has_col_input || !p.col_reduces.empty();
    p.prefetch = p.persistent;  // register double buffer, unless the ring below takes over
    p.min_ctas = d->options.min_ctas_per_sm;
    p.pairs = true;
    p.cache_wanted = tune.keep_values >= 0;
    // off unless the caller asked for fast math: the reference divides, and so do we (measured: softmax + argmax in one
    // pass 352 us with the division, 310 us with the reciprocal; softmax alone is at the memory bound either way)
    p.reciprocal_division = tune.reciprocal_division != 0 ? tune.reciprocal_division > 0 : p.fast_math;
    {
        // Ring of bulk-copied row buffers: needs 16-byte rows, as many stages as fit in 200 KB (at least 3, at most 8).
        const uint64_t teams = p.cta / p.team;
        size_t slot_bytes = 0;  // one row group of the CTA: every [rows, cols] input, TEAMS consecutive rows
        bool rows16 = true;
        for (size_t s = 0; s < p.inputs.size(); ++s)
            if (p.inputs[s].kind == THOR_B200_INPUT_TENSOR && p.input_shape[s] == FULL) {
                const size_t row_bytes = p.cols * dtypeSize(p.inputs[s].dtype);
                rows16 = rows16 && row_bytes % 16 == 0;
                slot_bytes += row_bytes * teams;
            }
        // Measured on B200, LayerNorm [32768, 8192] bf16.  Forward (two CTAs per SM): 3 buffers with round 1 pipelined
        // 164 us, against 175 us for the register double buffer, 183 us for 4 buffers and 186 us for 3 buffers
        // without the pipelining.  Backward (one CTA per SM, 64 accumulator registers): 4 buffers without pipelining
        // 311 us, against 321 us for the register double buffer, 316 / 314 us for 3 / 5 buffers and 324 us pipelined.
        const bool with_columns = !p.col_reduces.empty();
        const bool pipeline = (tune.pipeline_round_one != 0 ? tune.pipeline_round_one > 0 : !with_columns) && canPipeline(p);
        // A copy warpgroup beside the teams (see emit()): for programs that run one CTA of 256 team threads per SM, where
        // 2 x 240 + 24 registers per lane fit an SM sub-partition.  Measured on the backward program: 295 -> 285 us.
        const bool producer = (tune.copy_warpgroup != 0 ? tune.copy_warpgroup > 0 : with_columns) && with_columns && p.cta == 256;
        int wanted = tune.ring_buffers;  // 0 the measured default, -1 off, -2 as many buffers as fit, n >= 3 at most n
        if (wanted == 0) wanted = with_columns ? 4 : (pipeline ? 3 : -1);
        if (p.persistent && wanted != -1 && rows16 && slot_bytes > 0 && slot_bytes < (1u << 20)) {
            // programs without column reductions run two CTAs per SM, which share the SM's shared memory
            const int ctas_per_sm = p.col_reduces.empty() ? 2 : 1;
            const size_t budget = 200 * 1024 / ctas_per_sm;
            const size_t stage_bytes = slot_bytes;
            int stages = static_cast<int>(std::min<size_t>(8, budget / stage_bytes));
            if (wanted > 0) stages = std::min(stages, wanted);
            if (stages >= 3) {
                p.ring_stages = stages;
                p.ring_stage_bytes = stage_bytes;
                p.producer = producer;
                p.smem_bytes = stage_bytes * stages;
                p.prefetch = false;
                p.pipeline_wanted = pipeline;
                p.wait_limit_ms = tune.wait_limit_ms;
                p.drop_fill_iteration = tune.test_skip_fill > 0 ? tune.test_skip_fill : -1;
            }
        }
    }
    const uint64_t teams_per_cta = p.cta / p.team;
    const uint64_t ctas_for_rows = (p.rows + teams_per_cta - 1) / teams_per_cta;
    int sms = 148;
    {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) sms = v;
        else (void)cudaGetLastError();
        if (tune.reserve_sms < sms) sms -= tune.reserve_sms;
    }
    if (p.persistent) {
        // every extra CTA of a program with column reductions costs a [cols] fp32 partial row
        // measured on B200 (LayerNorm [32768, 8192] bf16): 2 CTAs per SM for the forward program, 1 for the
        // backward program whose per-column accumulators take most of the register file
        const uint64_t resident = p.col_reduces.empty() ? static_cast<uint64_t>(sms) * 2 : static_cast<uint64_t>(sms);
        p.grid = static_cast<uint32_t>(std::min<uint64_t>(ctas_for_rows, resident));
    } else {
        if (ctas_for_rows > 0x7FFFFFFFull) return fail(THOR_B200_UNSUPPORTED, "rowprog_compile: too many rows for one grid");
        p.grid = static_cast<uint32_t>(ctas_for_rows);
    }
    if (p.col_reduces.size() > static_cast<size_t>(kMaxColumnFolds))
        return fail(THOR_B200_UNSUPPORTED, "rowprog_compile: at most %d column reductions per program", kMaxColumnFolds);
    const std::string err = emit(p);
    if (!err.empty()) return fail(THOR_B200_UNSUPPORTED, "rowprog_compile: %s", err.c_str());
    h->workspace_bytes = p.col_reduces.empty() ? 1 : p.col_reduces.size() * static_cast<size_t>(p.grid) * teams_per_cta * p.cols * sizeof(float);
    if (int st = jit::compileSource(p.source, p.fast_math, "row_kernel", &h->module)) return st;
    if (!h->compile_only)
        if (int st = jit::ensureLoaded(*h->module)) return st;
    *workspace_bytes = h->workspace_bytes;
    *out_prog = h.release();
    return THOR_B200_OK;
}

int thor_b200_rowprog_launch(thor_b200_rowprog* h, const void* const* input_ptrs, const float* runtime_scalars, void* const* output_ptrs, void* workspace,
                             size_t workspace_bytes, void* stream_v) {
    return thor_b200_rowprog_launch_sharded(h, input_ptrs, runtime_scalars, output_ptrs, workspace, workspace_bytes, nullptr, stream_v);
}

int thor_b200_rowprog_launch_sharded(thor_b200_rowprog* h, const void* const* input_ptrs, const float* runtime_scalars, void* const* output_ptrs, void* workspace,
                                     size_t workspace_bytes, void* column_sums_f32, void* stream_v) {
    using namespace tb;
    using namespace tb::rowprog;
    TB_REQUIRE(h != nullptr, "rowprog_launch: null handle");
    TB_REQUIRE(!h->compile_only, "rowprog_launch: handle was compiled with compile_only");
    TB_REQUIRE(output_ptrs != nullptr, "rowprog_launch: output_ptrs is null");
    if (const uint32_t seen = h->expired_seen.load(std::memory_order_relaxed))
        return fail(THOR_B200_CUDA_ERROR,
                    "rowprog_launch: earlier launches of this program recorded %u expired device-side waits, so their outputs were invalid; "
                    "the program refuses further launches until the cause is found and it is compiled again",
                    seen);
    const Program& p = h->prog;
    TB_REQUIRE(workspace_bytes >= h->workspace_bytes, "rowprog_launch: workspace too small");
    TB_REQUIRE((p.col_reduces.empty() && p.all_reduces.empty()) || (workspace != nullptr && isAligned(workspace, 16)),
               "rowprog_launch: workspace must be a 16-byte aligned device pointer");
    if (int st = jit::ensureLoaded(*h->module)) return st;
    constexpr size_t kMaxArgs = 64;
    TB_REQUIRE(p.inputs.size() + p.outputs.size() + 1 <= kMaxArgs, "rowprog_launch: too many kernel arguments");
    void* args[kMaxArgs];
    const void* ptr_store[kMaxArgs];
    float scalar_store[kMaxArgs];
    size_t n = 0;
    for (size_t s = 0; s < p.inputs.size(); ++s) {
        if (p.inputs[s].kind == THOR_B200_INPUT_RUNTIME_SCALAR_FP32) {
            TB_REQUIRE(runtime_scalars != nullptr, "rowprog_launch: runtime_scalars is null");
            scalar_store[n] = runtime_scalars[s];
            args[n] = &scalar_store[n];
        } else {
            TB_REQUIRE(input_ptrs != nullptr && input_ptrs[s] != nullptr, "rowprog_launch: input %zu is null", s);
            if (p.inputs[s].kind == THOR_B200_INPUT_TENSOR && (p.input_shape[s] == FULL || p.input_shape[s] == COL))
                TB_REQUIRE(isAligned(input_ptrs[s], 16), "rowprog_launch: input %zu must be 16-byte aligned", s);
            ptr_store[n] = input_ptrs[s];
            args[n] = &ptr_store[n];
        }
        ++n;
    }
    for (size_t o = 0; o < p.outputs.size(); ++o) {
        TB_REQUIRE(output_ptrs[o] != nullptr, "rowprog_launch: output %zu is null", o);
        // column-reduction outputs are written by the fold kernel; the row kernel gets the pointer but does not use it
        if (p.shape[p.outputs[o].node] == FULL) TB_REQUIRE(isAligned(output_ptrs[o], 16), "rowprog_launch: output %zu must be 16-byte aligned", o);
        ptr_store[n] = output_ptrs[o];
        args[n] = &ptr_store[n];
        ++n;
    }
    const void* ws_ptr = workspace;
    args[n++] = &ws_ptr;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    if (p.smem_bytes > 0) {  // static shared memory counts against the 48 KB default too
        int dev = 0;
        TB_CUDA(cudaGetDevice(&dev));
        if (!h->smem_opted_in[dev & 63]) {
            TB_CUDA(cudaKernelSetAttributeForDevice(h->module->kernel.load(), cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(p.smem_bytes), dev));
            h->smem_opted_in[dev & 63] = true;
        }
    }
    TB_CUDA(launchDependentC(reinterpret_cast<const void*>(h->module->kernel.load()), dim3(p.grid), dim3(static_cast<unsigned>(p.cta + (p.ring_stages > 0 && p.producer ? 128 : 0))), args, p.smem_bytes, stream));
    countLaunch();
    if (!p.all_reduces.empty()) {
        // every group of up to kMaxFullFolds reductions is folded by one launch (one CTA per reduction)
        for (size_t first = 0; first < p.all_reduces.size(); first += kMaxFullFolds) {
            const size_t count = std::min<size_t>(kMaxFullFolds, p.all_reduces.size() - first);
            FullFoldArgs fold{};
            for (size_t i = 0; i < count; ++i) {
                const uint32_t k = p.all_reduces[first + i];
                size_t o = 0;
                for (; o < p.outputs.size(); ++o)
                    if (p.outputs[o].node == k) break;
                const uint16_t op = p.nodes[k].op;
                fold.out[i] = output_ptrs[o];
                fold.out_dtype[i] = p.outputs[o].dtype;
                fold.divisor[i] = op == THOR_B200_OP_REDUCE_AVG ? static_cast<float>(p.rows * p.cols) : 1.0f;
                fold.take_sqrt[i] = op == THOR_B200_OP_REDUCE_NORM2;
                fold.op[i] = op == THOR_B200_OP_REDUCE_PROD ? 1 : (op == THOR_B200_OP_REDUCE_MIN ? 2 : (op == THOR_B200_OP_REDUCE_MAX ? 3 : 0));
            }
            const float* part = static_cast<const float*>(workspace) + first * static_cast<size_t>(p.grid);
            TB_CUDA(launchDependent(foldFullPartials, dim3(static_cast<unsigned>(count)), dim3(1024), 0, stream, part, p.grid, fold));
            countLaunch();
        }
    }
    if (!p.col_reduces.empty()) {
        const uint32_t parts = p.grid * static_cast<uint32_t>(p.cta / p.team);
        ColumnFoldArgs fold{};
        size_t ci = 0;
        for (uint32_t k : p.col_reduces) {
            size_t o = 0;
            for (; o < p.outputs.size(); ++o)
                if (p.outputs[o].node == k) break;
            fold.out[ci] = output_ptrs[o];
            fold.out_dtype[ci] = p.outputs[o].dtype;
            fold.divisor[ci] = p.nodes[k].op == THOR_B200_OP_REDUCE_AVG ? static_cast<float>(p.rows) : 1.0f;
            ++ci;
        }
        const float* part = static_cast<const float*>(workspace);
        float* sums = static_cast<float*>(column_sums_f32);
        if (p.cols % 4 == 0)
            (void)launchDependent(foldColumnPartials<4>, dim3(static_cast<unsigned>((p.cols + 127) / 128), static_cast<unsigned>(ci)), dim3(256), 0, stream, part, parts, p.cols, fold, sums);
        else
            (void)launchDependent(foldColumnPartials<1>, dim3(static_cast<unsigned>((p.cols + 31) / 32), static_cast<unsigned>(ci)), dim3(256), 0, stream, part, parts, p.cols, fold, sums);
        TB_CUDA(cudaGetLastError());
        countLaunch();
    } else {
        TB_REQUIRE(column_sums_f32 == nullptr, "rowprog_launch: the program has no column reductions to report unrounded");
    }
    return THOR_B200_OK;
}

const char* thor_b200_rowprog_source(const thor_b200_rowprog* h) { return h ? h->prog.source.c_str() : ""; }

uint32_t thor_b200_rowprog_launch_count(const thor_b200_rowprog* h) {
    return h ? 1u + static_cast<uint32_t>((h->prog.col_reduces.empty() ? 0 : 1) + (h->prog.all_reduces.size() + tb::rowprog::kMaxFullFolds - 1) / tb::rowprog::kMaxFullFolds) : 0u;
}

int thor_b200_rowprog_waits_expired(thor_b200_rowprog* h, uint32_t* count) {
    TB_REQUIRE(h != nullptr && count != nullptr, "rowprog_waits_expired: null argument");
    *count = 0;
    if (h->prog.ring_stages == 0 || !h->module || h->module->kernel.load(std::memory_order_acquire) == nullptr) return THOR_B200_OK;  // never loaded
    void* flag = nullptr;
    size_t bytes = 0;
    TB_CUDA(cudaLibraryGetGlobal(&flag, &bytes, h->module->library, "tb_wait_expired"));
    TB_REQUIRE(bytes == sizeof(uint32_t), "rowprog_waits_expired: unexpected size of the device counter");
    TB_CUDA(cudaDeviceSynchronize());
    TB_CUDA(cudaMemcpy(count, flag, sizeof(uint32_t), cudaMemcpyDeviceToHost));
    h->expired_seen.store(*count, std::memory_order_relaxed);
    return THOR_B200_OK;
}

void thor_b200_rowprog_destroy(thor_b200_rowprog* h) { delete h; }

}  // extern "C"
