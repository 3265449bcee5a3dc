// Fused-stage emitter: turns a validated SSA node list (+ optional broadcast geometry) into the
// CUDA C++ source of one single-pass kernel and the launch geometry that goes with it.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

#include "thor_b200.h"

namespace tb::expr {

struct Stage {
    std::vector<thor_b200_expr_node> nodes;
    std::vector<thor_b200_expr_input> inputs;
    std::vector<thor_b200_expr_output> outputs;
    bool broadcast = false;
    uint32_t rank = 0;
    std::vector<uint64_t> dims;                 // [rank]
    std::vector<std::vector<int64_t>> strides;  // [n_inputs][rank] (tensor inputs only)
    bool fast_math = false;
    int rows_per_thread = 0;   // tuning overrides, 0 = automatic
    int min_ctas_per_sm = 0;
    int packs_per_thread = 0;
};

enum class Kind { FlatV2, FlatScalar, TiledV2, TiledScalar, Generic };

struct Emitted {
    std::string source;
    Kind kind = Kind::FlatScalar;
    int vec = 1;        // elements per pack
    int unroll = 1;     // packs (flat) or rows (tiled) per thread
    int threads = 256;
    // tiled / generic geometry (baked into the source as literals)
    uint64_t rows = 0, cols = 0, numel = 0;
    int tx = 0, ty = 0;
    bool linear_grid = false;  // tiled kernels: one-dimensional grid, column chunks of a row block in consecutive CTAs
    // pointer alignment (bytes) the kernel assumes for each tensor input / output; 1 = none
    std::vector<int> input_align;
    std::vector<int> output_align;
};

// Validates the stage.  Returns "" when it is well formed, else the reason.
std::string validate(const Stage& stage);

// Emits the fastest kernel shape the stage admits, or (force_generic) the element-wise fallback that
// makes no alignment or divisibility assumption.  Returns "" on success, else the reason.
std::string emit(const Stage& stage, bool force_generic, Emitted* out);

const char* kindName(Kind k);

// What the reference's emitter does to constants and identities before it emits a node
// (CudaSourceEmitter.cpp:1965-2076, 3478-3485, 3745-3782), applied to the node list itself:
//   - a subtree of literals under NEG / ADD / SUB / MUL / DIV is evaluated in double and becomes ONE literal, emitted as
//     a float literal and converted to the dtype the node's value is held in (not computed per node in a 16-bit type);
//   - x + 0, 0 + x, x - 0, x * 1, 1 * x and x / 1 compute nothing: the node's value is x converted to the node's dtype.
// Nodes listed in `keep` (stage outputs) keep their declared output dtype.  Returns how many nodes were rewritten.
size_t foldConstantsAndIdentities(std::vector<thor_b200_expr_node>& nodes, const std::vector<uint32_t>& keep);

// Building blocks shared with the row-program emitter.  A node's value lives in the variable "v<k>"
// typed as its output dtype; tensor inputs are "x<slot>", scalars "s<slot>".
std::string scalarNodeExpression(const std::vector<thor_b200_expr_node>& nodes, const std::vector<thor_b200_expr_input>& inputs, size_t k);
const char* cTypeName(int dtype);
// dtype in which node k's value is held inside a kernel (compute dtype for arithmetic nodes, output dtype for leaves and casts)
int nodeValueDType(const std::vector<thor_b200_expr_node>& nodes, size_t k);
std::string convertExpression(const std::string& e, int src, int dst);
bool isFusedStageOp(uint16_t op);

}  // namespace tb::expr
