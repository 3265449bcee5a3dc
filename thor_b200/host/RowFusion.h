// Physical fusion of "elementwise -> row reduction -> elementwise" chains into one single-pass row
// program (softmax, LayerNorm forward / backward, ...).  The reference never fuses across a
// reduction (EquationCompiler.cpp:684-688); this pass keeps its logical stage list and only
// replaces what launches.
#pragma once

#include <functional>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "FusedEquation.h"

namespace ThorB200 {

struct RowFusionContext {
    const PhysicalExpression& graph;
    const std::vector<NamedOutput>& outputs;
    const std::vector<std::vector<uint64_t>>& shape;
    const std::vector<RuntimeInputValue>& bound;  // by input slot
    int device_num;
    bool use_fast_math;
    RowProgramTuning tuning;
    bool unrounded_column_sums = false;
};

struct RowFusionMatch {
    std::string name;                                 // physical stage name, e.g. "row_program"
    std::string source;                               // generated CUDA source
    uint64_t launches = 1;
    std::vector<std::pair<uint32_t, bool>> produced;  // nodes the super-stage writes (node, is a requested output)
    std::vector<uint32_t> absorbed;                   // nodes that no longer need a stage of their own
    std::vector<std::string> scalar_names;            // per program input slot, "" for tensors
    std::shared_ptr<std::vector<float>> scalars;      // runtime scalar values by program input slot
    // Called once the produced tensors exist; returns the launch closure (no allocation inside it).
    std::function<std::function<void(void*)>(std::vector<Tensor>& node_tensor, std::vector<Tensor>& keep_alive, uint64_t& intermediate_bytes)> bind;
    // Device-side waits of the program that ran out of time so far (synchronises; 0 for programs without such waits).
    std::function<uint32_t()> waits_expired;
    // unrounded_column_sums: output names of the program's column reductions, and (after bind) the fp32 [names, cols] tensor
    std::vector<std::string> column_sum_names;
    std::shared_ptr<Tensor> column_sums;
};

// Tries to run the whole equation as one row program; returns no match when it does not fit.
std::vector<RowFusionMatch> matchRowFusions(const RowFusionContext& ctx);

}  // namespace ThorB200
