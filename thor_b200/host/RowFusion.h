// Physical fusion of "elementwise -> row reduction -> elementwise" chains into single-pass row
// kernels (softmax, LayerNorm forward / backward).  The reference never fuses across a reduction
// (EquationCompiler.cpp:684-688); this pass keeps its logical stage list and only replaces what
// launches.
#pragma once

#include <functional>
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
};

struct RowFusionMatch {
    std::string name;                                // physical stage name, e.g. "softmax_rows"
    uint64_t launches = 1;
    std::vector<std::pair<uint32_t, bool>> produced; // nodes the super-stage writes (node, is a requested output)
    std::vector<uint32_t> absorbed;                  // intermediate nodes that no longer need to exist
    // Called once the produced tensors exist; returns the launch closure (no allocation inside it).
    std::function<std::function<void(void*)>(std::vector<Tensor>& node_tensor, std::vector<Tensor>& keep_alive, uint64_t& intermediate_bytes)> bind;
};

std::vector<RowFusionMatch> matchRowFusions(const RowFusionContext& ctx);

}  // namespace ThorB200
