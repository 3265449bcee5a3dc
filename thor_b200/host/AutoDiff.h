// Reverse-mode graph transform over the Expression DAG (the reference's AutoDiff.h:16-63 /
// AutoDiff.cpp:3690-5930 restricted to the ops of this host layer).
#pragma once

#include <string>
#include <unordered_map>
#include <vector>

#include "Expression.h"

namespace ThorB200 {

// Builds outputs "<wrt>_grad" for each name in wrt_names.  The upstream gradient of forward output
// `o` is the tensor input "<upstream_prefix>" (single forward output) or "<upstream_prefix>_<o>".
// Forward sub-expressions are recomputed inside the backward graph (builder.cloneForward in the
// reference); broadcast operands are un-broadcast with reduce_sum + squeeze (sumToShape,
// AutoDiff.cpp:3403-3560), which needs the concrete forward input shapes.
// Each gradient is written in the dtype of the input it belongs to (the reference forces the terminal
// gradient node to preferredGradValueDType of the forward input, AutoDiff.cpp:5880-5915); internal
// compute keeps its promoted dtypes.
Outputs buildBackwardOutputs(const Outputs& forward, const std::vector<std::string>& wrt_names, const std::string& upstream_prefix,
                             const std::unordered_map<std::string, std::vector<uint64_t>>& input_dims,
                             const std::unordered_map<std::string, DataType>& input_dtypes);

}  // namespace ThorB200
