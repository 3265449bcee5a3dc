// Lane assignment for the stages of a stamped plan (the reference's detail::buildStampedExecutionSchedule,
// Utilities/Expression/StampedEquation.h:1634-1646; submission StampedEquation.cpp:4057-4205).  Lane 0 is the caller's
// stream; further lanes are helper streams for branches that can genuinely run beside it.  A pure function of the
// dependency lists, so the policy can be tested without a GPU.
#pragma once

#include <cstdint>
#include <vector>

namespace ThorB200 {

struct StampedExecutionSchedule {
    std::vector<uint32_t> stage_lane_indices;             // lane of every stage
    std::vector<uint32_t> lane_gpu_nums;                  // one entry per lane (all on the caller's GPU here)
    std::vector<bool> stage_has_downstream_dependency;    // some later stage consumes this stage
    std::vector<bool> stage_needs_completion_event;       // ... and runs on another lane: an event must be recorded behind it
    bool needs_caller_ready_event = false;                // a stage without dependencies runs on a helper lane
};

// dependencies[s] lists the stages whose results stage s consumes; every entry must be < s (stages are in a
// topological order), else std::runtime_error.  Policy: a stage continues the lane of a dependency that is still the last
// stage of its lane (the lowest such lane, so joins return to the caller's lane); otherwise -- a second consumer of a stage
// whose lane has moved on, or an independent root after the first -- it opens a new lane.
StampedExecutionSchedule buildStampedExecutionSchedule(const std::vector<std::vector<uint32_t>>& dependencies, uint32_t caller_gpu_num);

}  // namespace ThorB200
