#include "Schedule.h"

#include <limits>
#include <stdexcept>
#include <string>

namespace ThorB200 {

StampedExecutionSchedule buildStampedExecutionSchedule(const std::vector<std::vector<uint32_t>>& dependencies, uint32_t caller_gpu_num) {
    const uint32_t n = static_cast<uint32_t>(dependencies.size());
    StampedExecutionSchedule s;
    s.stage_lane_indices.assign(n, 0);
    s.stage_has_downstream_dependency.assign(n, false);
    s.stage_needs_completion_event.assign(n, false);
    constexpr uint32_t kNone = std::numeric_limits<uint32_t>::max();
    std::vector<uint32_t> lane_tail;  // last stage placed on each lane
    bool caller_lane_started = false;
    for (uint32_t stage = 0; stage < n; ++stage) {
        uint32_t lane = kNone;
        for (uint32_t dep : dependencies[stage]) {
            if (dep >= stage) throw std::runtime_error("stamped execution stage " + std::to_string(stage) + " depends on stage " + std::to_string(dep) + ", which does not precede it");
            s.stage_has_downstream_dependency[dep] = true;
            const uint32_t dep_lane = s.stage_lane_indices[dep];
            if (lane_tail[dep_lane] == dep && (lane == kNone || dep_lane < lane)) lane = dep_lane;
        }
        if (lane == kNone) {
            if (dependencies[stage].empty() && !caller_lane_started) {
                lane = 0;  // the first root starts the caller's lane
                if (lane_tail.empty()) lane_tail.push_back(kNone);
            } else {
                lane = static_cast<uint32_t>(lane_tail.size());
                if (lane == 0) {  // a dependent stage cannot come first, but keep lane 0 for the caller
                    lane_tail.push_back(kNone);
                    lane = 0;
                } else {
                    lane_tail.push_back(kNone);
                }
                if (dependencies[stage].empty()) s.needs_caller_ready_event = true;
            }
        }
        if (lane == 0) caller_lane_started = true;
        s.stage_lane_indices[stage] = lane;
        lane_tail[lane] = stage;
        for (uint32_t dep : dependencies[stage])
            if (s.stage_lane_indices[dep] != lane) s.stage_needs_completion_event[dep] = true;
    }
    s.lane_gpu_nums.assign(lane_tail.empty() ? 1 : lane_tail.size(), caller_gpu_num);
    return s;
}

}  // namespace ThorB200
