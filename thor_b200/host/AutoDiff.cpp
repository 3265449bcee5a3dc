#include "AutoDiff.h"

#include <stdexcept>

namespace ThorB200 {

Outputs buildBackwardOutputs(const Outputs&, const std::vector<std::string>&, const std::string&,
                             const std::unordered_map<std::string, std::vector<uint64_t>>&) {
    throw std::logic_error("buildBackwardOutputs: not built yet");
}

}  // namespace ThorB200
