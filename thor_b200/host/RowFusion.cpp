#include "RowFusion.h"

namespace ThorB200 {

std::vector<RowFusionMatch> matchRowFusions(const RowFusionContext&) { return {}; }

}  // namespace ThorB200
