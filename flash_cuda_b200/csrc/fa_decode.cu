// placeholder until the paged-decode kernel lands
#include "fa_internal.h"
#include "fa_sched.h"
namespace fa {
bool decode_supported(const PlanInput&) { return false; }
int launch_decode(const KParams&, const Plan&, int, cudaStream_t) { return -1; }
}  // namespace fa
