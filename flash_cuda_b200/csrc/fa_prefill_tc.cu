// placeholder until the tcgen05 prefill kernel lands
#include "fa_internal.h"
#include "fa_sched.h"
namespace fa {
bool prefill_tc_supported(const PlanInput&) { return false; }
int launch_prefill_tc(const KParams&, const Plan&, int, cudaStream_t) { return -1; }
}  // namespace fa
