// placeholder until the tcgen05 kernel lands
#include "common.cuh"
namespace wb {
bool gemm_tc_supports(const Weight &, int64_t) { return false; }
int plan_gemm_tc(wb_context *, const Weight &, int64_t, int, int, wb_plan *) { return fail(WB_ERR_UNSUPPORTED, "no tc"); }
int launch_gemm_tc(wb_context *, const Weight &, const void *, void *, const float *, int64_t, int, int, int, const wb_plan &) { return fail(WB_ERR_UNSUPPORTED, "no tc"); }
}
