// placeholder until the tcgen05 kernel lands
#include "gemm_tc.cuh"
bool tenmo_gemm_tc_supported(tenmo_ctx*, const TenmoGemmParams&, char* why, size_t n) { snprintf(why, n, "not built"); return false; }
bool tenmo_gemm_tc_profitable(tenmo_ctx*, const TenmoGemmParams&) { return false; }
int tenmo_gemm_tc_launch(tenmo_ctx* ctx, const TenmoGemmParams&) { return tenmo_set_error(ctx, TENMO_ERR_UNSUPPORTED, "not built"); }
