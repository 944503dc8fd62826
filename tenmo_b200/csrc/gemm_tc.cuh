// tcgen05 / TMEM 3xTF32 GEMM (see gemm_tc.cu).
#pragma once
#include "gemm_simt.cuh"

// True when the tensor-core kernel can serve the call; otherwise `why` says what rules it out.
bool tenmo_gemm_tc_supported(tenmo_ctx* ctx, const TenmoGemmParams& p, char* why, size_t why_len);
// Heuristic used by TENMO_ALGO_AUTO: is the problem large enough for the tensor-core kernel to win?
bool tenmo_gemm_tc_profitable(tenmo_ctx* ctx, const TenmoGemmParams& p);
int tenmo_gemm_tc_launch(tenmo_ctx* ctx, const TenmoGemmParams& p);
