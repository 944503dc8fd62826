// tcgen05 / TMEM 3xTF32 GEMM (see gemm_tc.cu).
#pragma once
#include "gemm_simt.cuh"

// True when the tensor-core kernel can serve the call; otherwise `why` says what rules it out.
bool tenmo_gemm_tc_supported(tenmo_ctx* ctx, const TenmoGemmParams& p, char* why, size_t why_len);
// Heuristic used by TENMO_ALGO_AUTO: is the problem large enough for the tensor-core kernel to win?
bool tenmo_gemm_tc_profitable(tenmo_ctx* ctx, const TenmoGemmParams& p);
int tenmo_gemm_tc_launch(tenmo_ctx* ctx, const TenmoGemmParams& p);
// lo plane of a strided (possibly batched) matrix, written compactly in the order of its storage
// (outer x inner rounded up to 4, batches back to back); floats_written receives the output length.
int tenmo_split_lo_launch(tenmo_ctx* ctx, const float* base, int64_t rows, int64_t cols, int64_t rs, int64_t cs,
                          const TenmoBatch& batch, const int64_t* bstrides, int64_t total_batch, float* out,
                          int64_t* floats_written);
