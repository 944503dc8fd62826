// tcgen05 / TMEM 3xTF32 GEMM (see gemm_tc.cu).
#pragma once
#include <cuda.h>

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

// ---- operand planning for kernels that read their operands through tensor maps (shared with the TMA-staged
// strict-fp32 kernel) ----
typedef CUresult (*TenmoEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct TenmoOperandPlan {
    bool mn_major;        // unit-stride axis is m / n (not k)
    int64_t inner, outer; // extents of the storage matrix (inner = unit-stride axis)
    int64_t ld;           // elements between consecutive `outer` indices
    int batched;          // 1: one slice per batch with a uniform stride, 0: broadcast
    int64_t batch_stride; // elements
    int64_t batches;      // slices that exist in memory (1 when broadcast)
    int64_t ld_lo, bstride_lo;
};

// Collapse an operand's (possibly broadcast) batch dims into "one uniform stride" or "broadcast".
bool tenmo_collapse_batch(const TenmoBatch& b, const int64_t* stride, int64_t total, int* batched, int64_t* bstride);
// rows x cols view; k is the row index when rows_are_k (operand B) else the column index (operand A).  False (and a
// reason in `why`) when the view has no unit-stride axis, is not 16-byte aligned or its batch does not collapse.
bool tenmo_plan_operand(int64_t rows, int64_t cols, int64_t rs, int64_t cs, bool rows_are_k, const float* ptr,
                        const TenmoBatch& b, const int64_t* bstrides, int64_t total_batch, TenmoOperandPlan* o,
                        const char* name, char* why, size_t why_len);
bool tenmo_make_plan(const TenmoGemmParams& p, TenmoOperandPlan* a, TenmoOperandPlan* b, char* why, size_t why_len);
// Fetches cuTensorMapEncodeTiled from the driver once per context (ctx->encode_tiled).
int tenmo_tma_init(tenmo_ctx* ctx);
