// Strict-FP32 SIMT GEMM: every output element is ONE k-ascending fmaf chain, which makes it
// bit-identical to tenmo's CPU paths 1a/1b (matmul_cpu.mojo:275-312: acc = fma(a_ik, b_kj, acc) for
// k ascending, partial sums parked exactly in C between k tiles).  Operands are arbitrary strided
// views (transposed views included) with NumPy-style broadcast batching decoded in the kernel, so
// nothing is materialised and no per-call offset table is uploaded (the reference uploads one per
// call, kernels/matmul_kernel.mojo:187-239).
#pragma once
#include "common.cuh"

struct TenmoBatch {
    int rank;
    int64_t shape[TENMO_MAX_BATCH_RANK];     // broadcast batch shape
    int64_t a_stride[TENMO_MAX_BATCH_RANK];  // 0 where A's dim is 1 or absent
    int64_t b_stride[TENMO_MAX_BATCH_RANK];
};

struct TenmoGemmParams {
    const float* A;  // already advanced by the view offset
    const float* B;
    float* C;
    int64_t M, N, K;
    int64_t a_rs, a_cs, b_rs, b_cs;
    int a_vec, b_vec;  // 16-byte vector loads legal along the operand's unit-stride axis
    int c_vec;         // float4 stores legal on C / aux
    float beta;
    const float* bias;
    int act;
    float* aux;
    // extended options (tenmo_gemm_f32_ex)
    const float* a_lo;      // precomputed lo planes of the operands' storage (tensor-core kernel only), or NULL
    const float* b_lo;
    float* c_lo;            // optional: lo plane of the stored result, row-major with leading dimension ld_clo
    int64_t ld_clo;
    const float* mul_mask;  // optional (total_batch, M, N): result is multiplied by it before beta / store
    const float* bias_m;    // optional M floats: per-row bias (the per-channel bias of a convolution)
    float* colsum;          // optional N floats: column sums of B over k, k ascending (the bias gradient riding along with
                            // dW = X^T . dY); honoured by the 64 / 32 tiles of the register-staged kernel only, see colsum_done
    size_t ws_skip;         // bytes at the start of the context workspace that belong to the caller (split-K partials)
    int tiles_m, tiles_n;
    int64_t total_batch;
    TenmoBatch batch;
};

// Picks the tile shape; large problems whose operands can be described by tensor maps (a unit-stride axis,
// 16-byte aligned base and leading stride, batch dims that collapse to one stride) go to the TMA-staged
// kernel of gemm_simt_tma.cu, everything else to the register-staged kernels of gemm_simt.cu.  Both give the
// same bits.
// *colsum_done (may be NULL) tells whether the kernel also wrote p.colsum; if not, the caller runs the column sum.
int tenmo_gemm_simt_launch(tenmo_ctx* ctx, const TenmoGemmParams& p, bool* colsum_done = nullptr);
bool tenmo_gemm_simt_tma_supported(tenmo_ctx* ctx, const TenmoGemmParams& p);
int tenmo_gemm_simt_tma_launch(tenmo_ctx* ctx, const TenmoGemmParams& p);
// Narrow results (N <= 32) over a long contraction (K >= 512), one matrix: gemm_skinny.cu, same bits.
bool tenmo_gemm_skinny_supported(const TenmoGemmParams& p);
int tenmo_gemm_skinny_launch(tenmo_ctx* ctx, const TenmoGemmParams& p);
