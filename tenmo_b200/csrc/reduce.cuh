// Column-sum kernels shared between entry points (see reduce.cu).
#pragma once
#include "common.cuh"

// Up to this many rows the column sum runs one thread per column in ascending row order
// (bit-identical to the reference's sequential CPU reduction).
#define TENMO_COLSUM_SEQ_ROWS 512

void tenmo_colsum_plan(int sm_count, int64_t M, int64_t N, bool vec, int* strips, int* slabs, int* rows_per_slab);
int tenmo_colsum_launch(tenmo_ctx* ctx, const float* x, int64_t M, int64_t N, int64_t ldx, float* out, float beta,
                        float* partials, unsigned int* tickets, int strips, int slabs, int rows_per_slab, bool vec);
int tenmo_colsum_scratch(tenmo_ctx* ctx, int slabs, int64_t N, int strips, float** partials, unsigned int** tickets);
