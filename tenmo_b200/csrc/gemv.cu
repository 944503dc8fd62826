// Matrix @ vector and vector @ matrix:  y[i] = sum_k A[i,k] x[k]   and   y[j] = sum_k x[k] A[k,j].
//
// Replaces MatrixVectorMulNd.forward (matrixvector.mojo:205-285) and VectorMatmulNd.forward (vectormatrix.mojo:210-340),
// which walk every output's k range with one scalar accumulator.  Both products read the matrix once and do two flops
// per element, so they are HBM-bound (4*M*K bytes); which kernel runs depends only on which axis of the matrix is
// contiguous in memory:
//   * the REDUCED axis is contiguous (row-major A in A.x, column-major A in x.A): a warp per output, lanes stride the
//     row with 16-byte loads (four in flight per lane), shuffle reduction at the end;
//   * the OUTPUT axis is contiguous (row-major A in x.A, column-major A in A.x): the weighted form of the split column
//     sum -- row slabs x 128-column strips, coalesced 16-byte loads, per-slab partials in scratch, the last CTA of a
//     strip (ticket) adds the partials in slab order, so the result does not depend on scheduling.
// Neither form adds in the reference's k-ascending order (a lane or a slab holds a strided subset of k), so results
// agree with the reference to rounding (about 1e-7 of sum |a||x|), not bit for bit; the GEMM with a unit dimension
// (tenmo_gemm_f32, strict-fp32 algorithm) is the bit-identical form and serves matrices without a unit-stride axis.
#include "common.cuh"
#include "reduce.cuh"

namespace {

constexpr int GV_THREADS = 256;
constexpr int GV_WARPS = GV_THREADS / 32;

// y[r] = sum_c A[r*ld + c] * x[c*incx]   (VEC = 4: 16-byte loads of A, and of x when incx == 1)
template <int VEC>
__global__ void __launch_bounds__(GV_THREADS) gemv_rowdot_kernel(const float* __restrict__ A, int64_t ld, const float* __restrict__ x,
                                                                int64_t incx, float* __restrict__ y, int64_t R, int64_t Cn,
                                                                float beta) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int64_t r = (int64_t)blockIdx.x * GV_WARPS + warp; r < R; r += (int64_t)gridDim.x * GV_WARPS) {
        const float* __restrict__ row = A + r * ld;
        float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
        int64_t c = 0;
        if (VEC == 4) {
            const int64_t vend = Cn & ~(int64_t)3;
            // four 16-byte loads per lane in flight: 2 KB per warp per step
            for (c = (int64_t)lane * 4; c + 3 * 128 < vend; c += 4 * 128) {
                float4 a[4], b[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) a[u] = __ldcs(reinterpret_cast<const float4*>(row + c + u * 128));
#pragma unroll
                for (int u = 0; u < 4; ++u) b[u] = __ldg(reinterpret_cast<const float4*>(x + c + u * 128));
                acc0 += a[0].x * b[0].x + a[0].y * b[0].y + a[0].z * b[0].z + a[0].w * b[0].w;
                acc1 += a[1].x * b[1].x + a[1].y * b[1].y + a[1].z * b[1].z + a[1].w * b[1].w;
                acc2 += a[2].x * b[2].x + a[2].y * b[2].y + a[2].z * b[2].z + a[2].w * b[2].w;
                acc3 += a[3].x * b[3].x + a[3].y * b[3].y + a[3].z * b[3].z + a[3].w * b[3].w;
            }
            for (; c < vend; c += 128) {
                const float4 a = __ldcs(reinterpret_cast<const float4*>(row + c));
                const float4 b = __ldg(reinterpret_cast<const float4*>(x + c));
                acc0 += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
            }
            c = vend + lane;  // ragged tail of at most three columns
            if (c < Cn) acc1 += __ldg(row + c) * __ldg(x + c);
        } else {
            for (c = lane; c < Cn; c += 32) acc0 += __ldg(row + c) * __ldg(x + c * incx);
        }
        const float s = tenmo_warp_sum((acc0 + acc1) + (acc2 + acc3));
        if (lane == 0) y[r] = beta != 0.f ? y[r] + s : s;
    }
}

// y[n] = sum_m w[m*incw] * X[m*ld + n]: the split column sum with a weight per row.
template <int VEC>
__global__ void __launch_bounds__(GV_THREADS)
gemv_colacc_kernel(const float* __restrict__ X, int64_t M, int64_t N, int64_t ld, const float* __restrict__ w, int64_t incw,
                   float* __restrict__ y, float beta, float* __restrict__ partials, unsigned int* __restrict__ tickets,
                   int rows_per_slab) {
    constexpr int STRIP = 32 * VEC;
    __shared__ float red[GV_WARPS][STRIP];
    __shared__ bool is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int strip = blockIdx.x, slab = blockIdx.y, slabs = gridDim.y;
    const int64_t n0 = (int64_t)strip * STRIP + lane * VEC;
    const int64_t m_begin = (int64_t)slab * rows_per_slab;
    const int64_t m_end = min(m_begin + (int64_t)rows_per_slab, M);
    float acc[VEC];
#pragma unroll
    for (int q = 0; q < VEC; ++q) acc[q] = 0.f;
    if (n0 < N) {
        int64_t m = m_begin + warp;
        for (; m + 3 * GV_WARPS < m_end; m += 4 * GV_WARPS) {  // four rows in flight per warp
            float wv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) wv[u] = __ldg(w + (m + u * GV_WARPS) * incw);
            if (VEC == 4) {
                float4 a[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) a[u] = __ldcs(reinterpret_cast<const float4*>(X + (m + u * GV_WARPS) * ld + n0));
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    acc[0] += wv[u] * a[u].x; acc[1 % VEC] += wv[u] * a[u].y;
                    acc[2 % VEC] += wv[u] * a[u].z; acc[3 % VEC] += wv[u] * a[u].w;
                }
            } else {
#pragma unroll
                for (int u = 0; u < 4; ++u) acc[0] += wv[u] * __ldg(X + (m + u * GV_WARPS) * ld + n0);
            }
        }
        for (; m < m_end; m += GV_WARPS) {
            const float wm = __ldg(w + m * incw);
            if (VEC == 4) {
                const float4 a = __ldcs(reinterpret_cast<const float4*>(X + m * ld + n0));
                acc[0] += wm * a.x; acc[1 % VEC] += wm * a.y; acc[2 % VEC] += wm * a.z; acc[3 % VEC] += wm * a.w;
            } else {
                acc[0] += wm * __ldg(X + m * ld + n0);
            }
        }
    }
#pragma unroll
    for (int q = 0; q < VEC; ++q) red[warp][lane * VEC + q] = acc[q];
    __syncthreads();
    if (threadIdx.x < STRIP) {
        float s = 0.f;
#pragma unroll
        for (int wi = 0; wi < GV_WARPS; ++wi) s += red[wi][threadIdx.x];
        const int64_t n = (int64_t)strip * STRIP + threadIdx.x;
        if (n < N) partials[(int64_t)slab * N + n] = s;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(&tickets[strip], 1u) == (unsigned int)slabs - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (threadIdx.x < STRIP) {
        const int64_t n = (int64_t)strip * STRIP + threadIdx.x;
        if (n < N) {
            float s = 0.f;
            for (int sl = 0; sl < slabs; ++sl) s += __ldcg(partials + (int64_t)sl * N + n);
            y[n] = beta != 0.f ? y[n] + s : s;
        }
    }
    if (threadIdx.x == 0) tickets[strip] = 0;  // ready for the next call
}

// out[o] = sum_r vec[r*inc] * Mtx[o*out_stride + r*red_stride], o < n_out, r < n_red
int gemv_dispatch(tenmo_ctx* ctx, const char* who, const float* Mtx, int64_t n_out, int64_t n_red, int64_t out_stride,
                  int64_t red_stride, const float* vec, int64_t inc, float* y, float beta) {
    if (n_out == 0) return TENMO_OK;
    if (n_red == 0) {
        if (beta == 0.f) TENMO_CUDA_TRY(ctx, cudaMemsetAsync(y, 0, (size_t)n_out * sizeof(float), ctx->stream));
        return TENMO_OK;
    }
    const bool base16 = (reinterpret_cast<uintptr_t>(Mtx) & 15u) == 0;
    if (red_stride == 1 || n_red == 1) {
        const bool v4 = base16 && inc == 1 && out_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(vec) & 15u) == 0 && n_red >= 4;
        const int64_t want = (n_out + GV_WARPS - 1) / GV_WARPS, cap = (int64_t)ctx->sm_count * 8;
        const unsigned grid = (unsigned)(want < cap ? want : cap);
        if (v4) gemv_rowdot_kernel<4><<<grid, GV_THREADS, 0, ctx->stream>>>(Mtx, out_stride, vec, inc, y, n_out, n_red, beta);
        else gemv_rowdot_kernel<1><<<grid, GV_THREADS, 0, ctx->stream>>>(Mtx, out_stride, vec, inc, y, n_out, n_red, beta);
        TENMO_LAUNCH_CHECK(ctx, "gemv_rowdot_kernel");
        return TENMO_OK;
    }
    if (out_stride == 1 || n_out == 1) {
        const bool v4 = base16 && n_out % 4 == 0 && red_stride % 4 == 0;
        int strips, slabs, rps;
        tenmo_colsum_plan(ctx->sm_count, n_red, n_out, v4, &strips, &slabs, &rps);
        float* partials = nullptr;
        unsigned int* tickets = nullptr;
        int st = tenmo_colsum_scratch(ctx, slabs, n_out, strips, &partials, &tickets);
        if (st != TENMO_OK) return st;
        dim3 grid((unsigned)strips, (unsigned)slabs);
        if (v4) gemv_colacc_kernel<4><<<grid, GV_THREADS, 0, ctx->stream>>>(Mtx, n_red, n_out, red_stride, vec, inc, y, beta, partials, tickets, rps);
        else gemv_colacc_kernel<1><<<grid, GV_THREADS, 0, ctx->stream>>>(Mtx, n_red, n_out, red_stride, vec, inc, y, beta, partials, tickets, rps);
        TENMO_LAUNCH_CHECK(ctx, "gemv_colacc_kernel");
        return TENMO_OK;
    }
    return tenmo_set_error(ctx, TENMO_ERR_UNSUPPORTED,
                           "%s: the matrix has no unit-stride axis (strides %lld, %lld); use tenmo_gemm_f32 with a unit dimension",
                           who, (long long)out_stride, (long long)red_stride);
}

int gemv_check(tenmo_ctx* ctx, const char* who, int64_t a, int64_t b, const tenmo_mat* A, const float* x, int64_t incx,
               const float* y, float beta) {
    if (a < 0 || b < 0) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "%s: negative shape", who);
    if (!A || (a > 0 && b > 0 && !A->ptr) || (b > 0 && !x) || (a > 0 && !y)) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "%s: NULL pointer", who);
    if (A->batch_rank != 0) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "%s: one matrix per call (batch_rank must be 0)", who);
    if (incx < 1) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "%s: the vector's stride must be >= 1", who);
    if (A->row_stride < 0 || A->col_stride < 0) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "%s: negative matrix stride", who);
    if (beta != 0.f && beta != 1.f) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "%s: beta must be 0 or 1", who);
    return TENMO_OK;
}

}  // namespace

extern "C" int tenmo_gemv_f32(tenmo_ctx* ctx, int64_t M, int64_t K, const tenmo_mat* A, const float* x, int64_t incx, float* y,
                              float beta) {
    TENMO_CHECK_CTX(ctx);
    int st = gemv_check(ctx, "gemv", M, K, A, x, incx, y, beta);
    if (st != TENMO_OK) return st;
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return gemv_dispatch(ctx, "gemv", A->ptr + A->offset, M, K, A->row_stride, A->col_stride, x, incx, y, beta);
}

extern "C" int tenmo_vecmat_f32(tenmo_ctx* ctx, int64_t K, int64_t N, const float* x, int64_t incx, const tenmo_mat* A, float* y,
                                float beta) {
    TENMO_CHECK_CTX(ctx);
    int st = gemv_check(ctx, "vecmat", N, K, A, x, incx, y, beta);
    if (st != TENMO_OK) return st;
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return gemv_dispatch(ctx, "vecmat", A->ptr + A->offset, N, K, A->col_stride, A->row_stride, x, incx, y, beta);
}
