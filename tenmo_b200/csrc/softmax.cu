// Softmax over the last axis, forward and backward -- the step between the two GEMMs of an attention
// block (scores -> weights).  Restates SoftmaxNdBuffer.softmax (tenmo/softmax.mojo:30-48: exp(x - max)
// divided by its sum) and SoftmaxBackwardDelegate (tenmo/softmax.mojo:206-213: y * (g - sum(g*y))).
// One warp per row; a row of up to 1024 values is read once and kept in registers, so the algorithmic
// traffic (forward 8 B, backward 12 B per element) is the real traffic.  HBM-bound.
#include "common.cuh"

namespace {

constexpr int SM_THREADS = 256;
constexpr int SM_WARPS = SM_THREADS / 32;
constexpr int SM_REG = 32;

__global__ void __launch_bounds__(SM_THREADS)
softmax_fwd_kernel(const float* __restrict__ x, int64_t ldx, float* __restrict__ y, int64_t M, int64_t C) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool cached = C <= 32 * SM_REG;
    for (int64_t row = (int64_t)blockIdx.x * SM_WARPS + warp; row < M; row += (int64_t)gridDim.x * SM_WARPS) {
        const float* xr = x + row * ldx;
        float* yr = y + row * C;
        float v[SM_REG];
        float mx = -3.4028234663852886e38f;
        if (cached) {
#pragma unroll
            for (int i = 0; i < SM_REG; ++i) {
                const int64_t c = lane + 32 * i;
                v[i] = c < C ? __ldg(xr + c) : -3.4028234663852886e38f;
                mx = fmaxf(mx, v[i]);
            }
        } else {
            for (int64_t c = lane; c < C; c += 32) mx = fmaxf(mx, __ldg(xr + c));
        }
        mx = tenmo_warp_max(mx);
        float s = 0.f;
        if (cached) {
#pragma unroll
            for (int i = 0; i < SM_REG; ++i) {
                const int64_t c = lane + 32 * i;
                if (c < C) { v[i] = expf(v[i] - mx); s += v[i]; }
            }
        } else {
            for (int64_t c = lane; c < C; c += 32) s += expf(__ldg(xr + c) - mx);
        }
        s = tenmo_warp_sum(s);
        if (cached) {
#pragma unroll
            for (int i = 0; i < SM_REG; ++i) {
                const int64_t c = lane + 32 * i;
                if (c < C) yr[c] = v[i] / s;
            }
        } else {
            for (int64_t c = lane; c < C; c += 32) yr[c] = expf(__ldg(xr + c) - mx) / s;
        }
    }
}

__global__ void __launch_bounds__(SM_THREADS)
softmax_bwd_kernel(const float* __restrict__ y, const float* __restrict__ g, float* __restrict__ dx, float beta, int64_t M,
                   int64_t C) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool cached = C <= 32 * SM_REG;
    for (int64_t row = (int64_t)blockIdx.x * SM_WARPS + warp; row < M; row += (int64_t)gridDim.x * SM_WARPS) {
        const float* yr = y + row * C;
        const float* gr = g + row * C;
        float* dr = dx + row * C;
        float yv[SM_REG], gv[SM_REG];
        float dot = 0.f;
        if (cached) {
#pragma unroll
            for (int i = 0; i < SM_REG; ++i) {
                const int64_t c = lane + 32 * i;
                yv[i] = c < C ? __ldg(yr + c) : 0.f;
                gv[i] = c < C ? __ldg(gr + c) : 0.f;
                dot += __fmul_rn(gv[i], yv[i]);
            }
        } else {
            for (int64_t c = lane; c < C; c += 32) dot += __fmul_rn(__ldg(gr + c), __ldg(yr + c));
        }
        dot = tenmo_warp_sum(dot);
        if (cached) {
#pragma unroll
            for (int i = 0; i < SM_REG; ++i) {
                const int64_t c = lane + 32 * i;
                if (c < C) {
                    const float r = __fmul_rn(yv[i], gv[i] - dot);
                    dr[c] = beta != 0.f ? dr[c] + r : r;
                }
            }
        } else {
            for (int64_t c = lane; c < C; c += 32) {
                const float r = __fmul_rn(__ldg(yr + c), __ldg(gr + c) - dot);
                dr[c] = beta != 0.f ? dr[c] + r : r;
            }
        }
    }
}

}  // namespace

extern "C" {

int tenmo_softmax_fwd_f32(tenmo_ctx* ctx, const float* x, int64_t ldx, float* y, int64_t M, int64_t C) {
    TENMO_CHECK_CTX(ctx);
    if (M < 0 || C <= 0) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "softmax_fwd: bad shape");
    if (M == 0) return TENMO_OK;
    if (!x || !y) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "softmax_fwd: NULL pointer");
    if (ldx < C) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "softmax_fwd: ldx < C");
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const int grid = tenmo_stream_grid(ctx, M, SM_WARPS, 8);
    softmax_fwd_kernel<<<grid, SM_THREADS, 0, ctx->stream>>>(x, ldx, y, M, C);
    TENMO_LAUNCH_CHECK(ctx, "softmax_fwd_kernel");
    return TENMO_OK;
}

int tenmo_softmax_bwd_f32(tenmo_ctx* ctx, const float* y, const float* g, float* dx, float beta, int64_t M, int64_t C) {
    TENMO_CHECK_CTX(ctx);
    if (M < 0 || C <= 0) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "softmax_bwd: bad shape");
    if (beta != 0.f && beta != 1.f) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "softmax_bwd: beta must be 0 or 1");
    if (M == 0) return TENMO_OK;
    if (!y || !g || !dx) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "softmax_bwd: NULL pointer");
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const int grid = tenmo_stream_grid(ctx, M, SM_WARPS, 8);
    softmax_bwd_kernel<<<grid, SM_THREADS, 0, ctx->stream>>>(y, g, dx, beta, M, C);
    TENMO_LAUNCH_CHECK(ctx, "softmax_bwd_kernel");
    return TENMO_OK;
}

}  // extern "C"
