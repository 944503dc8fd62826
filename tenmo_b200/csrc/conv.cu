// Convolution as GEMM and max pooling, NCHW (the CIFAR-shaped CNN of the reference's examples).
//
// tenmo's Conv2d forward is a direct convolution over a pre-padded image (cnn.mojo:404-507: the
// accumulator starts at the bias and adds img * kernel over (c_in, ky, kx) ascending), its kernel gradient
// is an explicit im2col followed by a matmul (cnn.mojo:716-809), its input gradient a scatter
// (cnn.mojo:812-950) and its bias gradient a per-channel sum (cnn.mojo:664-714).  Here every one of them
// is a GEMM of this library around four bandwidth-bound helpers:
//   im2col        patches[(n, oy, ox), (c, ky, kx)] = x[n, c, oy*s - p + ky*d, ox*s - p + kx*d]  (0 outside)
//   col2im        the adjoint gather: dx[n, c, y, x] = sum of the patch-gradient entries that read it
//   channel_sum   db[c] = sum over (n, y, x) of g[n, c, y, x]  (per-slab partial sums, then the slabs in order)
//   maxpool fwd / bwd   first-max-wins with an int64 argmax per output (pooling.mojo:301-402, 25-107)
// The k index of a patch runs (c, ky, kx), the layout of the (C_out, C_in, KH, KW) kernel tensor, so the
// weight matrix is the kernel tensor itself viewed as (C_out, C_in*KH*KW).
// Roofline: HBM.  im2col writes 4*N*Ho*Wo*C*KH*KW bytes (and reads the image once through L2); col2im reads
// as much; pooling reads 4 B and writes 4/k^2 + 8/k^2 B per input element.
#include "common.cuh"

namespace {

constexpr int CV_THREADS = 256;

struct ConvGeom {
    int64_t N, C, H, W;
    int KH, KW, stride, dil, pad;
    int64_t Ho, Wo;
};

// Division by a runtime constant as multiply + shift (n < 2^31, 1 <= d < 2^31): q = (n * M) >> k with
// k = 31 + ceil(log2 d), M = ceil(2^k / d) < 2^32.  The element index of these kernels is decoded with several
// divisions per element; as plain 64-bit divisions they, not the memory system, set the kernels' speed.
struct FastDiv {
    uint32_t d, M;
    int k;
    __device__ __forceinline__ uint32_t div(uint32_t n) const { return (uint32_t)(((uint64_t)n * M) >> k); }
    __device__ __forceinline__ void divmod(uint32_t n, uint32_t* q, uint32_t* r) const {
        *q = div(n);
        *r = n - *q * d;
    }
};

FastDiv make_fastdiv(int64_t d64) {
    FastDiv f;
    const uint32_t d = (uint32_t)d64;
    int l = 0;
    while ((1ull << l) < d) ++l;
    f.d = d;
    f.k = 31 + l;
    f.M = (uint32_t)(((1ull << f.k) + d - 1) / d);
    return f;
}

struct Im2colDivs {
    FastDiv K, KW, KH, Wo, Ho;
};

// One thread per patch element, consecutive threads along (c, ky, kx): the writes are fully coalesced, the reads
// gather from an image row that the neighbouring threads share.  SMALL: every index fits 31 bits.
template <bool SMALL>
__global__ void __launch_bounds__(CV_THREADS) im2col_kernel(const float* __restrict__ x, float* __restrict__ patches,
                                                            const ConvGeom g, const Im2colDivs dv) {
    const int64_t K = g.C * g.KH * g.KW;
    const int64_t total = g.N * g.Ho * g.Wo * K;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t n, c;
        int kx, ky;
        int64_t ox, oy;
        if (SMALL) {
            uint32_t pos, k, t, ukx, uky, uc, uox, uoy, un;
            dv.K.divmod((uint32_t)i, &pos, &k);
            dv.KW.divmod(k, &t, &ukx);
            dv.KH.divmod(t, &uc, &uky);
            dv.Wo.divmod(pos, &t, &uox);
            dv.Ho.divmod(t, &un, &uoy);
            n = un; c = uc; kx = (int)ukx; ky = (int)uky; ox = uox; oy = uoy;
        } else {
            const int64_t k = i % K, pos = i / K;
            kx = (int)(k % g.KW);
            ky = (int)((k / g.KW) % g.KH);
            c = k / (g.KW * g.KH);
            ox = pos % g.Wo;
            oy = (pos / g.Wo) % g.Ho;
            n = pos / (g.Wo * g.Ho);
        }
        const int64_t y = oy * g.stride - g.pad + (int64_t)ky * g.dil, xx = ox * g.stride - g.pad + (int64_t)kx * g.dil;
        float v = 0.f;
        if (y >= 0 && y < g.H && xx >= 0 && xx < g.W) v = __ldg(x + ((n * g.C + c) * g.H + y) * g.W + xx);
        patches[i] = v;
    }
}

struct Col2imDivs {
    FastDiv C, W, H;
};

// Gather form of the scatter in cnn.mojo:812-950: no atomics, every dx element is written once, its taps added in
// (ky, kx) order.  Threads run along the channel first: the taps of neighbouring channels lie KH*KW floats apart in
// a patch row, so a warp's reads fall into a few cache lines that its nine taps then use up completely (threads
// along x would touch one 4-byte word per K-float patch row).
template <bool SMALL>
__global__ void __launch_bounds__(CV_THREADS) col2im_kernel(const float* __restrict__ dpatches, float* __restrict__ dx,
                                                            const ConvGeom g, float beta, const Col2imDivs dv) {
    const int64_t K = g.C * g.KH * g.KW;
    const int64_t total = g.N * g.C * g.H * g.W;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t c, xx, y, n;  // i = ((n * H + y) * W + xx) * C + c
        if (SMALL) {
            uint32_t t, uc, ux, uy, un;
            dv.C.divmod((uint32_t)i, &t, &uc);
            dv.W.divmod(t, &t, &ux);
            dv.H.divmod(t, &un, &uy);
            c = uc; xx = ux; y = uy; n = un;
        } else {
            c = i % g.C;
            xx = (i / g.C) % g.W;
            y = (i / (g.C * g.W)) % g.H;
            n = i / (g.C * g.W * g.H);
        }
        float acc = 0.f;
        for (int ky = 0; ky < g.KH; ++ky) {
            const int64_t ty = y + g.pad - (int64_t)ky * g.dil;
            if (ty < 0) continue;
            int64_t oy = ty;
            if (g.stride != 1) {
                if (ty % g.stride != 0) continue;
                oy = ty / g.stride;
            }
            if (oy >= g.Ho) continue;
            for (int kx = 0; kx < g.KW; ++kx) {
                const int64_t tx = xx + g.pad - (int64_t)kx * g.dil;
                if (tx < 0) continue;
                int64_t ox = tx;
                if (g.stride != 1) {
                    if (tx % g.stride != 0) continue;
                    ox = tx / g.stride;
                }
                if (ox >= g.Wo) continue;
                acc += __ldg(dpatches + ((n * g.Ho + oy) * g.Wo + ox) * K + (c * g.KH + ky) * g.KW + kx);
            }
        }
        float* dst = dx + ((n * g.C + c) * g.H + y) * g.W + xx;
        *dst = beta != 0.f ? *dst + acc : acc;
    }
}

// Per-channel sum of g (N, C, S) in two steps with a fixed shape, so the result does not depend on scheduling:
// CTA (c, slab) adds the images of its slab (16-byte reads along S), then one thread per channel adds the slabs
// in order.
template <int VEC>
__global__ void __launch_bounds__(CV_THREADS) channel_sum_partial_kernel(const float* __restrict__ g, int64_t N, int64_t C,
                                                                         int64_t S, int imgs_per_slab,
                                                                         float* __restrict__ partials) {
    __shared__ float red[CV_THREADS / 32];
    const int64_t c = blockIdx.x;
    const int slab = blockIdx.y, slabs = gridDim.y;
    const int64_t n_begin = (int64_t)slab * imgs_per_slab;
    const int64_t n_end = min(n_begin + (int64_t)imgs_per_slab, N);
    float acc = 0.f;
    const int64_t per_img = S / VEC;
    for (int64_t n = n_begin; n < n_end; ++n) {
        const float* row = g + (n * C + c) * S;
        for (int64_t q = threadIdx.x; q < per_img; q += CV_THREADS) {
            if (VEC == 4) {
                const float4 v = __ldg(reinterpret_cast<const float4*>(row) + q);
                acc += (v.x + v.y) + (v.z + v.w);
            } else {
                acc += __ldg(row + q);
            }
        }
    }
    acc = tenmo_warp_sum(acc);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < CV_THREADS / 32; ++w) t += red[w];
        partials[c * slabs + slab] = t;
    }
}

__global__ void channel_sum_final_kernel(const float* __restrict__ partials, int64_t C, int slabs, float* __restrict__ out,
                                         float beta) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float t = 0.f;
    for (int s = 0; s < slabs; ++s) t += partials[c * slabs + s];
    out[c] = beta != 0.f ? out[c] + t : t;
}

__global__ void __launch_bounds__(CV_THREADS)
maxpool_fwd_kernel(const float* __restrict__ x, float* __restrict__ out, long long* __restrict__ argmax, int64_t NC, int64_t H,
                   int64_t W, int64_t Ho, int64_t Wo, int k, int stride, int pad) {
    const int64_t total = NC * Ho * Wo;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t ox = i % Wo, oy = (i / Wo) % Ho, nc = i / (Wo * Ho);
        const float* plane = x + nc * H * W;
        float best = -INFINITY;
        long long idx = -1;
        for (int ky = 0; ky < k; ++ky) {  // window walked row by row: the first maximum wins (strict >)
            const int64_t y = oy * stride - pad + ky;
            if (y < 0 || y >= H) continue;
            for (int kx = 0; kx < k; ++kx) {
                const int64_t xx = ox * stride - pad + kx;
                if (xx < 0 || xx >= W) continue;
                const float v = __ldg(plane + y * W + xx);
                if (v > best) { best = v; idx = y * W + xx; }
            }
        }
        out[i] = best;
        argmax[i] = idx;
    }
}

__global__ void __launch_bounds__(CV_THREADS)
maxpool_bwd_kernel(const float* __restrict__ g, const long long* __restrict__ argmax, float* __restrict__ dx, int64_t NC,
                   int64_t HW, int64_t HoWo) {
    const int64_t total = NC * HoWo;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const long long idx = argmax[i];
        if (idx >= 0) atomicAdd(dx + (i / HoWo) * HW + idx, __ldg(g + i));
    }
}

int check_geom(tenmo_ctx* ctx, const char* who, int64_t N, int64_t C, int64_t H, int64_t W, int KH, int KW, int stride, int dil,
               int pad, ConvGeom* g) {
    if (N < 0 || C <= 0 || H <= 0 || W <= 0 || KH <= 0 || KW <= 0 || stride <= 0 || dil <= 0 || pad < 0)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "%s: bad geometry", who);
    const int64_t eh = (int64_t)(KH - 1) * dil + 1, ew = (int64_t)(KW - 1) * dil + 1;
    if (H + 2 * pad < eh || W + 2 * pad < ew)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "%s: kernel (%d x %d, dilation %d) larger than the padded image", who, KH,
                               KW, dil);
    g->N = N; g->C = C; g->H = H; g->W = W;
    g->KH = KH; g->KW = KW; g->stride = stride; g->dil = dil; g->pad = pad;
    g->Ho = (H + 2 * pad - eh) / stride + 1;
    g->Wo = (W + 2 * pad - ew) / stride + 1;
    return TENMO_OK;
}

}  // namespace

extern "C" {

int tenmo_conv_out_size(int64_t in, int k, int stride, int dilation, int pad, int64_t* out) {
    const int64_t e = (int64_t)(k - 1) * dilation + 1;
    if (k <= 0 || stride <= 0 || dilation <= 0 || pad < 0 || in + 2 * pad < e || !out) return TENMO_ERR_INVALID;
    *out = (in + 2 * pad - e) / stride + 1;
    return TENMO_OK;
}

int tenmo_im2col_f32(tenmo_ctx* ctx, const float* x, int64_t N, int64_t C, int64_t H, int64_t W, int KH, int KW, int stride,
                     int dilation, int pad, float* patches) {
    TENMO_CHECK_CTX(ctx);
    ConvGeom g;
    int st = check_geom(ctx, "im2col", N, C, H, W, KH, KW, stride, dilation, pad, &g);
    if (st != TENMO_OK) return st;
    if (N == 0) return TENMO_OK;
    if (!x || !patches) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "im2col: NULL pointer");
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const int64_t total = g.N * g.Ho * g.Wo * g.C * g.KH * g.KW;
    const Im2colDivs dv{make_fastdiv(g.C * g.KH * g.KW), make_fastdiv(g.KW), make_fastdiv(g.KH), make_fastdiv(g.Wo),
                        make_fastdiv(g.Ho)};
    const int grid = tenmo_stream_grid(ctx, total, CV_THREADS * 4, 8);
    if (total < 0x7fffffffLL) im2col_kernel<true><<<grid, CV_THREADS, 0, ctx->stream>>>(x, patches, g, dv);
    else im2col_kernel<false><<<grid, CV_THREADS, 0, ctx->stream>>>(x, patches, g, dv);
    TENMO_LAUNCH_CHECK(ctx, "im2col_kernel");
    return TENMO_OK;
}

int tenmo_col2im_f32(tenmo_ctx* ctx, const float* dpatches, int64_t N, int64_t C, int64_t H, int64_t W, int KH, int KW,
                     int stride, int dilation, int pad, float* dx, float beta) {
    TENMO_CHECK_CTX(ctx);
    ConvGeom g;
    int st = check_geom(ctx, "col2im", N, C, H, W, KH, KW, stride, dilation, pad, &g);
    if (st != TENMO_OK) return st;
    if (beta != 0.f && beta != 1.f) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "col2im: beta must be 0 or 1");
    if (N == 0) return TENMO_OK;
    if (!dpatches || !dx) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "col2im: NULL pointer");
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const int64_t total = N * C * H * W;
    const Col2imDivs dv{make_fastdiv(C), make_fastdiv(W), make_fastdiv(H)};
    const int grid = tenmo_stream_grid(ctx, total, CV_THREADS * 2, 8);
    if (total < 0x7fffffffLL) col2im_kernel<true><<<grid, CV_THREADS, 0, ctx->stream>>>(dpatches, dx, g, beta, dv);
    else col2im_kernel<false><<<grid, CV_THREADS, 0, ctx->stream>>>(dpatches, dx, g, beta, dv);
    TENMO_LAUNCH_CHECK(ctx, "col2im_kernel");
    return TENMO_OK;
}

int tenmo_channel_sum_f32(tenmo_ctx* ctx, const float* g, int64_t N, int64_t C, int64_t S, float* out, float beta) {
    TENMO_CHECK_CTX(ctx);
    if (N < 0 || C <= 0 || S < 0) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "channel_sum: bad shape");
    if (beta != 0.f && beta != 1.f) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "channel_sum: beta must be 0 or 1");
    if (!out || (N * S > 0 && !g)) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "channel_sum: NULL pointer");
    if (C > 0x7fffffffLL) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "channel_sum: too many channels");
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    // enough (channel, slab) CTAs for four per SM, at least one image per slab
    int64_t slabs = (4LL * ctx->sm_count + C - 1) / C;
    if (slabs > N) slabs = N;
    if (slabs < 1) slabs = 1;
    if (slabs > 65535) slabs = 65535;
    const int imgs = (int)((N + slabs - 1) / slabs);
    slabs = N > 0 ? (N + imgs - 1) / imgs : 1;
    void* ws = nullptr;
    int st = tenmo_workspace(ctx, (size_t)C * (size_t)slabs * sizeof(float), &ws);
    if (st != TENMO_OK) return st;
    float* partials = static_cast<float*>(ws);
    const dim3 grid((unsigned)C, (unsigned)slabs);
    const bool vec = (S % 4 == 0) && ((reinterpret_cast<uintptr_t>(g) & 15u) == 0);
    if (vec) channel_sum_partial_kernel<4><<<grid, CV_THREADS, 0, ctx->stream>>>(g, N, C, S, imgs > 0 ? imgs : 1, partials);
    else channel_sum_partial_kernel<1><<<grid, CV_THREADS, 0, ctx->stream>>>(g, N, C, S, imgs > 0 ? imgs : 1, partials);
    TENMO_LAUNCH_CHECK(ctx, "channel_sum_partial_kernel");
    channel_sum_final_kernel<<<(unsigned)((C + 127) / 128), 128, 0, ctx->stream>>>(partials, C, (int)slabs, out, beta);
    TENMO_LAUNCH_CHECK(ctx, "channel_sum_final_kernel");
    return TENMO_OK;
}

int tenmo_maxpool2d_fwd_f32(tenmo_ctx* ctx, const float* x, int64_t N, int64_t C, int64_t H, int64_t W, int k, int stride,
                            int pad, float* out, int64_t* argmax) {
    TENMO_CHECK_CTX(ctx);
    if (N < 0 || C <= 0 || H <= 0 || W <= 0 || k <= 0 || stride <= 0 || pad < 0 || H + 2 * pad < k || W + 2 * pad < k)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "maxpool2d_fwd: bad geometry");
    if (N == 0) return TENMO_OK;
    if (!x || !out || !argmax) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "maxpool2d_fwd: NULL pointer");
    const int64_t Ho = (H + 2 * pad - k) / stride + 1, Wo = (W + 2 * pad - k) / stride + 1;
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    maxpool_fwd_kernel<<<tenmo_stream_grid(ctx, N * C * Ho * Wo, CV_THREADS * 2, 8), CV_THREADS, 0, ctx->stream>>>(
        x, out, reinterpret_cast<long long*>(argmax), N * C, H, W, Ho, Wo, k, stride, pad);
    TENMO_LAUNCH_CHECK(ctx, "maxpool_fwd_kernel");
    return TENMO_OK;
}

int tenmo_maxpool2d_bwd_f32(tenmo_ctx* ctx, const float* g, const int64_t* argmax, int64_t N, int64_t C, int64_t H, int64_t W,
                            int64_t Ho, int64_t Wo, float* dx) {
    TENMO_CHECK_CTX(ctx);
    if (N < 0 || C <= 0 || H <= 0 || W <= 0 || Ho <= 0 || Wo <= 0)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "maxpool2d_bwd: bad geometry");
    if (N == 0) return TENMO_OK;
    if (!g || !argmax || !dx) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "maxpool2d_bwd: NULL pointer");
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    TENMO_CUDA_TRY(ctx, cudaMemsetAsync(dx, 0, sizeof(float) * (size_t)(N * C * H * W), ctx->stream));
    maxpool_bwd_kernel<<<tenmo_stream_grid(ctx, N * C * Ho * Wo, CV_THREADS * 2, 8), CV_THREADS, 0, ctx->stream>>>(
        g, reinterpret_cast<const long long*>(argmax), dx, N * C, H * W, Ho * Wo);
    TENMO_LAUNCH_CHECK(ctx, "maxpool_bwd_kernel");
    return TENMO_OK;
}

}  // extern "C"
