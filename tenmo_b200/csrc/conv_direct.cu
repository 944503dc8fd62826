// Convolution as an IMPLICIT GEMM, NCHW, strict fp32: the patch matrix of im2col is never written.
//
// The reference's Conv2d (cnn.mojo:404-507) is out[n,co,oy,ox] = bias[co] + sum over (ci, ky, kx) ascending of
// img * kernel; its kernel gradient is grad(C_out, N*Ho*Wo) . patches(N*Ho*Wo, C_in*KH*KW) (cnn.mojo:716-809), its input
// gradient the scatter of kernel-weighted output gradients (cnn.mojo:812-950) and its bias gradient a per-channel sum
// (cnn.mojo:664-714).  All three are GEMMs whose patch operand is a gather from the image.  Here that gather happens
// in the operand load of the GEMM main loop: a CTA stages the image region its output tile reads (halo included, zeros
// for the padding) in shared memory once, and every multiply reads its patch element from there.
//
//   forward   3x3 / stride 1 / dilation 1 (any padding): CTA = (image, 32 output channels, 16x16 or 8x32 output pixels),
//             thread = 8 channels x 4 pixels in a row; per (ci, ky) a thread loads six image values and 24 weights and
//             issues 96 FMAs (packed fma.rn.f32x2, same bits as fmaf).  The accumulator starts at the bias and adds in
//             (ci, ky, kx) order: bit-identical to the reference's chain.  ReLU and its 0/1 mask ride in the epilogue.
//   dX        the same kernel: dX = conv(g, W'), W'[ci][co][ky][kx] = W[co][ci][KH-1-ky][KW-1-kx], padding KH-1-pad, with
//             the ReLU mask of the layer's output multiplied into g as it is staged.
//   dW, db    CTA = (slab of images, 32 output channels), thread = 4 channels x one input channel's 3x3 window (36
//             accumulators) over the pixels of its slice; per-CTA partial sums go to scratch and are added in slab order
//             by the sequential column sum, so the result does not depend on scheduling.  db is the pixel sum of the
//             same staged (masked) gradient tile.
//   any other geometry (stride, dilation, other kernel sizes) runs gather kernels without shared-memory staging: one
//   thread per output element for forward and dX, one CTA per kernel element for dW.
// Roofline: FP32 pipe (2 * N*Ho*Wo*C_out*C_in*KH*KW flop per pass); algorithmic HBM bytes are the image, the kernel and
// the output once each.
#include "common.cuh"
#include "reduce.cuh"

namespace {

constexpr int CD_THREADS = 256;
constexpr int CO_T = 32;  // output channels per CTA
constexpr int WS_P = 36;  // pitch of a staged weight row (32 channels): 16-byte aligned, and consecutive rows 4 banks apart

struct ConvArgs {
    const float* x;        // (N, Cin, H, W)
    const float* x_mask;   // optional (N, Cin, H, W) multiplier applied while x is staged (fused ReLU backward), or NULL
    const float* w;        // (Cout, Cin, KH, KW); the staged 3x3 kernel takes the repacked form of conv3x3_pack_weights_kernel
    const float* bias;     // (Cout) or NULL
    float* out;            // (N, Cout, Ho, Wo)
    float* mask;           // optional ReLU mask of the output
    int N, Cin, H, W, Cout, KH, KW, stride, dil, pad, Ho, Wo;
    int act;
    float beta;
    int tiles_x;
};

// Stages rows [ty0 - pad, +TH + 2) x columns [tx0 - pad, +TW + 2) of `nci` channels of image n (times an optional mask) into
// shared memory, zeros outside the image; column c of the region lands at index c + 3 of its row (pitch PW, plane stride
// PLANE).  With pad == 1 and W a multiple of 4 the interior columns are aligned 16-byte loads; every load of a thread is
// independent of the others, so several are in flight at once.
template <int TH, int TW, int PW, int PLANE>
__device__ __forceinline__ void stage_region(float* xs, const float* __restrict__ src, const float* __restrict__ msk, int n, int c_total,
                                             int ci0, int nci, int H, int W, int ty0, int tx0, int pad) {
    const int tid = threadIdx.x;
    if (pad == 1 && (W & 3) == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(msk)) & 15u) == 0) {
        constexpr int QW = TW / 4 + 1;  // float4 chunks of the interior + one unit for the two halo columns
        const int units = nci * (TH + 2) * QW;
#pragma unroll 4
        for (int u = tid; u < units; u += CD_THREADS) {
            const int q = u % QW, r = (u / QW) % (TH + 2), ci = u / (QW * (TH + 2));
            const int y = ty0 + r - 1;
            const bool row_ok = y >= 0 && y < H;
            const int64_t row_off = (((int64_t)n * c_total + ci0 + ci) * H + y) * W;
            float* dst = xs + ci * PLANE + r * PW;
            if (q < TW / 4) {
                const int xx = tx0 + 4 * q;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (row_ok && xx < W) {
                    v = __ldg(reinterpret_cast<const float4*>(src + row_off + xx));
                    if (msk) {
                        const float4 m = __ldg(reinterpret_cast<const float4*>(msk + row_off + xx));
                        v.x *= m.x; v.y *= m.y; v.z *= m.z; v.w *= m.w;
                    }
                }
                *reinterpret_cast<float4*>(dst + 4 + 4 * q) = v;
            } else {
                const int xl = tx0 - 1, xr = tx0 + TW;
                float vl = 0.f, vr = 0.f;
                if (row_ok && xl >= 0) { vl = __ldg(src + row_off + xl); if (msk) vl *= __ldg(msk + row_off + xl); }
                if (row_ok && xr < W) { vr = __ldg(src + row_off + xr); if (msk) vr *= __ldg(msk + row_off + xr); }
                dst[3] = vl;
                dst[TW + 4] = vr;
            }
        }
        return;
    }
#pragma unroll 4
    for (int i = tid; i < nci * (TH + 2) * (TW + 2); i += CD_THREADS) {
        const int c = i % (TW + 2), r = (i / (TW + 2)) % (TH + 2), ci = i / ((TW + 2) * (TH + 2));
        const int y = ty0 + r - pad, xx = tx0 + c - pad;
        float v = 0.f;
        if (y >= 0 && y < H && xx >= 0 && xx < W) {
            const int64_t gi = (((int64_t)n * c_total + ci0 + ci) * H + y) * W + xx;
            v = __ldg(src + gi);
            if (msk) v *= __ldg(msk + gi);
        }
        xs[ci * PLANE + r * PW + c + 3] = v;
    }
}

// The kernel tensor repacked for the staged forward kernel: wp[cb][ci][tap][c] = W[cb * 32 + c][ci][tap] (zeros beyond
// C_out), so that a CTA's weights for a run of input channels are one contiguous, 16-byte aligned block.  FLIP builds the
// kernel of the input-gradient convolution instead: wp[cb][co][tap][c] = W[co][cb * 32 + c][8 - tap] (roles of the channel
// axes exchanged, taps reversed).
template <bool FLIP>
__global__ void __launch_bounds__(CD_THREADS) conv3x3_pack_weights_kernel(const float* __restrict__ w, float* __restrict__ wp,
                                                                         int n_out, int n_in, int w_cout, int w_cin) {
    const int blocks = (n_out + CO_T - 1) / CO_T;
    const int total = blocks * n_in * 9 * CO_T;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int c = i % CO_T, t = (i / CO_T) % 9, ci = (i / (CO_T * 9)) % n_in, cb = i / (CO_T * 9 * n_in);
        const int o = cb * CO_T + c;
        float v = 0.f;
        if (o < n_out) v = FLIP ? __ldg(w + ((int64_t)ci * w_cin + o) * 9 + (8 - t)) : __ldg(w + ((int64_t)o * w_cin + ci) * 9 + t);
        wp[i] = v;
    }
    (void)w_cout;
}

// ---------------------------------------------------------------------------------------------------------------
// forward, 3x3 / stride 1 / dilation 1
// ---------------------------------------------------------------------------------------------------------------
template <int TH, int TW>
struct FwdCfg {
    static constexpr int CI_T = 32;            // input channels staged at a time
    static constexpr int PW = TW + 8;          // row pitch: input column c of the staged region sits at index c + 3, so
                                               // that columns 1..4 of a thread's six form an aligned float4
    static constexpr int PLANE_RAW = (TH + 2) * PW;
    static constexpr int PLANE = PLANE_RAW + ((36 - PLANE_RAW % 32) % 32);  // plane stride = 4 mod 32 floats
    static constexpr int SMEM = (CI_T * PLANE + CI_T * 9 * WS_P) * 4;
};

template <int TH, int TW>
__global__ void __launch_bounds__(CD_THREADS, 2) conv3x3_fwd_kernel(const ConvArgs a) {
    using Cfg = FwdCfg<TH, TW>;
    extern __shared__ float cd_smem[];
    float* xs = cd_smem;
    float* ws = cd_smem + Cfg::CI_T * Cfg::PLANE;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cg = warp & 3;                       // channel group: 8 of the CTA's 32 output channels
    const int pg = (warp >> 2) * 32 + lane;        // pixel group: 4 consecutive pixels of a row, 64 groups per tile
    const int row = pg / (TW / 4), col4 = (pg % (TW / 4)) * 4;
    const int n = blockIdx.z, co0 = blockIdx.y * CO_T;
    const int ty0 = (blockIdx.x / a.tiles_x) * TH, tx0 = (blockIdx.x % a.tiles_x) * TW;

    float2 acc[8][2];  // [channel][pixel pair]
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const int co = co0 + cg * 8 + c;
        const float b = (a.bias && co < a.Cout) ? __ldg(a.bias + co) : 0.f;  // the accumulator starts at the bias (cnn.mojo:435)
        acc[c][0] = make_float2(b, b);
        acc[c][1] = make_float2(b, b);
    }
    for (int ci0 = 0; ci0 < a.Cin; ci0 += Cfg::CI_T) {
        const int nci = min(Cfg::CI_T, a.Cin - ci0);
        __syncthreads();
        stage_region<TH, TW, Cfg::PW, Cfg::PLANE>(xs, a.x, a.x_mask, n, a.Cin, ci0, nci, a.H, a.W, ty0, tx0, a.pad);
        // the packed weights of this channel block and channel run: nci * 9 rows of 32 floats, one contiguous block
        {
            const float4* wsrc = reinterpret_cast<const float4*>(a.w + ((int64_t)blockIdx.y * a.Cin + ci0) * 9 * CO_T);
#pragma unroll 4
            for (int f = tid; f < nci * 9 * (CO_T / 4); f += CD_THREADS)
                *reinterpret_cast<float4*>(ws + (f >> 3) * WS_P + (f & 7) * 4) = __ldg(wsrc + f);
        }
        __syncthreads();
        for (int ci = 0; ci < nci; ++ci) {
#pragma unroll
            for (int ky = 0; ky < 3; ++ky) {
                const float* xr = xs + ci * Cfg::PLANE + (row + ky) * Cfg::PW + col4;
                float v[6];
                v[0] = xr[3];
                const float4 mid = *reinterpret_cast<const float4*>(xr + 4);
                v[1] = mid.x; v[2] = mid.y; v[3] = mid.z; v[4] = mid.w;
                v[5] = xr[8];
#pragma unroll
                for (int kx = 0; kx < 3; ++kx) {
                    const float* wp = ws + ((ci * 3 + ky) * 3 + kx) * WS_P + cg * 8;
                    const float4 w0 = *reinterpret_cast<const float4*>(wp), w1 = *reinterpret_cast<const float4*>(wp + 4);
                    const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        acc[c][0] = __ffma2_rn(make_float2(v[kx], v[kx + 1]), make_float2(w[c], w[c]), acc[c][0]);
                        acc[c][1] = __ffma2_rn(make_float2(v[kx + 2], v[kx + 3]), make_float2(w[c], w[c]), acc[c][1]);
                    }
                }
            }
        }
    }
    const int oy = ty0 + row, ox = tx0 + col4;
    if (oy >= a.Ho || ox >= a.Wo) return;
    const bool vec = (a.Wo % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.out) & 15u) == 0) &&
                     (!a.mask || (reinterpret_cast<uintptr_t>(a.mask) & 15u) == 0);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const int co = co0 + cg * 8 + c;
        if (co >= a.Cout) break;
        float o[4] = {acc[c][0].x, acc[c][0].y, acc[c][1].x, acc[c][1].y}, m[4];
        const int64_t base = (((int64_t)n * a.Cout + co) * a.Ho + oy) * a.Wo + ox;
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            m[p] = o[p] > 0.f ? 1.f : 0.f;
            if (a.act == TENMO_ACT_RELU) o[p] = o[p] > 0.f ? o[p] : 0.f;
            if (a.beta != 0.f && ox + p < a.Wo) o[p] += a.out[base + p];
        }
        if (vec) {
            *reinterpret_cast<float4*>(a.out + base) = make_float4(o[0], o[1], o[2], o[3]);
            if (a.mask) *reinterpret_cast<float4*>(a.mask + base) = make_float4(m[0], m[1], m[2], m[3]);
        } else {
            for (int p = 0; p < 4 && ox + p < a.Wo; ++p) {
                a.out[base + p] = o[p];
                if (a.mask) a.mask[base + p] = m[p];
            }
        }
    }
}

// forward, any geometry: one thread per output element, the reference's loop with the padding as a bounds check
__global__ void __launch_bounds__(CD_THREADS) conv_fwd_gather_kernel(const ConvArgs a) {
    const int64_t total = (int64_t)a.N * a.Cout * a.Ho * a.Wo;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int ox = (int)(i % a.Wo), oy = (int)((i / a.Wo) % a.Ho);
        const int co = (int)((i / ((int64_t)a.Wo * a.Ho)) % a.Cout), n = (int)(i / ((int64_t)a.Wo * a.Ho * a.Cout));
        float acc = a.bias ? __ldg(a.bias + co) : 0.f;
        for (int ci = 0; ci < a.Cin; ++ci)
            for (int ky = 0; ky < a.KH; ++ky) {
                const int y = oy * a.stride - a.pad + ky * a.dil;
                for (int kx = 0; kx < a.KW; ++kx) {
                    const int xx = ox * a.stride - a.pad + kx * a.dil;
                    float v = 0.f;
                    if (y >= 0 && y < a.H && xx >= 0 && xx < a.W) {
                        const int64_t gi = (((int64_t)n * a.Cin + ci) * a.H + y) * a.W + xx;
                        v = __ldg(a.x + gi);
                        if (a.x_mask) v *= __ldg(a.x_mask + gi);
                    }
                    acc = fmaf(v, __ldg(a.w + (((int64_t)co * a.Cin + ci) * a.KH + ky) * a.KW + kx), acc);
                }
            }
        const float m = acc > 0.f ? 1.f : 0.f;
        if (a.act == TENMO_ACT_RELU) acc = acc > 0.f ? acc : 0.f;
        if (a.beta != 0.f) acc += a.out[i];
        a.out[i] = acc;
        if (a.mask) a.mask[i] = m;
    }
}

// dX, any geometry: one thread per input element gathers the output gradients that read it (no atomics)
struct DxArgs {
    const float* g;
    const float* g_mask;
    const float* w;
    float* dx;
    int N, Cin, H, W, Cout, KH, KW, stride, dil, pad, Ho, Wo;
    float beta;
};
__global__ void __launch_bounds__(CD_THREADS) conv_dx_gather_kernel(const DxArgs a) {
    const int64_t total = (int64_t)a.N * a.Cin * a.H * a.W;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int xx = (int)(i % a.W), y = (int)((i / a.W) % a.H);
        const int ci = (int)((i / ((int64_t)a.W * a.H)) % a.Cin), n = (int)(i / ((int64_t)a.W * a.H * a.Cin));
        float acc = 0.f;
        for (int co = 0; co < a.Cout; ++co)
            for (int ky = 0; ky < a.KH; ++ky) {
                const int ty = y + a.pad - ky * a.dil;
                if (ty < 0 || ty % a.stride != 0 || ty / a.stride >= a.Ho) continue;
                for (int kx = 0; kx < a.KW; ++kx) {
                    const int tx = xx + a.pad - kx * a.dil;
                    if (tx < 0 || tx % a.stride != 0 || tx / a.stride >= a.Wo) continue;
                    const int64_t gi = (((int64_t)n * a.Cout + co) * a.Ho + ty / a.stride) * a.Wo + tx / a.stride;
                    float gv = __ldg(a.g + gi);
                    if (a.g_mask) gv *= __ldg(a.g_mask + gi);
                    acc = fmaf(gv, __ldg(a.w + (((int64_t)co * a.Cin + ci) * a.KH + ky) * a.KW + kx), acc);
                }
            }
        a.dx[i] = a.beta != 0.f ? a.dx[i] + acc : acc;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// dW and db, 3x3 / stride 1 / dilation 1
// ---------------------------------------------------------------------------------------------------------------
struct DwArgs {
    const float* x;       // (N, Cin, H, W)
    const float* g;       // (N, Cout, Ho, Wo)
    const float* g_mask;  // optional ReLU mask of the layer's output, multiplied into g as it is staged
    float* partials;      // (slabs, Cout*Cin*9 + Cout): per-slab partial dW followed by partial db
    int N, Cin, H, W, Cout, pad, Ho, Wo;
    int imgs_per_slab, tiles_x, tiles_y;
};

constexpr int DW_TH = 16, DW_TW = 16;
constexpr int DW_PW = DW_TW + 8;
constexpr int DW_PLANE_RAW = (DW_TH + 2) * DW_PW;                               // 432
constexpr int DW_PLANE = DW_PLANE_RAW + ((36 - DW_PLANE_RAW % 32) % 32);        // 452: stride = 4 mod 32 floats
constexpr int DW_GS = CO_T * DW_TH * DW_TW;                                      // staged gradient tile, floats

// CI_T: input channels staged at a time (a power of two <= 32); a warp's 32 lanes are CI_T channels x 32/CI_T row slices.
template <int CI_T>
__global__ void __launch_bounds__(CD_THREADS, 2) conv3x3_dw_kernel(const DwArgs a) {
    constexpr int PS = 32 / CI_T;
    extern __shared__ float cd_smem[];
    float* gs = cd_smem;                 // [32 co][16][16]
    float* xs = cd_smem + DW_GS;         // [CI_T][18][PW] (plane stride DW_PLANE)
    const int tid = threadIdx.x, lane = tid & 31, cg = tid >> 5;  // warp = group of 4 output channels
    const int ci_l = lane % CI_T, ps = lane / CI_T;
    const int slab = blockIdx.x, co0 = blockIdx.y * CO_T;
    const int K9 = a.Cin * 9;
    const int64_t row_len = (int64_t)a.Cout * K9 + a.Cout;
    float* part = a.partials + (int64_t)slab * row_len;
    const int n_begin = slab * a.imgs_per_slab, n_end = min(a.N, n_begin + a.imgs_per_slab);
    // db: thread (co = tid / 8, sub = tid % 8) adds 32 pixels of a staged tile; the eight partial sums meet by shuffle
    float db_acc = 0.f;

    for (int ci0 = 0; ci0 < a.Cin; ci0 += CI_T) {
        const int nci = min(CI_T, a.Cin - ci0);
        float acc[4][9];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int t = 0; t < 9; ++t) acc[j][t] = 0.f;
        for (int n = n_begin; n < n_end; ++n)
            for (int tile = 0; tile < a.tiles_x * a.tiles_y; ++tile) {
                const int ty0 = (tile / a.tiles_x) * DW_TH, tx0 = (tile % a.tiles_x) * DW_TW;
                __syncthreads();
                // gradient tile (zeros outside the output / beyond Cout), times the ReLU mask
                if ((a.Wo & 3) == 0 && ((reinterpret_cast<uintptr_t>(a.g) | reinterpret_cast<uintptr_t>(a.g_mask)) & 15u) == 0) {
#pragma unroll 4
                    for (int u = tid; u < DW_GS / 4; u += CD_THREADS) {
                        const int q = u % (DW_TW / 4), r = (u / (DW_TW / 4)) % DW_TH, co = u / ((DW_TW / 4) * DW_TH);
                        const int oy = ty0 + r, ox = tx0 + 4 * q;
                        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (oy < a.Ho && ox < a.Wo && co0 + co < a.Cout) {
                            const int64_t gi = (((int64_t)n * a.Cout + co0 + co) * a.Ho + oy) * a.Wo + ox;
                            v = __ldg(reinterpret_cast<const float4*>(a.g + gi));
                            if (a.g_mask) {
                                const float4 m = __ldg(reinterpret_cast<const float4*>(a.g_mask + gi));
                                v.x *= m.x; v.y *= m.y; v.z *= m.z; v.w *= m.w;
                            }
                        }
                        *reinterpret_cast<float4*>(gs + 4 * u) = v;
                    }
                } else {
#pragma unroll 4
                    for (int i = tid; i < DW_GS; i += CD_THREADS) {
                        const int c = i % DW_TW, r = (i / DW_TW) % DW_TH, co = i / (DW_TW * DW_TH);
                        const int oy = ty0 + r, ox = tx0 + c;
                        float v = 0.f;
                        if (oy < a.Ho && ox < a.Wo && co0 + co < a.Cout) {
                            const int64_t gi = (((int64_t)n * a.Cout + co0 + co) * a.Ho + oy) * a.Wo + ox;
                            v = __ldg(a.g + gi);
                            if (a.g_mask) v *= __ldg(a.g_mask + gi);
                        }
                        gs[i] = v;
                    }
                }
                stage_region<DW_TH, DW_TW, DW_PW, DW_PLANE>(xs, a.x, nullptr, n, a.Cin, ci0, nci, a.H, a.W, ty0, tx0, a.pad);
                __syncthreads();
                if (ci0 == 0) {  // bias gradient: once per (image, tile)
                    const int co = tid >> 3, sub = tid & 7;
                    float s = 0.f;
                    const float* gp = gs + co * (DW_TH * DW_TW) + sub * 32;
#pragma unroll 8
                    for (int q = 0; q < 32; ++q) s += gp[q];
                    s += __shfl_xor_sync(0xffffffffu, s, 4);
                    s += __shfl_xor_sync(0xffffffffu, s, 2);
                    s += __shfl_xor_sync(0xffffffffu, s, 1);
                    db_acc += s;
                }
                if (ci_l < nci) {
                    for (int r = ps; r < DW_TH; r += PS) {
#pragma unroll
                        for (int c4 = 0; c4 < DW_TW; c4 += 4) {
                            float4 g4[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                g4[j] = *reinterpret_cast<const float4*>(gs + (cg * 4 + j) * (DW_TH * DW_TW) + r * DW_TW + c4);
#pragma unroll
                            for (int ky = 0; ky < 3; ++ky) {
                                const float* xr = xs + ci_l * DW_PLANE + (r + ky) * DW_PW + c4;
                                float v[6];
                                v[0] = xr[3];
                                const float4 mid = *reinterpret_cast<const float4*>(xr + 4);
                                v[1] = mid.x; v[2] = mid.y; v[3] = mid.z; v[4] = mid.w;
                                v[5] = xr[8];
#pragma unroll
                                for (int kx = 0; kx < 3; ++kx)
#pragma unroll
                                    for (int j = 0; j < 4; ++j) {
                                        float s = acc[j][ky * 3 + kx];
                                        s = fmaf(g4[j].x, v[kx], s);
                                        s = fmaf(g4[j].y, v[kx + 1], s);
                                        s = fmaf(g4[j].z, v[kx + 2], s);
                                        s = fmaf(g4[j].w, v[kx + 3], s);
                                        acc[j][ky * 3 + kx] = s;
                                    }
                            }
                        }
                    }
                }
            }
        // the row slices of a warp meet in slice order (deterministic), then slice 0 writes the partial
        if (PS > 1) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int t = 0; t < 9; ++t) {
                    float s = acc[j][t];
                    for (int q = 1; q < PS; ++q) {
                        const float o = __shfl_sync(0xffffffffu, acc[j][t], q * CI_T + ci_l);
                        if (ps == 0) s += o;
                    }
                    acc[j][t] = s;
                }
        }
        if (ps == 0 && ci_l < nci) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int co = co0 + cg * 4 + j;
                if (co < a.Cout) {
#pragma unroll
                    for (int t = 0; t < 9; ++t) part[((int64_t)co * a.Cin + ci0 + ci_l) * 9 + t] = acc[j][t];
                }
            }
        }
    }
    if ((tid & 7) == 0) {
        const int co = co0 + (tid >> 3);
        if (co < a.Cout) part[(int64_t)a.Cout * K9 + co] = db_acc;
    }
}

// dW / db, any geometry: one CTA per kernel element (and one per channel for db), threads stride the (n, oy, ox) range,
// the 256 partial sums meet in a fixed tree.
struct DwGatherArgs {
    const float* x;
    const float* g;
    const float* g_mask;
    float* dw;
    float* db;
    int N, Cin, H, W, Cout, KH, KW, stride, dil, pad, Ho, Wo;
    float beta;
};
__global__ void __launch_bounds__(CD_THREADS) conv_dw_gather_kernel(const DwGatherArgs a) {
    __shared__ float red[CD_THREADS];
    const int n_w = a.Cout * a.Cin * a.KH * a.KW;
    const int e = blockIdx.x;
    const bool is_bias = e >= n_w;
    const int co = is_bias ? e - n_w : e / (a.Cin * a.KH * a.KW);
    const int kx = e % a.KW, ky = (e / a.KW) % a.KH, ci = (e / (a.KW * a.KH)) % a.Cin;
    const int64_t span = (int64_t)a.N * a.Ho * a.Wo;
    float acc = 0.f;
    for (int64_t i = threadIdx.x; i < span; i += CD_THREADS) {
        const int ox = (int)(i % a.Wo), oy = (int)((i / a.Wo) % a.Ho), n = (int)(i / ((int64_t)a.Wo * a.Ho));
        const int64_t gi = (((int64_t)n * a.Cout + co) * a.Ho + oy) * a.Wo + ox;
        float gv = __ldg(a.g + gi);
        if (a.g_mask) gv *= __ldg(a.g_mask + gi);
        if (is_bias) {
            acc += gv;
        } else {
            const int y = oy * a.stride - a.pad + ky * a.dil, xx = ox * a.stride - a.pad + kx * a.dil;
            if (y >= 0 && y < a.H && xx >= 0 && xx < a.W)
                acc = fmaf(gv, __ldg(a.x + (((int64_t)n * a.Cin + ci) * a.H + y) * a.W + xx), acc);
        }
    }
    red[threadIdx.x] = acc;
    __syncthreads();
    for (int s = CD_THREADS / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        float* dst = is_bias ? a.db + co : a.dw + e;
        *dst = a.beta != 0.f ? *dst + red[0] : red[0];
    }
}

// The per-slab partial rows [dW | db] added in slab order (one thread per column, sixteen loads in flight): one launch
// finishes both gradients.
__global__ void __launch_bounds__(CD_THREADS) conv_reduce_partials_kernel(const float* __restrict__ partials, int slabs, int n_w,
                                                                         int n_b, float* __restrict__ dw, float* __restrict__ db,
                                                                         float beta) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int row_len = n_w + n_b;
    if (c >= row_len) return;
    float acc = 0.f;
    int s = 0;
    for (; s + 16 <= slabs; s += 16) {
        float v[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) v[u] = __ldcs(partials + (int64_t)(s + u) * row_len + c);
#pragma unroll
        for (int u = 0; u < 16; ++u) acc += v[u];
    }
    for (; s < slabs; ++s) acc += __ldcs(partials + (int64_t)s * row_len + c);
    float* dst = c < n_w ? dw + c : db + (c - n_w);
    *dst = beta != 0.f ? *dst + acc : acc;
}

int conv_check(tenmo_ctx* ctx, const char* who, int64_t N, int64_t C, int64_t H, int64_t W, int64_t Cout, int KH, int KW, int stride,
               int dil, int pad, int64_t* Ho, int64_t* Wo) {
    if (N < 0 || C <= 0 || H <= 0 || W <= 0 || Cout <= 0 || KH <= 0 || KW <= 0 || stride <= 0 || dil <= 0 || pad < 0)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "%s: bad geometry", who);
    if (tenmo_conv_out_size(H, KH, stride, dil, pad, Ho) != TENMO_OK || tenmo_conv_out_size(W, KW, stride, dil, pad, Wo) != TENMO_OK ||
        *Ho <= 0 || *Wo <= 0)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "%s: the kernel does not fit the padded image", who);
    if (N * C * H * W >= ((int64_t)1 << 31) || N * Cout * *Ho * *Wo >= ((int64_t)1 << 31) || Cout * C * KH * KW >= ((int64_t)1 << 24))
        return tenmo_set_error(ctx, TENMO_ERR_UNSUPPORTED, "%s: tensors of 2^31 elements or more are not served", who);
    return TENMO_OK;
}

bool fast3x3(int KH, int KW, int stride, int dil) { return KH == 3 && KW == 3 && stride == 1 && dil == 1; }

template <int TH, int TW>
int launch_fwd3x3(tenmo_ctx* ctx, ConvArgs& a) {
    using Cfg = FwdCfg<TH, TW>;
    static bool attr_set[64] = {false};
    if (!attr_set[ctx->device & 63]) {
        TENMO_CUDA_TRY(ctx, cudaFuncSetAttribute(conv3x3_fwd_kernel<TH, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
        // two CTAs per SM need the large shared-memory split of the L1
        TENMO_CUDA_TRY(ctx, cudaFuncSetAttribute(conv3x3_fwd_kernel<TH, TW>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                                 cudaSharedmemCarveoutMaxShared));
        attr_set[ctx->device & 63] = true;
    }
    a.tiles_x = (a.Wo + TW - 1) / TW;
    const int tiles_y = (a.Ho + TH - 1) / TH;
    dim3 grid((unsigned)(a.tiles_x * tiles_y), (unsigned)((a.Cout + CO_T - 1) / CO_T), (unsigned)a.N);
    conv3x3_fwd_kernel<TH, TW><<<grid, CD_THREADS, Cfg::SMEM, ctx->stream>>>(a);
    TENMO_LAUNCH_CHECK(ctx, "conv3x3_fwd_kernel");
    return TENMO_OK;
}

// flip: the call computes an input gradient -- `a.w` is the layer's (a.Cin, a.Cout, 3, 3) kernel tensor, to be used with
// the channel axes exchanged and the taps reversed.
int launch_conv_fwd(tenmo_ctx* ctx, ConvArgs& a, bool flip) {
    if (a.N == 0) return TENMO_OK;
    if (a.N > 65535) return tenmo_set_error(ctx, TENMO_ERR_UNSUPPORTED, "conv2d: at most 65535 images per call");
    if (fast3x3(a.KH, a.KW, a.stride, a.dil)) {
        const int blocks = (a.Cout + CO_T - 1) / CO_T;
        const int n_wp = blocks * a.Cin * 9 * CO_T;
        void* ws = nullptr;
        int st = tenmo_workspace(ctx, (size_t)n_wp * sizeof(float), &ws);
        if (st != TENMO_OK) return st;
        const int grid = (n_wp + CD_THREADS - 1) / CD_THREADS;
        if (flip) conv3x3_pack_weights_kernel<true><<<grid, CD_THREADS, 0, ctx->stream>>>(a.w, static_cast<float*>(ws), a.Cout, a.Cin, a.Cin, a.Cout);
        else conv3x3_pack_weights_kernel<false><<<grid, CD_THREADS, 0, ctx->stream>>>(a.w, static_cast<float*>(ws), a.Cout, a.Cin, a.Cout, a.Cin);
        TENMO_LAUNCH_CHECK(ctx, "conv3x3_pack_weights_kernel");
        a.w = static_cast<const float*>(ws);
        return a.Wo <= 16 ? launch_fwd3x3<16, 16>(ctx, a) : launch_fwd3x3<8, 32>(ctx, a);
    }
    const int64_t total = (int64_t)a.N * a.Cout * a.Ho * a.Wo;
    conv_fwd_gather_kernel<<<tenmo_stream_grid(ctx, total, CD_THREADS, 8), CD_THREADS, 0, ctx->stream>>>(a);
    TENMO_LAUNCH_CHECK(ctx, "conv_fwd_gather_kernel");
    return TENMO_OK;
}

template <int CI_T>
int launch_dw3x3(tenmo_ctx* ctx, const DwArgs& a, int slabs) {
    constexpr int SMEM = (DW_GS + CI_T * DW_PLANE) * 4;
    static bool attr_set[64] = {false};
    if (!attr_set[ctx->device & 63]) {
        TENMO_CUDA_TRY(ctx, cudaFuncSetAttribute(conv3x3_dw_kernel<CI_T>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
        TENMO_CUDA_TRY(ctx, cudaFuncSetAttribute(conv3x3_dw_kernel<CI_T>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                                 cudaSharedmemCarveoutMaxShared));
        attr_set[ctx->device & 63] = true;
    }
    dim3 grid((unsigned)slabs, (unsigned)((a.Cout + CO_T - 1) / CO_T));
    conv3x3_dw_kernel<CI_T><<<grid, CD_THREADS, SMEM, ctx->stream>>>(a);
    TENMO_LAUNCH_CHECK(ctx, "conv3x3_dw_kernel");
    return TENMO_OK;
}

}  // namespace

extern "C" {

int tenmo_conv2d_fwd_f32(tenmo_ctx* ctx, const float* x, int64_t N, int64_t C, int64_t H, int64_t W, const float* weight,
                         const float* bias, int64_t Cout, int KH, int KW, int stride, int dilation, int pad, int act, float* out,
                         float* mask) {
    TENMO_CHECK_CTX(ctx);
    int64_t Ho, Wo;
    int st = conv_check(ctx, "conv2d_fwd", N, C, H, W, Cout, KH, KW, stride, dilation, pad, &Ho, &Wo);
    if (st != TENMO_OK) return st;
    if (!x || !weight || !out) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "conv2d_fwd: NULL pointer");
    if (act != TENMO_ACT_NONE && act != TENMO_ACT_RELU) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "conv2d_fwd: act must be none or ReLU");
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    ConvArgs a;
    memset(&a, 0, sizeof(a));
    a.x = x; a.w = weight; a.bias = bias; a.out = out; a.mask = mask;
    a.N = (int)N; a.Cin = (int)C; a.H = (int)H; a.W = (int)W; a.Cout = (int)Cout; a.KH = KH; a.KW = KW;
    a.stride = stride; a.dil = dilation; a.pad = pad; a.Ho = (int)Ho; a.Wo = (int)Wo; a.act = act;
    return launch_conv_fwd(ctx, a, false);
}

int tenmo_conv2d_bwd_input_f32(tenmo_ctx* ctx, const float* g, const float* g_mask, const float* weight, int64_t N, int64_t C,
                               int64_t H, int64_t W, int64_t Cout, int KH, int KW, int stride, int dilation, int pad, float* dx,
                               float beta) {
    TENMO_CHECK_CTX(ctx);
    int64_t Ho, Wo;
    int st = conv_check(ctx, "conv2d_bwd_input", N, C, H, W, Cout, KH, KW, stride, dilation, pad, &Ho, &Wo);
    if (st != TENMO_OK) return st;
    if (!g || !weight || !dx) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "conv2d_bwd_input: NULL pointer");
    if (beta != 0.f && beta != 1.f) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "conv2d_bwd_input: beta must be 0 or 1");
    if (N == 0) return TENMO_OK;
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    if (fast3x3(KH, KW, stride, dilation) && pad <= 2) {
        // dX = conv(g, W') with padding 2 - pad: an image of Ho x Wo gives back H x W
        ConvArgs a;
        memset(&a, 0, sizeof(a));
        a.x = g; a.x_mask = g_mask; a.w = weight; a.out = dx;
        a.N = (int)N; a.Cin = (int)Cout; a.H = (int)Ho; a.W = (int)Wo; a.Cout = (int)C; a.KH = 3; a.KW = 3;
        a.stride = 1; a.dil = 1; a.pad = 2 - pad; a.Ho = (int)H; a.Wo = (int)W; a.act = TENMO_ACT_NONE; a.beta = beta;
        return launch_conv_fwd(ctx, a, true);
    }
    DxArgs a;
    a.g = g; a.g_mask = g_mask; a.w = weight; a.dx = dx;
    a.N = (int)N; a.Cin = (int)C; a.H = (int)H; a.W = (int)W; a.Cout = (int)Cout; a.KH = KH; a.KW = KW;
    a.stride = stride; a.dil = dilation; a.pad = pad; a.Ho = (int)Ho; a.Wo = (int)Wo; a.beta = beta;
    conv_dx_gather_kernel<<<tenmo_stream_grid(ctx, N * C * H * W, CD_THREADS, 8), CD_THREADS, 0, ctx->stream>>>(a);
    TENMO_LAUNCH_CHECK(ctx, "conv_dx_gather_kernel");
    return TENMO_OK;
}

int tenmo_conv2d_bwd_weight_f32(tenmo_ctx* ctx, const float* x, const float* g, const float* g_mask, int64_t N, int64_t C, int64_t H,
                                int64_t W, int64_t Cout, int KH, int KW, int stride, int dilation, int pad, float* dW, float* db,
                                float beta) {
    TENMO_CHECK_CTX(ctx);
    int64_t Ho, Wo;
    int st = conv_check(ctx, "conv2d_bwd_weight", N, C, H, W, Cout, KH, KW, stride, dilation, pad, &Ho, &Wo);
    if (st != TENMO_OK) return st;
    if (!x || !g || !dW || !db) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "conv2d_bwd_weight: NULL pointer");
    if (beta != 0.f && beta != 1.f) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "conv2d_bwd_weight: beta must be 0 or 1");
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const int64_t n_w = Cout * C * KH * KW;
    if (N == 0) {
        if (beta == 0.f) {
            TENMO_CUDA_TRY(ctx, cudaMemsetAsync(dW, 0, (size_t)n_w * sizeof(float), ctx->stream));
            TENMO_CUDA_TRY(ctx, cudaMemsetAsync(db, 0, (size_t)Cout * sizeof(float), ctx->stream));
        }
        return TENMO_OK;
    }
    if (fast3x3(KH, KW, stride, dilation)) {
        const int co_blocks = (int)((Cout + CO_T - 1) / CO_T);
        // about two CTAs per SM in total, at most TENMO_COLSUM_SEQ_ROWS slabs
        int64_t slabs = (2 * (int64_t)ctx->sm_count + co_blocks - 1) / co_blocks;
        if (slabs > N) slabs = N;
        if (slabs > TENMO_COLSUM_SEQ_ROWS) slabs = TENMO_COLSUM_SEQ_ROWS;
        const int per = (int)((N + slabs - 1) / slabs);
        slabs = (N + per - 1) / per;
        const int64_t row_len = n_w + Cout;
        void* ws = nullptr;
        st = tenmo_workspace(ctx, (size_t)slabs * (size_t)row_len * sizeof(float), &ws);
        if (st != TENMO_OK) return st;
        DwArgs a;
        a.x = x; a.g = g; a.g_mask = g_mask; a.partials = static_cast<float*>(ws);
        a.N = (int)N; a.Cin = (int)C; a.H = (int)H; a.W = (int)W; a.Cout = (int)Cout; a.pad = pad; a.Ho = (int)Ho; a.Wo = (int)Wo;
        a.imgs_per_slab = per;
        a.tiles_x = (int)((Wo + DW_TW - 1) / DW_TW);
        a.tiles_y = (int)((Ho + DW_TH - 1) / DW_TH);
        if (C <= 4) st = launch_dw3x3<4>(ctx, a, (int)slabs);
        else if (C <= 8) st = launch_dw3x3<8>(ctx, a, (int)slabs);
        else if (C <= 16) st = launch_dw3x3<16>(ctx, a, (int)slabs);
        else st = launch_dw3x3<32>(ctx, a, (int)slabs);
        if (st != TENMO_OK) return st;
        // the slabs in ascending order, dW and db out of the same partial rows
        conv_reduce_partials_kernel<<<(unsigned)((row_len + CD_THREADS - 1) / CD_THREADS), CD_THREADS, 0, ctx->stream>>>(
            a.partials, (int)slabs, (int)n_w, (int)Cout, dW, db, beta);
        TENMO_LAUNCH_CHECK(ctx, "conv_reduce_partials_kernel");
        return TENMO_OK;
    }
    DwGatherArgs a;
    a.x = x; a.g = g; a.g_mask = g_mask; a.dw = dW; a.db = db;
    a.N = (int)N; a.Cin = (int)C; a.H = (int)H; a.W = (int)W; a.Cout = (int)Cout; a.KH = KH; a.KW = KW;
    a.stride = stride; a.dil = dilation; a.pad = pad; a.Ho = (int)Ho; a.Wo = (int)Wo; a.beta = beta;
    conv_dw_gather_kernel<<<(unsigned)(n_w + Cout), CD_THREADS, 0, ctx->stream>>>(a);
    TENMO_LAUNCH_CHECK(ctx, "conv_dw_gather_kernel");
    return TENMO_OK;
}

}  // extern "C"
