// Softmax cross-entropy with class-index targets: fused forward and backward.
//
// Forward (restates crossentropy.mojo:285-432): per row  max -> e = exp(x - max), sum -> loss ->
// softmax = e * (1/sum).  One warp owns a row; a row of up to 1024 classes is read from HBM once and
// kept in registers (32 values per lane), so the algorithmic traffic of 4*M*C read + 4*M*C written is
// also the real traffic.  Rows with few classes (C <= 32) are handled by one thread per row in
// ascending class order, which reproduces the reference's sequential sum exactly.
// The scalar loss is produced on the device by the last CTA to finish (ticket counter): for a batch of
// up to 256 rows it adds the per-row losses from a scratch row in ascending row order (the reference's
// sequential sum), beyond that every CTA leaves one (sum, count) partial and the last CTA adds those in a
// fixed order.  There is no host read-back between forward and backward (the reference synchronises and
// reads two scalars back, kernels/crossentropy_fused_kernel.mojo:359-375).
// Backward: one warp per row (label and scale read once per row, 16-byte accesses); rows of fewer than 32
// classes use a flat element-per-thread form.
// Roofline: HBM; forward 8*M*C + 8*M bytes, backward 8*M*C + 8*M bytes.
#include "common.cuh"

namespace {

constexpr int CE_THREADS = 256;
constexpr int CE_WARPS = CE_THREADS / 32;
constexpr int CE_REG = 32;  // cached classes per lane

struct CeFwdArgs {
    const float* logits;
    int64_t ld;
    const void* labels;
    int label_is_i64;
    int64_t M, C;
    int64_t ignore_index;
    float ls;
    int reduction;
    float* softmax;
    float* loss;          // 1 float (mean/sum) or M floats (none)
    int32_t* valid_count;
    float* row_loss;      // scratch, M floats (mean/sum with M <= CE_SEQ_ROWS only)
    float* part_loss;     // scratch, one partial loss sum per CTA (M > CE_SEQ_ROWS)
    int32_t* part_cnt;    // scratch, one counted-row total per CTA
    int vec;              // rows may be read / written as float4 (C % 4 == 0, ld % 4 == 0, 16-byte aligned bases)
    unsigned int* ticket; // one counter, zero between calls
    uint32_t* status;
    // fused backward of a small batch (NULL: off): the CTA that finishes the loss also writes
    // dlogits = ((softmax - (1-ls)*onehot) - ls/C) * valid * (upstream / scale), the arithmetic of ce_bwd_flat_kernel
    float* dlogits;
    const float* upstream;
};

constexpr int CE_SEQ_ROWS = 256;  // up to here the mean is the reference's row-ascending sequential sum
constexpr int64_t CE_FUSED_BWD_MAX = 16384;  // logits of a batch whose backward the forward kernel's last CTA also does

__device__ __forceinline__ int64_t load_label(const void* labels, int is_i64, int64_t row) {
    return is_i64 ? reinterpret_cast<const int64_t*>(labels)[row] : (int64_t) reinterpret_cast<const int32_t*>(labels)[row];
}

// loss of one row from its statistics (crossentropy.mojo:368-389); t = the row's label, logit_t = its logit
// (read early by the caller so that the two dependent loads overlap the row's own traffic);
// *counted = the row enters the mean's divisor
__device__ __forceinline__ float row_loss_from_stats(const CeFwdArgs& p, int64_t t, float logit_t, float mx, float sum_exp,
                                                     float sum_logits, int* counted) {
    *counted = 0;
    if (t == p.ignore_index) return 0.f;
    *counted = 1;
    if (t < 0 || t >= p.C) {
        atomicOr(p.status, TENMO_DEV_BAD_LABEL);
        return 0.f;
    }
    const float lse = logf(fmaxf(sum_exp, 1e-7f));
    float loss = -((logit_t - mx) - lse);
    if (p.ls > 0.f) {
        const float inv_c = 1.f / (float)p.C;
        const float mean_lsm = __fmul_rn(sum_logits, inv_c) - mx - lse;
        loss = __fmul_rn(1.f - p.ls, loss) - __fmul_rn(p.ls, mean_lsm);
    }
    return loss;
}

// Final reduction by the last CTA: ascending row order for small M (matches the reference's
// sequential `scalar_loss += loss`), fixed-shape tree otherwise.
__device__ void ce_finalize(const CeFwdArgs& p, float* red_smem) {
    const int tid = threadIdx.x;
    if (p.M <= CE_SEQ_ROWS) {
        // the reference's row-ascending sequential sum: all threads fetch (one row each), thread 0 adds in row order
        __shared__ float row_vals[CE_SEQ_ROWS];
        __shared__ int row_counted[CE_SEQ_ROWS];
        for (int r = tid; r < (int)p.M; r += CE_THREADS) {
            row_vals[r] = p.reduction != 2 ? __ldcg(p.row_loss + r) : 0.f;
            row_counted[r] = load_label(p.labels, p.label_is_i64, r) != p.ignore_index ? 1 : 0;
        }
        __syncthreads();
        if (tid == 0) {
            float s = 0.f;
            int cnt = 0;
            for (int r = 0; r < (int)p.M; ++r) {
                s += row_vals[r];
                cnt += row_counted[r];
            }
            if (p.reduction == 0 && cnt > 0) s = s / (float)cnt;
            if (p.reduction != 2) p.loss[0] = s;
            *p.valid_count = cnt;
        }
        return;
    }
    float s = 0.f;
    int cnt = 0;
    // per-CTA partials (each the sum of that CTA's rows in a fixed order), added in a fixed order
    for (int b = tid; b < (int)gridDim.x; b += CE_THREADS) {
        s += __ldcg(p.part_loss + b);
        cnt += __ldcg(p.part_cnt + b);
    }
    s = tenmo_warp_sum(s);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    int* cnt_smem = reinterpret_cast<int*>(red_smem + CE_WARPS);
    if ((tid & 31) == 0) { red_smem[tid >> 5] = s; cnt_smem[tid >> 5] = cnt; }
    __syncthreads();
    if (tid == 0) {
        float t = 0.f;
        int c = 0;
        for (int w = 0; w < CE_WARPS; ++w) { t += red_smem[w]; c += cnt_smem[w]; }
        if (p.reduction == 0 && c > 0) t = t / (float)c;
        if (p.reduction != 2) p.loss[0] = t;
        *p.valid_count = c;
    }
}

template <bool SMALL_C>
__global__ void __launch_bounds__(CE_THREADS, SMALL_C ? 2 : 3) ce_fwd_kernel(const CeFwdArgs p) {
    __shared__ float red_smem[2 * CE_WARPS];
    __shared__ bool is_last;
    tenmo_grid_dependency_sync();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool partials = p.M > CE_SEQ_ROWS;
    float part_loss = 0.f;  // this thread's rows, ascending
    int part_cnt = 0;
    if (SMALL_C) {
        // one thread per row, classes in ascending order
        for (int64_t row = (int64_t)blockIdx.x * CE_THREADS + threadIdx.x; row < p.M;
             row += (int64_t)gridDim.x * CE_THREADS) {
            const float* x = p.logits + row * p.ld;
            const int64_t t = load_label(p.labels, p.label_is_i64, row);
            const float logit_t = (t >= 0 && t < p.C) ? __ldg(x + t) : 0.f;
            float v[32];
            float mx = -3.4028234663852886e38f;
#pragma unroll
            for (int c = 0; c < 32; ++c)
                if (c < p.C) { v[c] = __ldg(x + c); mx = fmaxf(mx, v[c]); }
            float sum_exp = 0.f, sum_logits = 0.f;
#pragma unroll
            for (int c = 0; c < 32; ++c)
                if (c < p.C) { sum_logits += v[c]; v[c] = expf(v[c] - mx); sum_exp += v[c]; }
            int counted;
            const float loss = row_loss_from_stats(p, t, logit_t, mx, sum_exp, sum_logits, &counted);
            if (p.reduction == 2) p.loss[row] = loss; else if (!partials) p.row_loss[row] = loss;
            part_loss += loss;
            part_cnt += counted;
            if (p.softmax) {
                const float inv = 1.f / sum_exp;
#pragma unroll
                for (int c = 0; c < 32; ++c)
                    if (c < p.C) p.softmax[row * p.C + c] = v[c] * inv;
            }
        }
    } else {
        const bool cached = p.C <= 32 * CE_REG;
        const bool vec = cached && p.vec;
        for (int64_t row = (int64_t)blockIdx.x * CE_WARPS + warp; row < p.M; row += (int64_t)gridDim.x * CE_WARPS) {
            const float* x = p.logits + row * p.ld;
            // label first (same address in every lane: one broadcast load), its logit once the row's own loads are out:
            // the two dependent loads then overlap the row traffic instead of trailing it
            const int64_t t = load_label(p.labels, p.label_is_i64, row);
            float v[CE_REG];
            float mx = -3.4028234663852886e38f;
            if (vec) {
                // lane owns classes 4*(lane + 32*i) .. +3: eight 16-byte loads in flight per lane
                const float4* x4 = reinterpret_cast<const float4*>(x);
#pragma unroll
                for (int i = 0; i < CE_REG / 4; ++i) {
                    const int c = (lane + 32 * i) * 4;
                    float4 t = make_float4(mx, mx, mx, mx);
                    if (c < p.C) t = __ldg(x4 + lane + 32 * i);
                    v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
                }
#pragma unroll
                for (int i = 0; i < CE_REG; ++i) mx = fmaxf(mx, v[i]);
            } else if (cached) {
#pragma unroll
                for (int i = 0; i < CE_REG; ++i) {
                    const int64_t c = lane + 32 * i;
                    v[i] = c < p.C ? __ldg(x + c) : -3.4028234663852886e38f;
                    mx = fmaxf(mx, v[i]);
                }
            } else {
                for (int64_t c = lane; c < p.C; c += 32) mx = fmaxf(mx, __ldg(x + c));
            }
            mx = tenmo_warp_max(mx);
            const float logit_t = (t >= 0 && t < p.C) ? __ldg(x + t) : 0.f;
            float sum_exp = 0.f, sum_logits = 0.f;
            if (vec) {
#pragma unroll
                for (int i = 0; i < CE_REG; ++i) {
                    const int c = (lane + 32 * (i / 4)) * 4;
                    if (c < p.C) { sum_logits += v[i]; v[i] = expf(v[i] - mx); sum_exp += v[i]; }
                }
            } else if (cached) {
#pragma unroll
                for (int i = 0; i < CE_REG; ++i) {
                    const int64_t c = lane + 32 * i;
                    if (c < p.C) { sum_logits += v[i]; v[i] = expf(v[i] - mx); sum_exp += v[i]; }
                }
            } else {
                for (int64_t c = lane; c < p.C; c += 32) {
                    const float xv = __ldg(x + c);
                    sum_logits += xv;
                    sum_exp += expf(xv - mx);
                }
            }
            sum_exp = tenmo_warp_sum(sum_exp);
            sum_logits = tenmo_warp_sum(sum_logits);
            if (p.softmax) {
                const float inv = 1.f / sum_exp;
                float* sm = p.softmax + row * p.C;
                if (vec) {
                    float4* sm4 = reinterpret_cast<float4*>(sm);
#pragma unroll
                    for (int i = 0; i < CE_REG / 4; ++i) {
                        const int c = (lane + 32 * i) * 4;
                        if (c < p.C)
                            sm4[lane + 32 * i] = make_float4(v[4 * i] * inv, v[4 * i + 1] * inv, v[4 * i + 2] * inv, v[4 * i + 3] * inv);
                    }
                } else if (cached) {
#pragma unroll
                    for (int i = 0; i < CE_REG; ++i) {
                        const int64_t c = lane + 32 * i;
                        if (c < p.C) sm[c] = v[i] * inv;
                    }
                } else {
                    for (int64_t c = lane; c < p.C; c += 32) sm[c] = expf(__ldg(x + c) - mx) * inv;
                }
            }
            if (lane == 0) {
                int counted;
                const float loss = row_loss_from_stats(p, t, logit_t, mx, sum_exp, sum_logits, &counted);
                if (p.reduction == 2) p.loss[row] = loss; else if (!partials) p.row_loss[row] = loss;
                part_loss += loss;
                part_cnt += counted;
            }
        }
    }
    if (partials) {
        // this CTA's partial: lanes, then warps, in a fixed order
        part_loss = tenmo_warp_sum(part_loss);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) part_cnt += __shfl_xor_sync(0xffffffffu, part_cnt, o);
        int* cnt_smem = reinterpret_cast<int*>(red_smem + CE_WARPS);
        if (lane == 0) { red_smem[warp] = part_loss; cnt_smem[warp] = part_cnt; }
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = 0.f;
            int c = 0;
            for (int w = 0; w < CE_WARPS; ++w) { t += red_smem[w]; c += cnt_smem[w]; }
            p.part_loss[blockIdx.x] = t;
            p.part_cnt[blockIdx.x] = c;
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(p.ticket, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    ce_finalize(p, red_smem);
    if (threadIdx.x == 0) *p.ticket = 0;
    if (p.dlogits) {
        // every row's softmax is in memory (the other CTAs fenced before they drew their ticket) and so is the count
        __syncthreads();
        float scale_mul = 1.f;
        if (p.reduction != 2) {
            const float ug = p.upstream ? __ldg(p.upstream) : 1.f;
            const int vc = *reinterpret_cast<volatile int32_t*>(p.valid_count);
            const float scale = (p.reduction == 0 && vc > 0) ? (float)vc : 1.f;
            scale_mul = ug / scale;
        }
        const float ls_uniform = p.ls / (float)p.C;
        const int total = (int)(p.M * p.C), Ci = (int)p.C;
        for (int i = threadIdx.x; i < total; i += CE_THREADS) {
            const int row = i / Ci, c = i - row * Ci;
            const int64_t t = load_label(p.labels, p.label_is_i64, row);
            const bool ignored = t == p.ignore_index;
            const float onehot = (!ignored && t == c) ? 1.f : 0.f;
            float g = __ldcg(p.softmax + i);
            if (p.ls > 0.f) g = (g - __fmul_rn(onehot, 1.f - p.ls)) - ls_uniform;
            else g = g - onehot;
            g = g * (ignored ? 0.f : 1.f);
            const float m = p.reduction == 2 ? (p.upstream ? __ldg(p.upstream + row) : 1.f) : scale_mul;
            p.dlogits[i] = __fmul_rn(g, m);
        }
    }
}

// The forward pass for a large batch of wide, 16-byte aligned rows (33 <= C <= 1024, more rows than CE_SEQ_ROWS): the
// arithmetic of ce_fwd_kernel's row-in-registers path, bit for bit, with the NEXT row of a warp already on its way from
// HBM while the current one is reduced, exponentiated and written back.  A warp of the plain kernel alternates between
// a load phase and a compute phase and only the three CTAs of an SM overlap them; here every warp keeps 4 KB of loads in
// flight all the time (two CTAs of eight warps per SM, 64 row registers per lane).
__global__ void __launch_bounds__(CE_THREADS, 2) ce_fwd_stream_kernel(const CeFwdArgs p) {
    __shared__ float red_smem[2 * CE_WARPS];
    __shared__ bool is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float NEG = -3.4028234663852886e38f;
    float part_loss = 0.f;
    int part_cnt = 0;
    const int64_t stride = (int64_t)gridDim.x * CE_WARPS;
    auto load_row = [&](int64_t row, float (&v)[CE_REG]) {
        const float4* x4 = reinterpret_cast<const float4*>(p.logits + row * p.ld);
#pragma unroll
        for (int i = 0; i < CE_REG / 4; ++i) {
            const int c = (lane + 32 * i) * 4;
            float4 t = make_float4(NEG, NEG, NEG, NEG);
            if (c < p.C) t = __ldcs(x4 + lane + 32 * i);
            v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
        }
    };
    auto finish_row = [&](int64_t row, float (&v)[CE_REG]) {
        const int64_t t = load_label(p.labels, p.label_is_i64, row);
        const float logit_t = (t >= 0 && t < p.C) ? __ldg(p.logits + row * p.ld + t) : 0.f;
        float mx = NEG;
#pragma unroll
        for (int i = 0; i < CE_REG; ++i) mx = fmaxf(mx, v[i]);
        mx = tenmo_warp_max(mx);
        float sum_exp = 0.f, sum_logits = 0.f;
#pragma unroll
        for (int i = 0; i < CE_REG; ++i) {
            const int c = (lane + 32 * (i / 4)) * 4;
            if (c < p.C) { sum_logits += v[i]; v[i] = expf(v[i] - mx); sum_exp += v[i]; }
        }
        sum_exp = tenmo_warp_sum(sum_exp);
        sum_logits = tenmo_warp_sum(sum_logits);
        if (p.softmax) {
            const float inv = 1.f / sum_exp;
            float4* sm4 = reinterpret_cast<float4*>(p.softmax + row * p.C);
#pragma unroll
            for (int i = 0; i < CE_REG / 4; ++i) {
                const int c = (lane + 32 * i) * 4;
                if (c < p.C) sm4[lane + 32 * i] = make_float4(v[4 * i] * inv, v[4 * i + 1] * inv, v[4 * i + 2] * inv, v[4 * i + 3] * inv);
            }
        }
        if (lane == 0) {
            int counted;
            const float loss = row_loss_from_stats(p, t, logit_t, mx, sum_exp, sum_logits, &counted);
            if (p.reduction == 2) p.loss[row] = loss;
            part_loss += loss;
            part_cnt += counted;
        }
    };
    float va[CE_REG], vb[CE_REG];
    int64_t row = (int64_t)blockIdx.x * CE_WARPS + warp;
    if (row < p.M) load_row(row, va);
    while (row < p.M) {                       // two rows per turn, so that the buffers never have to be copied
        if (row + stride < p.M) load_row(row + stride, vb);
        finish_row(row, va);
        row += stride;
        if (row >= p.M) break;
        if (row + stride < p.M) load_row(row + stride, va);
        finish_row(row, vb);
        row += stride;
    }
    // this CTA's partial: lanes, then warps, in a fixed order (as in ce_fwd_kernel)
    part_loss = tenmo_warp_sum(part_loss);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part_cnt += __shfl_xor_sync(0xffffffffu, part_cnt, o);
    int* cnt_smem = reinterpret_cast<int*>(red_smem + CE_WARPS);
    if (lane == 0) { red_smem[warp] = part_loss; cnt_smem[warp] = part_cnt; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        int c = 0;
        for (int w = 0; w < CE_WARPS; ++w) { t += red_smem[w]; c += cnt_smem[w]; }
        p.part_loss[blockIdx.x] = t;
        p.part_cnt[blockIdx.x] = c;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(p.ticket, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    ce_finalize(p, red_smem);
    if (threadIdx.x == 0) *p.ticket = 0;
}

struct CeBwdArgs {
    const float* softmax;
    const void* labels;
    int label_is_i64;
    int64_t M, C;
    int64_t ignore_index;
    float ls;
    int reduction;
    const float* upstream;
    const int32_t* valid_count;
    float* dlogits;
    float beta;
    int vec;  // rows may be moved as float4
};

// one element: ((softmax - (1-ls)*onehot) - ls/C) * valid * (upstream / scale)   (crossentropy.mojo:742-766,473-481)
__device__ __forceinline__ float ce_bwd_value(const CeBwdArgs& p, float sm, bool hit, bool ignored, float ls_uniform, float m) {
    const float onehot = hit ? 1.f : 0.f;
    float g;
    if (p.ls > 0.f) g = (sm - __fmul_rn(onehot, 1.f - p.ls)) - ls_uniform;
    else g = sm - onehot;
    g = g * (ignored ? 0.f : 1.f);
    return __fmul_rn(g, m);
}

// One warp per row: the label and the row's scale are read once, the row moves as 16-byte accesses.
__global__ void __launch_bounds__(CE_THREADS) ce_bwd_kernel(const CeBwdArgs p) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float scale_mul = 1.f;
    if (p.reduction != 2) {
        const float ug = p.upstream ? __ldg(p.upstream) : 1.f;
        const int vc = p.valid_count ? *p.valid_count : 0;
        const float scale = (p.reduction == 0 && vc > 0) ? (float)vc : 1.f;
        scale_mul = ug / scale;
    }
    const float ls_uniform = p.ls / (float)p.C;
    const int64_t stride = (int64_t)gridDim.x * CE_WARPS;
    // two rows of a warp travel together (row and row + stride): twice the loads in flight per lane
    for (int64_t row = (int64_t)blockIdx.x * CE_WARPS + warp; row < p.M; row += 2 * stride) {
        const int64_t row_b = row + stride;
        const bool has_b = row_b < p.M;
        const int64_t ta = load_label(p.labels, p.label_is_i64, row);
        const int64_t tb = has_b ? load_label(p.labels, p.label_is_i64, row_b) : p.ignore_index;
        const bool ign_a = ta == p.ignore_index, ign_b = tb == p.ignore_index;
        const int64_t hit_a = ign_a ? -1 : ta, hit_b = ign_b ? -1 : tb;
        const float ma = p.reduction == 2 ? (p.upstream ? __ldg(p.upstream + row) : 1.f) : scale_mul;
        const float mb = p.reduction == 2 ? ((p.upstream && has_b) ? __ldg(p.upstream + row_b) : 1.f) : scale_mul;
        const float* sm_a = p.softmax + row * p.C;
        const float* sm_b = p.softmax + (has_b ? row_b : row) * p.C;
        float* dl_a = p.dlogits + row * p.C;
        float* dl_b = p.dlogits + (has_b ? row_b : row) * p.C;
        if (p.vec) {
            const float4* sa4 = reinterpret_cast<const float4*>(sm_a);
            const float4* sb4 = reinterpret_cast<const float4*>(sm_b);
            float4* da4 = reinterpret_cast<float4*>(dl_a);
            float4* db4 = reinterpret_cast<float4*>(dl_b);
            const int n4 = (int)(p.C >> 2);
#pragma unroll 4
            for (int q = lane; q < n4; q += 32) {
                const float4 s = __ldcs(sa4 + q);
                float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
                if (has_b) u = __ldcs(sb4 + q);
                const int64_t c = (int64_t)q * 4;
                float4 g, h;
                g.x = ce_bwd_value(p, s.x, c == hit_a, ign_a, ls_uniform, ma);
                g.y = ce_bwd_value(p, s.y, c + 1 == hit_a, ign_a, ls_uniform, ma);
                g.z = ce_bwd_value(p, s.z, c + 2 == hit_a, ign_a, ls_uniform, ma);
                g.w = ce_bwd_value(p, s.w, c + 3 == hit_a, ign_a, ls_uniform, ma);
                if (p.beta != 0.f) {
                    const float4 o = da4[q];
                    g.x += o.x; g.y += o.y; g.z += o.z; g.w += o.w;
                }
                da4[q] = g;
                if (has_b) {
                    h.x = ce_bwd_value(p, u.x, c == hit_b, ign_b, ls_uniform, mb);
                    h.y = ce_bwd_value(p, u.y, c + 1 == hit_b, ign_b, ls_uniform, mb);
                    h.z = ce_bwd_value(p, u.z, c + 2 == hit_b, ign_b, ls_uniform, mb);
                    h.w = ce_bwd_value(p, u.w, c + 3 == hit_b, ign_b, ls_uniform, mb);
                    if (p.beta != 0.f) {
                        const float4 o = db4[q];
                        h.x += o.x; h.y += o.y; h.z += o.z; h.w += o.w;
                    }
                    db4[q] = h;
                }
            }
        } else {
            for (int64_t c = lane; c < p.C; c += 32) {
                const float g = ce_bwd_value(p, __ldg(sm_a + c), c == hit_a, ign_a, ls_uniform, ma);
                dl_a[c] = p.beta != 0.f ? dl_a[c] + g : g;
                if (has_b) {
                    const float h = ce_bwd_value(p, __ldg(sm_b + c), c == hit_b, ign_b, ls_uniform, mb);
                    dl_b[c] = p.beta != 0.f ? dl_b[c] + h : h;
                }
            }
        }
    }
}

// Flat form for rows of fewer than 32 classes (a warp per row would idle most lanes).
// dlogits = ((softmax - (1-ls)*onehot) - ls/C) * valid * (upstream / scale)   (crossentropy.mojo:742-766,473-481)
__global__ void __launch_bounds__(CE_THREADS) ce_bwd_flat_kernel(const CeBwdArgs p) {
    const int64_t total = p.M * p.C;
    float scale_mul = 1.f;
    if (p.reduction != 2) {
        const float ug = p.upstream ? __ldg(p.upstream) : 1.f;
        const int vc = p.valid_count ? *p.valid_count : 0;
        const float scale = (p.reduction == 0 && vc > 0) ? (float)vc : 1.f;
        scale_mul = ug / scale;
    }
    const float ls_uniform = p.ls / (float)p.C;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / p.C, c = i - row * p.C;
        const int64_t t = load_label(p.labels, p.label_is_i64, row);
        const bool ignored = t == p.ignore_index;
        const float onehot = (!ignored && t == c) ? 1.f : 0.f;
        float g = __ldg(p.softmax + i);
        if (p.ls > 0.f) g = (g - __fmul_rn(onehot, 1.f - p.ls)) - ls_uniform;
        else g = g - onehot;
        g = g * (ignored ? 0.f : 1.f);
        const float m = p.reduction == 2 ? (p.upstream ? __ldg(p.upstream + row) : 1.f) : scale_mul;
        g = __fmul_rn(g, m);
        p.dlogits[i] = p.beta != 0.f ? p.dlogits[i] + g : g;
    }
}

}  // namespace

// upstream_dev / dlogits: the fused backward of a small batch, or NULL
static int ce_fwd_impl(tenmo_ctx* ctx, const float* logits, int64_t ld_logits, const void* labels, int label_is_i64,
                       int64_t M, int64_t C, int64_t ignore_index, float label_smoothing, int reduction,
                       float* softmax_out, float* loss_dev, int32_t* valid_count_dev, const float* upstream_dev,
                       float* dlogits) {
    TENMO_CHECK_CTX(ctx);
    if (M < 0 || C <= 0) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "ce_fwd: bad shape (M=%lld, C=%lld)", (long long)M, (long long)C);
    if (reduction < 0 || reduction > 2) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "ce_fwd: reduction must be 0 (mean), 1 (sum) or 2 (none)");
    if (label_smoothing < 0.f || label_smoothing > 1.f) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "ce_fwd: label_smoothing outside [0,1]");
    if (!loss_dev || !valid_count_dev || (M > 0 && (!logits || !labels)))
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "ce_fwd: NULL pointer");
    if (M > 0 && ld_logits < C) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "ce_fwd: ld_logits < C");
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    if (M == 0) {
        if (reduction != 2) TENMO_CUDA_TRY(ctx, cudaMemsetAsync(loss_dev, 0, sizeof(float), ctx->stream));
        TENMO_CUDA_TRY(ctx, cudaMemsetAsync(valid_count_dev, 0, sizeof(int32_t), ctx->stream));
        return TENMO_OK;
    }
    CeFwdArgs p;
    p.logits = logits; p.ld = ld_logits; p.labels = labels; p.label_is_i64 = label_is_i64;
    p.M = M; p.C = C; p.ignore_index = ignore_index; p.ls = label_smoothing; p.reduction = reduction;
    p.softmax = softmax_out; p.loss = loss_dev; p.valid_count = valid_count_dev;
    auto aligned16 = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; };
    p.vec = (C % 4 == 0) && (ld_logits % 4 == 0) && aligned16(logits) && (!softmax_out || aligned16(softmax_out));
    // large batches of wide aligned rows: the kernel that keeps the next row of every warp in flight (two CTAs per SM)
    const bool stream = C > 32 && C <= 32 * CE_REG && p.vec && M > 4 * (int64_t)ctx->sm_count * CE_WARPS && !dlogits;
    const int grid = C <= 32 ? tenmo_stream_grid(ctx, M, CE_THREADS, 4)
                             : (stream ? tenmo_stream_grid(ctx, M, CE_WARPS, 2) : tenmo_stream_grid(ctx, M, CE_WARPS, 8));
    // scratch: per-row losses for the sequential mean of a small batch, one (sum, count) pair per CTA beyond it
    p.row_loss = nullptr;
    p.part_loss = nullptr;
    p.part_cnt = nullptr;
    {
        const size_t rows = M <= CE_SEQ_ROWS ? (size_t)M : 0;
        void* ws = nullptr;
        int st = tenmo_workspace(ctx, (rows + 2 * (size_t)grid) * sizeof(float), &ws);
        if (st != TENMO_OK) return st;
        p.row_loss = static_cast<float*>(ws);
        p.part_loss = p.row_loss + rows;
        p.part_cnt = reinterpret_cast<int32_t*>(p.part_loss + grid);
    }
    p.ticket = reinterpret_cast<unsigned int*>(ctx->dev_status + 8);
    p.status = ctx->dev_status;
    p.dlogits = dlogits;
    p.upstream = upstream_dev;
    const bool pdl = tenmo_pdl_ok(ctx, grid);
    cudaError_t le;
    if (stream) le = tenmo_launch(ce_fwd_stream_kernel, (unsigned)grid, CE_THREADS, 0, ctx->stream, false, p);
    else le = C <= 32 ? tenmo_launch(ce_fwd_kernel<true>, (unsigned)grid, CE_THREADS, 0, ctx->stream, pdl, p)
                      : tenmo_launch(ce_fwd_kernel<false>, (unsigned)grid, CE_THREADS, 0, ctx->stream, pdl, p);
    if (le != cudaSuccess) return tenmo_set_error(ctx, TENMO_ERR_CUDA, "launch of ce_fwd_kernel failed: %s", cudaGetErrorString(le));
    TENMO_LAUNCH_CHECK(ctx, "ce_fwd_kernel");
    return TENMO_OK;
}

extern "C" {

int tenmo_ce_fwd_f32(tenmo_ctx* ctx, const float* logits, int64_t ld_logits, const void* labels, int label_is_i64,
                     int64_t M, int64_t C, int64_t ignore_index, float label_smoothing, int reduction,
                     float* softmax_out, float* loss_dev, int32_t* valid_count_dev) {
    return ce_fwd_impl(ctx, logits, ld_logits, labels, label_is_i64, M, C, ignore_index, label_smoothing, reduction,
                       softmax_out, loss_dev, valid_count_dev, nullptr, nullptr);
}

int tenmo_ce_fwd_bwd_f32(tenmo_ctx* ctx, const float* logits, int64_t ld_logits, const void* labels, int label_is_i64,
                         int64_t M, int64_t C, int64_t ignore_index, float label_smoothing, int reduction,
                         float* softmax_out, float* loss_dev, int32_t* valid_count_dev, const float* upstream_dev,
                         float* dlogits) {
    TENMO_CHECK_CTX(ctx);
    if (!softmax_out || (M > 0 && !dlogits)) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "ce_fwd_bwd: NULL pointer");
    // one launch while the CTA that finishes the loss can also sweep the batch; two launches beyond that
    if (M > 0 && M <= CE_SEQ_ROWS && M * C <= CE_FUSED_BWD_MAX)
        return ce_fwd_impl(ctx, logits, ld_logits, labels, label_is_i64, M, C, ignore_index, label_smoothing, reduction,
                           softmax_out, loss_dev, valid_count_dev, upstream_dev, dlogits);
    int st = ce_fwd_impl(ctx, logits, ld_logits, labels, label_is_i64, M, C, ignore_index, label_smoothing, reduction,
                         softmax_out, loss_dev, valid_count_dev, nullptr, nullptr);
    if (st != TENMO_OK) return st;
    return tenmo_ce_bwd_f32(ctx, softmax_out, labels, label_is_i64, M, C, ignore_index, label_smoothing, reduction,
                            upstream_dev, valid_count_dev, dlogits, 0.f);
}

int tenmo_ce_bwd_f32(tenmo_ctx* ctx, const float* softmax, const void* labels, int label_is_i64, int64_t M, int64_t C,
                     int64_t ignore_index, float label_smoothing, int reduction, const float* upstream_dev,
                     const int32_t* valid_count_dev, float* dlogits, float beta) {
    TENMO_CHECK_CTX(ctx);
    if (M < 0 || C <= 0) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "ce_bwd: bad shape");
    if (reduction < 0 || reduction > 2) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "ce_bwd: reduction must be 0, 1 or 2");
    if (beta != 0.f && beta != 1.f) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "ce_bwd: beta must be 0 or 1");
    if (M == 0) return TENMO_OK;
    if (!softmax || !labels || !dlogits) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "ce_bwd: NULL pointer");
    if (reduction == 0 && !valid_count_dev) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "ce_bwd: mean reduction needs valid_count_dev");
    CeBwdArgs p{softmax, labels, label_is_i64, M, C, ignore_index, label_smoothing, reduction, upstream_dev,
                valid_count_dev, dlogits, beta, 0};
    p.vec = (C % 4 == 0) && ((reinterpret_cast<uintptr_t>(softmax) | reinterpret_cast<uintptr_t>(dlogits)) & 15u) == 0;
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    if (C < 32) {
        const int grid = tenmo_stream_grid(ctx, M * C, CE_THREADS * 4, 8);
        ce_bwd_flat_kernel<<<grid, CE_THREADS, 0, ctx->stream>>>(p);
    } else {
        const int grid = tenmo_stream_grid(ctx, (M + 1) / 2, CE_WARPS, 8);  // a warp takes two rows at a time
        ce_bwd_kernel<<<grid, CE_THREADS, 0, ctx->stream>>>(p);
    }
    TENMO_LAUNCH_CHECK(ctx, "ce_bwd_kernel");
    return TENMO_OK;
}

}  // extern "C"
