// CPU oracle for the dense fp32 training path -- see tenmo_ref.h for what this is and is not.
// Every function cites the reference file:line it restates (paths relative to the reference root).
// Build: see oracle/Makefile (g++ -O2 -mavx2 -mfma -ffp-contract=off; FMAs are written explicitly).
#include "tenmo_ref.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstring>
#include <functional>
#include <thread>
#include <vector>

namespace {

constexpr int UNROLL = 4;  // matmul_cpu.mojo:30

inline float fma_chain(float a, float b, float acc) { return __builtin_fmaf(a, b, acc); }
// The reference's scalar sites read `acc += a * b` (matmul_cpu.mojo:349,466,539): whether that is
// contracted into an FMA is decided by the Mojo compiler, so it is a run-time option here.
inline float scalar_site(float a, float b, float acc, bool contract) {
    if (contract) return __builtin_fmaf(a, b, acc);
    volatile float prod = a * b;  // volatile: keep the rounding of the product
    return acc + prod;
}

// std.algorithm.parallelize over `n` work items with `threads` workers (matmul_cpu.mojo:353).
void parallel_for(int64_t n, int threads, const std::function<void(int64_t)>& fn) {
    if (threads <= 1 || n <= 1) {
        for (int64_t i = 0; i < n; ++i) fn(i);
        return;
    }
    int nt = (int)std::min<int64_t>(threads, n);
    std::atomic<int64_t> next{0};
    std::vector<std::thread> pool;
    pool.reserve(nt);
    for (int t = 0; t < nt; ++t)
        pool.emplace_back([&] {
            for (;;) {
                int64_t i = next.fetch_add(1);
                if (i >= n) break;
                fn(i);
            }
        });
    for (auto& th : pool) th.join();
}

struct Tiles { int64_t m, n, p; };
// matmul_cpu.mojo:87-89 (2D) and 577-579 (ND): each dimension picks its own tile.
Tiles pick_tiles(int64_t m, int64_t n, int64_t p) {
    Tiles t;
    t.m = m > 256 ? 128 : (m > 64 ? 64 : 32);
    t.n = n > 64 ? 64 : 32;
    t.p = p > 256 ? 256 : (p > 64 ? 128 : 64);
    return t;
}

// strides.mojo:239-264 / ndbuffer.mojo:523-524: exact C-order strides for every dim of size > 1.
bool is_contiguous_2d(int64_t rows, int64_t cols, int64_t s0, int64_t s1) {
    if (cols > 1 && s1 != 1) return false;
    if (rows > 1 && s0 != cols) return false;
    return true;
}

// One (row tile) of paths 1a / 1b: matmul_cpu.mojo:224-351 and 366-468 (identical but for the A address).
// B has unit column stride.  Loop order k_tile -> j_tile -> i -> j-strip -> k; partial sums are parked
// in C between k tiles, which is exact in fp32, so every C element is one k-ascending chain.
template <int W>
void rows_b_contig(const float* A, int64_t a_base, int64_t a_s0, int64_t a_s1, const float* B, int64_t b_base,
                   int64_t b_s0, float* C, int64_t i_start, int64_t i_end, int64_t n, int64_t p, Tiles T,
                   bool contract) {
    constexpr int SU = W * UNROLL;
    for (int64_t k_tile = 0; k_tile < n; k_tile += T.n) {
        const int64_t k_end = std::min(k_tile + T.n, n);
        for (int64_t j_tile = 0; j_tile < p; j_tile += T.p) {
            const int64_t j_end = std::min(j_tile + T.p, p);
            for (int64_t i = i_start; i < i_end; ++i) {
                const int64_t a_row = a_base + i * a_s0;
                float* c_row = C + i * p;
                int64_t j = j_tile;
                // UNROLL SIMD accumulators per strip (275-312)
                for (; j + SU <= j_end; j += SU) {
                    float acc[SU];
                    if (k_tile == 0) {
                        for (int q = 0; q < SU; ++q) acc[q] = 0.f;
                    } else {
                        for (int q = 0; q < SU; ++q) acc[q] = c_row[j + q];
                    }
                    for (int64_t k = k_tile; k < k_end; ++k) {
                        const float a = A[a_row + k * a_s1];
                        const float* b = B + b_base + k * b_s0 + j;
#pragma GCC ivdep
                        for (int q = 0; q < SU; ++q) acc[q] = fma_chain(a, b[q], acc[q]);
                    }
                    for (int q = 0; q < SU; ++q) c_row[j + q] = acc[q];
                }
                // single-vector tail (317-335)
                for (; j + W <= j_end; j += W) {
                    float acc[W];
                    if (k_tile == 0) {
                        for (int q = 0; q < W; ++q) acc[q] = 0.f;
                    } else {
                        for (int q = 0; q < W; ++q) acc[q] = c_row[j + q];
                    }
                    for (int64_t k = k_tile; k < k_end; ++k) {
                        const float a = A[a_row + k * a_s1];
                        const float* b = B + b_base + k * b_s0 + j;
#pragma GCC ivdep
                        for (int q = 0; q < W; ++q) acc[q] = fma_chain(a, b[q], acc[q]);
                    }
                    for (int q = 0; q < W; ++q) c_row[j + q] = acc[q];
                }
                // scalar tail (340-351)
                for (; j < j_end; ++j) {
                    float acc = (k_tile == 0) ? 0.f : c_row[j];
                    for (int64_t k = k_tile; k < k_end; ++k)
                        acc = scalar_site(A[a_row + k * a_s1], B[b_base + k * b_s0 + j], acc, contract);
                    c_row[j] = acc;
                }
            }
        }
    }
}

// Path 2, 2D form (matmul_cpu.mojo:504-543): i -> k_tile -> j_tile -> j -> k, scalar.
void rows_b_strided_2d(const float* A, int64_t a_base, int64_t a_s0, int64_t a_s1, const float* B, int64_t b_base,
                       int64_t b_s0, int64_t b_s1, float* C, int64_t i_start, int64_t i_end, int64_t n,
                       int64_t p, Tiles T, bool contract) {
    for (int64_t i = i_start; i < i_end; ++i) {
        const int64_t a_row = a_base + i * a_s0;
        float* c_row = C + i * p;
        for (int64_t k_tile = 0; k_tile < n; k_tile += T.n) {
            const int64_t k_end = std::min(k_tile + T.n, n);
            for (int64_t j_tile = 0; j_tile < p; j_tile += T.p) {
                const int64_t j_end = std::min(j_tile + T.p, p);
                for (int64_t j = j_tile; j < j_end; ++j) {
                    float acc = (k_tile == 0) ? 0.f : c_row[j];
                    for (int64_t k = k_tile; k < k_end; ++k)
                        acc = scalar_site(A[a_row + k * a_s1], B[b_base + k * b_s0 + j * b_s1], acc, contract);
                    c_row[j] = acc;
                }
            }
        }
    }
}

void rows_dispatch(bool a_contig, bool b_contig, const float* A, int64_t a_base, int64_t a_s0, int64_t a_s1,
                   const float* B, int64_t b_base, int64_t b_s0, int64_t b_s1, float* C, int64_t i_start,
                   int64_t i_end, int64_t n, int64_t p, Tiles T, const tenmo_ref_opts& o) {
    const bool contract = o.contract_scalar != 0;
    if (b_contig) {
        // 1a differs from 1b only by a_s1 == 1 (matmul_cpu.mojo:298-300 vs 422-424)
        const int64_t s1 = a_contig ? 1 : a_s1;
        if (o.simd_width == 16)
            rows_b_contig<16>(A, a_base, a_s0, s1, B, b_base, b_s0, C, i_start, i_end, n, p, T, contract);
        else
            rows_b_contig<8>(A, a_base, a_s0, s1, B, b_base, b_s0, C, i_start, i_end, n, p, T, contract);
    } else {
        rows_b_strided_2d(A, a_base, a_s0, a_s1, B, b_base, b_s0, b_s1, C, i_start, i_end, n, p, T, contract);
    }
}

tenmo_ref_opts default_opts(const tenmo_ref_opts* o) {
    tenmo_ref_opts r{8, 1, 1};
    if (o) r = *o;
    if (r.simd_width != 16) r.simd_width = 8;
    if (r.threads < 1) r.threads = 1;
    return r;
}

}  // namespace

extern "C" {

void tenmo_ref_matmul_2d(const tenmo_ref_mat* A, const tenmo_ref_mat* B, float* C, int64_t m, int64_t n, int64_t p,
                         const tenmo_ref_opts* opts) {
    const tenmo_ref_opts o = default_opts(opts);
    const Tiles T = pick_tiles(m, n, p);
    std::memset(C, 0, sizeof(float) * (size_t)(m * p));  // NDBuffer.zeros, matmul_cpu.mojo:183
    const bool a_contig = is_contiguous_2d(m, n, A->row_stride, A->col_stride);
    const bool b_contig = is_contiguous_2d(n, p, B->row_stride, B->col_stride);
    const int64_t tiles = (m + T.m - 1) / T.m;
    parallel_for(tiles, o.threads, [&](int64_t t) {
        const int64_t i0 = t * T.m, i1 = std::min(i0 + T.m, m);
        rows_dispatch(a_contig, b_contig, A->ptr, A->offset, A->row_stride, A->col_stride, B->ptr, B->offset,
                      B->row_stride, B->col_stride, C, i0, i1, n, p, T, o);
    });
}

int64_t tenmo_ref_matmul_nd(const tenmo_ref_mat* A, const tenmo_ref_mat* B, float* C, int64_t m, int64_t n,
                            int64_t p, const tenmo_ref_opts* opts) {
    const tenmo_ref_opts o = default_opts(opts);
    const Tiles T = pick_tiles(m, n, p);
    // ShapeBroadcaster.broadcast_shape over the batch dims (matmul_cpu.mojo:655-667)
    const int ra = A->batch_rank, rb = B->batch_rank, r = std::max(ra, rb);
    int64_t bshape[6];
    int64_t total = 1;
    for (int d = 0; d < r; ++d) {
        const int ad = d - (r - ra), bd = d - (r - rb);
        const int64_t sa = ad >= 0 ? A->batch_shape[ad] : 1;
        const int64_t sb = bd >= 0 ? B->batch_shape[bd] : 1;
        if (sa != sb && sa != 1 && sb != 1) return -1;
        bshape[d] = std::max(sa, sb);
        total *= bshape[d];
    }
    if (total == 0) total = 1;
    std::memset(C, 0, sizeof(float) * (size_t)(total * m * p));
    // NDBuffer.is_contiguous looks at the whole view including batch dims (ndbuffer.mojo:523-524)
    auto nd_contig = [](const tenmo_ref_mat* X, int64_t rows, int64_t cols) {
        if (!is_contiguous_2d(rows, cols, X->row_stride, X->col_stride)) return false;
        int64_t expect = rows * cols;
        for (int d = X->batch_rank - 1; d >= 0; --d) {
            if (X->batch_shape[d] > 1 && X->batch_stride[d] != expect) return false;
            expect *= X->batch_shape[d];
        }
        return true;
    };
    const bool a_contig = nd_contig(A, m, n), b_contig = nd_contig(B, n, p);
    const int64_t tiles_i = (m + T.m - 1) / T.m;
    parallel_for(total * tiles_i, o.threads, [&](int64_t flat) {
        const int64_t batch = flat / tiles_i, tile = flat % tiles_i;
        int64_t a_off = A->offset, b_off = B->offset;
        int64_t divisor = 1;  // right-to-left decode, matmul_cpu.mojo:710-724
        for (int d = r - 1; d >= 0; --d) {
            const int64_t coord = (batch / divisor) % bshape[d];
            const int ad = d - (r - ra), bd = d - (r - rb);
            if (ad >= 0 && A->batch_shape[ad] > 1) a_off += coord * A->batch_stride[ad];
            if (bd >= 0 && B->batch_shape[bd] > 1) b_off += coord * B->batch_stride[bd];
            divisor *= bshape[d];
        }
        float* c = C + batch * m * p;  // matmul_cpu.mojo:726
        const int64_t i0 = tile * T.m, i1 = std::min(i0 + T.m, m);
        if (b_contig) {
            rows_dispatch(a_contig, true, A->ptr, a_off, A->row_stride, A->col_stride, B->ptr, b_off, B->row_stride,
                          1, c, i0, i1, n, p, T, o);
        } else {
            // ND Path 2 is not j-tiled (matmul_cpu.mojo:931-952); per element it is the same k-ascending
            // scalar chain with partial sums parked in C between k tiles, so the 2D routine with one
            // full-width j tile reproduces it.
            Tiles T2 = T;
            T2.p = std::max<int64_t>(p, 1);
            rows_b_strided_2d(A->ptr, a_off, A->row_stride, A->col_stride, B->ptr, b_off, B->row_stride,
                              B->col_stride, c, i0, i1, n, p, T2, o.contract_scalar != 0);
        }
    });
    return total;
}

void tenmo_ref_matmul_naive(const tenmo_ref_mat* A, const tenmo_ref_mat* B, float* C, int64_t m, int64_t n,
                            int64_t p) {
    // tests/test_matmul_2d_verify.mojo:8-20: i, k, j with C[i,j] += A[i,k]*B[k,j]
    std::memset(C, 0, sizeof(float) * (size_t)(m * p));
    for (int64_t i = 0; i < m; ++i)
        for (int64_t k = 0; k < n; ++k) {
            const float a = A->ptr[A->offset + i * A->row_stride + k * A->col_stride];
            for (int64_t j = 0; j < p; ++j) {
                volatile float prod = a * B->ptr[B->offset + k * B->row_stride + j * B->col_stride];
                C[i * p + j] += prod;
            }
        }
}

void tenmo_ref_add_bias(const float* a, const float* b, float* out, int64_t M, int64_t N) {
    for (int64_t i = 0; i < M; ++i)
        for (int64_t j = 0; j < N; ++j) out[i * N + j] = a[i * N + j] + b[j];
}

void tenmo_ref_add_inplace(float* out, const float* in, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] += in[i];
}

void tenmo_ref_relu_fwd(const float* x, float* out, float* mask, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        const float v = x[i];
        out[i] = v > 0.f ? v : 0.f;  // max(x, 0): relu.mojo:121
        if (mask) mask[i] = v > 0.f ? 1.f : 0.f;
    }
}

void tenmo_ref_relu_bwd(const float* g, const float* mask, float* dx, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dx[i] = g[i] * mask[i];
}

void tenmo_ref_sigmoid_fwd(const float* x, float* y, int64_t n) {
    for (int64_t i = 0; i < n; ++i) y[i] = 1.f / (1.f + std::exp(-x[i]));
}

void tenmo_ref_sigmoid_bwd(const float* g, const float* y, float* dx, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        volatile float gy = g[i] * y[i];  // b * a * (one - a), left to right
        dx[i] = gy * (1.f - y[i]);
    }
}

void tenmo_ref_colsum(const float* x, float* out, int64_t M, int64_t N) {
    // coordinate-by-coordinate fallback: for each output n, accum += x[m,n], m ascending
    for (int64_t j = 0; j < N; ++j) {
        float accum = 0.f;
        for (int64_t i = 0; i < M; ++i) accum += x[i * N + j];
        out[j] = accum;
    }
}

int64_t tenmo_ref_ce_fwd(const float* logits, int64_t stride0, int64_t stride1, const int64_t* labels, int64_t M,
                         int64_t C, int64_t ignore_index, float label_smoothing, int reduction, float* softmax,
                         float* loss_out) {
    const bool has_ls = label_smoothing > 0.f;
    const bool none = reduction == 2;
    float scalar_loss = 0.f;
    int64_t valid = 0;
    for (int64_t row = 0; row < M; ++row) {
        const float* x = logits + row * stride0;
        float mx = -3.4028234663852886e38f;  // min_finite (crossentropy.mojo:333)
        for (int64_t c = 0; c < C; ++c) mx = std::max(mx, x[c * stride1]);
        float sum_exp = 0.f, sum_logits = 0.f;
        for (int64_t c = 0; c < C; ++c) {  // ascending c, sequential adds (346-366)
            const float v = x[c * stride1];
            const float e = std::exp(v - mx);
            sum_exp += e;
            if (has_ls) sum_logits += v;
            if (softmax) softmax[row * C + c] = e;
        }
        const float lse = std::log(std::max(sum_exp, 1e-7f));  // Epsilon[float32] = 1e-7 (common_utils.mojo:221)
        const bool is_valid = labels[row] != ignore_index;
        float loss = 0.f;
        if (is_valid) {
            const float logit_t = x[labels[row] * stride1];
            const float lsm_t = logit_t - mx - lse;
            loss = -lsm_t;
            if (has_ls) {
                const float inv_c = 1.f / (float)C;
                const float mean_lsm = sum_logits * inv_c - mx - lse;
                loss = (1.f - label_smoothing) * loss - label_smoothing * mean_lsm;
            }
            ++valid;
        }
        if (none) loss_out[row] = loss; else scalar_loss += loss;
        if (softmax) {
            const float inv = 1.f / sum_exp;  // multiply by the reciprocal (399-405)
            for (int64_t c = 0; c < C; ++c) softmax[row * C + c] *= inv;
        }
    }
    if (!none) {
        if (reduction == 0 && valid > 0) scalar_loss /= (float)valid;
        loss_out[0] = scalar_loss;
    }
    return valid;
}

void tenmo_ref_ce_bwd(const float* softmax, const int64_t* labels, int64_t M, int64_t C, int64_t ignore_index,
                      float label_smoothing, int reduction, const float* upstream, int64_t valid_count,
                      float* dlogits) {
    const float ls = label_smoothing;
    const float ls_uniform = ls / (float)C;
    float scale_mul = 0.f;
    if (reduction != 2) {
        const float scale = (float)((reduction == 0 && valid_count > 0) ? valid_count : 1);
        scale_mul = upstream[0] / scale;  // scalar_ops[Multiply](ug_scalar / scale), crossentropy.mojo:473-481
    }
    for (int64_t row = 0; row < M; ++row) {
        const bool ignored = labels[row] == ignore_index;
        const float mask = ignored ? 0.f : 1.f;
        for (int64_t c = 0; c < C; ++c) {
            const float onehot = (!ignored && labels[row] == c) ? 1.f : 0.f;  // ndbuffer.mojo:448-463
            float g = softmax[row * C + c];
            if (ls > 0.f) {
                volatile float oh = onehot * (1.f - ls);
                g = (g - oh) - ls_uniform;
            } else {
                g = g - onehot;
            }
            g = g * mask;
            g = g * (reduction == 2 ? upstream[row] : scale_mul);
            dlogits[row * C + c] = g;
        }
    }
}

void tenmo_ref_sgd_step(float* p, const float* g, float* v, int64_t n, float lr, float momentum, float wd) {
    // optim.mojo:100-158; products and sums rounded separately (Mojo's `a * b + c` on SIMD values
    // is written as two operations; no math.fma call there).
    for (int64_t k = 0; k < n; ++k) {
        float gk = g[k];
        const float pk = p[k];
        if (wd > 0.f) {
            volatile float t = pk * wd;
            gk += t;
        }
        if (momentum > 0.f) {
            volatile float mv = momentum * v[k];
            const float vk = mv + gk;
            v[k] = vk;
            volatile float step = lr * vk;
            p[k] = pk - step;
        } else {
            volatile float step = lr * gk;
            p[k] = pk - step;
        }
    }
}

int64_t tenmo_ref_accuracy(const float* logits, int64_t s0, int64_t s1, const int64_t* labels, int64_t M,
                           int64_t C) {
    int64_t correct = 0;
    for (int64_t row = 0; row < M; ++row) {
        const float* x = logits + row * s0;
        float mx = x[0];
        int64_t idx = 0;
        for (int64_t j = 1; j < C; ++j)
            if (x[j * s1] > mx) { mx = x[j * s1]; idx = j; }
        if (idx == labels[row]) ++correct;
    }
    return correct;
}

float tenmo_ref_mlp_step(int L, const int64_t* dims, float** W, float** b, float** vW, float** vb, float** dW,
                         float** db, const float* X, const int64_t* labels, int64_t batch, float lr,
                         float momentum, float wd, float grad_scale, int do_update, float* logits_out,
                         const tenmo_ref_opts* opts) {
    // Forward (net.mojo:1085-1092 -> 179-216): matmul, bias add, ReLU with a float mask between layers.
    std::vector<std::vector<float>> act(L + 1), mask(L);
    act[0].assign(X, X + batch * dims[0]);
    auto mat = [](const float* p, int64_t rs, int64_t cs) {
        tenmo_ref_mat m{};
        m.ptr = p; m.offset = 0; m.row_stride = rs; m.col_stride = cs; m.batch_rank = 0;
        return m;
    };
    for (int l = 0; l < L; ++l) {
        const int64_t in = dims[l], out = dims[l + 1];
        std::vector<float> z(batch * out);
        tenmo_ref_mat a = mat(act[l].data(), in, 1), w = mat(W[l], out, 1);
        tenmo_ref_matmul_2d(&a, &w, z.data(), batch, in, out, opts);
        if (b && b[l]) tenmo_ref_add_bias(z.data(), b[l], z.data(), batch, out);
        if (l + 1 < L) {
            act[l + 1].resize(batch * out);
            mask[l].resize(batch * out);
            tenmo_ref_relu_fwd(z.data(), act[l + 1].data(), mask[l].data(), batch * out);
        } else {
            act[l + 1] = std::move(z);
        }
    }
    const int64_t C = dims[L];
    if (logits_out) std::memcpy(logits_out, act[L].data(), sizeof(float) * batch * C);
    std::vector<float> sm(batch * C);
    float loss = 0.f;
    const int64_t valid = tenmo_ref_ce_fwd(act[L].data(), C, 1, labels, batch, C, -100, 0.f, 0, sm.data(), &loss);
    // Backward (tensor.mojo:3154-3247 order for this chain): CE, then per layer from the top:
    // add-broadcast (bias grad = column sum), matmul (dA = dC.B^T, dB = A^T.dC), ReLU (g*mask).
    std::vector<float> g(batch * C);
    const float one = 1.f;
    tenmo_ref_ce_bwd(sm.data(), labels, batch, C, -100, 0.f, 0, &one, valid, g.data());
    for (int l = L - 1; l >= 0; --l) {
        const int64_t in = dims[l], out = dims[l + 1];
        std::vector<float> gb(out), gw(in * out), ga;
        if (b && b[l]) tenmo_ref_colsum(g.data(), gb.data(), batch, out);
        tenmo_ref_mat dc = mat(g.data(), out, 1);
        if (l > 0) {  // the network input does not require grad (matmul.mojo:34)
            ga.resize(batch * in);
            tenmo_ref_mat wt = mat(W[l], 1, out);  // transpose view of (in,out): shape (out,in)
            tenmo_ref_matmul_2d(&dc, &wt, ga.data(), batch, out, in, opts);
        }
        tenmo_ref_mat at = mat(act[l].data(), 1, in);  // transpose view of (batch,in): shape (in,batch)
        tenmo_ref_matmul_2d(&at, &dc, gw.data(), in, batch, out, opts);
        if (dW && dW[l]) std::memcpy(dW[l], gw.data(), sizeof(float) * in * out);
        if (db && db[l] && b && b[l]) std::memcpy(db[l], gb.data(), sizeof(float) * out);
        if (do_update) {
            if (grad_scale != 1.f) {
                for (auto& x : gw) x *= grad_scale;
                for (auto& x : gb) x *= grad_scale;
            }
            tenmo_ref_sgd_step(W[l], gw.data(), vW[l], in * out, lr, momentum, wd);
            if (b && b[l]) tenmo_ref_sgd_step(b[l], gb.data(), vb[l], out, lr, momentum, wd);
        }
        if (l > 0) {
            g.resize(batch * in);
            tenmo_ref_relu_bwd(ga.data(), mask[l - 1].data(), g.data(), batch * in);
        }
    }
    return loss;
}

void tenmo_ref_conv2d_fwd(const float* img, const float* kernel, const float* bias, float* out, int64_t N, int64_t Cin,
                          int64_t Hp, int64_t Wp, int64_t Cout, int KH, int KW, int stride, int dilation, int contract) {
    const int64_t eh = (int64_t)(KH - 1) * dilation + 1, ew = (int64_t)(KW - 1) * dilation + 1;
    const int64_t Ho = (Hp - eh) / stride + 1, Wo = (Wp - ew) / stride + 1;
    for (int64_t n = 0; n < N; ++n)
        for (int64_t oy = 0; oy < Ho; ++oy)
            for (int64_t ox = 0; ox < Wo; ++ox)
                for (int64_t co = 0; co < Cout; ++co) {
                    float acc = bias ? bias[co] : 0.f;  // accumulator initialised with the bias (cnn.mojo:435)
                    for (int64_t ci = 0; ci < Cin; ++ci)
                        for (int ky = 0; ky < KH; ++ky)
                            for (int kx = 0; kx < KW; ++kx) {
                                const float v = img[((n * Cin + ci) * Hp + oy * stride + (int64_t)ky * dilation) * Wp +
                                                    ox * stride + (int64_t)kx * dilation];
                                const float w = kernel[((co * Cin + ci) * KH + ky) * KW + kx];
                                acc = scalar_site(v, w, acc, contract != 0);
                            }
                    out[((n * Cout + co) * Ho + oy) * Wo + ox] = acc;
                }
}

void tenmo_ref_conv2d_bwd(const float* grad, const float* img, const float* kernel, float* d_img, float* d_kernel,
                          float* d_bias, int64_t N, int64_t Cin, int64_t Hp, int64_t Wp, int64_t Cout, int KH, int KW,
                          int stride, int dilation) {
    const int64_t eh = (int64_t)(KH - 1) * dilation + 1, ew = (int64_t)(KW - 1) * dilation + 1;
    const int64_t Ho = (Hp - eh) / stride + 1, Wo = (Wp - ew) / stride + 1;
    if (d_bias)  // cnn.mojo:664-714: per channel, over n then the spatial positions
        for (int64_t co = 0; co < Cout; ++co) {
            float acc = 0.f;
            for (int64_t n = 0; n < N; ++n)
                for (int64_t s = 0; s < Ho * Wo; ++s) acc += grad[(n * Cout + co) * Ho * Wo + s];
            d_bias[co] = acc;
        }
    if (d_kernel)  // cnn.mojo:716-809: grad (C_out, N*Ho*Wo) . patches (N*Ho*Wo, C_in*KH*KW), patch index ascending
        for (int64_t co = 0; co < Cout; ++co)
            for (int64_t ci = 0; ci < Cin; ++ci)
                for (int ky = 0; ky < KH; ++ky)
                    for (int kx = 0; kx < KW; ++kx) {
                        float acc = 0.f;
                        for (int64_t n = 0; n < N; ++n)
                            for (int64_t oy = 0; oy < Ho; ++oy)
                                for (int64_t ox = 0; ox < Wo; ++ox)
                                    acc = fma_chain(grad[((n * Cout + co) * Ho + oy) * Wo + ox],
                                                    img[((n * Cin + ci) * Hp + oy * stride + (int64_t)ky * dilation) * Wp +
                                                        ox * stride + (int64_t)kx * dilation],
                                                    acc);
                        d_kernel[((co * Cin + ci) * KH + ky) * KW + kx] = acc;
                    }
    if (d_img) {  // cnn.mojo:812-950: scatter of kernel-weighted output gradients
        std::memset(d_img, 0, sizeof(float) * (size_t)(N * Cin * Hp * Wp));
        for (int64_t n = 0; n < N; ++n)
            for (int64_t co = 0; co < Cout; ++co)
                for (int64_t oy = 0; oy < Ho; ++oy)
                    for (int64_t ox = 0; ox < Wo; ++ox) {
                        const float g = grad[((n * Cout + co) * Ho + oy) * Wo + ox];
                        for (int64_t ci = 0; ci < Cin; ++ci)
                            for (int ky = 0; ky < KH; ++ky)
                                for (int kx = 0; kx < KW; ++kx)
                                    d_img[((n * Cin + ci) * Hp + oy * stride + (int64_t)ky * dilation) * Wp + ox * stride +
                                          (int64_t)kx * dilation] += g * kernel[((co * Cin + ci) * KH + ky) * KW + kx];
                    }
    }
}

void tenmo_ref_maxpool2d_fwd(const float* x, float* out, int64_t* argmax, int64_t NC, int64_t H, int64_t W, int k, int stride,
                             int pad) {
    const int64_t Ho = (H + 2 * pad - k) / stride + 1, Wo = (W + 2 * pad - k) / stride + 1;
    for (int64_t nc = 0; nc < NC; ++nc)
        for (int64_t oy = 0; oy < Ho; ++oy)
            for (int64_t ox = 0; ox < Wo; ++ox) {
                float best = -INFINITY;
                int64_t idx = -1;
                for (int ky = 0; ky < k; ++ky)
                    for (int kx = 0; kx < k; ++kx) {
                        const int64_t y = oy * stride - pad + ky, xx = ox * stride - pad + kx;
                        if (y < 0 || y >= H || xx < 0 || xx >= W) continue;
                        const float v = x[(nc * H + y) * W + xx];
                        if (v > best) { best = v; idx = y * W + xx; }
                    }
                out[(nc * Ho + oy) * Wo + ox] = best;
                argmax[(nc * Ho + oy) * Wo + ox] = idx;
            }
}

void tenmo_ref_maxpool2d_bwd(const float* g, const int64_t* argmax, float* dx, int64_t NC, int64_t H, int64_t W, int64_t Ho,
                             int64_t Wo) {
    std::memset(dx, 0, sizeof(float) * (size_t)(NC * H * W));
    for (int64_t nc = 0; nc < NC; ++nc)
        for (int64_t i = 0; i < Ho * Wo; ++i) {
            const int64_t idx = argmax[nc * Ho * Wo + i];
            if (idx >= 0) dx[nc * H * W + idx] += g[nc * Ho * Wo + i];
        }
}

// ---- softmax over the last axis of a contiguous (M, C) matrix -------------------------------------------------
// SoftmaxNdBuffer.softmax (softmax.mojo:30-48) = _softmax_components (:165-178: row max, x - max, exp) then
// SumMeanReduction.sum over the suffix axis, whose fast path is Buffer.sum (sum_mean_reduction.mojo:109-141 ->
// buffers.mojo:1304-1333): the row is walked in chunks of simd_width lanes, each chunk collapsed by reduce_add
// (restated as a halving tree, the order LLVM's reassociating vector reduction takes) and added to a scalar
// accumulator, then a scalar tail; finally exp / sum (a division, not a multiply by the reciprocal).
static float buffer_sum(const float* x, int64_t n, int simd) {
    float accum = 0.f;
    const int64_t vend = (n / simd) * simd;
    float lane[64];
    for (int64_t i = 0; i < vend; i += simd) {
        for (int l = 0; l < simd; ++l) lane[l] = x[i + l];
        for (int w = simd / 2; w >= 1; w /= 2)
            for (int l = 0; l < w; ++l) lane[l] = lane[l] + lane[l + w];
        accum += lane[0];
    }
    for (int64_t i = vend; i < n; ++i) accum += x[i];
    return accum;
}

void tenmo_ref_softmax_fwd(const float* x, float* y, int64_t M, int64_t C, int simd_width) {
    const int simd = (simd_width == 16) ? 16 : 8;
    std::vector<float> e((size_t)C);
    for (int64_t i = 0; i < M; ++i) {
        const float* row = x + i * C;
        float mx = row[0];
        for (int64_t j = 1; j < C; ++j) mx = row[j] > mx ? row[j] : mx;
        for (int64_t j = 0; j < C; ++j) e[(size_t)j] = std::exp(row[j] - mx);
        const float sum = buffer_sum(e.data(), C, simd);
        for (int64_t j = 0; j < C; ++j) y[i * C + j] = e[(size_t)j] / sum;
    }
}

// SoftmaxBackwardDelegate (softmax.mojo:206-213): gy = g * y; s = sum(gy) over the row (same Buffer.sum path);
// dx = y * (g - s).
void tenmo_ref_softmax_bwd(const float* g, const float* y, float* dx, int64_t M, int64_t C, int simd_width) {
    const int simd = (simd_width == 16) ? 16 : 8;
    std::vector<float> gy((size_t)C);
    for (int64_t i = 0; i < M; ++i) {
        for (int64_t j = 0; j < C; ++j) gy[(size_t)j] = g[i * C + j] * y[i * C + j];
        const float s = buffer_sum(gy.data(), C, simd);
        for (int64_t j = 0; j < C; ++j) dx[i * C + j] = y[i * C + j] * (g[i * C + j] - s);
    }
}

// ---- matrix @ vector and vector @ matrix -------------------------------------------------------------------------
// MatrixVectorMulNd.forward (matrixvector.mojo:269-282): out[i] = sum_j M[i,j] * v[j], one scalar accumulator per
// output, j ascending, `accumulator += m_val * v_val` (contraction is the compiler's choice, hence the option).
void tenmo_ref_mv(const float* Mx, int64_t m_s0, int64_t m_s1, const float* v, int64_t v_s, float* out, int64_t m,
                  int64_t k, int contract) {
    for (int64_t i = 0; i < m; ++i) {
        float acc = 0.f;
        for (int64_t j = 0; j < k; ++j) acc = scalar_site(Mx[i * m_s0 + j * m_s1], v[j * v_s], acc, contract != 0);
        out[i] = acc;
    }
}
// VectorMatmulNd.forward (vectormatrix.mojo:283-340): out[j] = sum_i v[i] * M[i,j]; the contiguous-row path keeps
// simd_width outputs in one vector accumulator and walks i ascending (`accumulator += v_val * m_vec`), the strided
// path does the same with scalars: either way every output is one i-ascending chain.
void tenmo_ref_vm(const float* v, int64_t v_s, const float* Mx, int64_t m_s0, int64_t m_s1, float* out, int64_t k,
                  int64_t n, int contract) {
    for (int64_t j = 0; j < n; ++j) {
        float acc = 0.f;
        for (int64_t i = 0; i < k; ++i) acc = scalar_site(v[i * v_s], Mx[i * m_s0 + j * m_s1], acc, contract != 0);
        out[j] = acc;
    }
}

}  // extern "C"
