// Strict-FP32 SIMT GEMM kernels (see gemm_simt.cuh).
//
// Tiling: a CTA of 256 threads owns a BM x BN tile of C and walks K in BK steps through two shared
// memory stages (global -> registers -> shared, so the next tile's loads are in flight while the
// current one is multiplied).  A thread owns a TM x TN register tile; for 8x8 it is split into four
// 4x4 quadrants so that the shared-memory reads of a warp are conflict-free 16-byte accesses.
// Roofline: FP32 pipe, 2*M*N*K flop against 2 * 128 lanes * SMs * clock.
#include <cstdlib>

#include "gemm_simt.cuh"

namespace {

constexpr int THREADS = 256;

template <int ROWS, int BK, bool INNER_K>
struct TileLoader {
    // A tile of ROWS (m or n index) x BK (k index), held in shared memory as [BK][ROWS + PAD].
    // Each thread moves groups of 4 elements that are consecutive along k (INNER_K) or along the
    // m/n index (!INNER_K); the caller picks the direction of the operand's unit stride so that the
    // global reads coalesce.
    static constexpr int PAD = 4;
    static constexpr int LD = ROWS + PAD;
    static constexpr int GROUPS = INNER_K ? BK / 4 : ROWS / 4;      // groups per line
    static constexpr int LINES_PER_PASS = THREADS / GROUPS;          // lines handled per pass
    static constexpr int LINES = INNER_K ? ROWS : BK;
    static constexpr int PASSES = LINES / LINES_PER_PASS;
    static_assert(LINES % LINES_PER_PASS == 0 && PASSES >= 1, "tile does not divide over 256 threads");

    float4 reg[PASSES];

    __device__ __forceinline__ void load(const float* __restrict__ base, int64_t s_mn, int64_t s_k, int64_t mn0,
                                         int64_t k0, int64_t MN, int64_t K, bool vec, int tid) {
        const int g = tid % GROUPS, line = tid / GROUPS;
#pragma unroll
        for (int p = 0; p < PASSES; ++p) {
            const int l = line + p * LINES_PER_PASS;
            int64_t mn, k;
            if (INNER_K) { mn = mn0 + l; k = k0 + g * 4; } else { mn = mn0 + g * 4; k = k0 + l; }
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            const float* ptr = base + mn * s_mn + k * s_k;
            if (INNER_K) {
                if (mn < MN) {
                    if (vec && k + 3 < K) {
                        v = __ldg(reinterpret_cast<const float4*>(ptr));
                    } else {
                        if (k + 0 < K) v.x = __ldg(ptr);
                        if (k + 1 < K) v.y = __ldg(ptr + s_k);
                        if (k + 2 < K) v.z = __ldg(ptr + 2 * s_k);
                        if (k + 3 < K) v.w = __ldg(ptr + 3 * s_k);
                    }
                }
            } else {
                if (k < K) {
                    if (vec && mn + 3 < MN) {
                        v = __ldg(reinterpret_cast<const float4*>(ptr));
                    } else {
                        if (mn + 0 < MN) v.x = __ldg(ptr);
                        if (mn + 1 < MN) v.y = __ldg(ptr + s_mn);
                        if (mn + 2 < MN) v.z = __ldg(ptr + 2 * s_mn);
                        if (mn + 3 < MN) v.w = __ldg(ptr + 3 * s_mn);
                    }
                }
            }
            reg[p] = v;
        }
    }

    __device__ __forceinline__ void store(float* __restrict__ tile, int tid) const {
        const int g = tid % GROUPS, line = tid / GROUPS;
#pragma unroll
        for (int p = 0; p < PASSES; ++p) {
            const int l = line + p * LINES_PER_PASS;
            if (INNER_K) {
                float* dst = tile + (g * 4) * LD + l;
                dst[0] = reg[p].x;
                dst[LD] = reg[p].y;
                dst[2 * LD] = reg[p].z;
                dst[3 * LD] = reg[p].w;
            } else {
                *reinterpret_cast<float4*>(tile + l * LD + g * 4) = reg[p];
            }
        }
    }
};

__device__ __forceinline__ float apply_act(float v, int act) {
    if (act == TENMO_ACT_RELU) return v > 0.f ? v : 0.f;
    if (act == TENMO_ACT_SIGMOID) return 1.f / (1.f + expf(-v));
    return v;
}

// Row / column owned by register index i of a thread (quadrant split for 8-wide register tiles).
template <int T, int B>
__device__ __forceinline__ int frag_index(int t, int i) {
    if (T == 8) return (i / 4) * (B / 2) + t * 4 + (i % 4);
    return t * T + i;
}

template <int BM, int BN, int BK, int TM, int TN, bool A_INNER_K, bool B_INNER_K>
__global__ void __launch_bounds__(THREADS, BM == 128 ? 2 : 1) gemm_simt_kernel(const TenmoGemmParams p) {
    static_assert((BM / TM) * (BN / TN) == THREADS, "thread tile must cover the CTA tile");
    using LoaderA = TileLoader<BM, BK, A_INNER_K>;
    using LoaderB = TileLoader<BN, BK, B_INNER_K>;
    __shared__ __align__(16) float As[2][BK * LoaderA::LD];
    __shared__ __align__(16) float Bs[2][BK * LoaderB::LD];
    tenmo_grid_dependency_sync();

    const int tid = threadIdx.x;
    // tile decode: blockIdx.x = (batch * tiles_m + tile_m) * tiles_n + tile_n
    int64_t bid = blockIdx.x;
    const int tile_n = (int)(bid % p.tiles_n);
    bid /= p.tiles_n;
    const int tile_m = (int)(bid % p.tiles_m);
    const int64_t batch = bid / p.tiles_m;

    // batch index decoded right to left; an operand's stride is 0 where it is broadcast
    const float* A = p.A;
    const float* B = p.B;
    {
        int64_t rem = batch;
#pragma unroll 1
        for (int d = p.batch.rank - 1; d >= 0; --d) {
            const int64_t coord = rem % p.batch.shape[d];
            rem /= p.batch.shape[d];
            A += coord * p.batch.a_stride[d];
            B += coord * p.batch.b_stride[d];
        }
    }
    float* C = p.C + batch * p.M * p.N;
    float* AUX = p.aux ? p.aux + batch * p.M * p.N : nullptr;

    const int64_t m0 = (int64_t)tile_m * BM, n0 = (int64_t)tile_n * BN;
    constexpr int TX = BN / TN;
    const int tx = tid % TX, ty = tid / TX;

    // accumulators as pairs of neighbouring columns: the k loop multiplies with the packed fma.rn.f32x2 (two
    // independent round-to-nearest fused multiply-adds, the same bits as two fmaf, half the instructions).  The
    // 128 x 128 tile holds its next tile in registers as well and spills in the packed form, so it keeps fmaf.
    constexpr bool PACKED = BM < 128;
    float2 acc[TM][TN / 2];
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        // a per-row bias is the accumulator's starting value, as in the reference's convolution (cnn.mojo:435)
        float init = 0.f;
        if (p.bias_m) {
            const int64_t m = m0 + frag_index<TM, BM>(ty, i);
            if (m < p.M) init = __ldg(p.bias_m + m);
        }
#pragma unroll
        for (int j = 0; j < TN / 2; ++j) acc[i][j] = make_float2(init, init);
    }

    // Column sums of B riding along (2-D calls only): the CTAs of the first tile row see every k of their columns pass
    // through shared memory; their ty == 0 threads add them in ascending k, the reference's sequential sum.
    constexpr bool CAN_COLSUM = BM < 128;
    const bool do_cs = CAN_COLSUM && p.colsum != nullptr && tile_m == 0 && ty == 0;
    float cs[TN];
#pragma unroll
    for (int j = 0; j < TN; ++j) cs[j] = 0.f;

    LoaderA la;
    LoaderB lb;
    const int64_t k_tiles = (p.K + BK - 1) / BK;
    la.load(A, p.a_rs, p.a_cs, m0, 0, p.M, p.K, p.a_vec != 0, tid);
    lb.load(B, p.b_cs, p.b_rs, n0, 0, p.N, p.K, p.b_vec != 0, tid);
    la.store(As[0], tid);
    lb.store(Bs[0], tid);
    __syncthreads();

    for (int64_t kt = 0; kt < k_tiles; ++kt) {
        const int cur = (int)(kt & 1);
        const bool has_next = kt + 1 < k_tiles;
        if (has_next) {
            la.load(A, p.a_rs, p.a_cs, m0, (kt + 1) * BK, p.M, p.K, p.a_vec != 0, tid);
            lb.load(B, p.b_cs, p.b_rs, n0, (kt + 1) * BK, p.N, p.K, p.b_vec != 0, tid);
        }
        const float* as = As[cur];
        const float* bs = Bs[cur];
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
            if (TM == 8) {
                *reinterpret_cast<float4*>(&a[0]) = *reinterpret_cast<const float4*>(as + kk * LoaderA::LD + ty * 4);
                *reinterpret_cast<float4*>(&a[4]) =
                    *reinterpret_cast<const float4*>(as + kk * LoaderA::LD + BM / 2 + ty * 4);
            } else if (TM == 4) {
                *reinterpret_cast<float4*>(&a[0]) = *reinterpret_cast<const float4*>(as + kk * LoaderA::LD + ty * 4);
            } else {
#pragma unroll
                for (int i = 0; i < TM; ++i) a[i] = as[kk * LoaderA::LD + ty * TM + i];
            }
            if (TN == 8) {
                *reinterpret_cast<float4*>(&b[0]) = *reinterpret_cast<const float4*>(bs + kk * LoaderB::LD + tx * 4);
                *reinterpret_cast<float4*>(&b[4]) =
                    *reinterpret_cast<const float4*>(bs + kk * LoaderB::LD + BN / 2 + tx * 4);
            } else if (TN == 4) {
                *reinterpret_cast<float4*>(&b[0]) = *reinterpret_cast<const float4*>(bs + kk * LoaderB::LD + tx * 4);
            } else {
#pragma unroll
                for (int j = 0; j < TN; ++j) b[j] = bs[kk * LoaderB::LD + tx * TN + j];
            }
            if (CAN_COLSUM && do_cs) {
#pragma unroll
                for (int j = 0; j < TN; ++j) cs[j] += b[j];
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN / 2; ++j)
                    acc[i][j] = PACKED ? __ffma2_rn(make_float2(a[i], a[i]), make_float2(b[2 * j], b[2 * j + 1]), acc[i][j])
                                       : make_float2(fmaf(a[i], b[2 * j], acc[i][j].x), fmaf(a[i], b[2 * j + 1], acc[i][j].y));
        }
        if (has_next) {
            la.store(As[cur ^ 1], tid);
            lb.store(Bs[cur ^ 1], tid);
        }
        __syncthreads();
    }

    if (CAN_COLSUM && do_cs) {
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int64_t n = n0 + frag_index<TN, BN>(tx, j);
            if (n < p.N) p.colsum[n] = p.beta != 0.f ? p.colsum[n] + cs[j] : cs[j];
        }
    }

    // Epilogue: bias, activation (+ mask), accumulate, store.
    constexpr int CW = (TN >= 4) ? 4 : TN;  // columns per store group
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int64_t m = m0 + frag_index<TM, BM>(ty, i);
        if (m >= p.M) continue;
#pragma unroll
        for (int jg = 0; jg < TN / CW; ++jg) {
            const int64_t n = n0 + frag_index<TN, BN>(tx, jg * CW);
            if (n >= p.N) continue;
            float v[CW], mk[CW];
#pragma unroll
            for (int q = 0; q < CW; ++q) {
                float x = ((jg * CW + q) & 1) ? acc[i][(jg * CW + q) >> 1].y : acc[i][(jg * CW + q) >> 1].x;
                if (p.bias && n + q < p.N) x += __ldg(p.bias + n + q);
                mk[q] = x > 0.f ? 1.f : 0.f;
                v[q] = apply_act(x, p.act);
            }
            float* dst = C + m * p.N + n;
            const bool extended = p.mul_mask != nullptr || p.c_lo != nullptr;
            if (CW == 4 && p.c_vec && n + 3 < p.N && !extended) {
                float4 o = make_float4(v[0], v[1], v[2], v[3]);
                if (p.beta != 0.f) {
                    const float4 old = *reinterpret_cast<const float4*>(dst);
                    o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4*>(dst) = o;
                if (AUX) *reinterpret_cast<float4*>(AUX + m * p.N + n) = make_float4(mk[0], mk[1], mk[2], mk[3]);
            } else {
#pragma unroll
                for (int q = 0; q < CW; ++q) {
                    if (n + q < p.N) {
                        float o = v[q];
                        if (p.mul_mask) o *= __ldg(p.mul_mask + (batch * p.M + m) * p.N + n + q);
                        if (p.beta != 0.f) o += dst[q];
                        dst[q] = o;
                        if (AUX) AUX[m * p.N + n + q] = mk[q];
                        if (p.c_lo) p.c_lo[(batch * p.M + m) * p.ld_clo + n + q] = tenmo_tf32_lo(o);
                    }
                }
            }
        }
    }
}

template <int BM, int BN, int BK, int TM, int TN>
cudaError_t launch_cfg(const TenmoGemmParams& p, bool a_inner_k, bool b_inner_k, int64_t grid, cudaStream_t s, bool pdl) {
    cudaError_t e;
    if (a_inner_k) {
        if (b_inner_k) e = tenmo_launch(gemm_simt_kernel<BM, BN, BK, TM, TN, true, true>, (unsigned)grid, THREADS, 0, s, pdl, p);
        else e = tenmo_launch(gemm_simt_kernel<BM, BN, BK, TM, TN, true, false>, (unsigned)grid, THREADS, 0, s, pdl, p);
    } else {
        if (b_inner_k) e = tenmo_launch(gemm_simt_kernel<BM, BN, BK, TM, TN, false, true>, (unsigned)grid, THREADS, 0, s, pdl, p);
        else e = tenmo_launch(gemm_simt_kernel<BM, BN, BK, TM, TN, false, false>, (unsigned)grid, THREADS, 0, s, pdl, p);
    }
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace

int tenmo_gemm_simt_launch(tenmo_ctx* ctx, const TenmoGemmParams& p_in, bool* colsum_done) {
    TenmoGemmParams p = p_in;
    if (colsum_done) *colsum_done = false;
    auto absl = [](int64_t v) { return v < 0 ? -v : v; };
    // Group loads along the axis with the smaller stride (the unit-stride axis when there is one).
    const bool a_inner_k = absl(p.a_cs) <= absl(p.a_rs);
    const bool b_inner_k = absl(p.b_rs) < absl(p.b_cs);
    // vector loads need unit stride on the grouped axis, a 16-byte aligned base and 16-byte multiples elsewhere
    auto aligned16 = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; };
    auto batch_ok = [&](const int64_t* st) {
        for (int d = 0; d < p.batch.rank; ++d)
            if (st[d] % 4 != 0) return false;
        return true;
    };
    p.a_vec = a_inner_k ? (p.a_cs == 1 && p.a_rs % 4 == 0) : (p.a_rs == 1 && p.a_cs % 4 == 0);
    p.a_vec = p.a_vec && aligned16(p.A) && batch_ok(p.batch.a_stride);
    p.b_vec = b_inner_k ? (p.b_rs == 1 && p.b_cs % 4 == 0) : (p.b_cs == 1 && p.b_rs % 4 == 0);
    p.b_vec = p.b_vec && aligned16(p.B) && batch_ok(p.batch.b_stride);
    p.c_vec = (p.N % 4 == 0) && aligned16(p.C) && (!p.aux || aligned16(p.aux));

    if (tenmo_gemm_skinny_supported(p)) return tenmo_gemm_skinny_launch(ctx, p);
    auto tiles = [&](int bm, int bn) {
        return ((p.M + bm - 1) / bm) * ((p.N + bn - 1) / bn) * p.total_batch;
    };
    int cfg;
    if (tiles(128, 128) >= ctx->sm_count) cfg = 128;
    else if (tiles(64, 64) >= ctx->sm_count / 2) cfg = 64;
    else cfg = 32;
    if (cfg == 128 && (p.M <= 64 || p.N <= 64)) cfg = 64;
    if (cfg == 64 && (p.M <= 32 || p.N <= 32)) cfg = 32;
    if (cfg == 128) p.colsum = nullptr;  // the 128 x 128 tiles leave the column sum to its own kernel
    if (cfg == 128 && p.K >= 64) {
        const char* env = getenv("TENMO_SIMT_TMA");  // "0" keeps the register-staged kernel (for comparisons)
        if (!(env && env[0] == '0') && tenmo_gemm_simt_tma_supported(ctx, p)) return tenmo_gemm_simt_tma_launch(ctx, p);
    }
    const int bm = cfg, bn = cfg;
    p.tiles_m = (int)((p.M + bm - 1) / bm);
    p.tiles_n = (int)((p.N + bn - 1) / bn);
    const int64_t grid = (int64_t)p.tiles_m * p.tiles_n * p.total_batch;
    if (grid <= 0 || grid > 0x7fffffffLL)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "gemm: grid of %lld tiles is out of range", (long long)grid);
    cudaError_t e;
    tenmo_prof_before(ctx);
    if (cfg == 128) e = launch_cfg<128, 128, 16, 8, 8>(p, a_inner_k, b_inner_k, grid, ctx->stream, tenmo_pdl_ok(ctx, grid));
    else if (cfg == 64) e = launch_cfg<64, 64, 16, 4, 4>(p, a_inner_k, b_inner_k, grid, ctx->stream, tenmo_pdl_ok(ctx, grid));
    else if (p.K <= 32) e = launch_cfg<32, 32, 32, 2, 2>(p, a_inner_k, b_inner_k, grid, ctx->stream, tenmo_pdl_ok(ctx, grid));
    else e = launch_cfg<32, 32, 64, 2, 2>(p, a_inner_k, b_inner_k, grid, ctx->stream, tenmo_pdl_ok(ctx, grid));  // deep k-tiles: fewer load round trips
    if (colsum_done) *colsum_done = p.colsum != nullptr;
    tenmo_prof_after(ctx);
    ctx->launches++;
    ctx->last_gemm_kernel = "gemm_simt_kernel";
    ctx->last_gemm_sk_units = 0;
    if (e != cudaSuccess)
        return tenmo_set_error(ctx, TENMO_ERR_CUDA, "launch of gemm_simt_kernel failed: %s", cudaGetErrorString(e));
    return TENMO_OK;
}
