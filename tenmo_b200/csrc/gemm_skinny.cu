// Strict-fp32 GEMM for a narrow result and a long contraction: C(M, N <= 32) = A(M, K) . B(K, N) with K in the thousands
// (the classifier layer of a CNN: (batch, 4096) . (4096, 10)).  Every output is still ONE k-ascending fmaf chain, as in
// the other strict kernels and in the reference's CPU loops (matmul_cpu.mojo:275-312), so the bits are the same; what
// changes is what sits between two links of the chain.  The square-tile kernel spends a global load, a shared-memory
// store and a block barrier per 64 links with a handful of CTAs in flight; here a CTA is eight rows (one warp each,
// lane = column), the next 256-deep slice of A and B is fetched into registers while the current one is multiplied out of
// shared memory, and a link costs one broadcast read, one conflict-free read and the FMA.
#include "gemm_simt.cuh"

namespace {

constexpr int SK_ROWS = 8;            // rows (= warps) per CTA
constexpr int SK_THREADS = SK_ROWS * 32;
constexpr int SK_KC = 256;            // k-slice staged at a time: its chain of 256 links outlasts the latency of the next fetch
constexpr int SK_BP = 33;             // pitch of a staged B row: lane n reads column n without conflicts

__device__ __forceinline__ float sk_act(float v, int act) {
    if (act == TENMO_ACT_RELU) return v > 0.f ? v : 0.f;
    if (act == TENMO_ACT_SIGMOID) return 1.f / (1.f + expf(-v));
    return v;
}

__global__ void __launch_bounds__(SK_THREADS) gemm_skinny_kernel(const TenmoGemmParams p) {
    __shared__ float as[SK_ROWS][SK_KC];
    __shared__ float bs[SK_KC * SK_BP];
    tenmo_grid_dependency_sync();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t m = (int64_t)blockIdx.x * SK_ROWS + warp;
    const int N = (int)p.N;
    const bool row_ok = m < p.M;
    constexpr int A_PER = SK_KC / 32;                       // A values per lane and slice
    constexpr int B_PER = SK_KC / SK_ROWS;                  // B values per lane and slice: warp w takes rows w, w + 8, ...
    float ra[A_PER], rb[B_PER];
    auto fetch = [&](int64_t k0) {
#pragma unroll
        for (int j = 0; j < A_PER; ++j) {
            const int64_t k = k0 + lane + 32 * j;
            ra[j] = (row_ok && k < p.K) ? __ldg(p.A + m * p.a_rs + k * p.a_cs) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < B_PER; ++j) {
            const int64_t k = k0 + warp + SK_ROWS * j;      // lane = column: a row of a row-major B is one coalesced read
            rb[j] = (lane < N && k < p.K) ? __ldg(p.B + k * p.b_rs + lane * p.b_cs) : 0.f;
        }
    };
    auto park = [&]() {
#pragma unroll
        for (int j = 0; j < A_PER; ++j) as[warp][lane + 32 * j] = ra[j];
#pragma unroll
        for (int j = 0; j < B_PER; ++j) bs[(warp + SK_ROWS * j) * SK_BP + lane] = rb[j];
    };
    float acc = (p.bias_m && row_ok) ? __ldg(p.bias_m + m) : 0.f;   // a per-row bias starts the chain (cnn.mojo:435)
    fetch(0);
    for (int64_t k0 = 0; k0 < p.K; k0 += SK_KC) {
        __syncthreads();          // the previous slice has been consumed
        park();
        __syncthreads();
        if (k0 + SK_KC < p.K) fetch(k0 + SK_KC);   // in flight while the chain below runs
        const int kn = (int)((p.K - k0) < SK_KC ? (p.K - k0) : SK_KC);
        if (lane < N) {
            if (kn == SK_KC) {
#pragma unroll 16
                for (int kk = 0; kk < SK_KC; ++kk) acc = fmaf(as[warp][kk], bs[kk * SK_BP + lane], acc);
            } else {
                for (int kk = 0; kk < kn; ++kk) acc = fmaf(as[warp][kk], bs[kk * SK_BP + lane], acc);
            }
        }
    }
    if (!row_ok || lane >= N) return;
    float x = acc;
    if (p.bias) x += __ldg(p.bias + lane);
    const float mk = x > 0.f ? 1.f : 0.f;
    float o = sk_act(x, p.act);
    const int64_t at = m * p.N + lane;
    if (p.mul_mask) o *= __ldg(p.mul_mask + at);
    if (p.beta != 0.f) o += p.C[at];
    p.C[at] = o;
    if (p.aux) p.aux[at] = mk;
    if (p.c_lo) p.c_lo[m * p.ld_clo + lane] = tenmo_tf32_lo(o);
}

}  // namespace

bool tenmo_gemm_skinny_supported(const TenmoGemmParams& p) {
    // one lane per column: N <= 32
    return p.total_batch == 1 && p.batch.rank == 0 && p.N >= 1 && p.N <= 32 && p.K >= 512 && p.M >= 1 && !p.colsum;
}

int tenmo_gemm_skinny_launch(tenmo_ctx* ctx, const TenmoGemmParams& p) {
    const int64_t grid = (p.M + SK_ROWS - 1) / SK_ROWS;
    if (grid > 0x7fffffffLL) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "gemm: too many rows for the narrow-result kernel");
    tenmo_prof_before(ctx);
    cudaError_t e = tenmo_launch(gemm_skinny_kernel, (unsigned)grid, SK_THREADS, 0, ctx->stream, tenmo_pdl_ok(ctx, grid), p);
    if (e == cudaSuccess) e = cudaGetLastError();
    tenmo_prof_after(ctx);
    ctx->launches++;
    ctx->last_gemm_kernel = "gemm_skinny_kernel";
    ctx->last_gemm_sk_units = 0;
    if (e != cudaSuccess) return tenmo_set_error(ctx, TENMO_ERR_CUDA, "launch of gemm_skinny_kernel failed: %s", cudaGetErrorString(e));
    return TENMO_OK;
}
