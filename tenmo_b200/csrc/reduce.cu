// Column sum  out[n] = sum_m x[m, n]  -- the bias gradient and the sum over a broadcast batch.
//
// HBM-bound: reads 4*M*N bytes once, coalesced (a warp reads 512 contiguous bytes of a row per step,
// where the reference's reduction kernel strides down a column, kernels/reduction_kernel.mojo:136-214).
// Two shapes of kernel:
//   * few rows (M <= COLSUM_SEQ_ROWS): one thread per column adds its rows in ascending order, which
//     is bit-identical to tenmo's CPU reduction (sum_mean_reduction.mojo:143-156);
//   * many rows: the rows are split over CTAs; each CTA reduces its slab of a 128-column strip and
//     parks a partial in scratch memory, and the last CTA of a strip to finish (ticket counter) adds
//     the partials in slab order, so the result does not depend on scheduling.
#include <atomic>

#include "common.cuh"
#include "reduce.cuh"

namespace {

constexpr int CS_THREADS = 256;
constexpr int CS_WARPS = CS_THREADS / 32;

__global__ void __launch_bounds__(CS_THREADS) colsum_seq_kernel(const float* __restrict__ x, int64_t M, int64_t N,
                                                               int64_t ldx, float* __restrict__ out, float beta) {
    const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    // rows are added in ascending order (the reference's sequential sum); sixteen loads are issued before the
    // first add so that the walk is not one memory latency per row
    float acc = 0.f;
    int64_t m = 0;
    for (; m + 16 <= M; m += 16) {
        float v[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) v[u] = __ldg(x + (m + u) * ldx + n);
#pragma unroll
        for (int u = 0; u < 16; ++u) acc += v[u];
    }
    for (; m < M; ++m) acc += __ldg(x + m * ldx + n);
    out[n] = beta != 0.f ? out[n] + acc : acc;
}

// VEC = 4: float4 loads (needs N % 4 == 0, ldx % 4 == 0, aligned base); VEC = 1: scalar loads.
template <int VEC>
__global__ void __launch_bounds__(CS_THREADS)
colsum_split_kernel(const float* __restrict__ x, int64_t M, int64_t N, int64_t ldx, float* __restrict__ out,
                    float beta, float* __restrict__ partials, unsigned int* __restrict__ tickets, int rows_per_slab) {
    constexpr int STRIP = 32 * VEC;
    __shared__ float red[CS_WARPS][STRIP];
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
        // 8 rows in flight per warp step (4 KB per warp with 16-byte loads) to cover HBM latency
        int64_t m = m_begin + warp;
        for (; m + 7 * CS_WARPS < m_end; m += 8 * CS_WARPS) {
            if (VEC == 4) {
                float4 r[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) r[u] = __ldcs(reinterpret_cast<const float4*>(x + (m + u * CS_WARPS) * ldx + n0));
                acc[0] += ((r[0].x + r[1].x) + (r[2].x + r[3].x)) + ((r[4].x + r[5].x) + (r[6].x + r[7].x));
                acc[1 % VEC] += ((r[0].y + r[1].y) + (r[2].y + r[3].y)) + ((r[4].y + r[5].y) + (r[6].y + r[7].y));
                acc[2 % VEC] += ((r[0].z + r[1].z) + (r[2].z + r[3].z)) + ((r[4].z + r[5].z) + (r[6].z + r[7].z));
                acc[3 % VEC] += ((r[0].w + r[1].w) + (r[2].w + r[3].w)) + ((r[4].w + r[5].w) + (r[6].w + r[7].w));
            } else {
                float r[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) r[u] = __ldg(x + (m + u * CS_WARPS) * ldx + n0);
                acc[0] += ((r[0] + r[1]) + (r[2] + r[3])) + ((r[4] + r[5]) + (r[6] + r[7]));
            }
        }
        for (; m + 3 * CS_WARPS < m_end; m += 4 * CS_WARPS) {
            if (VEC == 4) {
                const float4 a = __ldg(reinterpret_cast<const float4*>(x + m * ldx + n0));
                const float4 b = __ldg(reinterpret_cast<const float4*>(x + (m + CS_WARPS) * ldx + n0));
                const float4 c = __ldg(reinterpret_cast<const float4*>(x + (m + 2 * CS_WARPS) * ldx + n0));
                const float4 d = __ldg(reinterpret_cast<const float4*>(x + (m + 3 * CS_WARPS) * ldx + n0));
                acc[0] += (a.x + b.x) + (c.x + d.x);
                acc[1 % VEC] += (a.y + b.y) + (c.y + d.y);
                acc[2 % VEC] += (a.z + b.z) + (c.z + d.z);
                acc[3 % VEC] += (a.w + b.w) + (c.w + d.w);
            } else {
                const float a = __ldg(x + m * ldx + n0), b = __ldg(x + (m + CS_WARPS) * ldx + n0);
                const float c = __ldg(x + (m + 2 * CS_WARPS) * ldx + n0), d = __ldg(x + (m + 3 * CS_WARPS) * ldx + n0);
                acc[0] += (a + b) + (c + d);
            }
        }
        for (; m < m_end; m += CS_WARPS) {
            if (VEC == 4) {
                const float4 a = __ldg(reinterpret_cast<const float4*>(x + m * ldx + n0));
                acc[0] += a.x; acc[1 % VEC] += a.y; acc[2 % VEC] += a.z; acc[3 % VEC] += a.w;
            } else {
                acc[0] += __ldg(x + m * ldx + n0);
            }
        }
    }
#pragma unroll
    for (int q = 0; q < VEC; ++q) red[warp][lane * VEC + q] = acc[q];
    __syncthreads();
    // one partial per column of the strip for this slab
    if (threadIdx.x < STRIP) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < CS_WARPS; ++w) s += red[w][threadIdx.x];
        const int64_t n = (int64_t)strip * STRIP + threadIdx.x;
        if (n < N) partials[(int64_t)slab * N + n] = s;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int t = atomicAdd(&tickets[strip], 1u);
        is_last = (t == (unsigned int)slabs - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (threadIdx.x < STRIP) {
        const int64_t n = (int64_t)strip * STRIP + threadIdx.x;
        if (n < N) {
            float s = 0.f;
            for (int sl = 0; sl < slabs; ++sl) s += __ldcg(partials + (int64_t)sl * N + n);
            out[n] = beta != 0.f ? out[n] + s : s;
        }
    }
    if (threadIdx.x == 0) tickets[strip] = 0;  // ready for the next call
}

}  // namespace

void tenmo_colsum_plan(int sm_count, int64_t M, int64_t N, bool vec, int* strips, int* slabs, int* rows_per_slab) {
    const int strip_w = vec ? 128 : 32;
    const int64_t ns = (N + strip_w - 1) / strip_w;
    // aim for ~6 CTAs per SM in total, at least 64 rows per slab
    int64_t want = ((int64_t)sm_count * 6 + ns - 1) / ns;
    int64_t max_slabs = (M + 63) / 64;
    if (want > max_slabs) want = max_slabs;
    if (want < 1) want = 1;
    if (want > 1024) want = 1024;
    int64_t rps = (M + want - 1) / want;
    rps = (rps + CS_WARPS - 1) / CS_WARPS * CS_WARPS;
    *strips = (int)ns;
    *rows_per_slab = (int)rps;
    *slabs = (int)((M + rps - 1) / rps);
}

int tenmo_colsum_launch(tenmo_ctx* ctx, const float* x, int64_t M, int64_t N, int64_t ldx, float* out, float beta,
                        float* partials, unsigned int* tickets, int strips, int slabs, int rows_per_slab, bool vec) {
    dim3 grid((unsigned)strips, (unsigned)slabs);
    if (vec)
        colsum_split_kernel<4><<<grid, CS_THREADS, 0, ctx->stream>>>(x, M, N, ldx, out, beta, partials, tickets,
                                                                      rows_per_slab);
    else
        colsum_split_kernel<1><<<grid, CS_THREADS, 0, ctx->stream>>>(x, M, N, ldx, out, beta, partials, tickets,
                                                                      rows_per_slab);
    TENMO_LAUNCH_CHECK(ctx, "colsum_split_kernel");
    return TENMO_OK;
}

// Scratch of the split kernels: slabs*N partial sums (workspace) and one ticket counter per strip (kept at zero between calls).
int tenmo_colsum_scratch(tenmo_ctx* ctx, int slabs, int64_t N, int strips, float** partials, unsigned int** tickets) {
    void* ws = nullptr;
    int st = tenmo_workspace(ctx, (size_t)slabs * (size_t)N * sizeof(float), &ws);
    if (st != TENMO_OK) return st;
    if (strips > ctx->tickets_cap) {
        if (ctx->tickets) {
            TENMO_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
            cudaFree(ctx->tickets);
            ctx->tickets = nullptr;
            ctx->tickets_cap = 0;
        }
        const int cap = strips < 1024 ? 1024 : strips;
        TENMO_CUDA_TRY(ctx, cudaMalloc(&ctx->tickets, (size_t)cap * sizeof(unsigned int)));
        TENMO_CUDA_TRY(ctx, cudaMemset(ctx->tickets, 0, (size_t)cap * sizeof(unsigned int)));
        ctx->tickets_cap = cap;
    }
    *partials = static_cast<float*>(ws);
    *tickets = ctx->tickets;
    return TENMO_OK;
}

extern "C" int tenmo_colsum_f32(tenmo_ctx* ctx, const float* x, int64_t M, int64_t N, int64_t ldx, float* out,
                                float beta) {
    TENMO_CHECK_CTX(ctx);
    if (M < 0 || N < 0) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "colsum: negative shape");
    if (beta != 0.f && beta != 1.f) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "colsum: beta must be 0 or 1");
    if (N == 0) return TENMO_OK;
    if (!out || (M > 0 && !x)) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "colsum: NULL pointer");
    if (M > 0 && ldx < N) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "colsum: ldx (%lld) < N (%lld)", (long long)ldx, (long long)N);
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    if (M <= TENMO_COLSUM_SEQ_ROWS) {
        const int grid = (int)((N + CS_THREADS - 1) / CS_THREADS);
        colsum_seq_kernel<<<grid, CS_THREADS, 0, ctx->stream>>>(x, M, N, ldx, out, beta);
        TENMO_LAUNCH_CHECK(ctx, "colsum_seq_kernel");
        return TENMO_OK;
    }
    const bool vec = (N % 4 == 0) && (ldx % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15u) == 0);
    int strips, slabs, rps;
    tenmo_colsum_plan(ctx->sm_count, M, N, vec, &strips, &slabs, &rps);
    float* partials = nullptr;
    unsigned int* tickets = nullptr;
    int st = tenmo_colsum_scratch(ctx, slabs, N, strips, &partials, &tickets);
    if (st != TENMO_OK) return st;
    return tenmo_colsum_launch(ctx, x, M, N, ldx, out, beta, partials, tickets, strips, slabs, rps, vec);
}

// ---------------------------------------------------------------------------------------------------
// Column sum for callers that must not allocate.
//
// Some hosts of this library cannot let it call cudaMalloc: a runtime that has handed the whole device
// to its own buffer pool (tenmo's DeviceContext caches and re-issues device buffers, so a second
// allocator competing for what is left can fail at any time), or a serving / training loop that must
// not meet the device-wide synchronisation an allocation or a free implies.  The regular entry point
// grows a workspace on first use; this one keeps its scratch -- the per-slab partial sums and the
// per-strip ticket counters of the split kernel above -- in a fixed array that is part of the loaded
// module.  Every GPU that loads the library holds those TENMO_STATIC_SCRATCH_BYTES until exit.
// ---------------------------------------------------------------------------------------------------
#define TENMO_STATIC_MAX_COLS 16384   // widest matrix the fixed scratch serves
#define TENMO_STATIC_MAX_SLABS 64     // row slabs (partial sums per column)
#define TENMO_STATIC_MAX_STRIPS 512   // 16384 columns / 32-column scalar strips
#define TENMO_STATIC_PARTIAL_FLOATS (TENMO_STATIC_MAX_COLS * TENMO_STATIC_MAX_SLABS)
#define TENMO_STATIC_SCRATCH_BYTES (TENMO_STATIC_PARTIAL_FLOATS * 4 + TENMO_STATIC_MAX_STRIPS * 4)

// [0, PARTIAL_FLOATS) partial sums as float, then MAX_STRIPS ticket counters.  In host code this name is
// only a handle for cudaGetSymbolAddress; the kernel is always given the address obtained from it.
static __device__ __align__(256) unsigned int tenmo_static_scratch[TENMO_STATIC_PARTIAL_FLOATS + TENMO_STATIC_MAX_STRIPS];

namespace {
constexpr int STATIC_MAX_DEVICES = 64;
// Per device, published by its first call: the SM count is written first and the address is stored with release
// order, so a thread that reads a non-null address (acquire) also sees the SM count.  Two threads that race through
// the set-up both resolve the same address and store the same values.
std::atomic<void*> g_static_scratch_addr[STATIC_MAX_DEVICES];
std::atomic<int> g_static_sm_count[STATIC_MAX_DEVICES];
}  // namespace

extern "C" int tenmo_colsum_f32_static(const float* x, int64_t M, int64_t N, int64_t ldx, float* out, float beta,
                                       void* cuda_stream) {
    if (M < 0 || N < 0) return tenmo_set_error(nullptr, TENMO_ERR_INVALID, "colsum_static: negative shape");
    if (beta != 0.f && beta != 1.f) return tenmo_set_error(nullptr, TENMO_ERR_INVALID, "colsum_static: beta must be 0 or 1");
    if (N == 0) return TENMO_OK;
    if (!out || (M > 0 && !x)) return tenmo_set_error(nullptr, TENMO_ERR_INVALID, "colsum_static: NULL pointer");
    if (M > 0 && ldx < N)
        return tenmo_set_error(nullptr, TENMO_ERR_INVALID, "colsum_static: ldx (%lld) < N (%lld)", (long long)ldx, (long long)N);
    if (N > TENMO_STATIC_MAX_COLS)
        return tenmo_set_error(nullptr, TENMO_ERR_UNSUPPORTED,
                               "colsum_static: N = %lld exceeds the %d columns the fixed scratch serves; use tenmo_colsum_f32",
                               (long long)N, TENMO_STATIC_MAX_COLS);
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return tenmo_set_error(nullptr, TENMO_ERR_CUDA, "colsum_static: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= STATIC_MAX_DEVICES)
        return tenmo_set_error(nullptr, TENMO_ERR_UNSUPPORTED, "colsum_static: device ordinal %d is beyond %d", dev, STATIC_MAX_DEVICES);
    void* scratch = g_static_scratch_addr[dev].load(std::memory_order_acquire);
    if (!scratch) {
        // Set-up, once per device, with that device current: resolve the module's array to a device address.
        void* addr = nullptr;
        e = cudaGetSymbolAddress(&addr, tenmo_static_scratch);
        if (e != cudaSuccess || !addr)
            return tenmo_set_error(nullptr, TENMO_ERR_CUDA, "colsum_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess || sms <= 0)
            return tenmo_set_error(nullptr, TENMO_ERR_CUDA, "colsum_static: SM count query: %s", cudaGetErrorString(e));
        g_static_sm_count[dev].store(sms, std::memory_order_relaxed);
        g_static_scratch_addr[dev].store(addr, std::memory_order_release);
        scratch = addr;
    }
    if (M <= TENMO_COLSUM_SEQ_ROWS) {  // few rows: one thread per column, no scratch at all
        const int grid = (int)((N + CS_THREADS - 1) / CS_THREADS);
        colsum_seq_kernel<<<grid, CS_THREADS, 0, stream>>>(x, M, N, ldx, out, beta);
        e = cudaGetLastError();
        if (e != cudaSuccess) return tenmo_set_error(nullptr, TENMO_ERR_CUDA, "colsum_static: launch: %s", cudaGetErrorString(e));
        return TENMO_OK;
    }
    const bool vec = (N % 4 == 0) && (ldx % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15u) == 0);
    int strips, slabs, rps;
    tenmo_colsum_plan(g_static_sm_count[dev].load(std::memory_order_relaxed), M, N, vec, &strips, &slabs, &rps);
    if (slabs > TENMO_STATIC_MAX_SLABS) {  // fewer, taller slabs so that the partials fit
        const int64_t rows = (M + TENMO_STATIC_MAX_SLABS - 1) / TENMO_STATIC_MAX_SLABS;
        rps = (int)((rows + CS_WARPS - 1) / CS_WARPS * CS_WARPS);
        slabs = (int)((M + rps - 1) / rps);
    }
    if (strips > TENMO_STATIC_MAX_STRIPS || (int64_t)slabs * N > TENMO_STATIC_PARTIAL_FLOATS)
        return tenmo_set_error(nullptr, TENMO_ERR_UNSUPPORTED, "colsum_static: %d strips x %d slabs do not fit the fixed scratch", strips, slabs);
    float* partials = static_cast<float*>(scratch);
    unsigned int* tickets = static_cast<unsigned int*>(scratch) + TENMO_STATIC_PARTIAL_FLOATS;
    // The array keeps whatever the previous call left.  The partials are rewritten before they are read;
    // the tickets must start at zero, so they are cleared on the stream ahead of the kernel.
    e = cudaMemsetAsync(tickets, 0, (size_t)strips * sizeof(unsigned int), stream);
    if (e != cudaSuccess) return tenmo_set_error(nullptr, TENMO_ERR_CUDA, "colsum_static: clearing tickets: %s", cudaGetErrorString(e));
    dim3 grid((unsigned)strips, (unsigned)slabs);
    if (vec) colsum_split_kernel<4><<<grid, CS_THREADS, 0, stream>>>(x, M, N, ldx, out, beta, partials, tickets, rps);
    else colsum_split_kernel<1><<<grid, CS_THREADS, 0, stream>>>(x, M, N, ldx, out, beta, partials, tickets, rps);
    e = cudaGetLastError();
    if (e != cudaSuccess) return tenmo_set_error(nullptr, TENMO_ERR_CUDA, "colsum_static: launch: %s", cudaGetErrorString(e));
    return TENMO_OK;
}
