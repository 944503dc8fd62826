// Data-parallel gradient exchange over NVLink peer memory: a sum all-reduce written as ONE kernel per call.
//
// Why not only NCCL: one launch per layer does the reduce-scatter, (optionally) the optimiser on the rank's own shard and
// the all-gather, with peer loads and stores only, and it can be replayed from a captured CUDA graph.  Two geometries:
//   * stand-alone (default): 128 CTAs of 512 threads, eight 16-byte peer loads in flight per thread;
//   * co-resident (tenmo_dp_p2p_set_coresident): 128 CTAs of 128 threads at no more than 85 registers and without any
//     shared memory, so that one fits beside the persistent GEMM CTA of an SM (which leaves about 11 K of the 64 K
//     registers and 2 KB of shared memory free) when the exchange is issued on a side stream beside the backward GEMMs.
//     NCCL's CTAs cannot do that: they wait for GEMM CTAs to leave.  Measured, the overlap only pays while the GEMMs
//     beside it have several rounds of tiles; beside single-round GEMMs (1024 rows per rank) it costs more than it hides.
//
// Setup (one process per GPU): every rank allocates the gradient bucket and a small flag block with
// tenmo_dp_p2p_alloc, the ranks exchange the two CUDA IPC handles out of band (the host's job, like NCCL's unique id),
// and tenmo_dp_p2p_connect maps every peer's bucket and flags into this process.
// One call sums bucket[offset, offset + count) over the ranks in place:
//   wait until every peer's kernel for this call has started (its bucket holds its finished gradients: they were
//       written by earlier work on its stream);
//   reduce-scatter: rank r owns shard r of the range and adds the W copies of it in rank order 0..W-1 (peer copies
//       are read over NVLink with 16-byte loads) into its own bucket -- every element is added once, by its owner,
//       so all ranks end with identical bits;
//       and the owner writes each finished element straight into EVERY rank's bucket (plain peer stores: the all-gather
//       travels as pushes while the reduce-scatter's loads are still coming in, so both NVLink directions are busy);
//   wait until every peer has finished its shard: its pushes have then landed here (it fenced before it raised its flag)
//       and it has finished reading this rank's bucket (the next backward pass may overwrite it).
// The two waits are flags in peer memory, one word per (phase, source rank, CTA): CTA b of a rank only ever depends on
// CTA b of its peers (a shard is cut into chunks dealt round-robin to the CTAs, identically on every rank), so no
// grid-wide synchronisation is needed.  Flags carry the call's epoch (monotonic), so nothing is ever reset.
// The epoch lives on the device: a word of this rank's own flag block counts the calls that have completed, every CTA
// reads it on entry and the last CTA to leave advances it, so a call that is replayed from a captured CUDA graph
// takes the next epoch like an eagerly launched one.
// Every wait is bounded (2 s): on expiry the CTA raises the context status word and returns.
// No multicast, no TMA: plain peer loads and stores.  Roofline: NVLink, (W-1)/W * 4 * count bytes per rank in EACH
// direction (gradient copies read in, finished elements written out, at the same time).
//
// dp_p2p_kernel<.., true> is the same exchange with the optimiser sharded over the ranks (the bucket then holds the
// gradients AND the parameters): the owner of a shard adds the W gradient copies, applies SGD-momentum to its shard of
// the parameters (its velocities never leave the rank), and the all-gather phase distributes updated PARAMETERS
// instead of summed gradients, writing their 3xTF32 lo plane as they land.  Per rank the optimiser touches 1/W of the
// parameters instead of all of them, and no separate SGD launch follows the exchange.
#include <cstdlib>

#include "common.cuh"

namespace {

constexpr int P2P_CTAS = 128;
constexpr int P2P_THREADS = 128;      // co-resident form; the stand-alone form runs P2P_THREADS_BIG per CTA
constexpr int P2P_THREADS_BIG = 512;
constexpr int P2P_MAX_WORLD = 8;
constexpr int P2P_FLAG_WORDS = 3 * P2P_MAX_WORLD * P2P_CTAS;
constexpr int P2P_EPOCH_WORD = P2P_FLAG_WORDS;       // own block only: number of completed calls
constexpr int P2P_TICKET_WORD = P2P_FLAG_WORDS + 1;  // own block only: CTAs of the running call that have left
constexpr int P2P_FLAG_ALLOC_WORDS = P2P_FLAG_WORDS + 64;
constexpr uint64_t P2P_WAIT_LIMIT_NS = 2000000000ull;

struct P2PArgs {
    float* buf[P2P_MAX_WORLD];       // bucket of every rank, mapped into this process
    uint32_t* flags[P2P_MAX_WORLD];  // flag block of every rank
    int rank, world;
    int64_t off, count;
    uint32_t* status;
    // sharded-optimiser form only (dp_p2p_sgd_kernel): parameters at p_off of the same buckets, local velocities and
    // lo plane of the range, SGD constants
    int64_t p_off, lo_count;
    float* v;
    float* lo;
    float lr, momentum, wd, grad_scale;
};

__device__ __forceinline__ uint64_t p2p_now_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Signal "CTA b of this rank has reached `phase` of call `epoch`" to every rank, then wait for the same from every
// rank's CTA b.  False if a wait ran out.
__device__ bool p2p_barrier(const P2PArgs& a, uint32_t epoch, int phase) {
    __threadfence_system();  // this thread's bucket writes are visible system-wide before the flag is
    __syncthreads();
    const int t = threadIdx.x;
    int ok = 1;
    if (t < a.world) {
        uint32_t* dst = a.flags[t] + (phase * P2P_MAX_WORLD + a.rank) * P2P_CTAS + blockIdx.x;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(epoch) : "memory");
        const uint32_t* src = a.flags[a.rank] + (phase * P2P_MAX_WORLD + t) * P2P_CTAS + blockIdx.x;
        const uint64_t t0 = p2p_now_ns();
        for (uint32_t it = 0;; ++it) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(src) : "memory");
            if ((int32_t)(v - epoch) >= 0) break;
            if ((it & 63u) == 63u && p2p_now_ns() - t0 > P2P_WAIT_LIMIT_NS) {
                ok = 0;
                break;
            }
        }
    }
    return __syncthreads_and(ok) != 0;  // no shared memory: the kernel must fit beside a CTA that uses almost all of it
}

// Epoch of the running call: one more than the calls this rank has completed (every CTA reads the word before any
// CTA of the same call can advance it, because the advance happens after ALL of them have left).
__device__ uint32_t p2p_enter(const P2PArgs& a) {
    return *reinterpret_cast<volatile uint32_t*>(a.flags[a.rank] + P2P_EPOCH_WORD) + 1u;
}
// Every CTA leaves through here (also after a wait ran out): the last one advances the epoch and re-arms the ticket.
__device__ void p2p_leave(const P2PArgs& a, uint32_t epoch, bool timed_out) {
    __syncthreads();
    if (threadIdx.x == 0) {
        if (timed_out) atomicOr(a.status, TENMO_DEV_TIMEOUT);
        uint32_t* own = a.flags[a.rank];
        if (atomicAdd(own + P2P_TICKET_WORD, 1u) == gridDim.x - 1) {
            own[P2P_TICKET_WORD] = 0u;
            __threadfence();
            *reinterpret_cast<volatile uint32_t*>(own + P2P_EPOCH_WORD) = epoch;
        }
    }
}

__device__ __forceinline__ void p2p_sgd_one(float& p, float g, float& v, const P2PArgs& a, bool has_v) {
    // the arithmetic of sgd_kernel (optim.mojo:100-158), every product and sum rounded separately
    if (a.grad_scale != 1.f) g = __fmul_rn(g, a.grad_scale);
    if (a.wd > 0.f) g = __fadd_rn(g, __fmul_rn(p, a.wd));
    if (has_v) {
        v = __fadd_rn(__fmul_rn(a.momentum, v), g);
        p = __fsub_rn(p, __fmul_rn(a.lr, v));
    } else {
        p = __fsub_rn(p, __fmul_rn(a.lr, g));
    }
}

// One kernel body for both exchanges.  WT: the world size rounded up to 2, 4 or 8 (loop bounds known at compile time).
// SGD: the sharded-optimiser form.  A thread keeps 8 / WT chunks x WT copies = eight 16-byte gradient loads in flight per
// turn whatever the world size, so that the NVLink round trip (a few microseconds) is paid once per eight loads.
template <int WT, bool SGD, int THREADS>
__global__ void __launch_bounds__(THREADS, THREADS == P2P_THREADS ? 6 : 1) dp_p2p_kernel(const P2PArgs a) {
    constexpr int U = 8 / WT;
    constexpr int P2P_CHUNK = 4 * THREADS;  // floats per chunk: one float4 per thread
    const uint32_t epoch = p2p_enter(a);
    const int W = a.world, r = a.rank, b = blockIdx.x, t = threadIdx.x;
    // shards: equal sizes, multiples of a chunk's float4 granularity; the last may be short or empty
    const int64_t sz = ((a.count + W - 1) / W + 3) & ~(int64_t)3;
    auto shard_len = [&](int p) {
        const int64_t lo = (int64_t)p * sz;
        return lo >= a.count ? (int64_t)0 : (a.count - lo < sz ? a.count - lo : sz);
    };
    const bool has_v = SGD && a.momentum > 0.f;
    // buckets come from cudaMalloc: 16-byte alignment follows from the offsets
    const bool vec = ((a.off | a.p_off | sz) & 3) == 0 &&
                     (!SGD || ((reinterpret_cast<uintptr_t>(a.v) | reinterpret_cast<uintptr_t>(a.lo)) & 15u) == 0);
    const int64_t src_off = SGD ? a.p_off : a.off;       // what the all-gather phase distributes: parameters or sums
    float* const mine = a.buf[r] + src_off;              // this rank's copy of it
    const int64_t turn = (int64_t)gridDim.x * U * P2P_CHUNK;

    if (!p2p_barrier(a, epoch, 0)) { p2p_leave(a, epoch, true); return; }

    {   // own shard: the W gradient copies added in rank order (every element once, by its owner), then the optimiser
        const int64_t base = (int64_t)r * sz, len = shard_len(r);
        for (int64_t c0 = (int64_t)b * U * P2P_CHUNK; c0 < len; c0 += turn) {
            float4 gv[U][WT];
            bool full[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t j = c0 + (int64_t)u * P2P_CHUNK + 4 * t;
                full[u] = vec && j + 3 < len;
                if (full[u]) {
#pragma unroll
                    for (int p = 0; p < WT; ++p)
                        if (p < W) gv[u][p] = __ldcg(reinterpret_cast<const float4*>(a.buf[p] + a.off + base + j));
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t j = c0 + (int64_t)u * P2P_CHUNK + 4 * t;
                const int64_t i = base + j;  // index inside the range
                if (full[u]) {
                    float4 g = gv[u][0];
#pragma unroll
                    for (int p = 1; p < WT; ++p)
                        if (p < W) { g.x += gv[u][p].x; g.y += gv[u][p].y; g.z += gv[u][p].z; g.w += gv[u][p].w; }
                    if (!SGD) {
#pragma unroll
                        for (int p = 0; p < WT; ++p)  // the finished sum goes to every rank's bucket, this one's included
                            if (p < W) *reinterpret_cast<float4*>(a.buf[p] + src_off + i) = g;
                    } else {
                        float4 pp = __ldcs(reinterpret_cast<const float4*>(mine + i));
                        float4 vv = has_v ? __ldcs(reinterpret_cast<const float4*>(a.v + i)) : make_float4(0, 0, 0, 0);
                        p2p_sgd_one(pp.x, g.x, vv.x, a, has_v);
                        p2p_sgd_one(pp.y, g.y, vv.y, a, has_v);
                        p2p_sgd_one(pp.z, g.z, vv.z, a, has_v);
                        p2p_sgd_one(pp.w, g.w, vv.w, a, has_v);
#pragma unroll
                        for (int p = 0; p < WT; ++p)  // the updated parameters go to every rank's copy, this one's included
                            if (p < W) *reinterpret_cast<float4*>(a.buf[p] + src_off + i) = pp;
                        if (has_v) __stcs(reinterpret_cast<float4*>(a.v + i), vv);
                        if (i + 3 < a.lo_count) {
                            __stcs(reinterpret_cast<float4*>(a.lo + i),
                                   make_float4(tenmo_tf32_lo(pp.x), tenmo_tf32_lo(pp.y), tenmo_tf32_lo(pp.z), tenmo_tf32_lo(pp.w)));
                        } else {
                            const float e4[4] = {pp.x, pp.y, pp.z, pp.w};
                            for (int e = 0; e < 4; ++e)
                                if (i + e < a.lo_count) a.lo[i + e] = tenmo_tf32_lo(e4[e]);
                        }
                    }
                } else {
                    for (int e = 0; e < 4 && j + e < len; ++e) {
                        float g = __ldcg(a.buf[0] + a.off + i + e);
                        for (int p = 1; p < W; ++p) g += __ldcg(a.buf[p] + a.off + i + e);
                        if (!SGD) {
                            for (int p = 0; p < W; ++p) a.buf[p][src_off + i + e] = g;
                        } else {
                            float pp = mine[i + e], vv = has_v ? a.v[i + e] : 0.f;
                            p2p_sgd_one(pp, g, vv, a, has_v);
                            for (int p = 0; p < W; ++p) a.buf[p][src_off + i + e] = pp;
                            if (has_v) a.v[i + e] = vv;
                            if (i + e < a.lo_count) a.lo[i + e] = tenmo_tf32_lo(pp);
                        }
                    }
                }
            }
        }
    }

    // every rank's pushes into this rank's bucket have landed once its flag of this phase is seen (it fenced first); the
    // peers are also done reading this rank's gradients, which the next backward pass may now overwrite
    const bool ok = p2p_barrier(a, epoch, 1);
    if (ok && SGD && a.lo_count > 0) {
        // lo plane of the parameters the peers pushed (the own shard's was written with the update): a local pass over the
        // SAME chunks this CTA's counterparts on the peers wrote -- their flags are the only ones it has waited for
        for (int64_t c0 = (int64_t)b * U * P2P_CHUNK; c0 < sz; c0 += turn) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t j = c0 + (int64_t)u * P2P_CHUNK + 4 * t;
#pragma unroll
                for (int q = 1; q < WT; ++q) {
                    if (q < W) {
                        const int p = (r + q) % W;
                        const int64_t i = (int64_t)p * sz + j, len = shard_len(p);
                        if (vec && j + 3 < len && i + 3 < a.lo_count) {
                            const float4 x = __ldcg(reinterpret_cast<const float4*>(mine + i));
                            __stcs(reinterpret_cast<float4*>(a.lo + i),
                                   make_float4(tenmo_tf32_lo(x.x), tenmo_tf32_lo(x.y), tenmo_tf32_lo(x.z), tenmo_tf32_lo(x.w)));
                        } else {
                            for (int e = 0; e < 4 && j + e < len; ++e)
                                if (i + e < a.lo_count) a.lo[i + e] = tenmo_tf32_lo(__ldcg(mine + i + e));
                        }
                    }
                }
            }
        }
    }
    p2p_leave(a, epoch, !ok);
}

template <bool SGD>
void p2p_launch(const P2PArgs& a, int grid, cudaStream_t stream, bool big) {
    if (big) {
        if (a.world <= 2) dp_p2p_kernel<2, SGD, P2P_THREADS_BIG><<<grid, P2P_THREADS_BIG, 0, stream>>>(a);
        else if (a.world <= 4) dp_p2p_kernel<4, SGD, P2P_THREADS_BIG><<<grid, P2P_THREADS_BIG, 0, stream>>>(a);
        else dp_p2p_kernel<8, SGD, P2P_THREADS_BIG><<<grid, P2P_THREADS_BIG, 0, stream>>>(a);
    } else {
        if (a.world <= 2) dp_p2p_kernel<2, SGD, P2P_THREADS><<<grid, P2P_THREADS, 0, stream>>>(a);
        else if (a.world <= 4) dp_p2p_kernel<4, SGD, P2P_THREADS><<<grid, P2P_THREADS, 0, stream>>>(a);
        else dp_p2p_kernel<8, SGD, P2P_THREADS><<<grid, P2P_THREADS, 0, stream>>>(a);
    }
}

// CTAs per launch: P2P_CTAS unless TENMO_P2P_CTAS names fewer (every rank must use the same number: a CTA pairs with
// the CTA of the same index on its peers).
int p2p_grid() {
    static int grid = 0;
    if (!grid) {
        grid = P2P_CTAS;
        const char* env = getenv("TENMO_P2P_CTAS");
        if (env) {
            const int v = atoi(env);
            if (v >= 1 && v <= P2P_CTAS) grid = v;
        }
    }
    return grid;
}

void p2p_fill_args(tenmo_ctx* ctx, P2PArgs& a, int64_t offset, int64_t count) {
    memset(&a, 0, sizeof(a));
    for (int p = 0; p < P2P_MAX_WORLD; ++p) {
        a.buf[p] = static_cast<float*>(ctx->p2p_peer_buf[p]);
        a.flags[p] = static_cast<uint32_t*>(ctx->p2p_peer_flags[p]);
    }
    a.rank = ctx->p2p_rank; a.world = ctx->p2p_world;
    a.off = offset; a.count = count;
    a.status = ctx->dev_status;
}

}  // namespace

extern "C" {

int tenmo_dp_p2p_alloc(tenmo_ctx* ctx, int64_t count, float** buf_out, void* handles_out, size_t handles_bytes) {
    TENMO_CHECK_CTX(ctx);
    if (count <= 0 || !buf_out || !handles_out || handles_bytes < TENMO_DP_P2P_HANDLE_BYTES)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "dp_p2p_alloc: need count > 0, buf_out and %d bytes for the handles",
                               TENMO_DP_P2P_HANDLE_BYTES);
    if (ctx->p2p_buf) return tenmo_set_error(ctx, TENMO_ERR_STATE, "dp_p2p_alloc: already allocated");
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const size_t bytes = (((size_t)count * sizeof(float)) + 255) & ~(size_t)255;
    cudaIpcMemHandle_t hb, hf;
    cudaError_t e = cudaMalloc(&ctx->p2p_buf, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&ctx->p2p_flags, P2P_FLAG_ALLOC_WORDS * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(ctx->p2p_buf, 0, bytes);
    if (e == cudaSuccess) e = cudaMemset(ctx->p2p_flags, 0, P2P_FLAG_ALLOC_WORDS * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&hb, ctx->p2p_buf);
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&hf, ctx->p2p_flags);
    if (e != cudaSuccess) {  // nothing half-allocated is left behind
        if (ctx->p2p_buf) cudaFree(ctx->p2p_buf);
        if (ctx->p2p_flags) cudaFree(ctx->p2p_flags);
        ctx->p2p_buf = ctx->p2p_flags = nullptr;
        cudaGetLastError();
        return tenmo_set_error(ctx, TENMO_ERR_CUDA, "dp_p2p_alloc: %s", cudaGetErrorString(e));
    }
    static_assert(2 * sizeof(cudaIpcMemHandle_t) == TENMO_DP_P2P_HANDLE_BYTES, "handle block size");
    memcpy(handles_out, &hb, sizeof(hb));
    memcpy(static_cast<char*>(handles_out) + sizeof(hb), &hf, sizeof(hf));
    ctx->p2p_count = count;
    *buf_out = static_cast<float*>(ctx->p2p_buf);
    return TENMO_OK;
}

int tenmo_dp_p2p_connect(tenmo_ctx* ctx, int rank, int world, const void* all_handles, size_t handles_bytes) {
    TENMO_CHECK_CTX(ctx);
    if (!ctx->p2p_buf) return tenmo_set_error(ctx, TENMO_ERR_STATE, "dp_p2p_connect: call tenmo_dp_p2p_alloc first");
    if (ctx->p2p_world) return tenmo_set_error(ctx, TENMO_ERR_STATE, "dp_p2p_connect: already connected");
    if (world < 1 || world > P2P_MAX_WORLD || rank < 0 || rank >= world)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "dp_p2p_connect: rank %d / world %d (at most %d ranks)", rank, world,
                               P2P_MAX_WORLD);
    if (!all_handles || handles_bytes < (size_t)world * TENMO_DP_P2P_HANDLE_BYTES)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "dp_p2p_connect: need %d x %d handle bytes", world, TENMO_DP_P2P_HANDLE_BYTES);
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    for (int p = 0; p < world; ++p) {
        if (p == rank) {
            ctx->p2p_peer_buf[p] = ctx->p2p_buf;
            ctx->p2p_peer_flags[p] = ctx->p2p_flags;
            continue;
        }
        cudaIpcMemHandle_t hb, hf;
        const char* src = static_cast<const char*>(all_handles) + (size_t)p * TENMO_DP_P2P_HANDLE_BYTES;
        memcpy(&hb, src, sizeof(hb));
        memcpy(&hf, src + sizeof(hb), sizeof(hf));
        cudaError_t e = cudaIpcOpenMemHandle(&ctx->p2p_peer_buf[p], hb, cudaIpcMemLazyEnablePeerAccess);
        if (e == cudaSuccess) e = cudaIpcOpenMemHandle(&ctx->p2p_peer_flags[p], hf, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {  // unmap what was mapped so far; the bucket itself stays allocated
            for (int q = 0; q <= p; ++q) {
                if (q == rank) continue;
                if (ctx->p2p_peer_buf[q]) cudaIpcCloseMemHandle(ctx->p2p_peer_buf[q]);
                if (ctx->p2p_peer_flags[q]) cudaIpcCloseMemHandle(ctx->p2p_peer_flags[q]);
            }
            for (int q = 0; q < P2P_MAX_WORLD; ++q) ctx->p2p_peer_buf[q] = ctx->p2p_peer_flags[q] = nullptr;
            cudaGetLastError();
            return tenmo_set_error(ctx, TENMO_ERR_CUDA, "dp_p2p_connect: cannot map rank %d's bucket: %s", p, cudaGetErrorString(e));
        }
    }
    ctx->p2p_rank = rank;
    ctx->p2p_world = world;
    return TENMO_OK;
}

int tenmo_dp_p2p_allreduce_sum_f32(tenmo_ctx* ctx, int64_t offset, int64_t count) {
    TENMO_CHECK_CTX(ctx);
    if (!ctx->p2p_world) return tenmo_set_error(ctx, TENMO_ERR_STATE, "dp_p2p_allreduce: call tenmo_dp_p2p_connect first");
    if (offset < 0 || count < 0 || offset + count > ctx->p2p_count)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "dp_p2p_allreduce: [%lld, %lld) outside the bucket of %lld floats",
                               (long long)offset, (long long)(offset + count), (long long)ctx->p2p_count);
    if (ctx->p2p_world == 1 || count == 0) return TENMO_OK;
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    P2PArgs a;
    p2p_fill_args(ctx, a, offset, count);  // every rank makes the same calls in the same order
    p2p_launch<false>(a, p2p_grid(), ctx->stream, !ctx->p2p_small);
    TENMO_LAUNCH_CHECK(ctx, "dp_p2p_kernel");
    return TENMO_OK;
}

int tenmo_dp_p2p_sgd_step_f32(tenmo_ctx* ctx, int64_t grad_offset, int64_t param_offset, int64_t count, float* v, float* p_lo,
                              int64_t lo_count, float lr, float momentum, float weight_decay, float grad_scale) {
    TENMO_CHECK_CTX(ctx);
    if (!ctx->p2p_world) return tenmo_set_error(ctx, TENMO_ERR_STATE, "dp_p2p_sgd_step: call tenmo_dp_p2p_connect first");
    if (grad_offset < 0 || param_offset < 0 || count < 0 || grad_offset + count > ctx->p2p_count ||
        param_offset + count > ctx->p2p_count)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "dp_p2p_sgd_step: ranges [%lld, +%lld) and [%lld, +%lld) must lie in the bucket of %lld floats",
                               (long long)grad_offset, (long long)count, (long long)param_offset, (long long)count, (long long)ctx->p2p_count);
    if (grad_offset < param_offset + count && param_offset < grad_offset + count && count > 0)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "dp_p2p_sgd_step: the gradient and parameter ranges overlap");
    if (momentum > 0.f && !v) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "dp_p2p_sgd_step: momentum needs the velocity buffer");
    if (lo_count < 0 || lo_count > count || (lo_count > 0 && !p_lo))
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "dp_p2p_sgd_step: bad lo plane (0 <= lo_count <= count, pointer required)");
    if (count == 0) return TENMO_OK;
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    P2PArgs a;
    p2p_fill_args(ctx, a, grad_offset, count);
    a.p_off = param_offset;
    a.v = v; a.lo = lo_count > 0 ? p_lo : nullptr; a.lo_count = lo_count;
    a.lr = lr; a.momentum = momentum; a.wd = weight_decay; a.grad_scale = grad_scale;
    p2p_launch<true>(a, p2p_grid(), ctx->stream, !ctx->p2p_small);
    TENMO_LAUNCH_CHECK(ctx, "dp_p2p_kernel");
    return TENMO_OK;
}

int tenmo_dp_p2p_set_coresident(tenmo_ctx* ctx, int on) {
    TENMO_CHECK_CTX(ctx);
    ctx->p2p_small = on != 0;
    return TENMO_OK;
}

int tenmo_dp_p2p_close(tenmo_ctx* ctx) {
    TENMO_CHECK_CTX(ctx);
    if (!ctx->p2p_buf) return TENMO_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (int p = 0; p < ctx->p2p_world; ++p) {
        if (p == ctx->p2p_rank) continue;
        if (ctx->p2p_peer_buf[p]) cudaIpcCloseMemHandle(ctx->p2p_peer_buf[p]);
        if (ctx->p2p_peer_flags[p]) cudaIpcCloseMemHandle(ctx->p2p_peer_flags[p]);
    }
    for (int p = 0; p < P2P_MAX_WORLD; ++p) ctx->p2p_peer_buf[p] = ctx->p2p_peer_flags[p] = nullptr;
    cudaFree(ctx->p2p_buf);
    cudaFree(ctx->p2p_flags);
    ctx->p2p_buf = ctx->p2p_flags = nullptr;
    ctx->p2p_world = 0;
    ctx->p2p_count = 0;
    cudaGetLastError();
    return TENMO_OK;
}

}  // extern "C"
