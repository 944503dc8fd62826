// Data-parallel gradient exchange over NVLink peer memory: a sum all-reduce written as ONE kernel per call.
//
// Why not only NCCL: the exchange of a layer's gradients should run beside the backward GEMMs of the layers below,
// but the persistent GEMM kernel holds every SM with one large CTA, and NCCL's CTAs (hundreds of threads, ~100
// registers each) cannot share an SM with it, so they wait for GEMM CTAs to leave.  The kernel here is built to
// co-reside: 64 CTAs of 512 threads, 64 registers, no shared-memory tile.
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
//   wait until every peer has reduced its shard; all-gather: copy the peers' reduced shards into the own bucket;
//   wait until every peer has finished reading this rank's bucket (the next backward pass overwrites it).
// The three waits are flags in peer memory, one per (phase, source rank, CTA): CTA b of a rank only ever depends on
// CTA b of its peers (a shard is cut into chunks dealt round-robin to the CTAs, identically on every rank), so no
// grid-wide synchronisation is needed.  Flags carry the call's epoch (monotonic), so nothing is ever reset.
// The epoch lives on the device: a word of this rank's own flag block counts the calls that have completed, every CTA
// reads it on entry and the last CTA to leave advances it, so a call that is replayed from a captured CUDA graph
// takes the next epoch like an eagerly launched one.
// Every wait is bounded (2 s): on expiry the CTA raises the context status word and returns.
// No multicast, no TMA: plain peer loads and stores.  Roofline: NVLink, 2 * (W-1)/W * 4 * count bytes read per rank.
//
// dp_p2p_sgd_kernel is the same exchange with the optimiser sharded over the ranks (the bucket then holds the
// gradients AND the parameters): the owner of a shard adds the W gradient copies, applies SGD-momentum to its shard of
// the parameters (its velocities never leave the rank), and the all-gather phase distributes updated PARAMETERS
// instead of summed gradients, writing their 3xTF32 lo plane as they land.  Per rank the optimiser touches 1/W of the
// parameters instead of all of them, and no separate SGD launch follows the exchange.
#include "common.cuh"

namespace {

constexpr int P2P_CTAS = 64;
constexpr int P2P_THREADS = 512;
constexpr int P2P_MAX_WORLD = 8;
constexpr int P2P_FLAG_WORDS = 3 * P2P_MAX_WORLD * P2P_CTAS;
constexpr int P2P_EPOCH_WORD = P2P_FLAG_WORDS;       // own block only: number of completed calls
constexpr int P2P_TICKET_WORD = P2P_FLAG_WORDS + 1;  // own block only: CTAs of the running call that have left
constexpr int P2P_FLAG_ALLOC_WORDS = P2P_FLAG_WORDS + 64;
constexpr int P2P_CHUNK = 4 * P2P_THREADS;  // floats per chunk: one float4 per thread
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
__device__ bool p2p_barrier(const P2PArgs& a, uint32_t epoch, int phase, int* ok_smem) {
    __threadfence_system();  // this thread's bucket writes are visible system-wide before the flag is
    __syncthreads();
    const int t = threadIdx.x;
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
                *ok_smem = 0;
                break;
            }
        }
    }
    __syncthreads();
    return *ok_smem != 0;
}

// Epoch of the running call: one more than the calls this rank has completed (every CTA reads the word before any
// CTA of the same call can advance it, because the advance happens after ALL of them have left).
__device__ uint32_t p2p_enter(const P2PArgs& a, int* ok_smem, uint32_t* epoch_smem) {
    if (threadIdx.x == 0) {
        *ok_smem = 1;
        *epoch_smem = *reinterpret_cast<volatile uint32_t*>(a.flags[a.rank] + P2P_EPOCH_WORD) + 1u;
    }
    __syncthreads();
    return *epoch_smem;
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

__global__ void __launch_bounds__(P2P_THREADS) dp_p2p_allreduce_kernel(const P2PArgs a) {
    __shared__ int ok_smem;
    __shared__ uint32_t epoch_smem;
    const uint32_t epoch = p2p_enter(a, &ok_smem, &epoch_smem);
    const int W = a.world, r = a.rank, b = blockIdx.x, t = threadIdx.x;
    // shards: equal sizes, multiples of a chunk's float4 granularity; the last may be short or empty
    const int64_t sz = ((a.count + W - 1) / W + 3) & ~(int64_t)3;
    auto shard_len = [&](int p) {
        const int64_t lo = (int64_t)p * sz;
        return lo >= a.count ? (int64_t)0 : (a.count - lo < sz ? a.count - lo : sz);
    };
    const bool vec = ((a.off | sz) & 3) == 0;  // buckets come from cudaMalloc: 16-byte alignment follows from the offsets

    if (!p2p_barrier(a, epoch, 0, &ok_smem)) { p2p_leave(a, epoch, true); return; }

    {   // reduce-scatter: this rank's shard, chunks b, b + CTAS, ...
        const int64_t base = a.off + (int64_t)r * sz, len = shard_len(r);
        for (int64_t c0 = (int64_t)b * P2P_CHUNK; c0 < len; c0 += (int64_t)P2P_CTAS * P2P_CHUNK) {
            const int64_t j = c0 + 4 * t;
            if (j >= len) continue;
            if (vec && j + 3 < len) {
                // all W loads are issued before the first add: one NVLink round trip per element, not W
                float4 v[P2P_MAX_WORLD];
#pragma unroll
                for (int p = 0; p < P2P_MAX_WORLD; ++p)
                    if (p < W) v[p] = __ldcg(reinterpret_cast<const float4*>(a.buf[p] + base + j));
                float4 acc = v[0];
#pragma unroll
                for (int p = 1; p < P2P_MAX_WORLD; ++p)
                    if (p < W) { acc.x += v[p].x; acc.y += v[p].y; acc.z += v[p].z; acc.w += v[p].w; }
                *reinterpret_cast<float4*>(a.buf[r] + base + j) = acc;
            } else {
                for (int e = 0; e < 4 && j + e < len; ++e) {
                    float acc = __ldcg(a.buf[0] + base + j + e);
                    for (int p = 1; p < W; ++p) acc += __ldcg(a.buf[p] + base + j + e);
                    a.buf[r][base + j + e] = acc;
                }
            }
        }
    }

    if (!p2p_barrier(a, epoch, 1, &ok_smem)) { p2p_leave(a, epoch, true); return; }

    // all-gather: the peers' reduced shards (the same chunk of every peer in one go, so that W-1 loads are in flight)
    for (int64_t c0 = (int64_t)b * P2P_CHUNK; c0 < sz; c0 += (int64_t)P2P_CTAS * P2P_CHUNK) {
        const int64_t j = c0 + 4 * t;
        float4 v[P2P_MAX_WORLD];
        bool full[P2P_MAX_WORLD];
#pragma unroll
        for (int q = 1; q < P2P_MAX_WORLD; ++q) {
            full[q] = false;
            if (q < W) {
                const int p = (r + q) % W;  // start with the next rank: the ranks do not all read the same peer at once
                full[q] = vec && j + 3 < shard_len(p);
                if (full[q]) v[q] = __ldcg(reinterpret_cast<const float4*>(a.buf[p] + a.off + (int64_t)p * sz + j));
            }
        }
#pragma unroll
        for (int q = 1; q < P2P_MAX_WORLD; ++q) {
            if (q < W) {
                const int p = (r + q) % W;
                const int64_t base = a.off + (int64_t)p * sz, len = shard_len(p);
                if (full[q]) {
                    *reinterpret_cast<float4*>(a.buf[r] + base + j) = v[q];
                } else {
                    for (int e = 0; e < 4 && j + e < len; ++e) a.buf[r][base + j + e] = __ldcg(a.buf[p] + base + j + e);
                }
            }
        }
    }

    p2p_leave(a, epoch, !p2p_barrier(a, epoch, 2, &ok_smem));
}

// Reduce-scatter of the gradients, SGD-momentum on the own shard of the parameters, all-gather of the updated
// parameters (with their lo plane).  Same shards, chunks, flags and waits as the kernel above.
__global__ void __launch_bounds__(P2P_THREADS) dp_p2p_sgd_kernel(const P2PArgs a) {
    __shared__ int ok_smem;
    __shared__ uint32_t epoch_smem;
    const uint32_t epoch = p2p_enter(a, &ok_smem, &epoch_smem);
    const int W = a.world, r = a.rank, b = blockIdx.x, t = threadIdx.x;
    const int64_t sz = ((a.count + W - 1) / W + 3) & ~(int64_t)3;
    auto shard_len = [&](int p) {
        const int64_t lo = (int64_t)p * sz;
        return lo >= a.count ? (int64_t)0 : (a.count - lo < sz ? a.count - lo : sz);
    };
    const bool has_v = a.momentum > 0.f;
    const bool vec = ((a.off | a.p_off | sz) & 3) == 0 && ((reinterpret_cast<uintptr_t>(a.v) | reinterpret_cast<uintptr_t>(a.lo)) & 15u) == 0;
    float* const P = a.buf[r] + a.p_off;  // this rank's copy of the parameters of the range

    if (!p2p_barrier(a, epoch, 0, &ok_smem)) { p2p_leave(a, epoch, true); return; }

    {   // own shard: sum the W gradient copies in rank order, then the optimiser step
        const int64_t base = (int64_t)r * sz, len = shard_len(r);
        for (int64_t c0 = (int64_t)b * P2P_CHUNK; c0 < len; c0 += (int64_t)P2P_CTAS * P2P_CHUNK) {
            const int64_t j = c0 + 4 * t;
            if (j >= len) continue;
            const int64_t i = base + j;  // index inside the range
            if (vec && j + 3 < len) {
                float4 gv[P2P_MAX_WORLD];
#pragma unroll
                for (int p = 0; p < P2P_MAX_WORLD; ++p)
                    if (p < W) gv[p] = __ldcg(reinterpret_cast<const float4*>(a.buf[p] + a.off + i));
                float4 pp = *reinterpret_cast<const float4*>(P + i);
                float4 vv = has_v ? *reinterpret_cast<const float4*>(a.v + i) : make_float4(0, 0, 0, 0);
                float4 g = gv[0];
#pragma unroll
                for (int p = 1; p < P2P_MAX_WORLD; ++p)
                    if (p < W) { g.x += gv[p].x; g.y += gv[p].y; g.z += gv[p].z; g.w += gv[p].w; }
                p2p_sgd_one(pp.x, g.x, vv.x, a, has_v);
                p2p_sgd_one(pp.y, g.y, vv.y, a, has_v);
                p2p_sgd_one(pp.z, g.z, vv.z, a, has_v);
                p2p_sgd_one(pp.w, g.w, vv.w, a, has_v);
                *reinterpret_cast<float4*>(P + i) = pp;
                if (has_v) *reinterpret_cast<float4*>(a.v + i) = vv;
                if (i + 3 < a.lo_count) {
                    *reinterpret_cast<float4*>(a.lo + i) =
                        make_float4(tenmo_tf32_lo(pp.x), tenmo_tf32_lo(pp.y), tenmo_tf32_lo(pp.z), tenmo_tf32_lo(pp.w));
                } else {
                    const float e4[4] = {pp.x, pp.y, pp.z, pp.w};
                    for (int e = 0; e < 4; ++e)
                        if (i + e < a.lo_count) a.lo[i + e] = tenmo_tf32_lo(e4[e]);
                }
            } else {
                for (int e = 0; e < 4 && j + e < len; ++e) {
                    float g = __ldcg(a.buf[0] + a.off + i + e);
                    for (int p = 1; p < W; ++p) g += __ldcg(a.buf[p] + a.off + i + e);
                    float pp = P[i + e], vv = has_v ? a.v[i + e] : 0.f;
                    p2p_sgd_one(pp, g, vv, a, has_v);
                    P[i + e] = pp;
                    if (has_v) a.v[i + e] = vv;
                    if (i + e < a.lo_count) a.lo[i + e] = tenmo_tf32_lo(pp);
                }
            }
        }
    }

    if (!p2p_barrier(a, epoch, 1, &ok_smem)) { p2p_leave(a, epoch, true); return; }

    // all-gather of the updated parameters: the peers' shards, the same chunk of every peer in one go
    for (int64_t c0 = (int64_t)b * P2P_CHUNK; c0 < sz; c0 += (int64_t)P2P_CTAS * P2P_CHUNK) {
        const int64_t j = c0 + 4 * t;
        float4 pv[P2P_MAX_WORLD];
        bool full[P2P_MAX_WORLD];
#pragma unroll
        for (int q = 1; q < P2P_MAX_WORLD; ++q) {
            full[q] = false;
            if (q < W) {
                const int p = (r + q) % W;
                full[q] = vec && j + 3 < shard_len(p);
                if (full[q]) pv[q] = __ldcg(reinterpret_cast<const float4*>(a.buf[p] + a.p_off + (int64_t)p * sz + j));
            }
        }
#pragma unroll
        for (int q = 1; q < P2P_MAX_WORLD; ++q) {
            if (q < W) {
                const int p = (r + q) % W;
                const int64_t i = (int64_t)p * sz + j, len = shard_len(p);
                if (full[q]) {
                    *reinterpret_cast<float4*>(P + i) = pv[q];
                    if (i + 3 < a.lo_count) {
                        *reinterpret_cast<float4*>(a.lo + i) = make_float4(tenmo_tf32_lo(pv[q].x), tenmo_tf32_lo(pv[q].y),
                                                                           tenmo_tf32_lo(pv[q].z), tenmo_tf32_lo(pv[q].w));
                    } else {
                        const float e4[4] = {pv[q].x, pv[q].y, pv[q].z, pv[q].w};
                        for (int e = 0; e < 4; ++e)
                            if (i + e < a.lo_count) a.lo[i + e] = tenmo_tf32_lo(e4[e]);
                    }
                } else {
                    for (int e = 0; e < 4 && j + e < len; ++e) {
                        const float x = __ldcg(a.buf[p] + a.p_off + i + e);
                        P[i + e] = x;
                        if (i + e < a.lo_count) a.lo[i + e] = tenmo_tf32_lo(x);
                    }
                }
            }
        }
    }

    p2p_leave(a, epoch, !p2p_barrier(a, epoch, 2, &ok_smem));
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
    dp_p2p_allreduce_kernel<<<P2P_CTAS, P2P_THREADS, 0, ctx->stream>>>(a);
    TENMO_LAUNCH_CHECK(ctx, "dp_p2p_allreduce_kernel");
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
    dp_p2p_sgd_kernel<<<P2P_CTAS, P2P_THREADS, 0, ctx->stream>>>(a);
    TENMO_LAUNCH_CHECK(ctx, "dp_p2p_sgd_kernel");
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
