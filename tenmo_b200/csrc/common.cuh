// Shared declarations of libtenmo_cuda: the context object, error plumbing and small device helpers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../include/tenmo_cuda.h"

// Device status word bits (tenmo_cuda_check_device_status).
#define TENMO_DEV_TIMEOUT 1u    // a bounded mbarrier / flag wait ran out of iterations
#define TENMO_DEV_BAD_LABEL 2u  // cross-entropy saw a label outside [0, C) that is not ignore_index

// Layout of the small device scratch block (32-bit words): [0] status, [8] cross-entropy ticket, [64..127] tile counter
// pairs of the tensor-core GEMM, [256..511] fix-up flags of its stream-K tail (one per piece).
#define TENMO_DEV_STATUS_WORDS 512
#define TENMO_SK_FLAG_WORD0 256
#define TENMO_SK_MAX_UNITS 256
#define TENMO_MAX_BOUND_STREAMS 8

struct tenmo_ctx {
    int device = 0;
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
    int sm_clock_khz = 0;
    size_t smem_optin = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    cudaStream_t bound[8] = {nullptr};  // streams the context has been bound to, most recent first (tenmo_cuda_set_stream)
    int n_bound = 0;
    char err[512] = {0};
    int64_t launches = 0;
    int last_gemm_algo = -1;
    const char* last_gemm_kernel = "";
    int last_gemm_sk_units = 0;
    bool last_gemm_pair = false;  // the last tensor-core GEMM ran as CTA pairs (tcgen05 cta_group::2)
    bool pdl = true;  // programmatic dependent launch for small kernels (TENMO_PDL=0: off)
    // workspace (grown on demand, never shrunk): lo planes for the 3xTF32 kernel, reduction partials
    void* ws = nullptr;
    size_t ws_bytes = 0;
    // small fixed device scratch: [0] status word, [8..15] cross-entropy tickets/accumulators
    uint32_t* dev_status = nullptr;
    // ticket counters of the split column-sum kernel: zero between calls (the last CTA resets its own)
    unsigned int* tickets = nullptr;
    int tickets_cap = 0;
    // multi-tensor SGD descriptor staging (pinned host + device)
    void* sgd_desc_host = nullptr;
    void* sgd_desc_dev = nullptr;
    size_t sgd_desc_bytes = 0;
    // tcgen05 GEMM state (tensor-map encoder entry point, opt-in smem set)
    void* encode_tiled = nullptr;
    bool tc_ready = false;
    unsigned int tile_counter_next = 0;
    int reserve_sms = 0;  // persistent GEMM kernels launch sm_count - reserve_sms CTAs (tenmo_cuda_reserve_sms)
    // optional device timing of the GEMM kernels (tenmo_cuda_profile_begin/end)
    bool prof_on = false;
    cudaEvent_t* prof_ev = nullptr;  // pairs: [2*i] before, [2*i+1] after
    int prof_n = 0, prof_cap = 0;
    // NCCL
    void* nccl_lib = nullptr;
    void* nccl_comm = nullptr;
    int dp_rank = 0, dp_world = 1;
    // peer-memory exchange (dp_p2p.cu): own bucket + flag block, and every rank's, mapped through CUDA IPC
    void* p2p_buf = nullptr;
    void* p2p_flags = nullptr;
    void* p2p_peer_buf[8] = {nullptr};
    void* p2p_peer_flags[8] = {nullptr};
    int64_t p2p_count = 0;
    int p2p_rank = 0, p2p_world = 0;
    bool p2p_small = false;  // launch the exchange in its co-resident form (tenmo_dp_p2p_set_coresident)
};

int tenmo_set_error(tenmo_ctx* ctx, int status, const char* fmt, ...);
int tenmo_workspace(tenmo_ctx* ctx, size_t bytes, void** out);
// Event pair around a GEMM kernel launch while profiling is on (no-ops otherwise).
void tenmo_prof_before(tenmo_ctx* ctx);
void tenmo_prof_after(tenmo_ctx* ctx);

#define TENMO_CHECK_CTX(ctx)             \
    do {                                 \
        if (!(ctx)) return TENMO_ERR_INVALID; \
    } while (0)

#define TENMO_CUDA_TRY(ctx, expr)                                                                  \
    do {                                                                                           \
        cudaError_t _e = (expr);                                                                   \
        if (_e != cudaSuccess)                                                                     \
            return tenmo_set_error((ctx), TENMO_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

// Every launch goes through this so the context can count launches and surface launch errors.
#define TENMO_LAUNCH_CHECK(ctx, name)                                                              \
    do {                                                                                           \
        (ctx)->launches++;                                                                         \
        cudaError_t _e = cudaGetLastError();                                                       \
        if (_e != cudaSuccess)                                                                     \
            return tenmo_set_error((ctx), TENMO_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(_e)); \
    } while (0)

// Programmatic dependent launch for chains of small kernels (a latency-bound training step).  A kernel launched through
// tenmo_launch with pdl = true may be scheduled while its predecessor in the stream still runs: its CTAs become resident
// and then block in tenmo_grid_dependency_sync() until the predecessor has completed and its memory operations are
// visible, so the launch latency overlaps the predecessor instead of following it.  The kernel must call
// tenmo_grid_dependency_sync() before it touches global memory; launched with pdl = false the call does nothing.
// Only for grids that are resident at once (at most one CTA per SM): early CTAs of a large grid would take SM slots from
// the kernel they wait for.  TENMO_PDL=0 in the environment turns it off.
#ifdef __CUDACC__
__device__ __forceinline__ void tenmo_grid_dependency_sync() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the next kernel in the stream may start launching
}
template <typename... KArgs, typename... Args>
static inline cudaError_t tenmo_launch(void (*kernel)(KArgs...), unsigned grid, unsigned block, size_t smem, cudaStream_t s,
                                       bool pdl, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif
static inline bool tenmo_pdl_ok(const tenmo_ctx* ctx, int64_t grid) { return ctx->pdl && grid <= ctx->sm_count; }

// Grid size for grid-stride, bandwidth-bound kernels: a multiple of the SM count.
static inline int tenmo_stream_grid(const tenmo_ctx* ctx, int64_t work_items, int items_per_block, int ctas_per_sm) {
    int64_t want = (work_items + items_per_block - 1) / items_per_block;
    int64_t cap = (int64_t)ctx->sm_count * ctas_per_sm;
    if (want < 1) want = 1;
    return (int)(want < cap ? want : cap);
}

// lo plane of the 3xTF32 split: x = hi + lo with hi = x truncated to TF32 (what the tensor core reads from
// an fp32 word) and lo rounded to TF32.
__device__ __forceinline__ float tenmo_tf32_lo(float x) {
    const float hi = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
    const float d = x - hi;
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(d));
    return __uint_as_float(r);
}

__device__ __forceinline__ float tenmo_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float tenmo_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
