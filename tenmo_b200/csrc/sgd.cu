// SGD (with momentum / weight decay) over many parameter tensors in one launch.
//
// Restates optim.mojo:100-158:  g' = g (* grad_scale); if wd > 0: g' += p*wd;
//   momentum > 0:  v = momentum*v + g';  p -= lr*v        momentum == 0:  p -= lr*g'
// with every product and sum rounded separately (no FMA contraction), as the reference's SIMD
// expressions are.  The reference launches one kernel per tensor (kernels/sgd_kernel.mojo:54-128);
// here up to SGD_MAX_TENSORS tensors ride in the kernel parameters and one grid covers them all.
// Roofline: HBM, 20 bytes per parameter with momentum (read p,g,v; write p,v), 12 without.
#include "common.cuh"

namespace {

constexpr int SGD_THREADS = 256;
constexpr int SGD_MAX_TENSORS = 24;
constexpr int SGD_CHUNK = SGD_THREADS * 4 * 4;  // elements per CTA step

struct SgdBatch {
    float* p[SGD_MAX_TENSORS];
    const float* g[SGD_MAX_TENSORS];
    float* v[SGD_MAX_TENSORS];
    int64_t numel[SGD_MAX_TENSORS];
    float* lo[SGD_MAX_TENSORS];         // optional: 3xTF32 lo plane of the updated parameters, first lo_numel elements
    int64_t lo_numel[SGD_MAX_TENSORS];
    int64_t chunk_start[SGD_MAX_TENSORS + 1];  // prefix sum of chunks per tensor
    int n;
    float lr, momentum, wd, grad_scale;
};

__device__ __forceinline__ void sgd_one(float& p, float g, float& v, const SgdBatch& b, bool has_v) {
    if (b.grad_scale != 1.f) g = __fmul_rn(g, b.grad_scale);
    if (b.wd > 0.f) g = __fadd_rn(g, __fmul_rn(p, b.wd));
    if (has_v) {
        v = __fadd_rn(__fmul_rn(b.momentum, v), g);
        p = __fsub_rn(p, __fmul_rn(b.lr, v));
    } else {
        p = __fsub_rn(p, __fmul_rn(b.lr, g));
    }
}

__global__ void __launch_bounds__(SGD_THREADS) sgd_kernel(const SgdBatch b) {
    tenmo_grid_dependency_sync();
    const int64_t total_chunks = b.chunk_start[b.n];
    const bool has_v = b.momentum > 0.f;
    for (int64_t chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
        int t = 0;
        while (t + 1 < b.n && chunk >= b.chunk_start[t + 1]) ++t;
        const int64_t base = (chunk - b.chunk_start[t]) * SGD_CHUNK;
        const int64_t n = b.numel[t];
        float* __restrict__ p = b.p[t];
        const float* __restrict__ g = b.g[t];
        float* __restrict__ v = b.v[t];
        float* __restrict__ lo = b.lo[t];
        const int64_t n_lo = lo ? b.lo_numel[t] : 0;
        const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                           reinterpret_cast<uintptr_t>(v)) & 15u) == 0;
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int64_t i = base + ((int64_t)it * SGD_THREADS + threadIdx.x) * 4;
            if (i >= n) break;
            if (vec && i + 3 < n) {
                float4 pp = *reinterpret_cast<float4*>(p + i);
                const float4 gg = __ldg(reinterpret_cast<const float4*>(g + i));
                float4 vv = has_v ? *reinterpret_cast<float4*>(v + i) : make_float4(0, 0, 0, 0);
                sgd_one(pp.x, gg.x, vv.x, b, has_v);
                sgd_one(pp.y, gg.y, vv.y, b, has_v);
                sgd_one(pp.z, gg.z, vv.z, b, has_v);
                sgd_one(pp.w, gg.w, vv.w, b, has_v);
                *reinterpret_cast<float4*>(p + i) = pp;
                if (has_v) *reinterpret_cast<float4*>(v + i) = vv;
                if (i + 3 < n_lo) {
                    *reinterpret_cast<float4*>(lo + i) =
                        make_float4(tenmo_tf32_lo(pp.x), tenmo_tf32_lo(pp.y), tenmo_tf32_lo(pp.z), tenmo_tf32_lo(pp.w));
                } else {
                    const float e4[4] = {pp.x, pp.y, pp.z, pp.w};
                    for (int q = 0; q < 4; ++q)
                        if (i + q < n_lo) lo[i + q] = tenmo_tf32_lo(e4[q]);
                }
            } else {
                for (int q = 0; q < 4 && i + q < n; ++q) {
                    float pp = p[i + q], vv = has_v ? v[i + q] : 0.f;
                    sgd_one(pp, __ldg(g + i + q), vv, b, has_v);
                    p[i + q] = pp;
                    if (has_v) v[i + q] = vv;
                    if (i + q < n_lo) lo[i + q] = tenmo_tf32_lo(pp);
                }
            }
        }
    }
}

}  // namespace

static int sgd_launch(tenmo_ctx* ctx, int n_tensors, float* const* p, const float* const* g, float* const* v,
                      const int64_t* numel, float* const* p_lo, const int64_t* lo_numel, float lr, float momentum,
                      float weight_decay, float grad_scale) {
    TENMO_CHECK_CTX(ctx);
    if (n_tensors < 0) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "sgd: negative tensor count");
    if (n_tensors == 0) return TENMO_OK;
    if (!p || !g || !numel || (momentum > 0.f && !v)) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "sgd: NULL array");
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    int done = 0;
    while (done < n_tensors) {
        SgdBatch b;
        memset(&b, 0, sizeof(b));
        b.lr = lr; b.momentum = momentum; b.wd = weight_decay; b.grad_scale = grad_scale;
        int n = 0;
        int64_t chunks = 0;
        b.chunk_start[0] = 0;
        while (done < n_tensors && n < SGD_MAX_TENSORS) {
            const int64_t ne = numel[done];
            if (ne < 0) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "sgd: tensor %d has negative numel", done);
            if (ne > 0) {
                if (!p[done] || !g[done] || (momentum > 0.f && !v[done]))
                    return tenmo_set_error(ctx, TENMO_ERR_INVALID, "sgd: tensor %d has a NULL pointer", done);
                b.p[n] = p[done]; b.g[n] = g[done]; b.v[n] = momentum > 0.f ? v[done] : nullptr; b.numel[n] = ne;
                if (p_lo && p_lo[done]) {
                    if (!lo_numel || lo_numel[done] < 0 || lo_numel[done] > ne || (reinterpret_cast<uintptr_t>(p_lo[done]) & 15u))
                        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "sgd: tensor %d has a bad lo plane (0 <= lo_numel <= numel, 16-byte aligned)", done);
                    b.lo[n] = p_lo[done];
                    b.lo_numel[n] = lo_numel[done];
                }
                chunks += (ne + SGD_CHUNK - 1) / SGD_CHUNK;
                b.chunk_start[++n] = chunks;
            }
            ++done;
        }
        if (n == 0) continue;
        b.n = n;
        const int64_t cap = (int64_t)ctx->sm_count * 8;
        const int grid = (int)(chunks < cap ? chunks : cap);
        cudaError_t le = tenmo_launch(sgd_kernel, (unsigned)grid, SGD_THREADS, 0, ctx->stream, tenmo_pdl_ok(ctx, grid), b);
        if (le != cudaSuccess) return tenmo_set_error(ctx, TENMO_ERR_CUDA, "launch of sgd_kernel failed: %s", cudaGetErrorString(le));
        TENMO_LAUNCH_CHECK(ctx, "sgd_kernel");
    }
    return TENMO_OK;
}

extern "C" int tenmo_sgd_step_f32(tenmo_ctx* ctx, int n_tensors, float* const* p, const float* const* g,
                                  float* const* v, const int64_t* numel, float lr, float momentum,
                                  float weight_decay, float grad_scale) {
    return sgd_launch(ctx, n_tensors, p, g, v, numel, nullptr, nullptr, lr, momentum, weight_decay, grad_scale);
}

extern "C" int tenmo_sgd_step_lo_f32(tenmo_ctx* ctx, int n_tensors, float* const* p, const float* const* g,
                                     float* const* v, const int64_t* numel, float* const* p_lo, const int64_t* lo_numel,
                                     float lr, float momentum, float weight_decay, float grad_scale) {
    return sgd_launch(ctx, n_tensors, p, g, v, numel, p_lo, lo_numel, lr, momentum, weight_decay, grad_scale);
}
