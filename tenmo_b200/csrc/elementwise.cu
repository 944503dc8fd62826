// Bandwidth-bound elementwise neighbours of the GEMM, for a host that calls op by op.
// All are grid-stride kernels over float4 with a scalar tail; grid = a multiple of the SM count.
// Roofline: HBM.  Algorithmic bytes per element: add_bias 8, add_inplace 12, fill 4, relu_fwd 12
// (8 without the mask), relu_bwd / sigmoid_bwd 12 (16 accumulating), sigmoid_fwd 8.
#include "common.cuh"

namespace {

constexpr int EW_THREADS = 256;

enum EwOp { EW_ADD_INPLACE, EW_FILL, EW_RELU_FWD, EW_RELU_BWD, EW_SIGMOID_FWD, EW_SIGMOID_BWD };

struct EwArgs {
    const float* a;  // first input
    const float* b;  // second input
    float* out;
    float* out2;  // relu mask
    float scalar;
    float beta;
    int64_t n;
};

template <int OP>
__device__ __forceinline__ void ew_apply(float a, float b, float old, float old2, const EwArgs& p, float& o, float& o2) {
    (void)old2;
    o2 = 0.f;
    if (OP == EW_ADD_INPLACE) o = old + a;
    else if (OP == EW_FILL) o = p.scalar;
    else if (OP == EW_RELU_FWD) { o = a > 0.f ? a : 0.f; o2 = a > 0.f ? 1.f : 0.f; }
    else if (OP == EW_RELU_BWD) { o = a * b; if (p.beta != 0.f) o += old; }
    else if (OP == EW_SIGMOID_FWD) o = 1.f / (1.f + expf(-a));
    else { o = __fmul_rn(__fmul_rn(a, b), 1.f - b); if (p.beta != 0.f) o += old; }  // (g*y)*(1-y)
}

// NC: the inputs may be read through the non-coherent path (ld.global.nc).  That is only defined for memory the
// kernel does not write, so an in-place call (an input aliasing an output, e.g. relu_bwd(g, mask, g)) takes the
// instantiation with plain loads.
template <bool NC, typename T>
__device__ __forceinline__ T ew_load(const T* p) {
    return NC ? __ldg(p) : *p;
}

template <int OP, bool NC>
__global__ void __launch_bounds__(EW_THREADS) ew_kernel(const EwArgs p, const int vec_ok) {
    constexpr bool READ_A = OP != EW_FILL;
    constexpr bool READ_B = OP == EW_RELU_BWD || OP == EW_SIGMOID_BWD;
    const bool read_old = OP == EW_ADD_INPLACE || ((OP == EW_RELU_BWD || OP == EW_SIGMOID_BWD) && p.beta != 0.f);
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t n4 = vec_ok ? p.n / 4 : 0;
    for (int64_t i = tid; i < n4; i += stride) {
        float4 a = make_float4(0, 0, 0, 0), b = a, old = a, o, o2;
        if (READ_A) a = ew_load<NC>(reinterpret_cast<const float4*>(p.a) + i);
        if (READ_B) b = ew_load<NC>(reinterpret_cast<const float4*>(p.b) + i);
        if (read_old) old = reinterpret_cast<const float4*>(p.out)[i];
        ew_apply<OP>(a.x, b.x, old.x, 0.f, p, o.x, o2.x);
        ew_apply<OP>(a.y, b.y, old.y, 0.f, p, o.y, o2.y);
        ew_apply<OP>(a.z, b.z, old.z, 0.f, p, o.z, o2.z);
        ew_apply<OP>(a.w, b.w, old.w, 0.f, p, o.w, o2.w);
        reinterpret_cast<float4*>(p.out)[i] = o;
        if (OP == EW_RELU_FWD && p.out2) reinterpret_cast<float4*>(p.out2)[i] = o2;
    }
    for (int64_t i = n4 * 4 + tid; i < p.n; i += stride) {
        float a = 0.f, b = 0.f, old = 0.f, o, o2;
        if (READ_A) a = ew_load<NC>(p.a + i);
        if (READ_B) b = ew_load<NC>(p.b + i);
        if (read_old) old = p.out[i];
        ew_apply<OP>(a, b, old, 0.f, p, o, o2);
        p.out[i] = o;
        if (OP == EW_RELU_FWD && p.out2) p.out2[i] = o2;
    }
}

// out[m,n] = x[m,n] + bias[n]
// x and out may be the same buffer (each element is read and then written by the same thread), so x is read with
// plain loads and neither pointer is declared restrict.
__global__ void __launch_bounds__(EW_THREADS) add_bias_kernel(const float* x, const float* __restrict__ bias,
                                                             float* out, int64_t M, int64_t N, int vec_ok) {
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t total = M * N;
    if (vec_ok) {  // N % 4 == 0: a float4 never straddles a row
        const int64_t n4 = total / 4, row4 = N / 4;
        for (int64_t i = tid; i < n4; i += stride) {
            float4 v = reinterpret_cast<const float4*>(x)[i];
            const float4 b = __ldg(reinterpret_cast<const float4*>(bias) + (i % row4));
            v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
            reinterpret_cast<float4*>(out)[i] = v;
        }
    } else {
        for (int64_t i = tid; i < total; i += stride) out[i] = x[i] + __ldg(bias + (i % N));
    }
}

bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <int OP>
int launch_ew(tenmo_ctx* ctx, const EwArgs& p, const char* name) {
    if (p.n < 0) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "%s: negative length", name);
    if (p.n == 0) return TENMO_OK;
    if (!p.out || (OP != EW_FILL && !p.a) || ((OP == EW_RELU_BWD || OP == EW_SIGMOID_BWD) && !p.b))
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "%s: NULL pointer", name);
    const int vec_ok = al16(p.a) && al16(p.b) && al16(p.out) && al16(p.out2);
    const int grid = tenmo_stream_grid(ctx, p.n, EW_THREADS * 4 * 4, 8);
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    // inputs that overlap an output anywhere are read coherently (exact aliasing is the supported in-place form)
    auto overlaps = [&](const float* in, const float* out) {
        return in && out && in < out + p.n && out < in + p.n;
    };
    const bool aliased = overlaps(p.a, p.out) || overlaps(p.b, p.out) || overlaps(p.a, p.out2) || overlaps(p.b, p.out2);
    if (aliased) ew_kernel<OP, false><<<grid, EW_THREADS, 0, ctx->stream>>>(p, vec_ok);
    else ew_kernel<OP, true><<<grid, EW_THREADS, 0, ctx->stream>>>(p, vec_ok);
    TENMO_LAUNCH_CHECK(ctx, name);
    return TENMO_OK;
}

}  // namespace

extern "C" {

int tenmo_add_bias_f32(tenmo_ctx* ctx, const float* x, const float* bias, float* out, int64_t M, int64_t N) {
    TENMO_CHECK_CTX(ctx);
    if (M < 0 || N < 0) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "add_bias: negative shape");
    if (M == 0 || N == 0) return TENMO_OK;
    if (!x || !bias || !out) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "add_bias: NULL pointer");
    const int vec_ok = (N % 4 == 0) && al16(x) && al16(bias) && al16(out);
    const int grid = tenmo_stream_grid(ctx, M * N, EW_THREADS * 16, 8);
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    add_bias_kernel<<<grid, EW_THREADS, 0, ctx->stream>>>(x, bias, out, M, N, vec_ok);
    TENMO_LAUNCH_CHECK(ctx, "add_bias_kernel");
    return TENMO_OK;
}

int tenmo_add_inplace_f32(tenmo_ctx* ctx, float* out, const float* in, int64_t n) {
    TENMO_CHECK_CTX(ctx);
    EwArgs p{in, nullptr, out, nullptr, 0.f, 0.f, n};
    return launch_ew<EW_ADD_INPLACE>(ctx, p, "add_inplace");
}

int tenmo_fill_f32(tenmo_ctx* ctx, float* x, float value, int64_t n) {
    TENMO_CHECK_CTX(ctx);
    EwArgs p{nullptr, nullptr, x, nullptr, value, 0.f, n};
    return launch_ew<EW_FILL>(ctx, p, "fill");
}

int tenmo_relu_fwd_f32(tenmo_ctx* ctx, const float* x, float* out, float* mask, int64_t n) {
    TENMO_CHECK_CTX(ctx);
    EwArgs p{x, nullptr, out, mask, 0.f, 0.f, n};
    return launch_ew<EW_RELU_FWD>(ctx, p, "relu_fwd");
}

int tenmo_relu_bwd_f32(tenmo_ctx* ctx, const float* g, const float* mask, float* dx, float beta, int64_t n) {
    TENMO_CHECK_CTX(ctx);
    if (beta != 0.f && beta != 1.f) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "relu_bwd: beta must be 0 or 1");
    EwArgs p{g, mask, dx, nullptr, 0.f, beta, n};
    return launch_ew<EW_RELU_BWD>(ctx, p, "relu_bwd");
}

int tenmo_sigmoid_fwd_f32(tenmo_ctx* ctx, const float* x, float* y, int64_t n) {
    TENMO_CHECK_CTX(ctx);
    EwArgs p{x, nullptr, y, nullptr, 0.f, 0.f, n};
    return launch_ew<EW_SIGMOID_FWD>(ctx, p, "sigmoid_fwd");
}

int tenmo_sigmoid_bwd_f32(tenmo_ctx* ctx, const float* g, const float* y, float* dx, float beta, int64_t n) {
    TENMO_CHECK_CTX(ctx);
    if (beta != 0.f && beta != 1.f) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "sigmoid_bwd: beta must be 0 or 1");
    EwArgs p{g, y, dx, nullptr, 0.f, beta, n};
    return launch_ew<EW_SIGMOID_BWD>(ctx, p, "sigmoid_bwd");
}

}  // extern "C"
