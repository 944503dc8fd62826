// Accuracy: rows whose first-index argmax (strict >) equals the label (accuracy.mojo:20-66).
// One warp per row, any number of rows (the reference kernel is one block of batch_size threads and
// so stops at 1024 rows, kernels/accuracy_kernel.mojo:76-77).  The count is an integer atomic, so the
// result is exact whatever the scheduling.  HBM-bound: 4*M*C + 8*M bytes.
#include "common.cuh"

namespace {

constexpr int ACC_THREADS = 256;

__global__ void __launch_bounds__(ACC_THREADS)
accuracy_kernel(const float* __restrict__ logits, int64_t ld, const void* __restrict__ labels, int is_i64, int64_t M,
                int64_t C, unsigned long long* __restrict__ correct) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned int local = 0;
    for (int64_t row = (int64_t)blockIdx.x * (ACC_THREADS / 32) + warp; row < M;
         row += (int64_t)gridDim.x * (ACC_THREADS / 32)) {
        const float* x = logits + row * ld;
        // lane-local scan in ascending class order keeps the first maximum
        float best = 0.f;
        int64_t idx = -1;
        for (int64_t c = lane; c < C; c += 32) {
            const float v = __ldg(x + c);
            if (idx < 0 || v > best) { best = v; idx = c; }
        }
        // combine lanes: larger value wins, equal values -> smaller index
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int64_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (oi >= 0 && (idx < 0 || ob > best || (ob == best && oi < idx))) { best = ob; idx = oi; }
        }
        if (lane == 0) {
            const int64_t t = is_i64 ? reinterpret_cast<const int64_t*>(labels)[row]
                                     : (int64_t) reinterpret_cast<const int32_t*>(labels)[row];
            if (idx == t) ++local;
        }
    }
    if (lane == 0 && local) atomicAdd(correct, (unsigned long long)local);
}

}  // namespace

extern "C" int tenmo_accuracy_f32(tenmo_ctx* ctx, const float* logits, int64_t ld_logits, const void* labels,
                                  int label_is_i64, int64_t M, int64_t C, int64_t* correct_dev, int64_t* correct_host) {
    TENMO_CHECK_CTX(ctx);
    if (M < 0 || C <= 0) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "accuracy: bad shape");
    if (!correct_dev) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "accuracy: correct_dev is NULL");
    if (M > 0 && (!logits || !labels)) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "accuracy: NULL pointer");
    if (M > 0 && ld_logits < C) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "accuracy: ld_logits < C");
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    TENMO_CUDA_TRY(ctx, cudaMemsetAsync(correct_dev, 0, sizeof(int64_t), ctx->stream));
    if (M > 0) {
        const int grid = tenmo_stream_grid(ctx, M, ACC_THREADS / 32, 8);
        accuracy_kernel<<<grid, ACC_THREADS, 0, ctx->stream>>>(logits, ld_logits, labels, label_is_i64, M, C,
                                                               reinterpret_cast<unsigned long long*>(correct_dev));
        TENMO_LAUNCH_CHECK(ctx, "accuracy_kernel");
    }
    if (correct_host) {
        TENMO_CUDA_TRY(ctx, cudaMemcpyAsync(correct_host, correct_dev, sizeof(int64_t), cudaMemcpyDeviceToHost, ctx->stream));
        TENMO_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    }
    return TENMO_OK;
}
