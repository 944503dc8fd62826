// Context lifetime, error strings, stream binding, workspace.
#include "common.cuh"

// errors of calls that have no context (tenmo_cuda_init, tenmo_colsum_f32_static): one buffer per host thread
static thread_local char g_init_error[512] = {0};

int tenmo_set_error(tenmo_ctx* ctx, int status, const char* fmt, ...) {
    char* dst = ctx ? ctx->err : g_init_error;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(dst, 512, fmt, ap);
    va_end(ap);
    return status;
}

// Waits for every stream this context has been bound to (work that uses the workspace, the status block or the
// tickets may be queued on any of them).
static cudaError_t sync_bound_streams(tenmo_ctx* ctx) {
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    for (int i = 0; i < ctx->n_bound && e == cudaSuccess; ++i)
        if (ctx->bound[i] != ctx->stream) e = cudaStreamSynchronize(ctx->bound[i]);
    return e;
}

int tenmo_workspace(tenmo_ctx* ctx, size_t bytes, void** out) {
    if (bytes > ctx->ws_bytes) {
        // Growing frees the old block and allocates: neither is allowed while the stream records a CUDA graph.
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(ctx->stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
            return tenmo_set_error(ctx, TENMO_ERR_STATE,
                                   "the workspace must grow to %zu bytes but the stream is capturing: run the call once outside the capture first",
                                   bytes);
        // The old block may still be in use by work queued on any stream the context was bound to.
        if (ctx->ws) {
            cudaError_t e = sync_bound_streams(ctx);
            if (e != cudaSuccess) return tenmo_set_error(ctx, TENMO_ERR_CUDA, "workspace sync: %s", cudaGetErrorString(e));
            cudaFree(ctx->ws);
            ctx->ws = nullptr;
            ctx->ws_bytes = 0;
        }
        size_t want = (bytes + ((size_t)1 << 20) - 1) & ~(((size_t)1 << 20) - 1);
        cudaError_t e = cudaMalloc(&ctx->ws, want);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return tenmo_set_error(ctx, TENMO_ERR_NOMEM, "workspace of %zu bytes: %s", want, cudaGetErrorString(e));
        }
        ctx->ws_bytes = want;
    }
    *out = ctx->ws;
    return TENMO_OK;
}

void tenmo_prof_before(tenmo_ctx* ctx) {
    if (!ctx->prof_on || ctx->prof_n >= ctx->prof_cap) return;
    cudaEventRecord(ctx->prof_ev[2 * ctx->prof_n], ctx->stream);
}
void tenmo_prof_after(tenmo_ctx* ctx) {
    if (!ctx->prof_on || ctx->prof_n >= ctx->prof_cap) return;
    cudaEventRecord(ctx->prof_ev[2 * ctx->prof_n + 1], ctx->stream);
    ctx->prof_n++;
}

extern "C" {

int tenmo_cuda_profile_begin(tenmo_ctx* ctx) {
    TENMO_CHECK_CTX(ctx);
    if (!ctx->prof_ev) {
        const int cap = 4096;
        ctx->prof_ev = new cudaEvent_t[2 * cap];
        for (int i = 0; i < 2 * cap; ++i) TENMO_CUDA_TRY(ctx, cudaEventCreate(&ctx->prof_ev[i]));
        ctx->prof_cap = cap;
    }
    ctx->prof_n = 0;
    ctx->prof_on = true;
    return TENMO_OK;
}

int tenmo_cuda_profile_end(tenmo_ctx* ctx, int64_t* launches, double* total_ms) {
    TENMO_CHECK_CTX(ctx);
    ctx->prof_on = false;
    TENMO_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    double sum = 0.0;
    for (int i = 0; i < ctx->prof_n; ++i) {
        float ms = 0.f;
        TENMO_CUDA_TRY(ctx, cudaEventElapsedTime(&ms, ctx->prof_ev[2 * i], ctx->prof_ev[2 * i + 1]));
        sum += ms;
    }
    if (launches) *launches = ctx->prof_n;
    if (total_ms) *total_ms = sum;
    ctx->prof_n = 0;
    return TENMO_OK;
}

const char* tenmo_cuda_version(void) { return "tenmo_cuda 0.1 (sm_100a)"; }

int tenmo_cuda_init(int device, tenmo_ctx** out) {
    if (!out) return tenmo_set_error(nullptr, TENMO_ERR_INVALID, "tenmo_cuda_init: out is NULL");
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        cudaGetLastError();
        return tenmo_set_error(nullptr, TENMO_ERR_CUDA, "no CUDA device: %s", cudaGetErrorString(e));
    }
    if (device < 0 || device >= n)
        return tenmo_set_error(nullptr, TENMO_ERR_INVALID, "device %d out of range [0,%d)", device, n);
    e = cudaSetDevice(device);
    if (e != cudaSuccess) return tenmo_set_error(nullptr, TENMO_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(e));
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return tenmo_set_error(nullptr, TENMO_ERR_CUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    if (prop.major != 10)
        return tenmo_set_error(nullptr, TENMO_ERR_UNSUPPORTED,
                               "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major,
                               prop.minor);
    tenmo_ctx* ctx = new tenmo_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->cc_major = prop.major;
    ctx->cc_minor = prop.minor;
    ctx->smem_optin = prop.sharedMemPerBlockOptin;
    int khz = 0;
    cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, device);
    ctx->sm_clock_khz = khz;
    {
        const char* env_pdl = getenv("TENMO_PDL");
        ctx->pdl = !(env_pdl && atoi(env_pdl) == 0);
    }
    e = cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMalloc(&ctx->dev_status, TENMO_DEV_STATUS_WORDS * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(ctx->dev_status, 0, TENMO_DEV_STATUS_WORDS * sizeof(uint32_t));
    if (e != cudaSuccess) {
        tenmo_set_error(nullptr, TENMO_ERR_CUDA, "context set-up: %s", cudaGetErrorString(e));
        tenmo_cuda_destroy(ctx);
        return TENMO_ERR_CUDA;
    }
    ctx->stream = ctx->own_stream;
    *out = ctx;
    return TENMO_OK;
}

void tenmo_cuda_destroy(tenmo_ctx* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->nccl_comm) tenmo_dp_finalize(ctx);
    if (ctx->p2p_buf) tenmo_dp_p2p_close(ctx);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    if (ctx->ws) cudaFree(ctx->ws);
    if (ctx->dev_status) cudaFree(ctx->dev_status);
    if (ctx->tickets) cudaFree(ctx->tickets);
    if (ctx->sgd_desc_dev) cudaFree(ctx->sgd_desc_dev);
    if (ctx->sgd_desc_host) cudaFreeHost(ctx->sgd_desc_host);
    if (ctx->prof_ev) {
        for (int i = 0; i < 2 * ctx->prof_cap; ++i) cudaEventDestroy(ctx->prof_ev[i]);
        delete[] ctx->prof_ev;
    }
    if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
    delete ctx;
}

const char* tenmo_cuda_last_error(tenmo_ctx* ctx) { return ctx ? ctx->err : g_init_error; }

int tenmo_cuda_set_stream(tenmo_ctx* ctx, void* cuda_stream) {
    TENMO_CHECK_CTX(ctx);
    ctx->stream = cuda_stream == TENMO_STREAM_OWN ? ctx->own_stream : (cudaStream_t)cuda_stream;
    // remember the streams the context has run on (most recent first): a workspace growth and the status check wait for them
    int at = -1;
    for (int i = 0; i < ctx->n_bound; ++i)
        if (ctx->bound[i] == ctx->stream) at = i;
    if (at < 0) {
        if (ctx->n_bound < TENMO_MAX_BOUND_STREAMS) ++ctx->n_bound;
        at = ctx->n_bound - 1;
    }
    for (int i = at; i > 0; --i) ctx->bound[i] = ctx->bound[i - 1];
    ctx->bound[0] = ctx->stream;
    return TENMO_OK;
}

int tenmo_cuda_reserve_sms(tenmo_ctx* ctx, int n) {
    TENMO_CHECK_CTX(ctx);
    if (n < 0 || n >= ctx->sm_count)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "reserve_sms: %d is outside [0, %d)", n, ctx->sm_count);
    ctx->reserve_sms = n;
    return TENMO_OK;
}

int tenmo_cuda_synchronize(tenmo_ctx* ctx) {
    TENMO_CHECK_CTX(ctx);
    TENMO_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return TENMO_OK;
}

int tenmo_cuda_device_info(tenmo_ctx* ctx, int* sm_count, int* cc_major, int* cc_minor, int* sm_clock_khz) {
    TENMO_CHECK_CTX(ctx);
    if (sm_count) *sm_count = ctx->sm_count;
    if (cc_major) *cc_major = ctx->cc_major;
    if (cc_minor) *cc_minor = ctx->cc_minor;
    if (sm_clock_khz) *sm_clock_khz = ctx->sm_clock_khz;
    return TENMO_OK;
}

int tenmo_cuda_check_device_status(tenmo_ctx* ctx) {
    TENMO_CHECK_CTX(ctx);
    uint32_t word = 0;
    TENMO_CUDA_TRY(ctx, sync_bound_streams(ctx));
    TENMO_CUDA_TRY(ctx, cudaMemcpy(&word, ctx->dev_status, sizeof(word), cudaMemcpyDeviceToHost));
    if (word) {
        // an abandoned kernel may have left its tickets and tile counters dirty: clear the whole block
        TENMO_CUDA_TRY(ctx, cudaMemset(ctx->dev_status, 0, TENMO_DEV_STATUS_WORDS * sizeof(uint32_t)));
        if (word & TENMO_DEV_TIMEOUT)
            return tenmo_set_error(ctx, TENMO_ERR_TIMEOUT, "a device-side bounded wait gave up (status 0x%x)", word);
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "device status 0x%x: label outside [0,C) seen by cross-entropy",
                               word);
    }
    return TENMO_OK;
}

int64_t tenmo_cuda_launch_count(tenmo_ctx* ctx, int reset) {
    if (!ctx) return 0;
    int64_t n = ctx->launches;
    if (reset) ctx->launches = 0;
    return n;
}

}  // extern "C"
