// tenmo_gemm_f32 / tenmo_gemm_f32_ex: argument validation, batch broadcasting and kernel selection.
#include "gemm_simt.cuh"
#include "gemm_tc.cuh"
#include "reduce.cuh"

namespace {

int build_batch(tenmo_ctx* ctx, const tenmo_mat* A, const tenmo_mat* B, TenmoBatch* out, int64_t* total) {
    const int ra = A->batch_rank, rb = B ? B->batch_rank : 0;
    if (ra < 0 || rb < 0 || ra > TENMO_MAX_BATCH_RANK || rb > TENMO_MAX_BATCH_RANK)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "gemm: batch rank out of range (A %d, B %d, max %d)", ra, rb,
                               TENMO_MAX_BATCH_RANK);
    const int r = ra > rb ? ra : rb;
    out->rank = r;
    int64_t t = 1;
    for (int d = 0; d < r; ++d) {
        const int ad = d - (r - ra), bd = d - (r - rb);
        const int64_t sa = ad >= 0 ? A->batch_shape[ad] : 1;
        const int64_t sb = (B && bd >= 0) ? B->batch_shape[bd] : 1;
        if (sa < 0 || sb < 0 || (sa != sb && sa != 1 && sb != 1))
            return tenmo_set_error(ctx, TENMO_ERR_INVALID,
                                   "gemm: batch shapes not broadcastable at dim %d (%lld vs %lld)", d, (long long)sa,
                                   (long long)sb);
        out->shape[d] = sa > sb ? sa : sb;
        out->a_stride[d] = (ad >= 0 && sa > 1) ? A->batch_stride[ad] : 0;
        out->b_stride[d] = (B && bd >= 0 && sb > 1) ? B->batch_stride[bd] : 0;
        t *= out->shape[d];
    }
    for (int d = r; d < TENMO_MAX_BATCH_RANK; ++d) {
        out->shape[d] = 1;
        out->a_stride[d] = out->b_stride[d] = 0;
    }
    *total = t;
    return TENMO_OK;
}

}  // namespace

extern "C" {

// Split-K for the tensor-core kernel: a product with a small output and a very long k (the weight gradient of a narrow
// layer at a large batch, K = batch) leaves most SMs without a tile.  The k range is cut into S equal slices that run
// as the S batches of one batched GEMM (operand batch stride = one slice along k) into S partial results, which the
// sequential column-sum kernel then adds in slice order (deterministic) into C.  Only for calls without an epilogue and
// without caller-supplied lo planes; the strict-fp32 kernel never splits (one k-ascending chain per output is its contract).
static int tc_split_k(tenmo_ctx* ctx, const TenmoGemmParams& p, const tenmo_gemm_opts* o, bool* done) {
    *done = false;
    if (p.total_batch != 1 || p.batch.rank != 0) return TENMO_OK;
    if (o->bias || o->act != TENMO_ACT_NONE || o->aux || o->mul_mask || o->c_lo || o->bias_m || o->a_lo || o->b_lo) return TENMO_OK;
    const int64_t tiles = ((p.M + 127) / 128) * ((p.N + 127) / 128);
    if (p.K < 4096 || tiles * 2 > ctx->sm_count) return TENMO_OK;
    // slices: enough for about 1.5 work units per SM, each at least 512 long and a multiple of the k-block, K = S * slice
    const int64_t want = (3 * (int64_t)ctx->sm_count / 2 + tiles - 1) / tiles;
    const int64_t s_max = p.K / 512 < TENMO_COLSUM_SEQ_ROWS ? p.K / 512 : TENMO_COLSUM_SEQ_ROWS;
    auto fits = [&](int64_t s) { return s >= 2 && p.K % s == 0 && (p.K / s) % 32 == 0; };
    int64_t S = 0;
    for (int64_t s = want; s <= s_max && S == 0; ++s)
        if (fits(s)) S = s;
    for (int64_t s = (want < s_max ? want : s_max); s >= 2 && S == 0; --s)
        if (fits(s)) S = s;
    if (S == 0) return TENMO_OK;
    const int64_t Ks = p.K / S;
    TenmoGemmParams q = p;
    q.K = Ks;
    q.total_batch = S;
    q.batch.rank = 1;
    q.batch.shape[0] = S;
    q.batch.a_stride[0] = Ks * p.a_cs;
    q.batch.b_stride[0] = Ks * p.b_rs;
    q.beta = 0.f;
    char why[160];
    if (!tenmo_gemm_tc_supported(ctx, q, why, sizeof(why))) return TENMO_OK;
    const size_t part_bytes = (((size_t)S * (size_t)p.M * (size_t)p.N * sizeof(float)) + 1023) & ~(size_t)1023;
    // reserve partials + lo planes in one request so that the kernel launch below does not move the block
    const size_t lo_bytes = ((size_t)(p.M + 4) * (size_t)(p.K + 4) + (size_t)(p.N + 4) * (size_t)(p.K + 4)) * sizeof(float) + 8192;
    void* ws = nullptr;
    int st = tenmo_workspace(ctx, part_bytes + lo_bytes, &ws);
    if (st != TENMO_OK) return st;
    q.C = static_cast<float*>(ws);
    q.ws_skip = part_bytes;
    st = tenmo_gemm_tc_launch(ctx, q);
    if (st != TENMO_OK) return st;
    st = tenmo_colsum_f32(ctx, q.C, S, p.M * p.N, p.M * p.N, p.C, p.beta);
    if (st != TENMO_OK) return st;
    *done = true;
    return TENMO_OK;
}

int tenmo_gemm_last_algo(tenmo_ctx* ctx) { return ctx ? ctx->last_gemm_algo : -1; }
const char* tenmo_gemm_last_kernel(tenmo_ctx* ctx) { return ctx ? ctx->last_gemm_kernel : ""; }
int tenmo_gemm_last_stream_k(tenmo_ctx* ctx) { return ctx ? ctx->last_gemm_sk_units : 0; }

int tenmo_gemm_f32_ex(tenmo_ctx* ctx, int algo, int64_t M, int64_t N, int64_t K, const tenmo_mat* A, const tenmo_mat* B,
                      float* C, const tenmo_gemm_opts* o) {
    TENMO_CHECK_CTX(ctx);
    tenmo_gemm_opts none;
    memset(&none, 0, sizeof(none));
    if (!o) o = &none;
    if (!A || !B) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "gemm: NULL operand descriptor");
    if (M < 0 || N < 0 || K < 0)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "gemm: negative dimension (M=%lld N=%lld K=%lld)", (long long)M,
                               (long long)N, (long long)K);
    if (algo < TENMO_ALGO_AUTO || algo > TENMO_ALGO_TC_3XTF32)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "gemm: unknown algo %d", algo);
    if (o->act < TENMO_ACT_NONE || o->act > TENMO_ACT_SIGMOID)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "gemm: unknown activation %d", o->act);
    if (o->beta != 0.f && o->beta != 1.f) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "gemm: beta must be 0 or 1");
    TenmoGemmParams p;
    memset(&p, 0, sizeof(p));
    int st = build_batch(ctx, A, B, &p.batch, &p.total_batch);
    if (st != TENMO_OK) return st;
    if (o->colsum && p.batch.rank != 0)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "gemm: colsum output is defined for 2-D operands only");
    if (M == 0 || N == 0 || p.total_batch == 0) return TENMO_OK;  // empty output: nothing to do
    if (!C) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "gemm: C is NULL");
    if (K > 0 && (!A->ptr || !B->ptr)) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "gemm: NULL operand pointer");
    p.A = A->ptr ? A->ptr + A->offset : nullptr;
    p.B = B->ptr ? B->ptr + B->offset : nullptr;
    p.C = C;
    p.M = M; p.N = N; p.K = K;
    p.a_rs = A->row_stride; p.a_cs = A->col_stride;
    p.b_rs = B->row_stride; p.b_cs = B->col_stride;
    p.beta = o->beta; p.bias = o->bias; p.act = o->act; p.aux = o->aux;
    p.a_lo = o->a_lo; p.b_lo = o->b_lo; p.c_lo = o->c_lo; p.mul_mask = o->mul_mask;
    p.ld_clo = (N + 3) / 4 * 4;
    p.bias_m = o->bias_m;

    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    int chosen = TENMO_ALGO_SIMT_FP32;
    if (algo != TENMO_ALGO_SIMT_FP32) {
        char why[160] = {0};
        const bool ok = tenmo_gemm_tc_supported(ctx, p, why, sizeof(why));
        if (algo == TENMO_ALGO_TC_3XTF32 && !ok)
            return tenmo_set_error(ctx, TENMO_ERR_UNSUPPORTED, "gemm: tensor-core kernel cannot take this call: %s", why);
        if (ok && (algo == TENMO_ALGO_TC_3XTF32 || tenmo_gemm_tc_profitable(ctx, p))) chosen = TENMO_ALGO_TC_3XTF32;
    }
    bool colsum_done = false;
    if (chosen == TENMO_ALGO_TC_3XTF32) {
        bool split_done = false;
        st = tc_split_k(ctx, p, o, &split_done);
        if (st == TENMO_OK && !split_done) st = tenmo_gemm_tc_launch(ctx, p);
    } else {
        // up to TENMO_COLSUM_SEQ_ROWS rows the column sum is the sequential one, which the GEMM kernel can produce itself
        if (o->colsum && B->col_stride == 1 && K <= TENMO_COLSUM_SEQ_ROWS && K > 0) p.colsum = o->colsum;
        st = tenmo_gemm_simt_launch(ctx, p, &colsum_done);
    }
    if (st != TENMO_OK) return st;
    ctx->last_gemm_algo = chosen;
    if (o->colsum && !colsum_done) {
        // column sums of the right operand: db when this call is dW = X^T . dY
        if (B->col_stride != 1)
            return tenmo_set_error(ctx, TENMO_ERR_UNSUPPORTED, "gemm: colsum needs a unit column stride on B");
        st = tenmo_colsum_f32(ctx, p.B, K, N, B->row_stride, o->colsum, o->beta);
    }
    return st;
}

int tenmo_gemm_f32(tenmo_ctx* ctx, int algo, int64_t M, int64_t N, int64_t K, const tenmo_mat* A, const tenmo_mat* B,
                   float* C, float beta, const float* bias, int act, float* aux, float* colsum) {
    tenmo_gemm_opts o;
    memset(&o, 0, sizeof(o));
    o.beta = beta; o.bias = bias; o.act = act; o.aux = aux; o.colsum = colsum;
    return tenmo_gemm_f32_ex(ctx, algo, M, N, K, A, B, C, &o);
}

int tenmo_gemm_last_pair(tenmo_ctx* ctx) { return ctx && ctx->last_gemm_pair ? 1 : 0; }

int tenmo_split_lo_f32(tenmo_ctx* ctx, const tenmo_mat* X, int64_t rows, int64_t cols, float* lo_out, int64_t capacity) {
    TENMO_CHECK_CTX(ctx);
    if (!X || !X->ptr || !lo_out) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "split_lo: NULL pointer");
    if (rows <= 0 || cols <= 0) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "split_lo: empty matrix");
    TenmoBatch batch;
    int64_t total = 1;
    int st = build_batch(ctx, X, nullptr, &batch, &total);
    if (st != TENMO_OK) return st;
    const int64_t inner = (X->col_stride == 1 || cols == 1) ? cols : rows, outer = inner == cols ? rows : cols;
    const int64_t need = total * outer * ((inner + 3) / 4 * 4);
    if (capacity < need)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "split_lo: output holds %lld floats, %lld needed", (long long)capacity,
                               (long long)need);
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return tenmo_split_lo_launch(ctx, X->ptr + X->offset, rows, cols, X->row_stride, X->col_stride, batch, batch.a_stride, total,
                                 lo_out, nullptr);
}

}  // extern "C"
