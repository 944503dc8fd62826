// Data-parallel gradient exchange: a sum all-reduce over one process per GPU, NCCL over NVLink 5 /
// NVSwitch.  The reference has no distributed layer; this is the exchange step of batch-sharded
// training.  NCCL is bound at run time with dlopen (the same libnccl.so.2 a PyTorch process already
// has loaded), so the library itself has no link-time dependency on it.
#include <dlfcn.h>

#include <cstdlib>

#include "common.cuh"

namespace {

typedef struct { char internal[128]; } nccl_unique_id;
typedef void* nccl_comm_t;
enum { NCCL_FLOAT32 = 7, NCCL_SUM = 0 };

struct NcclApi {
    int (*GetUniqueId)(nccl_unique_id*);
    int (*CommInitRank)(nccl_comm_t*, int, nccl_unique_id, int);
    int (*AllReduce)(const void*, void*, size_t, int, int, nccl_comm_t, cudaStream_t);
    int (*CommDestroy)(nccl_comm_t);
    int (*CommAbort)(nccl_comm_t);
    const char* (*GetErrorString)(int);
    int (*CommGetAsyncError)(nccl_comm_t, int*);
};
NcclApi g_nccl;
bool g_nccl_loaded = false;

int load_nccl(tenmo_ctx* ctx) {
    if (g_nccl_loaded) return TENMO_OK;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    const char* env = getenv("TENMO_NCCL_PATH");
    if (env) h = dlopen(env, RTLD_NOW | RTLD_GLOBAL);
    for (int i = 0; !h && i < 2; ++i) h = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
    if (!h) return tenmo_set_error(ctx, TENMO_ERR_NCCL, "cannot load libnccl.so.2 (set TENMO_NCCL_PATH): %s", dlerror());
#define BIND(field, sym)                                                                    \
    *(void**)(&g_nccl.field) = dlsym(h, sym);                                               \
    if (!g_nccl.field) return tenmo_set_error(ctx, TENMO_ERR_NCCL, "libnccl lacks %s", sym);
    BIND(GetUniqueId, "ncclGetUniqueId");
    BIND(CommInitRank, "ncclCommInitRank");
    BIND(AllReduce, "ncclAllReduce");
    BIND(CommDestroy, "ncclCommDestroy");
    BIND(CommAbort, "ncclCommAbort");
    BIND(GetErrorString, "ncclGetErrorString");
    BIND(CommGetAsyncError, "ncclCommGetAsyncError");
#undef BIND
    ctx->nccl_lib = h;
    g_nccl_loaded = true;
    return TENMO_OK;
}

}  // namespace

extern "C" {

int tenmo_dp_get_unique_id(tenmo_ctx* ctx, void* id_out, size_t id_bytes) {
    TENMO_CHECK_CTX(ctx);
    if (!id_out || id_bytes < TENMO_DP_ID_BYTES)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "dp_get_unique_id: need a buffer of %d bytes", TENMO_DP_ID_BYTES);
    int st = load_nccl(ctx);
    if (st != TENMO_OK) return st;
    nccl_unique_id id;
    int r = g_nccl.GetUniqueId(&id);
    if (r != 0) return tenmo_set_error(ctx, TENMO_ERR_NCCL, "ncclGetUniqueId: %s", g_nccl.GetErrorString(r));
    memcpy(id_out, &id, sizeof(id));
    return TENMO_OK;
}

int tenmo_dp_init(tenmo_ctx* ctx, int rank, int world, const void* id, size_t id_bytes) {
    TENMO_CHECK_CTX(ctx);
    if (world < 1 || rank < 0 || rank >= world)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "dp_init: rank %d / world %d", rank, world);
    if (ctx->nccl_comm) return tenmo_set_error(ctx, TENMO_ERR_STATE, "dp_init: already initialised");
    ctx->dp_rank = rank;
    ctx->dp_world = world;
    if (world == 1) return TENMO_OK;  // nothing to exchange
    if (!id || id_bytes < TENMO_DP_ID_BYTES) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "dp_init: bad unique id");
    int st = load_nccl(ctx);
    if (st != TENMO_OK) return st;
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    nccl_unique_id uid;
    memcpy(&uid, id, sizeof(uid));
    nccl_comm_t comm = nullptr;
    int r = g_nccl.CommInitRank(&comm, world, uid, rank);
    if (r != 0) return tenmo_set_error(ctx, TENMO_ERR_NCCL, "ncclCommInitRank: %s", g_nccl.GetErrorString(r));
    ctx->nccl_comm = comm;
    return TENMO_OK;
}

int tenmo_dp_allreduce_sum_f32(tenmo_ctx* ctx, float* buf, int64_t count) {
    TENMO_CHECK_CTX(ctx);
    if (count < 0) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "dp_allreduce: negative count");
    if (ctx->dp_world == 1 || count == 0) return TENMO_OK;
    if (!ctx->nccl_comm) return tenmo_set_error(ctx, TENMO_ERR_STATE, "dp_allreduce: call tenmo_dp_init first");
    if (!buf) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "dp_allreduce: NULL buffer");
    int r = g_nccl.AllReduce(buf, buf, (size_t)count, NCCL_FLOAT32, NCCL_SUM, ctx->nccl_comm, ctx->stream);
    if (r != 0) return tenmo_set_error(ctx, TENMO_ERR_NCCL, "ncclAllReduce: %s", g_nccl.GetErrorString(r));
    return TENMO_OK;
}

int tenmo_dp_finalize(tenmo_ctx* ctx) {
    TENMO_CHECK_CTX(ctx);
    if (ctx->nccl_comm) {
        cudaStreamSynchronize(ctx->stream);
        g_nccl.CommDestroy(ctx->nccl_comm);
        ctx->nccl_comm = nullptr;
    }
    ctx->dp_world = 1;
    ctx->dp_rank = 0;
    return TENMO_OK;
}

}  // extern "C"
