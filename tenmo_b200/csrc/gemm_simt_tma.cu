// Strict-FP32 SIMT GEMM with TMA-staged shared-memory tiles.
//
// Same arithmetic contract as gemm_simt.cu: every output element is one k-ascending fmaf chain, so the two
// kernels give identical bits.  What differs is how the 128 x 128 x 16 tiles reach shared memory and how the
// multiplies are issued.
//   * Staging: one elected thread issues two tiled bulk copies (cp.async.bulk.tensor, no multicast) per k-tile
//     into a ring of four 16 KB stages guarded by full / empty mbarriers, so the k loop holds no global load,
//     no address arithmetic, no staging store and no block-wide barrier.
//   * Multiply: the packed fma.rn.f32x2 (two independent round-to-nearest FMAs per lane and instruction, the
//     same bits as two fmaf).  The FP32 pipe takes one warp-level FFMA per cycle per scheduler, which is also
//     the issue limit, so with scalar fmaf every fragment read displaces an FFMA and three-operand delivery
//     shows up as dispatch stalls (0.61-0.66 of peak); the packed form needs half the instructions and runs
//     into the pipe itself (0.74-0.83).  It wants one operand as a pair of neighbouring registers.
// Shared-memory layouts (what the copy engine writes) and the fragment reads that go with them:
//   unit stride along m / n ("MN-major", e.g. row-major B or a transposed view of A): box {128, 16} ->
//       [k][128] rows of 512 B; per k a thread reads its 8 values as two float4 (columns tx*4.. and 64+tx*4..);
//       neighbouring columns are neighbouring registers, so B supplies the pairs and a value of A is used twice.
//   unit stride along k ("K-major", e.g. row-major A): box {16, 128} -> [row][16] rows of 64 B, written with
//       the 64-byte swizzle (16-byte chunk index ^= (row >> 1) & 3).  The copy engine cannot transpose 32-bit
//       elements.  Operand A: each warp only multiplies with 16 rows of the tile, and transposes those for
//       itself into a private [k][16] block (two 16-byte reads, eight 4-byte writes per lane and k-tile, a
//       __syncwarp), after which its fragments read like the MN-major ones.  Operand B (all 128 rows are needed
//       by every warp): fragments are read as float2 ALONG k from the swizzled tile, a thread's columns are
//       interleaved (n = tx + 16 j: 16 consecutive rows spread over the banks), the pairs run down the rows of A
//       and a value of B is used twice.
// Fragments are shared inside a warp by same-address shared-memory reads (a broadcast costs no extra
// wavefront); a shuffle-based exchange would put one more instruction per value into the issue stream.
// Every mbarrier wait is bounded (2 s); on expiry the kernel raises the context status word, waits for the
// copies it has in flight and returns without storing.
// Roofline: FP32 pipe, 2*M*N*K flop against 2 * 128 lanes * SMs * clock.
#include <cstdlib>

#include "gemm_tc.cuh"
#include "tma_util.cuh"

namespace {

constexpr int ST_BM = 128, ST_BN = 128, ST_BK = 16;
constexpr int ST_STAGES = 4;
constexpr int ST_THREADS = 256;
constexpr int ST_TILE = 128 * ST_BK * 4;  // bytes of one operand tile
constexpr int ST_STAGE = 2 * ST_TILE;
constexpr int ST_LDT = 20;                          // floats per k row of a warp's transposed A fragment block
constexpr int ST_TBUF = ST_BK * ST_LDT * 4;         // bytes of that block (one per warp)
constexpr int ST_SMEM = ST_STAGES * ST_STAGE + 1024 /*alignment slack*/ + 128 /*barriers, abort flag*/ +
                        (ST_THREADS / 32) * ST_TBUF;
constexpr int ST_GROUP_M = 16;  // tile order: groups of 16 row tiles walked column by column (L2 reuse)

struct StParams {
    float* C;
    float* aux;
    const float* bias;
    const float* bias_m;
    const float* mul_mask;
    float* c_lo;
    int64_t ld_clo;
    int64_t M, N, K;
    int tiles_m, tiles_n;
    int a_batched, b_batched;
    float beta;
    int act;
    int c_vec;
    uint32_t* status;
};

__device__ __forceinline__ float st_act(float v, int act) {
    if (act == TENMO_ACT_RELU) return v > 0.f ? v : 0.f;
    if (act == TENMO_ACT_SIGMOID) return 1.f / (1.f + expf(-v));
    return v;
}

__device__ __forceinline__ float4 lds128(const uint8_t* p) { return *reinterpret_cast<const float4*>(p); }

// row / column of register index i in the quadrant split (two runs of four, 64 apart)
__device__ __forceinline__ int quad_index(int t, int i) { return (i >> 2) * 64 + t * 4 + (i & 3); }

// Two independent fused multiply-adds: one packed fma.rn.f32x2 (both halves rounded to
// nearest exactly like fmaf, so the bits do not change) or, for comparison, two scalar fmaf.
template <bool PACKED>
__device__ __forceinline__ float2 fma_pair(float a0, float a1, float b0, float b1, float2 c) {
    if (PACKED) return __ffma2_rn(make_float2(a0, a1), make_float2(b0, b1), c);
    return make_float2(fmaf(a0, b0, c.x), fmaf(a1, b1, c.y));
}

// A_K / B_K: the operand's unit-stride axis is k.  PACKED: the k loop multiplies with fma.rn.f32x2.
template <bool A_K, bool B_K, bool PACKED>
__global__ void __launch_bounds__(ST_THREADS, 2)
gemm_simt_tma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const StParams p) {
    extern __shared__ uint8_t st_smem_raw[];
    const uint32_t smem_base = (smem_u32(st_smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = st_smem_raw + (smem_base - smem_u32(st_smem_raw));
    const uint32_t bar_base = smem_base + ST_STAGES * ST_STAGE;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (ST_STAGES + s); };
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + ST_STAGES * ST_STAGE + 8 * 2 * ST_STAGES);

    const int tid = threadIdx.x, lane = tid & 31;
    const int tx = tid & 15, ty = tid >> 4;

    // tile decode
    const int64_t per_batch = (int64_t)p.tiles_m * p.tiles_n;
    const int64_t batch = (int64_t)blockIdx.x / per_batch;
    int tile_m, tile_n;
    {
        const int t = (int)((int64_t)blockIdx.x % per_batch);
        const int group = t / (ST_GROUP_M * p.tiles_n);
        const int first_m = group * ST_GROUP_M;
        const int rows = min(ST_GROUP_M, p.tiles_m - first_m);
        const int in_group = t - group * ST_GROUP_M * p.tiles_n;
        tile_m = first_m + in_group % rows;
        tile_n = in_group / rows;
    }
    const int m0 = tile_m * ST_BM, n0 = tile_n * ST_BN;
    const int ba = p.a_batched ? (int)batch : 0, bb = p.b_batched ? (int)batch : 0;
    const int k_tiles = (int)((p.K + ST_BK - 1) / ST_BK);

    auto issue = [&](int kt) {  // both operand tiles of k-tile kt into stage kt % ST_STAGES (one thread)
        const int s = kt % ST_STAGES;
        const uint32_t sa = smem_base + s * ST_STAGE, sb = sa + ST_TILE;
        const uint32_t bar = full_bar(s);
        mbar_expect_tx(bar, (uint32_t)ST_STAGE);
        if (A_K) tma_load_3d(sa, &map_a, bar, kt * ST_BK, m0, ba);
        else tma_load_3d(sa, &map_a, bar, m0, kt * ST_BK, ba);
        if (B_K) tma_load_3d(sb, &map_b, bar, kt * ST_BK, n0, bb);
        else tma_load_3d(sb, &map_b, bar, n0, kt * ST_BK, bb);
    };

    if (tid == 0) {
        for (int s = 0; s < ST_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), ST_THREADS / 32); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    int issued = 0;  // thread 0 only
    if (tid == 0) {
        const int pre = k_tiles < ST_STAGES ? k_tiles : ST_STAGES;
        for (; issued < pre; ++issued) issue(issued);
    }

    // 32 accumulator pairs.  With B read as [k][n] (its pairs of neighbouring columns are neighbouring registers)
    // a pair holds (row i, columns 2jj and 2jj+1) at index i*4 + jj; with B read along k the pairs run down the
    // rows instead, (rows 2ii and 2ii+1, column j) at index ii*8 + j, and the row values of A form the pair.
    constexpr bool PAIR_ROWS = B_K;
    float2 acc[32];
    {
        float init[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            // a per-row bias is the accumulator's starting value, as in the reference's convolution (cnn.mojo:435)
            init[i] = 0.f;
            if (p.bias_m) {
                const int64_t m = (int64_t)m0 + quad_index(ty, i);
                if (m < p.M) init[i] = __ldg(p.bias_m + m);
            }
        }
#pragma unroll
        for (int q = 0; q < 32; ++q)
            acc[q] = PAIR_ROWS ? make_float2(init[2 * (q >> 3)], init[2 * (q >> 3) + 1]) : make_float2(init[q >> 2], init[q >> 2]);
    }

    // per-thread constants of the fragment addresses
    const int warp = tid >> 5, ty_l = ty & 1;
    const int b_base = B_K ? tx * 64 : tx * 16;    // K-major: row tx (rows tx + 16 j); MN-major: column tx*4
    const int sb = (tx >> 1) & 3;                   // swizzle term (row >> 1) & 3 of rows tx + 16 j
    // A K-major tile is transposed by each warp for itself (see below): lane = (local row lr, 16-byte chunk c)
    uint8_t* Tw = smem_gen + ST_STAGES * ST_STAGE + 128 + warp * ST_TBUF;
    const int lr = lane >> 2, lc = lane & 3;
    const int t_src = (8 * warp + lr) * 64 + ((lc ^ ((lr >> 1) & 3)) << 4);  // chunk lc of row 8w + lr (+ 64 rows: + 4096 B)
    // k = 4*lc + e lands in row k of the block; column = 4 * (quad ^ swap) + (lr & 3), quad = 2*pass + (lr >> 2),
    // swap = 2 for k >= 8
    const int t_dst0 = ((4 * lc) * ST_LDT + (((lr >> 2) ^ ((lc >> 1) << 1)) << 2) + (lr & 3)) * 4;
    const int t_dst1 = ((4 * lc) * ST_LDT + (((2 + (lr >> 2)) ^ ((lc >> 1) << 1)) << 2) + (lr & 3)) * 4;

    int kt = 0;
    for (; kt < k_tiles; ++kt) {
        const int s = kt % ST_STAGES;
        if (!mbar_wait(full_bar(s), (uint32_t)((kt / ST_STAGES) & 1), abort_flag)) break;
        const uint8_t* As = smem_gen + s * ST_STAGE;
        const uint8_t* Bs = As + ST_TILE;
        if (A_K) {
            // The copy engine cannot transpose 32-bit elements, and a fragment along m must be neighbouring registers
            // (float4 reads, register pairs for the packed FMA).  Each warp therefore transposes the 16 rows of A it
            // multiplies with (rows 8w..8w+7 and 64+8w..64+8w+7) from [row][16 k] into its own [k][16 rows] block:
            // two 16-byte reads and eight 4-byte writes per lane and k-tile, synchronised inside the warp only.  With
            // 20 floats per k row and the two 8-row halves swapped for k >= 8 the 32 writes of a step hit 32 banks.
#pragma unroll
            for (int pass = 0; pass < 2; ++pass) {
                const float4 v = lds128(As + pass * 4096 + t_src);
                float* dst = reinterpret_cast<float*>(Tw + (pass ? t_dst1 : t_dst0));
                dst[0 * ST_LDT] = v.x;
                dst[1 * ST_LDT] = v.y;
                dst[2 * ST_LDT] = v.z;
                dst[3 * ST_LDT] = v.w;
            }
            __syncwarp();
        }
        // a fragment of k: rows ty*4..+3 and 64+ty*4..+3
        const uint8_t* Af = A_K ? Tw + ty_l * 16 : As + ty * 16;
        constexpr int A_ROW = A_K ? ST_LDT * 4 : 512;
        auto a_lo = [&](int k) { return Af + k * A_ROW + (A_K && k >= 8 ? 32 : 0); };   // rows ty*4 .. ty*4+3
        auto a_hi = [&](int k) { return Af + k * A_ROW + (A_K ? (k >= 8 ? 0 : 32) : 256); };  // rows 64+ty*4 ..
#pragma unroll
        for (int k2 = 0; k2 < ST_BK / 2; ++k2) {  // two k steps at a time: K-major B fragments are read as float2 along k
            if (k2 == 2 && tid == 0 && kt >= 1 && issued < k_tiles) {
                // refill the stage k-tile kt-1 used, once all eight warps have released it
                const int prev = kt - 1;
                if (mbar_wait(empty_bar(prev % ST_STAGES), (uint32_t)((prev / ST_STAGES) & 1), abort_flag)) {
                    issue(issued);
                    ++issued;
                }
            }
            if (!B_K) {
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
                    float a[8], b[8];
                    *reinterpret_cast<float4*>(&a[0]) = lds128(a_lo(k2 * 2 + kk));
                    *reinterpret_cast<float4*>(&a[4]) = lds128(a_hi(k2 * 2 + kk));
                    *reinterpret_cast<float4*>(&b[0]) = lds128(Bs + (k2 * 2 + kk) * 512 + b_base);
                    *reinterpret_cast<float4*>(&b[4]) = lds128(Bs + (k2 * 2 + kk) * 512 + b_base + 256);
#pragma unroll
                    for (int i = 0; i < 8; ++i)
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj)
                            acc[i * 4 + jj] = fma_pair<PACKED>(a[i], a[i], b[2 * jj], b[2 * jj + 1], acc[i * 4 + jj]);
                }
            } else {
                // byte offset of k = 2*k2 inside a 64-byte K-major row: swizzled 16-byte chunk, then the half of the chunk
                const int xb = (((k2 >> 1) ^ sb) << 4) + (k2 & 1) * 8;
                float bf[8][2];  // bf[j][kk] = B[2*k2 + kk][column tx + 16 j]
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    *reinterpret_cast<float2*>(&bf[j][0]) = *reinterpret_cast<const float2*>(Bs + b_base + j * 1024 + xb);
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
                    float a[8];
                    *reinterpret_cast<float4*>(&a[0]) = lds128(a_lo(k2 * 2 + kk));
                    *reinterpret_cast<float4*>(&a[4]) = lds128(a_hi(k2 * 2 + kk));
#pragma unroll
                    for (int ii = 0; ii < 4; ++ii)
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            acc[ii * 8 + j] = fma_pair<PACKED>(a[2 * ii], a[2 * ii + 1], bf[j][kk], bf[j][kk], acc[ii * 8 + j]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(s));
    }

    __syncthreads();  // every wait above is bounded, so all threads arrive here
    if (*abort_flag) {
        if (tid == 0) {
            // copies still in flight target this CTA's shared memory: wait for them (bounded) before leaving
            for (int t = kt; t < issued; ++t) {
                const uint64_t t0 = globaltimer_ns();
                while (!mbar_try_wait(full_bar(t % ST_STAGES), (uint32_t)((t / ST_STAGES) & 1)))
                    if (globaltimer_ns() - t0 > TENMO_WAIT_LIMIT_NS) break;
            }
            atomicOr(p.status, TENMO_DEV_TIMEOUT);
        }
        return;
    }

    // Epilogue: bias, activation (+ mask), multiplier, accumulate, store.
    float* C = p.C + batch * p.M * p.N;
    float* AUX = p.aux ? p.aux + batch * p.M * p.N : nullptr;
    const float* MASK = p.mul_mask ? p.mul_mask + batch * p.M * p.N : nullptr;
    float* CLO = p.c_lo ? p.c_lo + batch * p.M * p.ld_clo : nullptr;
    const bool extended = MASK != nullptr || CLO != nullptr;
    auto acc_at = [&](int i, int j) {  // indices are compile-time constants after unrolling
        if (PAIR_ROWS) return (i & 1) ? acc[(i >> 1) * 8 + j].y : acc[(i >> 1) * 8 + j].x;
        return (j & 1) ? acc[i * 4 + (j >> 1)].y : acc[i * 4 + (j >> 1)].x;
    };
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int64_t m = (int64_t)m0 + quad_index(ty, i);
        if (m >= p.M) continue;
        if (!B_K && p.c_vec && !extended) {
#pragma unroll
            for (int jg = 0; jg < 2; ++jg) {
                const int64_t n = (int64_t)n0 + jg * 64 + tx * 4;
                if (n >= p.N) continue;  // N % 4 == 0 on this path, so n < N covers n + 3
                float v[4], mk[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    float x = acc_at(i, jg * 4 + q);
                    if (p.bias) x += __ldg(p.bias + n + q);
                    mk[q] = x > 0.f ? 1.f : 0.f;
                    v[q] = st_act(x, p.act);
                }
                float* dst = C + m * p.N + n;
                float4 o = make_float4(v[0], v[1], v[2], v[3]);
                if (p.beta != 0.f) {
                    const float4 old = *reinterpret_cast<const float4*>(dst);
                    o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4*>(dst) = o;
                if (AUX) *reinterpret_cast<float4*>(AUX + m * p.N + n) = make_float4(mk[0], mk[1], mk[2], mk[3]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int64_t n = (int64_t)n0 + (B_K ? tx + 16 * j : quad_index(tx, j));
                if (n >= p.N) continue;
                float x = acc_at(i, j);
                if (p.bias) x += __ldg(p.bias + n);
                const float mk = x > 0.f ? 1.f : 0.f;
                float o = st_act(x, p.act);
                if (MASK) o *= __ldg(MASK + m * p.N + n);
                float* dst = C + m * p.N + n;
                if (p.beta != 0.f) o += *dst;
                *dst = o;
                if (AUX) AUX[m * p.N + n] = mk;
                if (CLO) CLO[m * p.ld_clo + n] = tenmo_tf32_lo(o);
            }
        }
    }
}

// K-major operand: box {16 k, 128 rows}, 64-byte swizzle; MN-major: box {128, 16 k}, no swizzle (the rows of
// 512 B are read 16 bytes per lane, which is conflict-free as it lies).  Out-of-range elements read as zero.
int st_encode_map(tenmo_ctx* ctx, CUtensorMap* map, const float* base, const TenmoOperandPlan& o) {
    TenmoEncodeTiledFn fn = reinterpret_cast<TenmoEncodeTiledFn>(ctx->encode_tiled);
    cuuint64_t dims[3] = {(cuuint64_t)o.inner, (cuuint64_t)o.outer, (cuuint64_t)o.batches};
    cuuint64_t strides[2] = {(cuuint64_t)o.ld * 4, (cuuint64_t)(o.batched ? o.batch_stride : o.ld * o.outer) * 4};
    if (strides[1] % 16 != 0) strides[1] = (strides[1] + 15) / 16 * 16;  // unused when there is one slice
    cuuint32_t box[3] = {o.mn_major ? 128u : (cuuint32_t)ST_BK, o.mn_major ? (cuuint32_t)ST_BK : 128u, 1u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, o.mn_major ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_64B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return tenmo_set_error(ctx, TENMO_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d (inner %lld outer %lld ld %lld)",
                               (int)r, (long long)o.inner, (long long)o.outer, (long long)o.ld);
    return TENMO_OK;
}

template <bool PACKED>
cudaError_t st_launch(bool a_k, bool b_k, unsigned grid, cudaStream_t s, const CUtensorMap& ma, const CUtensorMap& mb,
                      const StParams& sp) {
#define ST_LAUNCH(AK, BKM)                                                                                             \
    {                                                                                                                  \
        cudaError_t e = cudaFuncSetAttribute(gemm_simt_tma_kernel<AK, BKM, PACKED>,                                   \
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, ST_SMEM);                    \
        if (e == cudaSuccess) /* two CTAs per SM need the large shared-memory split of the L1 */                      \
            e = cudaFuncSetAttribute(gemm_simt_tma_kernel<AK, BKM, PACKED>, cudaFuncAttributePreferredSharedMemoryCarveout, \
                                     cudaSharedmemCarveoutMaxShared);                                                  \
        if (e != cudaSuccess) return e;                                                                                \
        gemm_simt_tma_kernel<AK, BKM, PACKED><<<grid, ST_THREADS, ST_SMEM, s>>>(ma, mb, sp);                          \
    }
    if (a_k) { if (b_k) ST_LAUNCH(true, true) else ST_LAUNCH(true, false) }
    else { if (b_k) ST_LAUNCH(false, true) else ST_LAUNCH(false, false) }
#undef ST_LAUNCH
    return cudaGetLastError();
}

}  // namespace

bool tenmo_gemm_simt_tma_supported(tenmo_ctx* ctx, const TenmoGemmParams& p) {
    (void)ctx;
    TenmoOperandPlan a, b;
    char why[160];
    if (p.M < 1 || p.N < 1) return false;
    return tenmo_make_plan(p, &a, &b, why, sizeof(why));
}

int tenmo_gemm_simt_tma_launch(tenmo_ctx* ctx, const TenmoGemmParams& p) {
    int st = tenmo_tma_init(ctx);
    if (st != TENMO_OK) return st;
    TenmoOperandPlan a, b;
    char why[160];
    if (!tenmo_make_plan(p, &a, &b, why, sizeof(why))) return tenmo_set_error(ctx, TENMO_ERR_UNSUPPORTED, "gemm_simt_tma: %s", why);
    CUtensorMap ma, mb;
    if ((st = st_encode_map(ctx, &ma, p.A, a)) != TENMO_OK) return st;
    if ((st = st_encode_map(ctx, &mb, p.B, b)) != TENMO_OK) return st;

    StParams sp;
    sp.C = p.C; sp.aux = p.aux; sp.bias = p.bias; sp.bias_m = p.bias_m; sp.mul_mask = p.mul_mask;
    sp.c_lo = p.c_lo; sp.ld_clo = p.ld_clo;
    sp.M = p.M; sp.N = p.N; sp.K = p.K;
    sp.tiles_m = (int)((p.M + ST_BM - 1) / ST_BM);
    sp.tiles_n = (int)((p.N + ST_BN - 1) / ST_BN);
    sp.a_batched = a.batched; sp.b_batched = b.batched;
    sp.beta = p.beta; sp.act = p.act;
    sp.c_vec = (p.N % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15u) == 0) &&
               (!p.aux || (reinterpret_cast<uintptr_t>(p.aux) & 15u) == 0);
    sp.status = ctx->dev_status;
    const int64_t grid = (int64_t)sp.tiles_m * sp.tiles_n * p.total_batch;
    if (grid <= 0 || grid > 0x7fffffffLL)
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "gemm_simt_tma: grid of %lld tiles is out of range", (long long)grid);
    // TENMO_SIMT_FFMA2=0 switches the k loop to scalar fmaf (same bits; kept for comparisons).
    bool packed = true;
    const char* env = getenv("TENMO_SIMT_FFMA2");
    if (env && (env[0] == '0' || env[0] == '1')) packed = env[0] == '1';
    tenmo_prof_before(ctx);
    cudaError_t e = packed ? st_launch<true>(!a.mn_major, !b.mn_major, (unsigned)grid, ctx->stream, ma, mb, sp)
                            : st_launch<false>(!a.mn_major, !b.mn_major, (unsigned)grid, ctx->stream, ma, mb, sp);
    tenmo_prof_after(ctx);
    ctx->launches++;
    ctx->last_gemm_kernel = "gemm_simt_tma_kernel";
    ctx->last_gemm_sk_units = 0;
    if (e != cudaSuccess)
        return tenmo_set_error(ctx, TENMO_ERR_CUDA, "launch of gemm_simt_tma_kernel failed: %s", cudaGetErrorString(e));
    return TENMO_OK;
}
