// tcgen05 / TMEM tensor-core GEMM with 3xTF32 error compensation (fp32 in, fp32 out).
//
// Arithmetic.  Each fp32 operand x is split as x = hi + lo with hi = x truncated to TF32 (the tensor
// core reads only the top 19 bits of an fp32 word, so the raw operand IS the hi plane) and
// lo = tf32(x - hi).  A product a*b is formed as  a_lo*b_hi + a_hi*b_lo + a_hi*b_hi  by three
// tcgen05.mma.kind::tf32 instructions into one fp32 accumulator in tensor memory; the dropped
// a_lo*b_lo term is below 2^-20 relative.  The lo planes are produced by a bandwidth-bound split
// kernel into the context workspace (one read + one write per operand element).
//
// Kernel.  Persistent, one CTA per SM, 320 threads, warp-specialised:
//   warp 0   TMA producer   cp.async.bulk.tensor (no multicast) of the A, A_lo, B, B_lo tiles of a
//                           k-block into a ring of shared-memory stages, 128-byte swizzle
//   warp 1   MMA issuer     one elected thread issues 4 k-steps x 3 products of 128 x BN x 8 per stage,
//                           tcgen05.commit releases the stage and, at the end of a tile, publishes the
//                           accumulator; also owns the TMEM allocation (2 accumulators, double buffered)
//   warps 2-9 epilogue      tcgen05.ld the accumulator (one TMEM lane = one row per thread), add bias,
//                           activation / ReLU mask / beta accumulate, store to C
// Scheduling.  Work is handed out by the producer warp through a small shared-memory ring as segments (tile, range of
// k-blocks, action).  Normally a segment is a whole tile.  When the tiles would leave the last wave of CTAs partly
// empty, the k-blocks of the last tiles are cut into one equal piece per CTA (stream-K): a piece that ends inside a tile
// parks its accumulator in the workspace, the piece that holds the tile's end adds the parked ones in ascending k and
// runs the epilogue.  Pieces depend only on lower-numbered pieces and are drawn in ascending order.
// Long sums.  The tensor core adds into its fp32 accumulator with truncation, so the error of one chain of same-signed
// products grows with its length.  A k-range above 96 k-blocks therefore travels as several segments whose accumulators
// the epilogue warps add up in fp32 (round to nearest), the running sum kept where the result goes (C or the parking slot).
// Operand layouts.  "K-major" = the contraction index is the unit-stride axis (row-major A, or B given
// as a transposed view); "MN-major" = the other axis is (A given as a transposed view, row-major B).
// Both are native tcgen05 shared-memory layouts, so transposed stride views need no copy: only the
// tensor-map box and the descriptor change (this is what the two backward GEMMs use).
// Every wait on an mbarrier is bounded in wall-clock time; on expiry the kernel raises the context's
// device status word, drains its outstanding copies, frees its tensor memory and returns.
// Roofline: tensor pipe; the useful work is 2*M*N*K flop (the 3x is not counted).
#include <cuda.h>

#include <cstdlib>

#include "gemm_tc.cuh"
#include "tma_util.cuh"

namespace {

constexpr int TC_THREADS = 320;                // producer warp, MMA warp, eight epilogue warps
constexpr int EPI_WARPS = 8;
constexpr int BM = 128;
#ifndef TENMO_TC_BK
#define TENMO_TC_BK 32
#endif
constexpr int BK = TENMO_TC_BK;  // fp32 elements per k-block: 32 = one 128-byte swizzle row, 16 = one 64-byte row
static_assert(BK == 32 || BK == 16, "BK must be 16 or 32");
constexpr int UMMA_K = 8;                    // tf32 k per instruction
constexpr int SQ = 4;                        // depth of the tile-id ring between the scheduler and its consumers
constexpr int TILE_COUNTERS = 32;            // ring of global tile counters, one per GEMM launch in flight

constexpr int EP_LD = 32;  // floats per row of an epilogue warp's 32 x 32 staging block; 16-byte chunk q of row r sits at
                           // chunk q ^ (r & 7), which keeps the row-wise writes and the 4-rows-at-a-time reads conflict-free

// PAIR: two CTAs on neighbouring SMs (a cluster of two) work on one 256 x BN tile with tcgen05.mma.cta_group::2: each holds
// its own 128 rows of A and HALF of the B tile, the tensor cores read the other half from the partner's shared memory.
// A stage is then 64 KB instead of 96 KB at BN = 256, so three stages fit where the single-CTA kernel has two, and every
// byte of B is fetched from L2 once per pair instead of once per CTA.
template <int BN, bool PAIR = false>
struct TcCfg {
    static constexpr int A_TILE = BM * BK * 4;   // bytes of one plane of A per stage
    static constexpr int B_ROWS = PAIR ? BN / 2 : BN;  // columns of the B tile this CTA stages
    static constexpr int B_TILE = B_ROWS * BK * 4;
    static constexpr int STAGE = 2 * A_TILE + 2 * B_TILE;
    static constexpr int STAGES = (PAIR ? 3 : ((BN == 256) ? 2 : (BN == 128 ? 3 : 4))) * (32 / BK);
    // No alignment slack: the dynamic array is declared 1024-byte aligned and is the CTA's only shared memory.  With BN = 256
    // this leaves 2 KB of the SM's shared memory free, which is what lets a small CTA of another kernel (the data-parallel
    // exchange) share the SM with this one.
    static constexpr int SMEM = STAGES * STAGE + 256 /*barriers*/ + EPI_WARPS * 32 * EP_LD * 4 /*epilogue staging*/;
    static constexpr int TMEM_COLS = 2 * BN;     // two accumulators
};

struct TcParams {
    float* C;
    float* aux;
    const float* bias;
    const float* mul_mask;  // optional elementwise multiplier of the result (fused ReLU backward)
    const float* bias_m;    // optional per-row bias
    float* c_lo;            // optional lo plane of the stored result
    int64_t ld_clo;
    int64_t M, N, K;
    int64_t total_batch;
    int tiles_m, tiles_n;
    int a_batched, b_batched;  // 0: operand is broadcast over the batch (coordinate 0), 1: one slice per batch
    float beta;
    int act;
    int c_vec;
    uint32_t* status;
    unsigned int* tile_counter;  // zero at launch; hands out tiles gridDim.x, gridDim.x + 1, ...
    // stream-K tail (sk_units == 0: off).  Tiles [0, dp_tiles) are worked whole; the k-blocks of the tiles
    // [dp_tiles, tiles) form one linear range that is cut into sk_units equal pieces.
    int sk_units;
    int64_t dp_tiles;
    float* sk_partials;          // sk_units slots of BM x BN floats
    unsigned int* sk_flags;      // sk_units words, zero between launches: epilogue warps that have stored their part of slot u
    // Longest run of k-blocks that is summed in one tensor-memory accumulator (0: no limit).  The tensor core adds into its
    // fp32 accumulator with truncation, so on same-signed data the error of a chain grows in proportion to its length;
    // longer ranges are cut into sub-ranges whose sums the epilogue warps add up in fp32 (round to nearest).
    int chunk_kb;
    int group_m;  // row tiles per group of the tile order
};

// What travels from the scheduler to the MMA and epilogue warps: a tile, a range of its k-blocks, and what to do with the
// accumulator: the normal epilogue (after adding `npred` partial accumulators found in slots slot, slot + 1, ...), or
// park it as a partial in `slot`.
constexpr int SEG_PARTIAL = 1;
// A k-range longer than TcParams::chunk_kb travels as several segments: all but the last only add their accumulator to a
// running sum (CARRY_OUT) that the following ones pick up (CARRY_IN).  The running sum lives where the range's result goes:
// in the piece's parking slot, or in C itself.
constexpr int SEG_CARRY_IN = 2;
constexpr int SEG_CARRY_OUT = 4;
__device__ __forceinline__ int seg_info(int kind, int npred, int slot) { return kind | (npred << 4) | (slot << 8); }

// ---------------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// ---- the same for a CTA pair (cluster of two) ----
__device__ __forceinline__ void umma_tf32_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives on the barrier at the same shared-memory offset in BOTH CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(mask)
                 : "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// address of this CTA's shared-memory location `addr` as seen in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t cluster_bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// tiled bulk copy whose completion is counted on a barrier of the pair's leader CTA (no multicast: the data lands in this
// CTA's shared memory only)
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (sm_100 format): start address, leading / stride byte offsets in
// 16-byte units, descriptor version 1, 128-byte swizzle.
// layout_type: 2 = 128-byte swizzle of 16-byte chunks (K-major tiles), 1 = 128-byte swizzle of 32-byte
// chunks, the only swizzled layout tcgen05 takes for an MN-major 32-bit operand.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout_type) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;  // version
    d |= (uint64_t)layout_type << 61;
    return d;
}

__device__ __forceinline__ float act_apply(float v, int act) {
    if (act == TENMO_ACT_RELU) return v > 0.f ? v : 0.f;
    if (act == TENMO_ACT_SIGMOID) return 1.f / (1.f + expf(-v));
    return v;
}

// Tile order: groups of GROUP_M row tiles are walked column by column, so that the tiles running at
// the same time share A and B panels in L2.
__device__ __forceinline__ void tile_coords(int64_t tile, int tiles_m, int tiles_n, int GROUP_M, int64_t* batch, int* tm, int* tn) {
    const int64_t per_batch = (int64_t)tiles_m * tiles_n;
    *batch = tile / per_batch;
    const int t = (int)(tile % per_batch);
    const int group = t / (GROUP_M * tiles_n);
    const int first_m = group * GROUP_M;
    const int rows = min(GROUP_M, tiles_m - first_m);
    const int in_group = t - group * GROUP_M * tiles_n;
    *tm = first_m + in_group % rows;
    *tn = in_group / rows;
}

// A_MN / B_MN: the operand's unit-stride axis is m (resp. n) instead of k.
template <int BN, bool A_MN, bool B_MN, bool PAIR = false>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_a_lo,
               const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_b_lo, const TcParams p) {
    using Cfg = TcCfg<BN, PAIR>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = smem_u32(smem_raw);  // 128B swizzle wants 1024-byte alignment
    uint8_t* smem_gen = smem_raw;
    if (smem_base & 1023u) {  // cannot happen with the declaration above; checked because a misaligned tile would be garbage
        if (threadIdx.x == 0) atomicOr(p.status, TENMO_DEV_TIMEOUT);
        return;
    }
    const uint32_t bar_base = smem_base + Cfg::STAGES * Cfg::STAGE;
    // barrier layout (8 bytes each): full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], sched_full[SQ],
    // sched_empty[SQ]; then the segment ring (4 ints per entry), the tmem pointer and the abort flag
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (Cfg::STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * Cfg::STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * Cfg::STAGES + 2 + a); };
    auto sfull_bar = [&](int q) { return bar_base + 8u * (2 * Cfg::STAGES + 4 + q); };
    auto sempty_bar = [&](int q) { return bar_base + 8u * (2 * Cfg::STAGES + 4 + SQ + q); };
    volatile int* sched_tiles =
        reinterpret_cast<volatile int*>(smem_gen + Cfg::STAGES * Cfg::STAGE + 8 * (2 * Cfg::STAGES + 4 + 2 * SQ));
    uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(const_cast<int*>(sched_tiles) + 4 * SQ);
    static_assert(8 * (2 * Cfg::STAGES + 4 + 2 * SQ) + 16 * SQ + 8 <= 256, "barrier block overflows its 256 bytes");
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // PAIR: p.tiles_m counts 256-row tiles; rank 0 of the cluster (the leader) issues the MMAs for both CTAs, owns the
    // barriers the loads of both CTAs complete on (full) and the one both epilogues release an accumulator on (tempty)
    const uint32_t crank = PAIR ? cluster_ctarank() : 0u;
    const bool leader = crank == 0u;
    const int64_t num_tiles = (int64_t)p.tiles_m * p.tiles_n * p.total_batch;
    const int num_kb = (int)((p.K + BK - 1) / BK);

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) { mbar_init(full_bar(s), PAIR ? 2 : 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), PAIR ? 2 * EPI_WARPS : EPI_WARPS); }
        for (int q = 0; q < SQ; ++q) { mbar_init(sfull_bar(q), 1); mbar_init(sempty_bar(q), 1 + EPI_WARPS); }  // MMA thread + the epilogue warps
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if (PAIR) {  // the pair allocates the same columns in both tensor memories: one warp of each CTA takes part
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_ptr_smem)),
                         "r"((uint32_t)Cfg::TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_ptr_smem)),
                         "r"((uint32_t)Cfg::TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();  // the partner's barriers are initialised before anything arrives on them
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_ptr_smem;

    if (warp == 0) {
        // ------------------------------- TMA producer -------------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t armed = 0;  // stages whose full barrier was armed at least once
            bool ok = true;
            // Tile scheduler: the first tile of a CTA is its block index, every further one comes from a
            // global counter, so a CTA that starts late (its SM was busy with another stream's kernel) or runs
            // slow simply takes fewer tiles.  Tile ids travel to the MMA and epilogue warps through a small
            // shared-memory ring; -1 ends the stream.
            int sq = 0;
            uint32_t sphase = 0;
            auto publish = [&](int tile, int kb0, int kb1, int info) -> bool {
                if (!mbar_wait(sempty_bar(sq), sphase ^ 1u, abort_flag)) return false;
                sched_tiles[4 * sq + 0] = tile;
                sched_tiles[4 * sq + 1] = kb0;
                sched_tiles[4 * sq + 2] = kb1;
                sched_tiles[4 * sq + 3] = info;
                mbar_arrive(sfull_bar(sq));
                if (++sq == SQ) { sq = 0; sphase ^= 1u; }
                return true;
            };
            auto load = [&](int64_t tile, int kb0, int kb1) -> bool {
                int64_t batch; int tm, tn;
                tile_coords(tile, p.tiles_m, p.tiles_n, p.group_m, &batch, &tm, &tn);
                // PAIR: this CTA's 128 rows of the 256-row tile and its half of the tile's columns
                const int m0 = PAIR ? tm * (2 * BM) + (int)crank * BM : tm * BM;
                const int n0 = tn * BN + (PAIR ? (int)crank * (BN / 2) : 0);
                const int ba = p.a_batched ? (int)batch : 0, bb = p.b_batched ? (int)batch : 0;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) return false;
                    const uint32_t sa = smem_base + stage * Cfg::STAGE;
                    const uint32_t sal = sa + Cfg::A_TILE, sb = sa + 2 * Cfg::A_TILE, sbl = sb + Cfg::B_TILE;
                    // the copies of BOTH CTAs of a pair complete on the leader's barrier: each CTA announces its own bytes
                    const uint32_t bar = PAIR ? map_to_cta(full_bar(stage), 0u) : full_bar(stage);
                    if (PAIR) mbar_expect_tx_cluster(bar, (uint32_t)Cfg::STAGE);
                    else mbar_expect_tx(bar, (uint32_t)Cfg::STAGE);
                    armed |= 1u << stage;
                    const int k0 = kb * BK;
                    auto ld = [&](uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2) {
                        if (PAIR) tma_load_3d_pair(dst, map, bar, c0, c1, c2);
                        else tma_load_3d(dst, map, bar, c0, c1, c2);
                    };
                    if (!A_MN) {
                        ld(sa, &map_a, k0, m0, ba);
                        ld(sal, &map_a_lo, k0, m0, ba);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / 32; ++j) {
                            ld(sa + j * (BK * 128), &map_a, m0 + 32 * j, k0, ba);
                            ld(sal + j * (BK * 128), &map_a_lo, m0 + 32 * j, k0, ba);
                        }
                    }
                    if (!B_MN) {
                        ld(sb, &map_b, k0, n0, bb);
                        ld(sbl, &map_b_lo, k0, n0, bb);
                    } else {
#pragma unroll
                        for (int j = 0; j < Cfg::B_ROWS / 32; ++j) {
                            ld(sb + j * (BK * 128), &map_b, n0 + 32 * j, k0, bb);
                            ld(sbl + j * (BK * 128), &map_b_lo, n0 + 32 * j, k0, bb);
                        }
                    }
                    if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1u; }
                }
                return true;
            };
            // One k-range of a tile as one segment, or as several that carry a running sum (see SEG_CARRY_*).  Each segment is
            // published just before its own loads: the ring is short.
            auto emit = [&](int64_t tile, int kb0, int kb1, int info) -> bool {
                const int len = kb1 - kb0;
                const int n = (p.chunk_kb > 0 && len > p.chunk_kb) ? (len + p.chunk_kb - 1) / p.chunk_kb : 1;
                // a result that is added to the old C (beta = 1) takes the old C as the first carry
                const bool first_carry = !(info & SEG_PARTIAL) && p.beta != 0.f;
                int a = kb0;
                for (int s = 0; s < n; ++s) {
                    const int b = kb0 + (int)((int64_t)len * (s + 1) / n);
                    int f;
                    if (s == n - 1) f = info | (n > 1 ? SEG_CARRY_IN : 0);
                    else f = (info & SEG_PARTIAL) | (info & ~0xFF) | SEG_CARRY_OUT | ((s > 0 || first_carry) ? SEG_CARRY_IN : 0);
                    if (!publish((int)tile, a, b, f)) return false;
                    if (!load(tile, a, b)) return false;
                    a = b;
                }
                return true;
            };
            // Work units: tiles [0, dp_tiles) whole, then sk_units pieces of the linear k-block range of the remaining
            // tiles.  Units are drawn in ascending order and a piece only ever depends on pieces with a lower number,
            // which some running CTA has already drawn, so the waits of the fix-up cannot form a cycle even when not all
            // CTAs are resident.  For that the first unit must come from the counter too unless it is a whole tile.
            const int64_t num_units = p.dp_tiles + p.sk_units;
            const int64_t unit_base = (p.dp_tiles >= (int64_t)gridDim.x) ? (int64_t)gridDim.x : 0;
            // A pair cannot draw from the counter (its two CTAs must see the same sequence without talking to each other):
            // its units are fixed by its index -- whole tiles round-robin over the pairs, then the piece of its own number.
            int64_t s_next = blockIdx.x / 2;
            bool s_piece_taken = false;
            auto draw = [&]() -> int64_t {
                if (!PAIR) return unit_base + (int64_t)atomicAdd(p.tile_counter, 1u);
                if (s_next < p.dp_tiles) { const int64_t u = s_next; s_next += gridDim.x / 2; return u; }
                if (!s_piece_taken) {
                    s_piece_taken = true;
                    const int64_t j = blockIdx.x / 2;
                    if (j < p.sk_units) return p.dp_tiles + j;
                }
                return p.dp_tiles + p.sk_units;  // nothing left
            };
            const int64_t sk_total = (num_tiles - p.dp_tiles) * (int64_t)num_kb;
            const int64_t sk_q = p.sk_units ? sk_total / p.sk_units : 0, sk_r = p.sk_units ? sk_total % p.sk_units : 0;
            int64_t unit = PAIR ? draw() : (unit_base ? (int64_t)blockIdx.x : draw());
            while (ok) {
                if (unit >= num_units) { if (!publish(-1, 0, 0, 0)) ok = false; break; }
                int64_t next = -1;
                if (unit < p.dp_tiles) {
                    next = draw();  // fetched early: the latency hides under the loads
                    if (!emit(unit, 0, num_kb, 0)) { ok = false; break; }
                } else {
                    // piece j covers [begin, end) of the linear range.  Its tiles are walked from the last to the first: the
                    // part that does not reach its tile's end (a partial for piece j + 1 to pick up) goes first, the part
                    // that completes a tile begun by earlier pieces goes last, when their partials have long been stored.
                    const int64_t j = unit - p.dp_tiles;
                    const int64_t begin = j * sk_q + (j < sk_r ? j : sk_r);
                    int64_t hi = begin + sk_q + (j < sk_r ? 1 : 0);
                    while (hi > begin) {
                        const int64_t t = (hi - 1) / num_kb, base = t * (int64_t)num_kb;
                        const int64_t lo = begin > base ? begin : base;
                        int info = 0;
                        if (hi - base < num_kb) {
                            info = seg_info(SEG_PARTIAL, 0, (int)j);
                        } else if (lo > base) {
                            const int64_t cut = sk_r * (sk_q + 1);  // pieces below sk_r are one k-block longer
                            const int64_t first = base < cut ? base / (sk_q + 1) : sk_r + (base - cut) / sk_q;
                            info = seg_info(0, (int)(j - first), (int)first);
                        }
                        if (next < 0) next = draw();
                        if (!emit(p.dp_tiles + t, (int)(lo - base), (int)(hi - base), info)) { ok = false; break; }
                        hi = lo;
                    }
                }
                unit = next;
            }
            if (!ok && (!PAIR || leader)) {
                // Drain: let every copy already issued land before the CTA gives its shared memory back (the leader of a
                // pair waits for both CTAs' copies, and the pair leaves together).
                // A stage's last armed phase: stages < `stage` were armed in the current phase, the rest in the previous.
                for (int s = 0; s < Cfg::STAGES; ++s) {
                    if (!(armed & (1u << s))) continue;
                    const uint32_t ph = (s < stage) ? phase : (phase ^ 1u);
                    const uint64_t t0 = globaltimer_ns();
                    for (;;) {
                        uint32_t done;
                        asm volatile(
                            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                            : "=r"(done) : "r"(full_bar(s)), "r"(ph) : "memory");
                        if (done || globaltimer_ns() - t0 > TENMO_WAIT_LIMIT_NS) break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------- MMA issuer -------------------------------
        if (lane == 0) {
            // instruction shape: M = 128 (one CTA) or 256 (a pair: 128 rows in each CTA's tensor memory), N = BN
            constexpr uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_MN ? 1u : 0u) << 15) |
                                       ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) |
                                       ((uint32_t)((PAIR ? 2 * BM : BM) >> 4) << 24);
            // K-major: rows of 128 B, 8-row groups 1024 B apart (SBO), k-step = 32 B inside the swizzle row.
            // MN-major: a tile is [32-wide mn chunk][k row of 128 B]; chunks are 4096 B apart (LBO), the
            // swizzle pattern repeats every 4 k rows = 512 B (SBO), one k-step of 8 rows = 1024 B.
            // With BK = 16 a K-major row is 64 B (64-byte swizzle, 8-row groups 512 B apart) and an MN-major chunk
            // holds 16 k rows (2048 B).
            constexpr uint32_t K_SBO = 8u * BK * 4u, K_LT = BK == 32 ? 2u : 4u, MN_LBO = BK * 128u;
            constexpr uint32_t A_LBO = A_MN ? MN_LBO : 16u, A_SBO = A_MN ? 512u : K_SBO, A_KSTEP = A_MN ? 1024u : 32u;
            constexpr uint32_t B_LBO = B_MN ? MN_LBO : 16u, B_SBO = B_MN ? 512u : K_SBO, B_KSTEP = B_MN ? 1024u : 32u;
            constexpr uint32_t A_LT = A_MN ? 1u : K_LT, B_LT = B_MN ? 1u : K_LT;
            int stage = 0;
            uint32_t phase = 0;
            uint32_t acc_phase[2] = {0, 0};
            int acc = 0;
            bool ok = true;
            int sq = 0;
            uint32_t sphase = 0;
            while (ok) {
                if (!mbar_wait(sfull_bar(sq), sphase, abort_flag)) { ok = false; break; }
                const int tile = sched_tiles[4 * sq], kb0 = sched_tiles[4 * sq + 1], kb1 = sched_tiles[4 * sq + 2];
                mbar_arrive(sempty_bar(sq));
                if (++sq == SQ) { sq = 0; sphase ^= 1u; }
                if (tile < 0) break;
                if (PAIR && !leader) continue;  // the partner's warp only keeps the segment ring moving
                if (!mbar_wait(tempty_bar(acc), acc_phase[acc] ^ 1u, abort_flag)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t sa = smem_base + stage * Cfg::STAGE;
                    const uint32_t sal = sa + Cfg::A_TILE, sb = sa + 2 * Cfg::A_TILE, sbl = sb + Cfg::B_TILE;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t da = make_desc(sa + k * A_KSTEP, A_LBO, A_SBO, A_LT);
                        const uint64_t dal = make_desc(sal + k * A_KSTEP, A_LBO, A_SBO, A_LT);
                        const uint64_t db = make_desc(sb + k * B_KSTEP, B_LBO, B_SBO, B_LT);
                        const uint64_t dbl = make_desc(sbl + k * B_KSTEP, B_LBO, B_SBO, B_LT);
                        if (PAIR) {
                            umma_tf32_pair(d_tmem, dal, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);  // a_lo * b_hi
                            umma_tf32_pair(d_tmem, da, dbl, idesc, 1u);                             // a_hi * b_lo
                            umma_tf32_pair(d_tmem, da, db, idesc, 1u);                              // a_hi * b_hi
                        } else {
                            umma_tf32(d_tmem, dal, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);  // a_lo * b_hi
                            umma_tf32(d_tmem, da, dbl, idesc, 1u);                             // a_hi * b_lo
                            umma_tf32(d_tmem, da, db, idesc, 1u);                              // a_hi * b_hi
                        }
                    }
                    // stage is free once these MMAs have read it (a pair: in both CTAs)
                    if (PAIR) umma_commit_pair(empty_bar(stage)); else umma_commit(empty_bar(stage));
                    if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                if (PAIR) umma_commit_pair(tfull_bar(acc)); else umma_commit(tfull_bar(acc));  // accumulator complete
                acc_phase[acc] ^= 1u;
                acc ^= 1;
            }
        }
    } else {
        // ------------------------------- epilogue (warps 2..9) -------------------------------
        // Two warps per TMEM lane quarter: warp w and w + 4 take the even and the odd 32-column blocks of their 32 rows.
        // The epilogue of a short-k tile is a chain of dependent instructions per warp; with one warp per scheduler
        // nothing hides their latency, with two the drain of a tile takes half as long.
        const int quarter = warp & 3;  // a warp may only touch TMEM lanes [32*(warp%4), +32)
        float* ebuf = reinterpret_cast<float*>(smem_gen + Cfg::STAGES * Cfg::STAGE + 256) + (warp - 2) * (32 * EP_LD);
        const int half = (warp - 2) >> 2;
        uint32_t acc_phase[2] = {0, 0};
        int acc = 0;
        bool ok = true;
        int sq = 0;
        uint32_t sphase = 0;
        // Lane 0 does the waiting and the warp follows its result, so the warp never diverges around the
        // warp-collective tcgen05.ld below, not even when a wait is abandoned.
        auto warp_wait = [&](uint32_t bar, uint32_t parity) -> bool {
            int got = 1;
            if (lane == 0) got = mbar_wait(bar, parity, abort_flag) ? 1 : 0;
            return __shfl_sync(0xffffffffu, got, 0) != 0;
        };
        while (ok) {
            if (!warp_wait(sfull_bar(sq), sphase)) { ok = false; break; }
            int tile = 0, info = 0;
            if (lane == 0) {
                tile = sched_tiles[4 * sq];
                info = sched_tiles[4 * sq + 3];
                mbar_arrive(sempty_bar(sq));
            }
            tile = __shfl_sync(0xffffffffu, tile, 0);
            info = __shfl_sync(0xffffffffu, info, 0);
            if (++sq == SQ) { sq = 0; sphase ^= 1u; }
            if (tile < 0) break;
            const bool partial = (info & SEG_PARTIAL) != 0;
            const bool carry_in = (info & SEG_CARRY_IN) != 0, carry_out = (info & SEG_CARRY_OUT) != 0;
            const float beta = carry_in ? 0.f : p.beta;  // the old C came in with the carry
            int npred = (info >> 4) & 15;
            const int slot = info >> 8;
            int64_t batch; int tm, tn;
            tile_coords(tile, p.tiles_m, p.tiles_n, p.group_m, &batch, &tm, &tn);
            if (PAIR) tm = 2 * tm + (int)crank;  // this CTA's 128 rows of the pair's 256-row tile
            if (!warp_wait(tfull_bar(acc), acc_phase[acc])) { ok = false; break; }
            tcgen05_fence_after();
            // A thread's tcgen05.ld delivers 32 consecutive columns of ONE row, so storing straight from those
            // registers would make every warp-wide store touch 32 rows, 16 bytes each.  The 32 x 32 block goes through a
            // per-warp shared-memory buffer instead (16-byte chunks XOR-swizzled by row: conflict-free both ways) and comes back
            // as (row = 4i + lane/8, columns 4*(lane%8)..+3): a warp-wide access then covers four full 128-byte row
            // segments, for the result as for the mask, the old C, the ReLU mask and the lo plane.
            const int64_t m_warp = (int64_t)tm * BM + quarter * 32;
            const int64_t n_base = (int64_t)tn * BN;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
            const int col4 = (lane & 7) * 4, row_sub = lane >> 3;
            // element offsets of row (m_warp + row_sub); the other seven rows of a lane lie 4 rows further each
            const int64_t row_off0 = (batch * p.M + m_warp + row_sub) * p.N;
            const int64_t clo_off0 = (batch * p.M + m_warp + row_sub) * p.ld_clo;
            const bool plain = !p.bias && !p.bias_m && p.act == TENMO_ACT_NONE && !p.aux && !p.mul_mask && !p.c_lo &&
                               beta == 0.f && p.c_vec;
            // Stream-K fix-up.  A partial accumulator is parked in its slot in the order the registers come out of tensor
            // memory: float4 number (8 c + q) * 128 + row, so that a warp's store covers 512 contiguous bytes; the warp of
            // the completing CTA that owns the same rows and columns reads it back the same way.  A slot's flag counts the
            // epilogue warps that have stored their part.
            // a pair parks two halves per piece: slot 2 j + rank
            constexpr int SLOT_MUL = PAIR ? 2 : 1;
            const int slot_add = PAIR ? (int)crank : 0;
            float4* const part = reinterpret_cast<float4*>(p.sk_partials + (size_t)(slot * SLOT_MUL + slot_add) * (BM * BN)) + quarter * 32 + lane;
            if (npred) {
                int got = 1;
                if (lane == 0) {
                    const uint64_t t0 = globaltimer_ns();
                    for (int s = 0; s < npred && got; ++s) {
                        const unsigned int* f = p.sk_flags + (slot + s) * SLOT_MUL + slot_add;
                        for (uint32_t it = 0;; ++it) {
                            unsigned int v;
                            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
                            if (v >= (unsigned int)EPI_WARPS) break;
                            if (*abort_flag || ((it & 63u) == 63u && globaltimer_ns() - t0 > TENMO_WAIT_LIMIT_NS)) {
                                *abort_flag = 1;
                                got = 0;
                                break;
                            }
                        }
                    }
                }
                if (!__shfl_sync(0xffffffffu, got, 0)) npred = 0;  // gave up: finish the tile without them, the status word tells
            }
#pragma unroll 1
            for (int c = half; c < BN / 32; c += 2) {
                const int64_t n0 = n_base + c * 32;
                if (n0 >= p.N) break;  // uniform: the rest of the tile lies outside the matrix
                uint32_t r[32];
                tmem_ld32(taddr + (uint32_t)(c * 32), r);
                tmem_ld_wait();
                if (partial) {
                    // (a carried sum is re-read by the thread that wrote it: program order suffices)
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        float4 x = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                               __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
                        if (carry_in) {
                            const float4 o = part[(c * 8 + q) * 128];
                            x.x += o.x; x.y += o.y; x.z += o.z; x.w += o.w;
                        }
                        part[(c * 8 + q) * 128] = x;
                    }
                    continue;
                }
                for (int s = 0; s < npred; ++s) {  // ascending k: own + partial of the first piece + the next ...
                    const float4* src = part + (size_t)s * SLOT_MUL * (BM * BN / 4) + (c * 8) * 128;
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        const float4 x = __ldcg(src + q * 128);
                        r[4 * q] = __float_as_uint(__uint_as_float(r[4 * q]) + x.x);
                        r[4 * q + 1] = __float_as_uint(__uint_as_float(r[4 * q + 1]) + x.y);
                        r[4 * q + 2] = __float_as_uint(__uint_as_float(r[4 * q + 2]) + x.z);
                        r[4 * q + 3] = __float_as_uint(__uint_as_float(r[4 * q + 3]) + x.w);
                    }
                }
#pragma unroll
                for (int q = 0; q < 32; q += 4)
                    *reinterpret_cast<float4*>(ebuf + lane * EP_LD + ((((q >> 2) ^ (lane & 7))) << 2)) =
                        make_float4(__uint_as_float(r[q]), __uint_as_float(r[q + 1]), __uint_as_float(r[q + 2]),
                                    __uint_as_float(r[q + 3]));
                __syncwarp();
                const int64_t n = n0 + col4;
                if (carry_out) {
                    // not the last sub-range of its k-range: the running sum is kept in C (each element by the thread that
                    // will read it again)
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rl = 4 * i + row_sub;
                        float4 x4 = *reinterpret_cast<const float4*>(ebuf + rl * EP_LD + ((((lane & 7) ^ (rl & 7))) << 2));
                        if (m_warp + rl >= p.M || n >= p.N) continue;
                        float* d = p.C + row_off0 + (int64_t)(4 * i) * p.N + n;
                        if (p.c_vec && n + 3 < p.N) {
                            if (carry_in) {
                                const float4 o = *reinterpret_cast<const float4*>(d);
                                x4.x += o.x; x4.y += o.y; x4.z += o.z; x4.w += o.w;
                            }
                            *reinterpret_cast<float4*>(d) = x4;
                        } else {
                            const float xs[4] = {x4.x, x4.y, x4.z, x4.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                if (n + e < p.N) d[e] = carry_in ? xs[e] + d[e] : xs[e];
                        }
                    }
                    __syncwarp();
                    continue;
                }
                if (plain) {
                    // no epilogue options: the block goes out as it is (a handful of instructions per 16 bytes; the
                    // general path below spends ~25 per element on option checks with one warp per scheduler)
                    float* dst = p.C + row_off0 + n;
                    const int64_t step = 4 * p.N;
                    if (n < p.N) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int rl = 4 * i + row_sub;
                            float4 x4 = *reinterpret_cast<const float4*>(ebuf + rl * EP_LD + ((((lane & 7) ^ (rl & 7))) << 2));
                            if (m_warp + 4 * i + row_sub < p.M) {
                                if (carry_in) {
                                    const float4 o = *reinterpret_cast<const float4*>(dst + i * step);
                                    x4.x += o.x; x4.y += o.y; x4.z += o.z; x4.w += o.w;
                                }
                                *reinterpret_cast<float4*>(dst + i * step) = x4;
                            }
                        }
                    }
                    __syncwarp();
                    continue;
                }
                float cb[4] = {0.f, 0.f, 0.f, 0.f};
                if (p.bias) {
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (n + e < p.N) cb[e] = __ldg(p.bias + n + e);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int row_l = 4 * i + row_sub;
                    const int64_t m = m_warp + row_l;
                    const float4 x4 = *reinterpret_cast<const float4*>(ebuf + row_l * EP_LD + ((((lane & 7) ^ (row_l & 7))) << 2));
                    if (m >= p.M || n >= p.N) continue;
                    const float row_bias = p.bias_m ? __ldg(p.bias_m + m) : 0.f;
                    const int64_t row_off = row_off0 + (int64_t)(4 * i) * p.N;
                    float* crow = p.C + row_off;
                    float xs[4] = {x4.x, x4.y, x4.z, x4.w};
                    if (carry_in) {
                        if (p.c_vec && n + 3 < p.N) {
                            const float4 o = *reinterpret_cast<const float4*>(crow + n);
                            xs[0] += o.x; xs[1] += o.y; xs[2] += o.z; xs[3] += o.w;
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                if (n + e < p.N) xs[e] += crow[n + e];
                        }
                    }
                    float v[4], mk[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float x = xs[e] + row_bias + cb[e];
                        mk[e] = x > 0.f ? 1.f : 0.f;
                        v[e] = act_apply(x, p.act);
                    }
                    if (p.c_vec && n + 3 < p.N) {
                        float4 o = make_float4(v[0], v[1], v[2], v[3]);
                        if (p.mul_mask) {
                            const float4 mm = __ldg(reinterpret_cast<const float4*>(p.mul_mask + row_off + n));
                            o.x *= mm.x; o.y *= mm.y; o.z *= mm.z; o.w *= mm.w;
                        }
                        if (beta != 0.f) {
                            const float4 old = *reinterpret_cast<const float4*>(crow + n);
                            o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                        }
                        *reinterpret_cast<float4*>(crow + n) = o;
                        if (p.aux) *reinterpret_cast<float4*>(p.aux + row_off + n) = make_float4(mk[0], mk[1], mk[2], mk[3]);
                        if (p.c_lo)
                            *reinterpret_cast<float4*>(p.c_lo + clo_off0 + (int64_t)(4 * i) * p.ld_clo + n) =
                                make_float4(tenmo_tf32_lo(o.x), tenmo_tf32_lo(o.y), tenmo_tf32_lo(o.z), tenmo_tf32_lo(o.w));
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            if (n + e < p.N) {
                                float o = v[e];
                                if (p.mul_mask) o *= __ldg(p.mul_mask + row_off + n + e);
                                if (beta != 0.f) o += crow[n + e];
                                crow[n + e] = o;
                                if (p.aux) p.aux[row_off + n + e] = mk[e];
                                if (p.c_lo) p.c_lo[clo_off0 + (int64_t)(4 * i) * p.ld_clo + n + e] = tenmo_tf32_lo(o);
                            }
                    }
                }
                __syncwarp();  // the buffer is rewritten by the next chunk
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (PAIR) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0u));  // both epilogues release it on the leader's barrier
                else mbar_arrive(tempty_bar(acc));
                if (partial && !carry_out) {
                    __threadfence();  // the warp's stores (ordered before this by the __syncwarp) are visible before the count
                    atomicAdd(p.sk_flags + slot * SLOT_MUL + slot_add, 1u);
                }
            }
            acc_phase[acc] ^= 1u;
            acc ^= 1;
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();  // neither CTA gives back shared or tensor memory the other may still be addressing
    if (threadIdx.x == 0) {
        if (*abort_flag) atomicOr(p.status, TENMO_DEV_TIMEOUT);
        // every CTA has finished drawing tiles (and reading flags) once it is here; the last one re-arms the counter pair
        // and the fix-up flags, so that no memset sits in front of the next launch and a captured graph can be replayed
        __threadfence();
        if (atomicAdd(p.tile_counter + 1, 1u) == gridDim.x - 1) {
            __threadfence();
            for (int u = 0; u < p.sk_units * (PAIR ? 2 : 1); ++u) p.sk_flags[u] = 0;
            p.tile_counter[0] = 0;
            p.tile_counter[1] = 0;
            __threadfence();
        }
    }
    if (warp == 1) {
        tcgen05_fence_after();
        if (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::TMEM_COLS)
                         : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::TMEM_COLS)
                         : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------
// lo-plane split:  lo = tf32_rna(x - trunc_tf32(x)), written compactly (rows x inner, ld = ld_lo)
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ float tf32_lo(float x) { return tenmo_tf32_lo(x); }

__global__ void __launch_bounds__(256)
split_lo_kernel(const float* __restrict__ src, float* __restrict__ dst, int64_t rows, int64_t inner, int64_t ld_src,
                int64_t ld_dst, int64_t batches, int64_t bstride_src, int64_t bstride_dst) {
    const int64_t vec_per_row = ld_dst / 4;  // ld_dst is a multiple of 4; the pad columns are written as zeros
    const int64_t total = batches * rows * vec_per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t v = i % vec_per_row;
        const int64_t rb = i / vec_per_row;
        const int64_t r = rb % rows, b = rb / rows;
        const int64_t c = v * 4;
        const float* s = src + b * bstride_src + r * ld_src + c;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c + 3 < inner) {
            x = __ldg(reinterpret_cast<const float4*>(s));
        } else {
            if (c + 0 < inner) x.x = __ldg(s);
            if (c + 1 < inner) x.y = __ldg(s + 1);
            if (c + 2 < inner) x.z = __ldg(s + 2);
        }
        float4 o = make_float4(tf32_lo(x.x), tf32_lo(x.y), tf32_lo(x.z), tf32_lo(x.w));
        *reinterpret_cast<float4*>(dst + b * bstride_dst + r * ld_dst + c) = o;
    }
}

// ---------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------
}  // namespace

// Collapse an operand's (possibly broadcast) batch dims into "one uniform stride" or "broadcast".
bool tenmo_collapse_batch(const TenmoBatch& b, const int64_t* stride, int64_t total, int* batched, int64_t* bstride) {
    if (total == 1) { *batched = 0; *bstride = 0; return true; }
    bool all_zero = true;
    for (int d = 0; d < b.rank; ++d)
        if (b.shape[d] > 1 && stride[d] != 0) all_zero = false;
    if (all_zero) { *batched = 0; *bstride = 0; return true; }
    // every dim of extent > 1 must be present with stride = stride[next] * shape[next]
    int64_t expect = -1;
    for (int d = b.rank - 1; d >= 0; --d) {
        if (b.shape[d] == 1) continue;
        if (stride[d] == 0) return false;  // broadcast in some dims only
        if (expect < 0) { *bstride = stride[d]; expect = stride[d] * b.shape[d]; }
        else { if (stride[d] != expect) return false; expect *= b.shape[d]; }
    }
    *batched = 1;
    return true;
}

bool tenmo_plan_operand(int64_t rows, int64_t cols, int64_t rs, int64_t cs, bool rows_are_k, const float* ptr,
                  const TenmoBatch& b, const int64_t* bstrides, int64_t total_batch, TenmoOperandPlan* o, const char* name,
                  char* why, size_t why_len) {
    // rows x cols view; k is the row index when rows_are_k (operand B) else the column index (operand A)
    bool unit_cols = (cs == 1) || cols == 1, unit_rows = (rs == 1) || rows == 1;
    int64_t inner, outer, ld;
    bool inner_is_k;
    if (unit_cols && (rs >= cols || rows == 1)) { inner = cols; outer = rows; ld = rows == 1 ? cols : rs; inner_is_k = !rows_are_k; }
    else if (unit_rows && (cs >= rows || cols == 1)) { inner = rows; outer = cols; ld = cols == 1 ? rows : cs; inner_is_k = rows_are_k; }
    else { snprintf(why, why_len, "%s has no unit-stride axis", name); return false; }
    if (ld % 4 != 0 || (reinterpret_cast<uintptr_t>(ptr) & 15u) != 0) {
        snprintf(why, why_len, "%s is not 16-byte aligned (leading stride %lld elements)", name, (long long)ld);
        return false;
    }
    if (ld < inner) { snprintf(why, why_len, "%s rows overlap", name); return false; }
    if (!tenmo_collapse_batch(b, bstrides, total_batch, &o->batched, &o->batch_stride)) {
        snprintf(why, why_len, "%s batch dims do not collapse to one stride", name);
        return false;
    }
    if (o->batched && (o->batch_stride % 4 != 0 || o->batch_stride <= 0)) {
        snprintf(why, why_len, "%s batch stride is not a positive multiple of 4 elements", name);
        return false;
    }
    o->mn_major = !inner_is_k;
    o->inner = inner; o->outer = outer; o->ld = ld;
    o->batches = o->batched ? total_batch : 1;
    o->ld_lo = (inner + 3) / 4 * 4;
    o->bstride_lo = o->ld_lo * outer;
    return true;
}

bool tenmo_make_plan(const TenmoGemmParams& p, TenmoOperandPlan* a, TenmoOperandPlan* b, char* why, size_t why_len) {
    if (p.K < 1) { snprintf(why, why_len, "K == 0"); return false; }
    if (p.M > 0x7fffffffLL || p.N > 0x7fffffffLL || p.K > 0x7fffffffLL || p.total_batch > 0x7fffffffLL) {
        snprintf(why, why_len, "dimension exceeds 2^31"); return false;
    }
    if (!tenmo_plan_operand(p.M, p.K, p.a_rs, p.a_cs, false, p.A, p.batch, p.batch.a_stride, p.total_batch, a, "A", why, why_len)) return false;
    if (!tenmo_plan_operand(p.K, p.N, p.b_rs, p.b_cs, true, p.B, p.batch, p.batch.b_stride, p.total_batch, b, "B", why, why_len)) return false;
    return true;
}

namespace {

int encode_map(tenmo_ctx* ctx, CUtensorMap* map, const float* base, const TenmoOperandPlan& o, bool lo, int box_outer) {
    TenmoEncodeTiledFn fn = reinterpret_cast<TenmoEncodeTiledFn>(ctx->encode_tiled);
    const int64_t ld = lo ? o.ld_lo : o.ld;
    const int64_t bs = lo ? o.bstride_lo : (o.batched ? o.batch_stride : ld * o.outer);
    cuuint64_t dims[3] = {(cuuint64_t)o.inner, (cuuint64_t)o.outer, (cuuint64_t)o.batches};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 4, (cuuint64_t)bs * 4};
    if (o.batches == 1) strides[1] = (cuuint64_t)ld * 4 * (cuuint64_t)o.outer;  // unused, but must be a legal stride
    if (strides[1] % 16 != 0) strides[1] = (strides[1] + 15) / 16 * 16;
    cuuint32_t box[3] = {o.mn_major ? 32u : (cuuint32_t)BK, (cuuint32_t)box_outer, 1u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE,
                    o.mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : (BK == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B),
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return tenmo_set_error(ctx, TENMO_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d (inner %lld outer %lld ld %lld)", (int)r,
                               (long long)o.inner, (long long)o.outer, (long long)ld);
    return TENMO_OK;
}

template <int BN>
cudaError_t launch_tc(bool a_mn, bool b_mn, int grid, cudaStream_t s, const CUtensorMap& ma, const CUtensorMap& mal,
                      const CUtensorMap& mb, const CUtensorMap& mbl, const TcParams& tp) {
    const int smem = TcCfg<BN>::SMEM;
#define TC_LAUNCH(AM, BMJ)                                                                                          \
    {                                                                                                               \
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, AM, BMJ>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
        if (e != cudaSuccess) return e;                                                                             \
        gemm_tc_kernel<BN, AM, BMJ><<<grid, TC_THREADS, smem, s>>>(ma, mal, mb, mbl, tp);                           \
    }
    if (a_mn) { if (b_mn) TC_LAUNCH(true, true) else TC_LAUNCH(true, false) }
    else { if (b_mn) TC_LAUNCH(false, true) else TC_LAUNCH(false, false) }
#undef TC_LAUNCH
    return cudaGetLastError();
}

// The CTA-pair form (BN = 256 only): `grid` CTAs in clusters of two.
cudaError_t launch_tc_pair(bool a_mn, bool b_mn, int grid, cudaStream_t s, const CUtensorMap& ma, const CUtensorMap& mal,
                           const CUtensorMap& mb, const CUtensorMap& mbl, const TcParams& tp) {
    const int smem = TcCfg<256, true>::SMEM;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
#define TC_LAUNCH_PAIR(AM, BMJ)                                                                                        \
    {                                                                                                                  \
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<256, AM, BMJ, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
        if (e != cudaSuccess) return e;                                                                                \
        e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<256, AM, BMJ, true>, ma, mal, mb, mbl, tp);                       \
        if (e != cudaSuccess) return e;                                                                                \
    }
    if (a_mn) { if (b_mn) TC_LAUNCH_PAIR(true, true) else TC_LAUNCH_PAIR(true, false) }
    else { if (b_mn) TC_LAUNCH_PAIR(false, true) else TC_LAUNCH_PAIR(false, false) }
#undef TC_LAUNCH_PAIR
    return cudaGetLastError();
}

}  // namespace

int tenmo_tma_init(tenmo_ctx* ctx) {
    if (ctx->tc_ready) return TENMO_OK;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
        cudaGetLastError();
        return tenmo_set_error(ctx, TENMO_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    }
    ctx->encode_tiled = fn;
    ctx->tc_ready = true;
    return TENMO_OK;
}


namespace {
// One thread waits on an mbarrier nothing will ever arrive on, with the wait routine the GEMM kernels use and a short
// limit: the expiry path (give up, raise the status word, leave) as a normal, returning kernel.
__global__ void wait_probe_kernel(uint64_t limit_ns, uint32_t* status) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (!mbar_wait(smem_u32(&bar), 0, &abort_flag, limit_ns)) atomicOr(status, TENMO_DEV_TIMEOUT);
}
}  // namespace

extern "C" int tenmo_cuda_wait_probe(tenmo_ctx* ctx, int limit_us) {
    TENMO_CHECK_CTX(ctx);
    if (limit_us < 1 || limit_us > 1000000) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "wait_probe: limit must be 1 us .. 1 s");
    TENMO_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    wait_probe_kernel<<<1, 1, 0, ctx->stream>>>((uint64_t)limit_us * 1000ull, ctx->dev_status);
    TENMO_LAUNCH_CHECK(ctx, "wait_probe_kernel");
    return TENMO_OK;
}

bool tenmo_gemm_tc_supported(tenmo_ctx* ctx, const TenmoGemmParams& p, char* why, size_t why_len) {
    (void)ctx;
    TenmoOperandPlan a, b;
    return tenmo_make_plan(p, &a, &b, why, why_len);
}

bool tenmo_gemm_tc_profitable(tenmo_ctx* ctx, const TenmoGemmParams& p) {
    (void)ctx;
    const double flop = 2.0 * (double)p.M * (double)p.N * (double)p.K * (double)p.total_batch;
    return flop >= 2.0e9 && p.M >= 128 && p.N >= 64 && p.K >= 64;
}

int tenmo_split_lo_launch(tenmo_ctx* ctx, const float* base, int64_t rows, int64_t cols, int64_t rs, int64_t cs,
                          const TenmoBatch& batch, const int64_t* bstrides, int64_t total_batch, float* out,
                          int64_t* floats_written) {
    TenmoOperandPlan o;
    char why[160];
    if (!tenmo_plan_operand(rows, cols, rs, cs, false, base, batch, bstrides, total_batch, &o, "X", why, sizeof(why)))
        return tenmo_set_error(ctx, TENMO_ERR_UNSUPPORTED, "split_lo: %s", why);
    if (reinterpret_cast<uintptr_t>(out) & 15u) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "split_lo: output is not 16-byte aligned");
    const int64_t work = o.batches * o.outer * (o.ld_lo / 4);
    const int grid = tenmo_stream_grid(ctx, work, 256 * 4, 8);
    split_lo_kernel<<<grid, 256, 0, ctx->stream>>>(base, out, o.outer, o.inner, o.ld, o.ld_lo, o.batches,
                                                   o.batched ? o.batch_stride : 0, o.bstride_lo);
    TENMO_LAUNCH_CHECK(ctx, "split_lo_kernel");
    if (floats_written) *floats_written = o.bstride_lo * o.batches;
    return TENMO_OK;
}

int tenmo_gemm_tc_launch(tenmo_ctx* ctx, const TenmoGemmParams& p) {
    int st = tenmo_tma_init(ctx);
    if (st != TENMO_OK) return st;
    TenmoOperandPlan a, b;
    char why[160];
    if (!tenmo_make_plan(p, &a, &b, why, sizeof(why))) return tenmo_set_error(ctx, TENMO_ERR_UNSUPPORTED, "gemm_tc: %s", why);

    // Tile width: 128 x 256 unless that leaves most SMs without a tile, then 128 x 128, then 128 x 64
    // (e.g. the 1000-class output layer at batch 1024: 32 tiles -> 64 -> 128).
    int ctas = ctx->sm_count - ctx->reserve_sms;  // SMs left free for a collective running beside the GEMM
    if (ctas < 1) ctas = 1;
    auto tiles_for = [&](int w) { return ((p.M + BM - 1) / BM) * ((p.N + w - 1) / w) * p.total_batch; };
    int bn = 256;
    if (tiles_for(256) * 4 < (int64_t)ctas * 3) bn = tiles_for(128) * 4 < (int64_t)ctas * 3 ? 64 : 128;
    if (p.N <= 64) bn = 64;
    else if (p.N <= 128 && bn > 128) bn = 128;
    const char* env_bn = getenv("TENMO_TC_BN");
    if (env_bn && (atoi(env_bn) == 64 || atoi(env_bn) == 128 || atoi(env_bn) == 256)) bn = atoi(env_bn);

    // Stream-K tail.  With T tiles on P CTAs the last wave is only partly filled (128 tiles on 148 SMs: 14 % of the
    // machine idle; 512 tiles: 3.46 waves run as 4).  When that costs more than 5 %, the k-blocks of the last tiles are
    // handed out as P equal pieces of one linear range; a piece that ends inside a tile parks its accumulator in the
    // workspace and the piece holding the tile's end adds it.  The cut depends only on the shape and the CTA count, so
    // results are reproducible.
    // Which tiles: pieces run at different k positions, so they share less of the operand panels in L2 than whole tiles
    // walking k in step; measured on 4096-wide layers, cutting the last 1.x waves pays up to x = .6 (+6 .. +14 %), above
    // that only the last, partial wave should be cut (1.73 waves as pieces: -6 %; its last .73: +6 %).  Pieces under 48
    // k-blocks do not repay the fix-up.
    int64_t tiles = tiles_for(bn);
    if (tiles > 0x7fffffffLL) return tenmo_set_error(ctx, TENMO_ERR_INVALID, "gemm_tc: %lld tiles is out of range", (long long)tiles);
    // CTA pairs (256 x 256 tiles on two SMs, three 64 KB stages, B fetched once per pair): whenever the 256-wide tile was
    // chosen and there is at least one such tile for every other pair.  The pairs take whole tiles in a fixed round-robin
    // (their two CTAs must agree on the sequence without talking) and, like the single-CTA form, cut the k-range of the
    // last tiles into one piece per pair when the last round would be short.  TENMO_TC_PAIR=0 / 1 forces it off / on.
    const int pairs = ctas / 2;
    const int64_t tiles2 = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + 255) / 256) * p.total_batch;
    bool use_pair = bn == 256 && pairs >= 1 && tiles2 * 2 >= (int64_t)pairs;
    {
        const char* env_pair = getenv("TENMO_TC_PAIR");
        if (env_pair && bn == 256 && pairs >= 1) use_pair = atoi(env_pair) != 0;
    }
    if (use_pair) tiles = tiles2;
    const int workers = use_pair ? pairs : ctas;   // units that work on tiles side by side
    int sk_units = 0;
    int64_t dp_tiles = tiles;
    {
        const int64_t num_kb = (p.K + BK - 1) / BK;
        const int64_t waves = (tiles + workers - 1) / workers;
        const char* env_sk = getenv("TENMO_TC_STREAMK");
        bool allowed = !(env_sk && atoi(env_sk) == 0) && p.ws_skip == 0 && workers * (use_pair ? 2 : 1) <= TENMO_SK_MAX_UNITS;
        // Pairs park and re-read two 128 KB halves per piece, so their tail pays in fewer cases (measured on 4096-wide
        // layers): not from two full rounds up (4096^3: 260 TFLOP/s in fixed rounds, 246 with the tail), and not when a
        // single round is already four fifths full.
        if (use_pair && (tiles >= 2 * (int64_t)workers || (tiles < workers && tiles * 5 >= (int64_t)workers * 4))) allowed = false;
        if (allowed && tiles % workers != 0 && (double)tiles < 0.95 * (double)(waves * workers)) {
            const int64_t full = tiles / workers;
            int64_t dp = 0;
            if (full >= 1) dp = ((tiles - (full - 1) * workers) * 10 <= (int64_t)workers * 16) ? (full - 1) * workers : full * workers;
            const int64_t q = (tiles - dp) * num_kb / workers;
            // and at most 8 partials to add into one tile
            if (q >= 48 && q * 8 >= num_kb) { sk_units = workers; dp_tiles = dp; }
        }
    }
    const size_t sk_bytes = (size_t)sk_units * (use_pair ? 2 : 1) * BM * bn * 4;

    // lo planes: taken from the caller when supplied (same storage geometry: outer x inner rounded up to 4,
    // batches back to back), else split here into the workspace [A_lo | B_lo]
    const size_t a_lo_bytes = p.a_lo ? 0 : (((size_t)a.bstride_lo * a.batches * 4 + 1023) & ~(size_t)1023);
    const size_t b_lo_bytes = p.b_lo ? 0 : (((size_t)b.bstride_lo * b.batches * 4 + 1023) & ~(size_t)1023);
    void* ws = nullptr;
    if (a_lo_bytes + b_lo_bytes + sk_bytes > 0) {
        st = tenmo_workspace(ctx, p.ws_skip + a_lo_bytes + b_lo_bytes + sk_bytes, &ws);
        if (st != TENMO_OK) return st;
        ws = static_cast<char*>(ws) + p.ws_skip;
    }
    const float* a_lo = p.a_lo ? p.a_lo : static_cast<float*>(ws);
    const float* b_lo = p.b_lo ? p.b_lo : reinterpret_cast<float*>(static_cast<char*>(ws) + a_lo_bytes);
    if ((p.a_lo && (reinterpret_cast<uintptr_t>(p.a_lo) & 15u)) || (p.b_lo && (reinterpret_cast<uintptr_t>(p.b_lo) & 15u)))
        return tenmo_set_error(ctx, TENMO_ERR_INVALID, "gemm_tc: a supplied lo plane is not 16-byte aligned");

    auto split = [&](const float* src, float* dst, const TenmoOperandPlan& o) -> int {
        const int64_t work = o.batches * o.outer * (o.ld_lo / 4);
        const int grid = tenmo_stream_grid(ctx, work, 256 * 4, 8);
        split_lo_kernel<<<grid, 256, 0, ctx->stream>>>(src, dst, o.outer, o.inner, o.ld, o.ld_lo, o.batches,
                                                       o.batched ? o.batch_stride : 0, o.bstride_lo);
        TENMO_LAUNCH_CHECK(ctx, "split_lo_kernel");
        return TENMO_OK;
    };
    if (!p.a_lo && (st = split(p.A, const_cast<float*>(a_lo), a)) != TENMO_OK) return st;
    if (!p.b_lo && (st = split(p.B, const_cast<float*>(b_lo), b)) != TENMO_OK) return st;

    CUtensorMap ma, mal, mb, mbl;
    const int a_box = a.mn_major ? BK : BM;
    const int b_box = b.mn_major ? BK : (use_pair ? bn / 2 : bn);  // a CTA of a pair stages half of the tile's columns
    if ((st = encode_map(ctx, &ma, p.A, a, false, a_box)) != TENMO_OK) return st;
    if ((st = encode_map(ctx, &mal, a_lo, a, true, a_box)) != TENMO_OK) return st;
    if ((st = encode_map(ctx, &mb, p.B, b, false, b_box)) != TENMO_OK) return st;
    if ((st = encode_map(ctx, &mbl, b_lo, b, true, b_box)) != TENMO_OK) return st;

    TcParams tp;
    tp.C = p.C; tp.aux = p.aux; tp.bias = p.bias;
    tp.mul_mask = p.mul_mask; tp.c_lo = p.c_lo; tp.ld_clo = p.ld_clo; tp.bias_m = p.bias_m;
    tp.M = p.M; tp.N = p.N; tp.K = p.K; tp.total_batch = p.total_batch;
    tp.tiles_m = use_pair ? (int)((p.M + 2 * BM - 1) / (2 * BM)) : (int)((p.M + BM - 1) / BM);
    tp.tiles_n = (int)((p.N + bn - 1) / bn);
    tp.a_batched = a.batched; tp.b_batched = b.batched;
    tp.beta = p.beta; tp.act = p.act;
    tp.c_vec = (p.N % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15u) == 0) &&
               (!p.aux || (reinterpret_cast<uintptr_t>(p.aux) & 15u) == 0) &&
               (!p.mul_mask || (reinterpret_cast<uintptr_t>(p.mul_mask) & 15u) == 0) &&
               (!p.c_lo || ((reinterpret_cast<uintptr_t>(p.c_lo) & 15u) == 0 && p.ld_clo % 4 == 0));
    tp.status = ctx->dev_status;
    tp.sk_units = sk_units;
    tp.dp_tiles = dp_tiles;
    tp.sk_partials = sk_units ? reinterpret_cast<float*>(static_cast<char*>(ws) + a_lo_bytes + b_lo_bytes) : nullptr;
    tp.sk_flags = reinterpret_cast<unsigned int*>(ctx->dev_status) + TENMO_SK_FLAG_WORD0;
    // Accumulation chains of at most 96 k-blocks (K = 3072); a longer range is cut into equal sub-ranges.  Measured on a
    // weight gradient of post-ReLU activations against softmax gradients at K = 8192: one chain is off by 1.2e-4 of
    // sum |a||b| (the bar is 1e-4), chains of 64 k-blocks by 2.9e-5.  The extra passes of the epilogue warps run beside the
    // next sub-range's MMAs: 8192^3 is unchanged within the run-to-run spread, a K = 4096 product (two sub-ranges) loses
    // 3.5 %.  TENMO_TC_CHUNK=<k-blocks> overrides (0: never cut).  Not when the old C is added after an activation or a
    // mask: there C cannot hold the running sum.
    // Tile order: groups of 16 row tiles walked column by column.  Measured at 8192^3 with CTA pairs: groups of 16 / 8 / 4
    // read 10.2 / 9.3 / 12.0 GB from DRAM per launch, speeds within the run-to-run spread.  TENMO_TC_GROUP_M overrides.
    tp.group_m = 16;
    {
        const char* env_gm = getenv("TENMO_TC_GROUP_M");
        if (env_gm && atoi(env_gm) >= 1) tp.group_m = atoi(env_gm);
    }
    tp.chunk_kb = 3072 / BK;
    {
        const char* env_ck = getenv("TENMO_TC_CHUNK");
        if (env_ck && atoi(env_ck) >= 0) tp.chunk_kb = atoi(env_ck);
    }
    if (p.beta != 0.f && (p.act != TENMO_ACT_NONE || p.mul_mask)) tp.chunk_kb = 0;
    const int grid = use_pair ? 2 * (sk_units ? pairs : (int)(tiles < pairs ? tiles : pairs))
                              : (sk_units ? ctas : (int)(tiles < ctas ? tiles : ctas));
    // a tile counter pair for this launch (dev_status words 64..127: [next tile, CTAs finished] x 32).  Both words
    // are zero between launches: the last CTA to leave clears them, so no memset sits in front of the kernel.
    tp.tile_counter = reinterpret_cast<unsigned int*>(ctx->dev_status) + 64 + 2 * (ctx->tile_counter_next++ % TILE_COUNTERS);
    tenmo_prof_before(ctx);
    cudaError_t e = use_pair      ? launch_tc_pair(a.mn_major, b.mn_major, grid, ctx->stream, ma, mal, mb, mbl, tp)
                    : (bn == 256) ? launch_tc<256>(a.mn_major, b.mn_major, grid, ctx->stream, ma, mal, mb, mbl, tp)
                    : (bn == 128) ? launch_tc<128>(a.mn_major, b.mn_major, grid, ctx->stream, ma, mal, mb, mbl, tp)
                                  : launch_tc<64>(a.mn_major, b.mn_major, grid, ctx->stream, ma, mal, mb, mbl, tp);
    tenmo_prof_after(ctx);
    ctx->launches++;
    ctx->last_gemm_kernel = "gemm_tc_kernel";
    ctx->last_gemm_sk_units = sk_units;
    ctx->last_gemm_pair = use_pair;
    if (e != cudaSuccess) return tenmo_set_error(ctx, TENMO_ERR_CUDA, "launch of gemm_tc_kernel failed: %s", cudaGetErrorString(e));
    return TENMO_OK;
}
