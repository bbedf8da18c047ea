// Gated block multiply for DENSE macro tiles on pairs of SMs (tcgen05 cta_group::2), sm_100a only.
//
// The one-SM kernel moves 24 KiB of operands into shared memory per 128 x 256 x 32 step and its issuing thread
// pays ~110 cycles per instruction; both limit it to about 0.6 of the tensor-pipe rate.  When a macro tile and its
// vertical neighbour are both dense (every k, all rows, all columns -- the list builder marks that), the two are
// multiplied as ONE 256 x 256 tile by a cluster of two blocks: each block loads its own 128 rows of A (8 KiB per
// step) and HALF of B's 256 columns (8 KiB), the leader block issues tcgen05.mma.cta_group::2 (M=256, N=256, K=16),
// which reads A from each block's own shared memory and B from both, and writes each block's 128 x 256 accumulator
// in that block's tensor memory.  Per SM that is 16 KiB of copies and half an instruction issue per step.
//
// Roles per block: warp 0 producer (bulk copies of 4 consecutive steps per ring stage), warp 1 the MMA issuer
// in the leader block and a relay in the other (waits for its block's copies, then arrives on the leader's barrier
// through the cluster's shared-memory window), warps 2-5 epilogue.  A stage is released in both blocks at once by
// tcgen05.commit with cluster multicast; no load is multicast.  The schedule is static: cluster c takes the
// eligible pairs c, c + #clusters, ... of a band-wise order, so the two blocks need no scheduling traffic.
// Every wait is bounded; on expiry the block records the error, drains and leaves.
#include "tc_utils.cuh"

namespace spamm {

constexpr int P_SPS = 4;                                        // steps per ring stage
constexpr int P_STEP_BYTES = A_SLAB_BYTES + B_SLAB_BYTES / 2;   // 16 KiB: own rows of A, half the columns of B
constexpr int P_STAGE_BYTES = P_SPS * P_STEP_BYTES;             // 64 KiB
constexpr int P_STAGES = 3;
constexpr int P_THREADS = 192;
constexpr int P_CTRL_BYTES = 256;
constexpr int P_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + P_CTRL_BYTES + 4 * EPI_WARP_BYTES + 128;
constexpr uint32_t P_TMEM_COLS = 512;
constexpr uint32_t P_ACC_COLS = MT_C * TILE;                    // 256

struct PairCtrl {
    unsigned long long full[P_STAGES];        // this block's copies of a stage have landed; in the leader: both blocks'
    unsigned long long empty[P_STAGES];       // the multiplies that read the stage are done (multicast commit)
    unsigned long long tmem_full[2];          // accumulator complete (multicast commit)
    unsigned long long tmem_empty[2];         // (leader only) both blocks have drained the accumulator
    unsigned long long drain;
    uint32_t tmem_base;
    uint32_t abort_flag;
};
static_assert(sizeof(PairCtrl) <= P_CTRL_BYTES, "control block too large");

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on the barrier at the same shared-memory offset in block `cta` of the cluster
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar, uint32_t cta)
{
    asm volatile(
        "{\n\t.reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
        "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}" ::"r"(bar),
        "r"(cta)
        : "memory");
}
// waits with cluster scope, for barriers another block of the cluster arrives on
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
static __device__ __noinline__ bool wait_bounded_cluster(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                                  int32_t *err, int code)
{
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if (*abort_flag) return false;
        if (global_ns() - t0 > WAIT_LIMIT_NS) {
            *abort_flag = 1;
            atomicCAS(err, 0, code);
            return false;
        }
    }
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, 1, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc)
        : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar)
{
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
        "h"((uint16_t)3)
        : "memory");
}

enum { PERR_EMPTY = 11, PERR_FULL = 12, PERR_TMEM_EMPTY = 14, PERR_TMEM_FULL = 15 };

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
gated_multiply_pair_kernel(const uint8_t *__restrict__ half_a, const uint8_t *__restrict__ half_b,
                           const int32_t *__restrict__ step_counts, spamm_list_scalars *__restrict__ sc, int row_tiles,
                           int k_tiles, int n_tiles, float *__restrict__ c, int64_t ldc)
{
    const int mi_n = (row_tiles + MT_R - 1) / MT_R;
    const int mj_n = (n_tiles + MT_C - 1) / MT_C;
    const unsigned int n_mt = (unsigned int)(mi_n * mj_n);
    // same test as in the one-SM kernel: below half dense macro tiles this kernel does nothing
    if (mi_n < 2 || sc->dense_count * 2u < n_mt) return;

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    PairCtrl *ctrl = reinterpret_cast<PairCtrl *>(smem + P_STAGES * P_STAGE_BYTES);
    volatile uint32_t *abort_flag = &ctrl->abort_flag;
    int32_t *err = &sc->error;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader (upper macro tile), 1 = lower macro tile
    const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    const int rows_total = row_tiles * TILE;
    const int pair_rows = mi_n >> 1;                  // vertical pairs of macro-tile rows
    const int n_pairs = pair_rows * mj_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < P_STAGES; s++) {
            // the leader's barrier also counts the other block's "my copies have landed" (one wait per stage)
            mbar_init(smem_u32(&ctrl->full[s]), rank == 0 ? 2 : 1);
            mbar_init(smem_u32(&ctrl->empty[s]), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(smem_u32(&ctrl->tmem_full[b]), 1);
            mbar_init(smem_u32(&ctrl->tmem_empty[b]), 8);     // one lane of each of the 2 x 4 epilogue warps
        }
        mbar_init(smem_u32(&ctrl->drain), 1);
        ctrl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&ctrl->tmem_base)),
                     "r"(P_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = ctrl->tmem_base;
    if (warp >= 2) {
        const uint32_t q = (uint32_t)(warp & 3);
        for (uint32_t col = 0; col < P_TMEM_COLS; col += 32) tmem_st32_zero(tmem_base + ((q * 32u) << 16) + col);
        tmem_wait_st();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();

    // pair p of the band-wise order: bands of 8 pair rows (16 macro-tile rows), walked column by column
    auto pair_at = [&](int p, int *pr, int *mj) {
        const int band_rows = 8;
        const int per_band = band_rows * mj_n;
        const int band = p / per_band, in_band = p % per_band;
        const int rows_here = min(band_rows, pair_rows - band * band_rows);
        *mj = in_band / rows_here;
        *pr = band * band_rows + in_band % rows_here;
    };
    // the last band may have fewer rows: recompute the index range of each band
    auto eligible = [&](int pr, int mj) -> bool {
        return step_list_dense(step_counts[(2 * pr) * mj_n + mj]) && step_list_dense(step_counts[(2 * pr + 1) * mj_n + mj]);
    };
    const int stages_per_tile = (k_tiles + P_SPS - 1) / P_SPS;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer (lane 0)
        if (lane == 0) {
            uint32_t slot = 0;
            bool ok = true;
            for (int p = cluster_id; p < n_pairs && ok; p += n_clusters) {
                int pr, mj;
                pair_at(p, &pr, &mj);
                if (!eligible(pr, mj)) continue;
                const int mi = 2 * pr + (int)rank;
                const uint8_t *a_base = half_a + (int64_t)mi * k_tiles * A_SLAB_BYTES;
                const uint8_t *b_base = half_b + (int64_t)mj * B_SLAB_BYTES + (int64_t)rank * (B_SLAB_BYTES / 2);
                for (int g = 0; g < stages_per_tile; g++) {
                    const uint32_t s = slot % P_STAGES, ph = (slot / P_STAGES) & 1u;
                    ok = wait_bounded(smem_u32(&ctrl->empty[s]), ph ^ 1u, abort_flag, err, PERR_EMPTY);
                    if (!ok) break;
                    const int k0 = g * P_SPS, ns = min(P_SPS, k_tiles - k0);
                    const uint32_t bar = smem_u32(&ctrl->full[s]);
                    const uint32_t a_stage = smem_u32(smem + s * P_STAGE_BYTES);
                    const uint32_t b_stage = a_stage + P_SPS * A_SLAB_BYTES;
                    mbar_arrive_expect_tx(bar, (uint32_t)ns * P_STEP_BYTES);
                    // the A slabs of consecutive k are neighbours in memory: one copy for the stage
                    bulk_g2s(a_stage, a_base + (int64_t)k0 * A_SLAB_BYTES, (uint32_t)ns * A_SLAB_BYTES, bar);
                    for (int t = 0; t < ns; t++)
                        bulk_g2s(b_stage + t * (B_SLAB_BYTES / 2), b_base + (int64_t)(k0 + t) * mj_n * B_SLAB_BYTES,
                                 B_SLAB_BYTES / 2, bar);
                    slot++;
                }
            }
            if (*abort_flag) {
                const uint32_t first = slot > P_STAGES ? slot - P_STAGES : 0;
                for (uint32_t sl = first; sl < slot; sl++) {
                    const uint32_t s = sl % P_STAGES, ph = (sl / P_STAGES) & 1u;
                    const unsigned long long t0 = global_ns();
                    while (!mbar_try_wait(smem_u32(&ctrl->full[s]), ph) && global_ns() - t0 < WAIT_LIMIT_NS) {}
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // In the leader every lane of the warp runs the loop and lane 0 issues: addresses and descriptors are then
        // the same in all lanes (measured: 8 % more tensor throughput than a loop inside `if (lane == 0)`).
        if (rank == 0 || lane == 0) {
            uint32_t slot = 0, acc_iter = 0;
            bool ok = true;
            if (rank == 0) {
                // -------------------------------------------------------------- leader: tensor-core issue
                const uint64_t desc0 = smem_desc(0);
                const uint32_t stage0 = smem_u32(smem);
                constexpr uint32_t IDESC = (1u << 4) | ((256u >> 3) << 17) | ((256u >> 4) << 24);   // M=256, N=256
                for (int p = cluster_id; p < n_pairs && ok; p += n_clusters) {
                    int pr, mj;
                    pair_at(p, &pr, &mj);
                    if (!eligible(pr, mj)) continue;
                    const uint32_t buf = acc_iter & 1u;
                    ok = wait_bounded_cluster(smem_u32(&ctrl->tmem_empty[buf]), ((acc_iter >> 1) & 1u) ^ 1u, abort_flag,
                                              err, PERR_TMEM_EMPTY);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t d = tmem_base + buf * P_ACC_COLS;
                    for (int g = 0; g < stages_per_tile; g++) {
                        const uint32_t s = slot % P_STAGES, ph = (slot / P_STAGES) & 1u;
                        ok = wait_bounded_cluster(smem_u32(&ctrl->full[s]), ph, abort_flag, err, PERR_FULL);
                        if (!ok) break;
                        tc_fence_after();
                        const int ns = min(P_SPS, k_tiles - g * P_SPS);
                        const uint32_t a_stage = stage0 + s * P_STAGE_BYTES;
                        const uint32_t b_stage = a_stage + P_SPS * A_SLAB_BYTES;
                        if (lane == 0) {
                            for (int t = 0; t < ns; t++) {
                                const uint64_t da = desc0 + (uint64_t)((a_stage + t * A_SLAB_BYTES) >> 4);
                                const uint64_t db = desc0 + (uint64_t)((b_stage + t * (B_SLAB_BYTES / 2)) >> 4);
                                umma_f16_pair(d, da, db, IDESC);
                                umma_f16_pair(d, da + 16u, db + 16u, IDESC);
                            }
                            umma_commit_pair(smem_u32(&ctrl->empty[s]));
                        }
                        __syncwarp();
                        slot++;
                    }
                    if (!ok) break;
                    if (lane == 0) umma_commit_pair(smem_u32(&ctrl->tmem_full[buf]));
                    acc_iter++;
                }
                if (*abort_flag && lane == 0) {
                    umma_commit_pair(smem_u32(&ctrl->drain));
                    const unsigned long long t0 = global_ns();
                    while (!mbar_try_wait(smem_u32(&ctrl->drain), 0) && global_ns() - t0 < WAIT_LIMIT_NS) {}
                }
            } else {
                // -------------------------------------------------------------- other block: relay "my copies landed"
                for (int p = cluster_id; p < n_pairs && ok; p += n_clusters) {
                    int pr, mj;
                    pair_at(p, &pr, &mj);
                    if (!eligible(pr, mj)) continue;
                    for (int g = 0; g < stages_per_tile; g++) {
                        const uint32_t s = slot % P_STAGES, ph = (slot / P_STAGES) & 1u;
                        ok = wait_bounded(smem_u32(&ctrl->full[s]), ph, abort_flag, err, PERR_FULL);
                        if (!ok) break;
                        mbar_arrive_remote(smem_u32(&ctrl->full[s]), 0u);
                        slot++;
                    }
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue (4 warps per block)
        const uint32_t q = (uint32_t)(warp & 3);
        uint8_t *epi_tile = smem + P_STAGES * P_STAGE_BYTES + P_CTRL_BYTES + (warp - 2) * EPI_WARP_BYTES;
        uint32_t acc_iter = 0;
        unsigned int done = 0;
        bool ok = true;
        for (int p = cluster_id; p < n_pairs && ok; p += n_clusters) {
            int pr, mj;
            pair_at(p, &pr, &mj);
            if (!eligible(pr, mj)) continue;
            const int mi = 2 * pr + (int)rank;
            const uint32_t buf = acc_iter & 1u;
            ok = wait_bounded(smem_u32(&ctrl->tmem_full[buf]), (acc_iter >> 1) & 1u, abort_flag, err, PERR_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int row = mi * (MT_R * TILE) + (int)q * TILE + lane;
            const bool row_ok = row < rows_total;
            // first row of this warp's 32-row block of C, first column of the macro tile
            float *cblock = c + (int64_t)(row - lane) * ldc + (int64_t)mj * (MT_C * TILE);
#pragma unroll 1
            for (int cc = 0; cc < MT_C; cc++) {
                const uint32_t taddr = tmem_base + ((q * 32u) << 16) + buf * P_ACC_COLS + (uint32_t)cc * TILE;
                uint32_t v[32];
                tmem_ld32(taddr, v);
                tmem_wait_ld();
                tmem_st32_zero(taddr);
                if (row_ok && mj * MT_C + cc < n_tiles) store_block_coalesced(epi_tile, v, cblock + cc * TILE, ldc, lane);
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(smem_u32(&ctrl->tmem_empty[buf]), 0u);   // the leader's barrier
            acc_iter++;
            done++;
        }
        if (warp == 2 && lane == 0 && done) atomicAdd(&sc->pair_done, done);            // macro tiles written
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                       // nobody frees tensor memory while the other block may still use it
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(P_TMEM_COLS)
                     : "memory");
    }
}

int gated_multiply_pair_launch(const void *d_half_a, const void *d_half_b, const int32_t *d_step_counts,
                               spamm_list_scalars *d_scalars, int row_tiles, int k_tiles, int n_tiles, float *d_c,
                               int64_t ldc, cudaStream_t stream)
{
    const int mi_n = ceil_div(row_tiles, MT_R), mj_n = ceil_div(n_tiles, MT_C);
    if (mi_n < 2 || mj_n == 0 || k_tiles == 0) return SPAMM_OK;
    static int sm_count_of[64] = {};
    int dev = 0;
    SPAMM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SPAMM_ERR_UNSUPPORTED;
    if (sm_count_of[dev] == 0) {
        int sms = 0;
        SPAMM_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        SPAMM_CUDA_TRY(cudaFuncSetAttribute(gated_multiply_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            P_SMEM_BYTES));
        sm_count_of[dev] = sms;
    }
    const int64_t n_pairs = (int64_t)(mi_n / 2) * mj_n;
    int clusters = sm_count_of[dev] / 2;
    if (clusters > n_pairs) clusters = (int)n_pairs;
    if (clusters < 1) return SPAMM_OK;
    gated_multiply_pair_kernel<<<2 * clusters, P_THREADS, P_SMEM_BYTES, stream>>>(
        static_cast<const uint8_t *>(d_half_a), static_cast<const uint8_t *>(d_half_b), d_step_counts, d_scalars,
        row_tiles, k_tiles, n_tiles, d_c, ldc);
    SPAMM_CUDA_TRY(cudaGetLastError());
    return SPAMM_OK;
}

}  // namespace spamm
