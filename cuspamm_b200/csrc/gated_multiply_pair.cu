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
//
// The kernel comes in two widths (template parameter NB = macro-tile columns per pair of SMs).  NB = 1 is the form
// described above.  NB = 2 multiplies FOUR dense macro tiles (two rows x two columns, 256 x 512 of C) per pair: what
// bounds the dense limit is the traffic from L2 into shared memory, and with twice the columns each byte of A is used
// twice.  Per k and SM: 8 KiB of A and one WHOLE 16 KiB slab of B (block 0 the left macro-tile column's, block 1 the
// right one's), 24 KiB for twice the products of NB = 1's 16 KiB.  An instruction's 256 columns are the FIRST (then
// the SECOND) 128 columns of both slabs, so every copy of B is one contiguous slab; the epilogue undoes that
// interleaving when it stores.  The 128 x 512 float accumulator fills tensor memory, so the epilogue of a unit does
// not overlap the next unit's multiplies (the copies for them are already under way); the first instruction of a unit
// overwrites the accumulator, so nothing has to clear it.  The launcher runs NB = 2 first, then NB = 1 for the dense
// pairs no quad covers (an odd last column, a neighbour that is not dense).
#include "tc_utils.cuh"

namespace spamm {

template <int NB>
struct PairCfg {
    static constexpr int SPS = NB == 2 ? 2 : 4;                              // k per ring stage
    static constexpr int B_BYTES = NB == 2 ? B_SLAB_BYTES : B_SLAB_BYTES / 2;   // of B per k and block
    static constexpr int STEP_BYTES = A_SLAB_BYTES + B_BYTES;               // 16 KiB / 24 KiB
    static constexpr int STAGE_BYTES = SPS * STEP_BYTES;                     // 64 KiB / 48 KiB
    static constexpr int STAGES = NB == 2 ? 4 : 3;                           // 192 KiB either way
    static constexpr int ACC_BUFS = NB == 2 ? 1 : 2;                         // accumulators in tensor memory
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 256 + 4 * EPI_WARP_BYTES + 128;
};
constexpr int P_MAX_STAGES = 4;
constexpr int P_THREADS = 192;
constexpr int P_CTRL_BYTES = 256;
constexpr uint32_t P_TMEM_COLS = 512;
constexpr uint32_t P_ACC_COLS = MT_C * TILE;                    // 256

struct PairCtrl {
    unsigned long long full[P_MAX_STAGES];    // this block's copies of a stage have landed; in the leader: both blocks'
    unsigned long long empty[P_MAX_STAGES];   // the multiplies that read the stage are done (multicast commit)
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
    if (mbar_try_wait_cluster(bar, parity) || mbar_try_wait_cluster(bar, parity) || mbar_try_wait_cluster(bar, parity))
        return true;
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
// `accumulate` == 0: the product replaces what the accumulator holds
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate = 1u)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
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

template <int NB>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
gated_multiply_pair_kernel(const uint8_t *__restrict__ half_a, const uint8_t *__restrict__ half_b,
                           const int32_t *__restrict__ step_counts, spamm_list_scalars *__restrict__ sc, int row_tiles,
                           int k_tiles, int n_tiles, float *__restrict__ c, int64_t ldc)
{
    using Cfg = PairCfg<NB>;
    constexpr int SPS = Cfg::SPS, STAGES = Cfg::STAGES, STAGE_BYTES = Cfg::STAGE_BYTES, ACC_BUFS = Cfg::ACC_BUFS;
    const int mi_n = (row_tiles + MT_R - 1) / MT_R;
    const int mj_n = (n_tiles + MT_C - 1) / MT_C;
    const unsigned int n_mt = (unsigned int)(mi_n * mj_n);
    // same test as in the one-SM kernel: below half dense macro tiles this kernel does nothing
    if (mi_n < 2 || sc->dense_count * 2u < n_mt) return;

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    PairCtrl *ctrl = reinterpret_cast<PairCtrl *>(smem + STAGES * STAGE_BYTES);
    volatile uint32_t *abort_flag = &ctrl->abort_flag;
    int32_t *err = &sc->error;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader (upper macro tiles), 1 = lower macro tiles
    const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    const int rows_total = row_tiles * TILE;
    const int pair_rows = mi_n >> 1;                  // vertical pairs of macro-tile rows
    const int unit_cols = NB == 2 ? (mj_n >> 1) : mj_n;   // units per pair row: quads (two columns) or single columns
    const int n_units = pair_rows * unit_cols;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
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

    // unit u of the band-wise order: bands of 8 pair rows (16 macro-tile rows), walked column by column
    auto unit_at = [&](int u, int *pr, int *uc) {
        const int band_rows = 8;
        const int per_band = band_rows * unit_cols;
        const int band = u / per_band, in_band = u % per_band;
        const int rows_here = min(band_rows, pair_rows - band * band_rows);
        *uc = in_band / rows_here;
        *pr = band * band_rows + in_band % rows_here;
    };
    auto pair_dense = [&](int pr, int mj) -> bool {
        return step_list_dense(step_counts[(2 * pr) * mj_n + mj]) && step_list_dense(step_counts[(2 * pr + 1) * mj_n + mj]);
    };
    // NB = 2 takes the quads whose four macro tiles are dense; NB = 1 the dense pairs that no such quad covers
    auto eligible = [&](int pr, int uc) -> bool {
        if (NB == 2) return pair_dense(pr, 2 * uc) && pair_dense(pr, 2 * uc + 1);
        if (!pair_dense(pr, uc)) return false;
        const int q = uc >> 1;
        return !(q < (mj_n >> 1) && pair_dense(pr, 2 * q) && pair_dense(pr, 2 * q + 1));
    };
    const int stages_per_unit = (k_tiles + SPS - 1) / SPS;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer (lane 0)
        if (lane == 0) {
            uint32_t slot = 0;
            bool ok = true;
            for (int u = cluster_id; u < n_units && ok; u += n_clusters) {
                int pr, uc;
                unit_at(u, &pr, &uc);
                if (!eligible(pr, uc)) continue;
                const int mi = 2 * pr + (int)rank;
                const uint8_t *a_base = half_a + (int64_t)mi * k_tiles * A_SLAB_BYTES;
                // NB = 1: this block's half of the one slab of B; NB = 2: the whole slab of this block's column
                const uint8_t *b_base = NB == 2 ? half_b + (int64_t)(2 * uc + (int)rank) * B_SLAB_BYTES
                                                : half_b + (int64_t)uc * B_SLAB_BYTES + (int64_t)rank * (B_SLAB_BYTES / 2);
                for (int g = 0; g < stages_per_unit; g++) {
                    const uint32_t s = slot % STAGES, ph = (slot / STAGES) & 1u;
                    ok = wait_bounded(smem_u32(&ctrl->empty[s]), ph ^ 1u, abort_flag, err, PERR_EMPTY);
                    if (!ok) break;
                    const int k0 = g * SPS, ns = min(SPS, k_tiles - k0);
                    const uint32_t bar = smem_u32(&ctrl->full[s]);
                    const uint32_t a_stage = smem_u32(smem + s * STAGE_BYTES);
                    const uint32_t b_stage = a_stage + SPS * A_SLAB_BYTES;
                    mbar_arrive_expect_tx(bar, (uint32_t)ns * Cfg::STEP_BYTES);
                    // the A slabs of consecutive k are neighbours in memory: one copy for the stage
                    bulk_g2s(a_stage, a_base + (int64_t)k0 * A_SLAB_BYTES, (uint32_t)ns * A_SLAB_BYTES, bar);
                    for (int t = 0; t < ns; t++)
                        bulk_g2s(b_stage + t * Cfg::B_BYTES, b_base + (int64_t)(k0 + t) * mj_n * B_SLAB_BYTES, Cfg::B_BYTES,
                                 bar);
                    slot++;
                }
            }
            if (*abort_flag) {
                const uint32_t first = slot > STAGES ? slot - STAGES : 0;
                for (uint32_t sl = first; sl < slot; sl++) {
                    const uint32_t s = sl % STAGES, ph = (sl / STAGES) & 1u;
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
                for (int u = cluster_id; u < n_units && ok; u += n_clusters) {
                    int pr, uc;
                    unit_at(u, &pr, &uc);
                    if (!eligible(pr, uc)) continue;
                    const uint32_t buf = acc_iter % ACC_BUFS;
                    ok = wait_bounded_cluster(smem_u32(&ctrl->tmem_empty[buf]), ((acc_iter / ACC_BUFS) & 1u) ^ 1u,
                                              abort_flag, err, PERR_TMEM_EMPTY);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t d = tmem_base + buf * P_ACC_COLS;
                    for (int g = 0; g < stages_per_unit; g++) {
                        const uint32_t s = slot % STAGES, ph = (slot / STAGES) & 1u;
                        ok = wait_bounded_cluster(smem_u32(&ctrl->full[s]), ph, abort_flag, err, PERR_FULL);
                        if (!ok) break;
                        tc_fence_after();
                        const int ns = min(SPS, k_tiles - g * SPS);
                        const uint32_t a_stage = stage0 + s * STAGE_BYTES;
                        const uint32_t b_stage = a_stage + SPS * A_SLAB_BYTES;
                        if (lane == 0) {
                            for (int t = 0; t < ns; t++) {
                                const uint64_t da = desc0 + (uint64_t)((a_stage + t * A_SLAB_BYTES) >> 4);
                                const uint64_t db = desc0 + (uint64_t)((b_stage + t * Cfg::B_BYTES) >> 4);
                                // the first instruction on each part of the accumulator replaces its contents
                                const uint32_t acc = (g == 0 && t == 0) ? 0u : 1u;
                                umma_f16_pair(d, da, db, IDESC, acc);
                                umma_f16_pair(d, da + 16u, db + 16u, IDESC, 1u);
                                if (NB == 2) {
                                    // columns 128-255 of both blocks' slabs, into the second half of tensor memory
                                    const uint64_t db2 = db + (uint64_t)((B_SLAB_BYTES / 2) >> 4);
                                    umma_f16_pair(d + P_ACC_COLS, da, db2, IDESC, acc);
                                    umma_f16_pair(d + P_ACC_COLS, da + 16u, db2 + 16u, IDESC, 1u);
                                }
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
                for (int u = cluster_id; u < n_units && ok; u += n_clusters) {
                    int pr, uc;
                    unit_at(u, &pr, &uc);
                    if (!eligible(pr, uc)) continue;
                    for (int g = 0; g < stages_per_unit; g++) {
                        const uint32_t s = slot % STAGES, ph = (slot / STAGES) & 1u;
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
        uint8_t *epi_tile = smem + STAGES * STAGE_BYTES + P_CTRL_BYTES + (warp - 2) * EPI_WARP_BYTES;
        uint32_t acc_iter = 0;
        unsigned int done = 0;
        bool ok = true;
        for (int u = cluster_id; u < n_units && ok; u += n_clusters) {
            int pr, uc;
            unit_at(u, &pr, &uc);
            if (!eligible(pr, uc)) continue;
            const int mi = 2 * pr + (int)rank;
            const uint32_t buf = acc_iter % ACC_BUFS;
            ok = wait_bounded(smem_u32(&ctrl->tmem_full[buf]), (acc_iter / ACC_BUFS) & 1u, abort_flag, err,
                              PERR_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int row = mi * (MT_R * TILE) + (int)q * TILE + lane;
            const bool row_ok = row < rows_total;
            // first row of this warp's 32-row block of C
            float *crow = c + (int64_t)(row - lane) * ldc;
            // which 32 columns of C the accumulator's 32-column block cc is.  NB = 2: the accumulator holds, in chunks of
            // 128 columns, [left 0-127 | right 0-127 | left 128-255 | right 128-255]
            auto c_tile_of = [&](int cc) -> int {
                if (NB == 2) {
                    const int chunk = cc >> 2;
                    return (2 * uc + (chunk & 1)) * MT_C + (chunk >> 1) * 4 + (cc & 3);
                }
                return uc * MT_C + cc;
            };
            const uint32_t tbase = tmem_base + ((q * 32u) << 16) + buf * P_ACC_COLS;
            // two register sets: the load of the next block is under way while the current one is stored
            uint32_t v0[32], v1[32];
            tmem_ld32(tbase, v0);
#pragma unroll 1
            for (int cc = 0; cc < NB * MT_C; cc += 2) {
                tmem_wait_ld();
                tmem_ld32(tbase + (uint32_t)(cc + 1) * TILE, v1);
                int ct = c_tile_of(cc);
                if (row_ok && ct < n_tiles) store_block_coalesced(epi_tile, v0, crow + (int64_t)ct * TILE, ldc, lane);
                tmem_wait_ld();
                if (cc + 2 < NB * MT_C) tmem_ld32(tbase + (uint32_t)(cc + 2) * TILE, v0);
                ct = c_tile_of(cc + 1);
                if (row_ok && ct < n_tiles) store_block_coalesced(epi_tile, v1, crow + (int64_t)ct * TILE, ldc, lane);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(smem_u32(&ctrl->tmem_empty[buf]), 0u);   // the leader's barrier
            acc_iter++;
            done += NB;
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

template <int NB>
static int launch_width(const void *d_half_a, const void *d_half_b, const int32_t *d_step_counts,
                        spamm_list_scalars *d_scalars, int row_tiles, int k_tiles, int n_tiles, float *d_c, int64_t ldc,
                        int sms, int64_t n_units, cudaStream_t stream)
{
    int clusters = sms / 2;
    if (clusters > n_units) clusters = (int)n_units;
    if (clusters < 1) return SPAMM_OK;
    gated_multiply_pair_kernel<NB><<<2 * clusters, P_THREADS, PairCfg<NB>::SMEM_BYTES, stream>>>(
        static_cast<const uint8_t *>(d_half_a), static_cast<const uint8_t *>(d_half_b), d_step_counts, d_scalars,
        row_tiles, k_tiles, n_tiles, d_c, ldc);
    SPAMM_CUDA_TRY(cudaGetLastError());
    return SPAMM_OK;
}

int gated_multiply_pair_launch(const void *d_half_a, const void *d_half_b, const int32_t *d_step_counts,
                               spamm_list_scalars *d_scalars, int row_tiles, int k_tiles, int n_tiles, float *d_c,
                               int64_t ldc, cudaStream_t stream)
{
    const int mi_n = ceil_div(row_tiles, MT_R), mj_n = ceil_div(n_tiles, MT_C);
    if (mi_n < 2 || mj_n == 0 || k_tiles == 0) return SPAMM_OK;
    static int sm_count_of[64] = {};        // per device, written once with the same value by whoever comes first
    int dev = 0;
    SPAMM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SPAMM_ERR_UNSUPPORTED;
    if (sm_count_of[dev] == 0) {
        int sms = 0;
        SPAMM_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        SPAMM_CUDA_TRY(cudaFuncSetAttribute(gated_multiply_pair_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            PairCfg<1>::SMEM_BYTES));
        SPAMM_CUDA_TRY(cudaFuncSetAttribute(gated_multiply_pair_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            PairCfg<2>::SMEM_BYTES));
        sm_count_of[dev] = sms;
    }
    const int64_t pair_rows = mi_n / 2;
    int st;
    // quads first (two macro-tile columns per pair of SMs), then the dense pairs that no quad covers
    if (mj_n >= 2 &&
        (st = launch_width<2>(d_half_a, d_half_b, d_step_counts, d_scalars, row_tiles, k_tiles, n_tiles, d_c, ldc,
                              sm_count_of[dev], pair_rows * (mj_n / 2), stream)))
        return st;
    return launch_width<1>(d_half_a, d_half_b, d_step_counts, d_scalars, row_tiles, k_tiles, n_tiles, d_c, ldc,
                           sm_count_of[dev], pair_rows * mj_n, stream);
}

// Loads this file's kernels onto the current device now (kernels are loaded lazily, at their first launch, and such
// a load can wait for kernels that are running; a kernel of one GPU that waits for a peer must not find the peer stuck
// in the load of a kernel it needs).
int preload_multiply_pair()
{
    cudaFuncAttributes a;
    SPAMM_CUDA_TRY(cudaFuncGetAttributes(&a, gated_multiply_pair_kernel<1>));
    SPAMM_CUDA_TRY(cudaFuncGetAttributes(&a, gated_multiply_pair_kernel<2>));
    return SPAMM_OK;
}

}  // namespace spamm
