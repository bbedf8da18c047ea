// Gated block multiply on PAIRS of SMs (tcgen05 cta_group::2), sm_100a only: the half-full workloads.
//
// The one-SM kernel (gated_multiply.cu) moves up to 24 KiB from L2 into shared memory per k of a 128 x 256 macro tile.
// When most macro tiles have long lists (a density matrix on a lattice: hundreds of k per tile, a third of the
// products of a step surviving), all SMs pull operands at once and the traffic from L2 into the SMs is what bounds the
// multiply.  Here two vertically adjacent macro tiles (256 x 256 of C) are multiplied by a cluster of two blocks that
// SHARE the tiles of B: per k each block loads its own rows of A (8 KiB) and HALF of the columns of B the k needs,
// and one tcgen05.mma.cta_group::2 (M = 256) reads A from each block's own shared memory and B from both.
//
// The skip lists stay what the list builder wrote (one list of steps per 128 x 256 macro tile, gated_multiply.cu);
// for this kernel a second small kernel (pair_runs_kernel) writes, per pair of macro tiles and per k that has any
// surviving product in it, one 16-byte RECORD: k and up to 8 RUNS.  It evaluates the same rounded float products
// against the same threshold as the list builder (one k per lane, 8 x 8 products), so both describe the same set.
// For one k the record holds the row set of every tile column (4 bits for the upper macro tile's rows, 4 for the
// lower's); a maximal range of adjacent columns with the same non-empty row set is a run: one instruction (two, for
// the two K = 16 halves of a tile) with N = 32 * length, whose disable-output-lane mask (8 words: 4 per block) leaves
// out the tile rows that are not in the set -- so no product outside the lists is ever added.  A run's columns are
// split between the blocks the way the instruction reads them: the first half of its bytes goes to block 0, the
// second to block 1, both at the same offset of their stage slot (1 KiB per column tile of the range), one bulk copy
// each.
//
// Roles per block: warp 0 producer (reads the records 32 at a time, lane 0 issues copies), warp 1 the MMA issuer in the
// leader block and a relay in the other (its block's copies have landed -> arrives on the leader's barrier), warps
// 2-5 epilogue (tensor memory -> shared-memory turn -> whole rows of C; clears the accumulator behind itself, since
// every instruction accumulates).  Two accumulators alternate.  Units (pairs of macro tiles) are dealt out round-robin
// in a band-wise order; the last macro-tile row of an odd count is left to the one-SM kernel, which runs afterwards.
// Every wait is bounded; on expiry the block records the error, drains and leaves.
#include "tc_utils.cuh"

namespace spamm {

constexpr int G_SPS = 2;                                        // k per ring stage
constexpr int G_SLOT_BYTES = A_SLAB_BYTES + B_SLAB_BYTES / 2;   // 16 KiB: own rows of A, half of the columns of B
constexpr int G_STAGE_BYTES = G_SPS * G_SLOT_BYTES;             // 32 KiB
constexpr int G_STAGES = 6;                                     // 192 KiB
constexpr int G_RUNS = 8;                                       // most runs of one k (8 tile columns)
constexpr int G_THREADS = 192;
constexpr int G_CTRL_BYTES = 512;
constexpr int G_SMEM_BYTES = G_STAGES * G_STAGE_BYTES + G_CTRL_BYTES + 4 * EPI_WARP_BYTES + 128;
constexpr uint32_t G_TMEM_COLS = 512;
constexpr uint32_t G_ACC_COLS = MT_C * TILE;                    // 256

struct GCtrl {
    unsigned long long full[G_STAGES];        // this block's copies of a stage have landed; in the leader: both blocks'
    unsigned long long empty[G_STAGES];       // the multiplies that read the stage are done (multicast commit)
    unsigned long long tmem_full[2];          // accumulator complete (multicast commit)
    unsigned long long tmem_empty[2];         // (leader only) both blocks have drained the accumulator
    unsigned long long drain;
    uint4 rec[G_STAGES][G_SPS];               // per stage slot: the record of one k (x == 0xffffffff: slot not used)
    uint32_t stage_last[G_STAGES];            // this stage ends its unit
    uint32_t tmem_base;
    uint32_t abort_flag;
};
static_assert(sizeof(GCtrl) <= G_CTRL_BYTES, "control block too large");

// Record of one k of one pair of macro tiles, 128 bits: bits 0-15 k, then 8 runs of 14 bits each
// (bits 0-7 row set: 4 upper + 4 lower tile rows; bits 8-10 first tile column; bits 11-13 length - 1); a run with an
// empty row set ends the record.
__device__ __forceinline__ uint32_t rec_run(const uint4 &r, int i)
{
    const int o = 16 + 14 * i, wi = o >> 5, sh = o & 31;
    const uint32_t lo = wi == 0 ? r.x : wi == 1 ? r.y : wi == 2 ? r.z : r.w;
    const uint32_t hi = wi == 0 ? r.y : wi == 1 ? r.z : wi == 2 ? r.w : 0u;
    return __funnelshift_r(lo, hi, sh) & 0x3fffu;
}
__device__ __forceinline__ void rec_set_run(uint4 &r, int i, uint32_t run)
{
    const int o = 16 + 14 * i, wi = o >> 5, sh = o & 31;
    const uint64_t v = (uint64_t)run << sh;
    const uint32_t lo = (uint32_t)v, hi = (uint32_t)(v >> 32);
    if (wi == 0) { r.x |= lo; r.y |= hi; }
    else if (wi == 1) { r.y |= lo; r.z |= hi; }
    else if (wi == 2) { r.z |= lo; r.w |= hi; }
    else { r.w |= lo; }
}

__device__ __forceinline__ uint32_t g_cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void g_cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void g_mbar_arrive_remote(uint32_t bar, uint32_t cta)
{
    asm volatile(
        "{\n\t.reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
        "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}" ::"r"(bar),
        "r"(cta)
        : "memory");
}
__device__ __forceinline__ bool g_mbar_try_wait_cluster(uint32_t bar, uint32_t parity)
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
static __device__ __noinline__ bool g_wait_cluster(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag, int32_t *err,
                                                    int code)
{
    if (g_mbar_try_wait_cluster(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        if (g_mbar_try_wait_cluster(bar, parity)) return true;
        if (*abort_flag) return false;
        if (global_ns() - t0 > WAIT_LIMIT_NS) {
            *abort_flag = 1;
            atomicCAS(err, 0, code);
            return false;
        }
    }
}
// M = 256 over both blocks; m[0..3] mask the lanes of block 0's accumulator, m[4..7] block 1's (a set bit = not written)
__device__ __forceinline__ void g_umma_masked(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              const uint32_t *m)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, 1, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%4, %5, %6, %7, %8, %9, %10, %11}, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(m[0]), "r"(m[1]), "r"(m[2]), "r"(m[3]), "r"(m[4]), "r"(m[5]), "r"(m[6]),
        "r"(m[7])
        : "memory");
}
__device__ __forceinline__ void g_umma_commit(uint32_t bar)
{
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
        "h"((uint16_t)3)
        : "memory");
}

enum { GERR_EMPTY = 21, GERR_FULL = 22, GERR_TMEM_EMPTY = 24, GERR_TMEM_FULL = 25 };

// Records for the two-SM kernel: one warp per pair of macro tiles, one k per lane.  amax / bmax are the chunk maxima
// the list builder's first kernel left (largest norm per 4 tile rows of A / 8 tile columns of B and 32 k): a chunk
// whose largest product is below the threshold holds no survivor and is not read (rounded float multiplication is
// monotone in each factor).
__global__ void __launch_bounds__(128)
pair_runs_kernel(const float *__restrict__ norm_a, const float *__restrict__ norm_b, int row_tiles, int k_tiles,
                 int n_tiles, float tau, const float *__restrict__ amax, const float *__restrict__ bmax,
                 uint4 *__restrict__ recs, int32_t *__restrict__ rec_counts)
{
    const int lane = threadIdx.x & 31;
    const int mi_n = (row_tiles + MT_R - 1) / MT_R;
    const int mj_n = (n_tiles + MT_C - 1) / MT_C;
    const int kc_n = (k_tiles + 31) / 32;
    const int unit = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (unit >= (mi_n >> 1) * mj_n) return;
    const int pr = unit / mj_n, mj = unit % mj_n;
    uint4 *out = recs + (int64_t)unit * k_tiles;
    int n_out = 0;
    const bool b_vec = ((n_tiles & 3) == 0) && (mj * MT_C + MT_C <= n_tiles) &&
                       ((reinterpret_cast<uintptr_t>(norm_b) & 15) == 0);
    for (int g0 = 0; g0 < kc_n; g0 += 32) {
        bool alive = false;
        if (g0 + lane < kc_n) {
            const float bm = bmax[(int64_t)(g0 + lane) * mj_n + mj];
            const float p0 = __fmul_rn(amax[(int64_t)(2 * pr) * kc_n + g0 + lane], bm);
            const float p1 = __fmul_rn(amax[(int64_t)(2 * pr + 1) * kc_n + g0 + lane], bm);
            alive = !(p0 < tau) || !(p1 < tau);
        }
        uint32_t chunks = __ballot_sync(0xffffffffu, alive);
        while (chunks) {
            const int kb = (g0 + __ffs(chunks) - 1) * 32;
            chunks &= chunks - 1;
            const int k = kb + lane;
            uint4 rec = make_uint4(0u, 0u, 0u, 0u);
            bool any = false;
            if (k < k_tiles) {
                float a[2 * MT_R], b[MT_C];
#pragma unroll
                for (int r = 0; r < 2 * MT_R; r++) {
                    const int row = pr * 2 * MT_R + r;
                    a[r] = (row < row_tiles) ? __ldg(norm_a + (int64_t)row * k_tiles + k) : 0.0f;
                }
                const float *brow = norm_b + (int64_t)k * n_tiles + mj * MT_C;
                if (b_vec) {
                    const float4 b0 = __ldg(reinterpret_cast<const float4 *>(brow));
                    const float4 b1 = __ldg(reinterpret_cast<const float4 *>(brow) + 1);
                    b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w;
                    b[4] = b1.x; b[5] = b1.y; b[6] = b1.z; b[7] = b1.w;
                } else {
#pragma unroll
                    for (int cc = 0; cc < MT_C; cc++) b[cc] = (mj * MT_C + cc < n_tiles) ? __ldg(brow + cc) : 0.0f;
                }
                // row set of every column, then the runs: adjacent columns with the same non-empty set
                uint32_t prev = 0, c0 = 0, len = 0;
                int n_runs = 0;
#pragma unroll
                for (int cc = 0; cc <= MT_C; cc++) {
                    uint32_t rows = 0;
                    if (cc < MT_C && mj * MT_C + cc < n_tiles) {
#pragma unroll
                        for (int r = 0; r < 2 * MT_R; r++) {
                            const int row = pr * 2 * MT_R + r;
                            if (row < row_tiles && __fmul_rn(a[r], b[cc]) >= tau) rows |= 1u << r;
                        }
                    }
                    if (rows != prev || cc == MT_C) {
                        if (prev) {
                            rec_set_run(rec, n_runs, prev | (c0 << 8) | ((len - 1u) << 11));
                            n_runs++;
                        }
                        prev = rows;
                        c0 = (uint32_t)cc;
                        len = 0;
                    }
                    len++;
                }
                any = n_runs > 0;
                rec.x |= (uint32_t)k;
            }
            const uint32_t have = __ballot_sync(0xffffffffu, any);
            if (any) out[n_out + __popc(have & ((1u << lane) - 1u))] = rec;
            n_out += __popc(have);
        }
    }
    if (lane == 0) rec_counts[unit] = n_out;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(G_THREADS, 1)
gated_multiply_gpair_kernel(const uint8_t *__restrict__ half_a, const uint8_t *__restrict__ half_b,
                            const int32_t *__restrict__ step_counts,
                            const uint4 *__restrict__ recs, const int32_t *__restrict__ rec_counts,
                            spamm_list_scalars *__restrict__ sc, int row_tiles, int k_tiles, int n_tiles,
                            float *__restrict__ c, int64_t ldc, int mode)
{
    const bool c_zeroed = (mode & GM_C_ZEROED) != 0;        // leave units without steps alone
    const bool accumulate = (mode & GM_ACCUMULATE) != 0;    // add to C
    const float acc_scale = (mode & GM_LOW_OPERAND) ? 1.0f / SPLIT_LOW_SCALE : 1.0f;
    const int mi_n = (row_tiles + MT_R - 1) / MT_R;
    const int mj_n = (n_tiles + MT_C - 1) / MT_C;

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    GCtrl *ctrl = reinterpret_cast<GCtrl *>(smem + G_STAGES * G_STAGE_BYTES);
    volatile uint32_t *abort_flag = &ctrl->abort_flag;
    int32_t *err = &sc->error;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = g_cluster_ctarank();        // 0 = leader (upper macro tile), 1 = lower macro tile
    const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    const int rows_total = row_tiles * TILE;
    const int pair_rows = mi_n >> 1;                  // vertical pairs of macro-tile rows
    const int n_units = pair_rows * mj_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < G_STAGES; s++) {
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
                     "r"(G_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    g_cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = ctrl->tmem_base;
    if (warp >= 2) {
        // clear both accumulators: every multiply accumulates
        const uint32_t q = (uint32_t)(warp & 3);
        for (uint32_t col = 0; col < G_TMEM_COLS; col += 32) tmem_st32_zero(tmem_base + ((q * 32u) << 16) + col);
        tmem_wait_st();
    }
    tc_fence_before();
    __syncthreads();
    g_cluster_sync_all();
    tc_fence_after();

    // unit u of the band-wise order: bands of 8 pair rows (16 macro-tile rows), walked column by column
    auto unit_at = [&](int u, int *pr, int *mj) {
        const int band_rows = 8;
        const int per_band = band_rows * mj_n;
        const int band = u / per_band, in_band = u % per_band;
        const int rows_here = min(band_rows, pair_rows - band * band_rows);
        *mj = in_band / rows_here;
        *pr = band * band_rows + in_band % rows_here;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        // The warp reads the unit's records 32 at a time (one per lane, the next 32 fetched meanwhile); every lane
        // follows them (the values are the same in all lanes), lane 0 issues the copies.
        uint32_t slot = 0;
        bool ok = true;
        for (int u = cluster_id; u < n_units && ok; u += n_clusters) {
            int pr, mj;
            unit_at(u, &pr, &mj);
            const int unit = pr * mj_n + mj;
            const int cnt = rec_counts[unit];
            if (cnt == 0) continue;
            const uint4 *list = recs + (int64_t)unit * k_tiles;
            const int mi = 2 * pr + (int)rank;
            const uint8_t *a_base = half_a + (int64_t)mi * k_tiles * A_SLAB_BYTES;
            const uint8_t *b_base = half_b + (int64_t)mj * B_SLAB_BYTES;
            const uint4 none = make_uint4(0u, 0u, 0u, 0u);
            uint4 next = lane < cnt ? __ldg(list + lane) : none;
            for (int i0 = 0; i0 < cnt && ok; i0 += 32) {
                const uint4 mine = next;
                next = i0 + 32 + lane < cnt ? __ldg(list + i0 + 32 + lane) : none;
                const int nb = min(32, cnt - i0);
                for (int j = 0; j < nb && ok; j++) {
                    uint4 rec;
                    rec.x = __shfl_sync(0xffffffffu, mine.x, j);
                    rec.y = __shfl_sync(0xffffffffu, mine.y, j);
                    rec.z = __shfl_sync(0xffffffffu, mine.z, j);
                    rec.w = __shfl_sync(0xffffffffu, mine.w, j);
                    const int t = (i0 + j) % G_SPS;                 // slot inside the stage
                    const bool last = i0 + j == cnt - 1;
                    const uint32_t s = slot % G_STAGES;
                    if (lane == 0) {
                        if (t == 0) {
                            // a new stage: wait until the multiplies that read its previous contents are done
                            ok = wait_bounded(smem_u32(&ctrl->empty[s]), ((slot / G_STAGES) & 1u) ^ 1u, abort_flag, err,
                                              GERR_EMPTY);
                        }
                        if (ok) {
                            const uint32_t bar = smem_u32(&ctrl->full[s]);
                            const uint32_t a_slot = smem_u32(smem + s * G_STAGE_BYTES) + t * A_SLAB_BYTES;
                            const uint32_t b_slot = smem_u32(smem + s * G_STAGE_BYTES) + G_SPS * A_SLAB_BYTES +
                                                    t * (B_SLAB_BYTES / 2);
                            const uint32_t k = rec.x & 0xffffu;
                            const uint8_t *b_src = b_base + (int64_t)k * mj_n * B_SLAB_BYTES;
                            uint32_t bytes = 0, rows_any = 0;
#pragma unroll 1
                            for (int r = 0; r < G_RUNS; r++) {
                                const uint32_t run = rec_run(rec, r);
                                if ((run & 0xffu) == 0u) break;
                                const uint32_t c0 = (run >> 8) & 7u, len = ((run >> 11) & 7u) + 1u;
                                rows_any |= run & 0xffu;
                                // the run's 2 KiB tiles are adjacent in B's slab: the first half of the bytes to block 0,
                                // the second to block 1, both at 1 KiB per tile of the range from the slot's start
                                bulk_g2s(b_slot + c0 * (TILE_BYTES / 2), b_src + c0 * TILE_BYTES + rank * len * (TILE_BYTES / 2),
                                         len * (TILE_BYTES / 2), bar);
                                bytes += len * (TILE_BYTES / 2);
                            }
                            // the rows of A this block owns: one tile when a single row takes part, else the slab
                            const uint32_t own = (rows_any >> (4 * rank)) & 0xfu;
                            if (own) {
                                const uint8_t *a_src = a_base + (int64_t)k * A_SLAB_BYTES;
                                if (__popc(own) == 1) {
                                    const uint32_t q = (uint32_t)(__ffs(own) - 1);
                                    bulk_g2s(a_slot + q * TILE_BYTES, a_src + q * TILE_BYTES, TILE_BYTES, bar);
                                    bytes += TILE_BYTES;
                                } else {
                                    bulk_g2s(a_slot, a_src, A_SLAB_BYTES, bar);
                                    bytes += A_SLAB_BYTES;
                                }
                            }
                            ctrl->rec[s][t] = rec;
                            // a copy may complete before the bytes it brings are announced: the barrier's count of
                            // pending bytes is signed, and its phase cannot end before the arrival below
                            if (t == G_SPS - 1 || last) {
                                if (t < G_SPS - 1) ctrl->rec[s][t + 1].x = 0xffffffffu;
                                ctrl->stage_last[s] = last ? 1u : 0u;
                                mbar_arrive_expect_tx(bar, bytes);
                            } else {
                                asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes)
                                             : "memory");
                            }
                        }
                    }
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (t == G_SPS - 1 || last) slot++;
                }
            }
        }
        if (lane == 0 && *abort_flag) {
            const uint32_t first = slot > G_STAGES ? slot - G_STAGES : 0;
            for (uint32_t sl = first; sl < slot; sl++) {
                const uint32_t s = sl % G_STAGES, ph = (sl / G_STAGES) & 1u;
                const unsigned long long t0 = global_ns();
                while (!mbar_try_wait(smem_u32(&ctrl->full[s]), ph) && global_ns() - t0 < WAIT_LIMIT_NS) {}
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (rank == 0 || lane == 0) {
            uint32_t slot = 0, acc_iter = 0;
            bool ok = true;
            if (rank == 0) {
                // -------------------------------------------------------------- leader: tensor-core issue
                const uint64_t desc0 = smem_desc(0);
                const uint32_t stage0 = smem_u32(smem);
                for (int u = cluster_id; u < n_units && ok; u += n_clusters) {
                    int pr, mj;
                    unit_at(u, &pr, &mj);
                    if (rec_counts[pr * mj_n + mj] == 0) continue;
                    const uint32_t buf = acc_iter & 1u;
                    ok = g_wait_cluster(smem_u32(&ctrl->tmem_empty[buf]), ((acc_iter >> 1) & 1u) ^ 1u, abort_flag, err,
                                        GERR_TMEM_EMPTY);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t dbase = tmem_base + buf * G_ACC_COLS;
                    for (bool last = false; !last;) {
                        const uint32_t s = slot % G_STAGES, ph = (slot / G_STAGES) & 1u;
                        ok = g_wait_cluster(smem_u32(&ctrl->full[s]), ph, abort_flag, err, GERR_FULL);
                        if (!ok) break;
                        tc_fence_after();
                        last = ctrl->stage_last[s] != 0u;
                        const uint32_t a_stage = stage0 + s * G_STAGE_BYTES;
                        const uint32_t b_stage = a_stage + G_SPS * A_SLAB_BYTES;
                        __syncwarp();
                        if (lane == 0) {
#pragma unroll 1
                            for (int t = 0; t < G_SPS; t++) {
                                const uint4 rec = ctrl->rec[s][t];
                                if (rec.x == 0xffffffffu) break;       // a stage that is not full: no further slots
                                const uint64_t da = desc0 + (uint64_t)((a_stage + t * A_SLAB_BYTES) >> 4);
                                const uint32_t b_slot = b_stage + t * (B_SLAB_BYTES / 2);
#pragma unroll 1
                                for (int r = 0; r < G_RUNS; r++) {
                                    const uint32_t run = rec_run(rec, r);
                                    const uint32_t rows8 = run & 0xffu;
                                    if (rows8 == 0u) break;
                                    const uint32_t c0 = (run >> 8) & 7u, len = ((run >> 11) & 7u) + 1u;
                                    uint32_t m[8];
#pragma unroll
                                    for (int i = 0; i < 8; i++) m[i] = ((rows8 >> i) & 1u) ? 0u : 0xffffffffu;
                                    const uint32_t n = len * TILE;
                                    const uint32_t idesc = (1u << 4) | ((n >> 3) << 17) | ((256u >> 4) << 24);
                                    const uint64_t db = desc0 + (uint64_t)((b_slot + c0 * (TILE_BYTES / 2)) >> 4);
                                    const uint32_t dcol = dbase + c0 * TILE;
                                    g_umma_masked(dcol, da, db, idesc, m);
                                    g_umma_masked(dcol, da + 16u, db + 16u, idesc, m);
                                }
                            }
                            g_umma_commit(smem_u32(&ctrl->empty[s]));
                        }
                        __syncwarp();
                        slot++;
                    }
                    if (!ok) break;
                    if (lane == 0) g_umma_commit(smem_u32(&ctrl->tmem_full[buf]));
                    acc_iter++;
                }
                if (*abort_flag && lane == 0) {
                    g_umma_commit(smem_u32(&ctrl->drain));
                    const unsigned long long t0 = global_ns();
                    while (!mbar_try_wait(smem_u32(&ctrl->drain), 0) && global_ns() - t0 < WAIT_LIMIT_NS) {}
                }
            } else {
                // -------------------------------------------------------------- other block: relay "my copies landed"
                for (int u = cluster_id; u < n_units && ok; u += n_clusters) {
                    int pr, mj;
                    unit_at(u, &pr, &mj);
                    if (rec_counts[pr * mj_n + mj] == 0) continue;
                    for (bool last = false; !last;) {
                        const uint32_t s = slot % G_STAGES, ph = (slot / G_STAGES) & 1u;
                        ok = wait_bounded(smem_u32(&ctrl->full[s]), ph, abort_flag, err, GERR_FULL);
                        if (!ok) break;
                        last = ctrl->stage_last[s] != 0u;
                        g_mbar_arrive_remote(smem_u32(&ctrl->full[s]), 0u);
                        slot++;
                    }
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue (4 warps per block)
        const uint32_t q = (uint32_t)(warp & 3);
        const int e = threadIdx.x - 64;
        uint8_t *epi_tile = smem + G_STAGES * G_STAGE_BYTES + G_CTRL_BYTES + (warp - 2) * EPI_WARP_BYTES;
        uint32_t acc_iter = 0;
        unsigned int done = 0;
        bool ok = true;
        for (int u = cluster_id; u < n_units && ok; u += n_clusters) {
            int pr, mj;
            unit_at(u, &pr, &mj);
            const int mi = 2 * pr + (int)rank;
            done++;
            if (rec_counts[pr * mj_n + mj] == 0) {
                // nothing survives in either macro tile: zeros, unless C was cleared beforehand
                if (!c_zeroed) {
                    // zero_fill (see gated_multiply.cu): 128 threads, 64 columns of float4 each pass
                    const int col = mj * (MT_C * TILE) + (e & 63) * 4;
                    if (col < n_tiles * TILE) {
                        const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
                        for (int rr = (e >> 6); rr < MT_R * TILE; rr += 2) {
                            const int row = mi * (MT_R * TILE) + rr;
                            if (row < rows_total) __stcs(reinterpret_cast<float4 *>(c + (int64_t)row * ldc + col), z);
                        }
                    }
                }
                continue;
            }
            const uint32_t buf = acc_iter & 1u;
            ok = wait_bounded(smem_u32(&ctrl->tmem_full[buf]), (acc_iter >> 1) & 1u, abort_flag, err, GERR_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int row = mi * (MT_R * TILE) + (int)q * TILE + lane;
            const bool row_ok = row < rows_total;
            // this block's own macro tile may be one without steps while its partner's has some: with C cleared
            // beforehand (or holding a partial result) it is left alone, but the accumulator is still cleared
            const bool write = !(c_zeroed && step_count_of(step_counts[mi * mj_n + mj]) == 0);
            float *cblock = c + (int64_t)(row - lane) * ldc + (int64_t)mj * (MT_C * TILE);
#pragma unroll 1
            for (int cc = 0; cc < MT_C; cc++) {
                const uint32_t taddr = tmem_base + ((q * 32u) << 16) + buf * G_ACC_COLS + (uint32_t)cc * TILE;
                uint32_t v[32];
                tmem_ld32(taddr, v);
                tmem_wait_ld();
                tmem_st32_zero(taddr);
                if (write && row_ok && mj * MT_C + cc < n_tiles)
                    store_block_coalesced(epi_tile, v, cblock + cc * TILE, ldc, lane, accumulate, acc_scale);
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) g_mbar_arrive_remote(smem_u32(&ctrl->tmem_empty[buf]), 0u);   // the leader's barrier
            acc_iter++;
        }
        if (warp == 2 && lane == 0 && done) atomicAdd(&sc->pair_done, done);            // macro tiles taken care of
    }

    tc_fence_before();
    __syncthreads();
    g_cluster_sync_all();                     // nobody frees tensor memory while the other block may still use it
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(G_TMEM_COLS)
                     : "memory");
    }
}

size_t gated_multiply_gpair_scratch_bytes(int row_tiles, int k_tiles, int n_tiles)
{
    const size_t units = (size_t)(ceil_div(row_tiles, MT_R) / 2) * ceil_div(n_tiles, MT_C);
    return units * ((size_t)k_tiles * sizeof(uint4) + 16);
}

int gated_multiply_gpair_launch(const void *d_half_a, const void *d_half_b, const float *d_norm_a, const float *d_norm_b,
                                float tau, const void *d_chunk_max, const int32_t *d_step_counts, void *d_scratch,
                                bool build_records, spamm_list_scalars *d_scalars, int row_tiles, int k_tiles,
                                int n_tiles, float *d_c, int64_t ldc, int mode, cudaStream_t stream)
{
    const int mi_n = ceil_div(row_tiles, MT_R), mj_n = ceil_div(n_tiles, MT_C);
    if (mi_n < 2 || mj_n == 0 || k_tiles == 0) return SPAMM_OK;
    if (!d_scratch || !d_norm_a || !d_norm_b || !d_chunk_max || (reinterpret_cast<uintptr_t>(d_scratch) & 15))
        return SPAMM_ERR_INVALID;
    static int sm_count_of[64] = {};        // per device, written once with the same value by whoever comes first
    int dev = 0;
    SPAMM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SPAMM_ERR_UNSUPPORTED;
    if (sm_count_of[dev] == 0) {
        int sms = 0;
        SPAMM_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        SPAMM_CUDA_TRY(cudaFuncSetAttribute(gated_multiply_gpair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            G_SMEM_BYTES));
        sm_count_of[dev] = sms;
    }
    const int64_t n_units = (int64_t)(mi_n / 2) * mj_n;
    // scratch: the records of every unit (k_tiles each), then the units' record counts
    uint4 *recs = static_cast<uint4 *>(d_scratch);
    int32_t *rec_counts = reinterpret_cast<int32_t *>(recs + n_units * k_tiles);
    if (build_records) {
        const int kc_n = ceil_div(k_tiles, 32);
        const float *amax = static_cast<const float *>(d_chunk_max);
        const float *bmax = amax + (size_t)mi_n * kc_n;
        pair_runs_kernel<<<(unsigned)((n_units + 3) / 4), 128, 0, stream>>>(d_norm_a, d_norm_b, row_tiles, k_tiles, n_tiles,
                                                                           tau, amax, bmax, recs, rec_counts);
    }
    int clusters = sm_count_of[dev] / 2;
    if (clusters > n_units) clusters = (int)n_units;
    if (clusters < 1) return SPAMM_OK;
    gated_multiply_gpair_kernel<<<2 * clusters, G_THREADS, G_SMEM_BYTES, stream>>>(
        static_cast<const uint8_t *>(d_half_a), static_cast<const uint8_t *>(d_half_b), d_step_counts, recs, rec_counts,
        d_scalars, row_tiles, k_tiles, n_tiles, d_c, ldc, mode);
    SPAMM_CUDA_TRY(cudaGetLastError());
    return SPAMM_OK;
}

// Loads this file's kernels onto the current device now (kernels are loaded lazily, at their first launch, and such
// a load can wait for kernels that are running; a kernel of one GPU that waits for a peer must not find the peer stuck
// in the load of a kernel it needs).
int preload_multiply_gpair()
{
    cudaFuncAttributes a;
    SPAMM_CUDA_TRY(cudaFuncGetAttributes(&a, pair_runs_kernel));
    SPAMM_CUDA_TRY(cudaFuncGetAttributes(&a, gated_multiply_gpair_kernel));
    return SPAMM_OK;
}

}  // namespace spamm
