// Gated block multiply on the 5th-generation tensor cores (tcgen05 + tensor memory), sm_100a only.
//
// Stands in for get_C_FP16_B32 (reference cuSpAMM.cu:336-391): for every C tile, the sum over the surviving k of
// half(A(i,k)) * half(B(k,j)) with float accumulation; tiles with an empty list are written as zeros
// (cuSpAMM.cu:300,391).  The reference runs one 128-thread block per 32x32 C tile with 16x16x16 WMMA fragments.
// Here a persistent block per SM walks macro tiles of 128 x 256 C elements (4 x 8 tiles):
//
//   warp 0      scheduler + producer: claims macro tiles from a device-wide work counter (those with steps first),
//               publishes them to the other warps through a small ring, then reads the macro tile's step list 32
//               steps at a time, ONE STEP PER LANE: slot and stage boundaries, the copy extents of every slot and
//               the list of multiplies every step stands for come out of ballots, shuffles and one prefix sum; the
//               first lane of a slot issues the slot's bulk copies (cp.async.bulk, completion on an mbarrier) of
//               the packed half tiles into a ring of shared-memory stages, every lane writes the ready-made
//               multiplies of its step (instruction descriptor, operand descriptors, accumulator column, row set)
//               into the stage's control block; the steps of one k share their copies;
//   warp 1      follows the stages and issues what the control block lists: tcgen05.mma (M=128, N=32*run, K=16),
//               two per entry; the step's row set is the instruction's disable-output-lane mask, so tile rows
//               that did not survive are not touched -- no product outside the lists is ever added.  The warp
//               does no decoding: one thread that decodes steps AND issues was the limit of this kernel on long
//               half-full lists (the loop over a stage's entries runs in all lanes, lane 0 issues);
//   warps 6-9   fillers: when few macro tiles have steps, write the all-zero macro tiles from the start, in
//               parallel with the pipeline;
//   warps 2-5   epilogue: read the 128x256 float accumulator from tensor memory (tcgen05.ld), turn it through a
//               small shared-memory tile so that whole rows are stored to C, clear it for the next macro tile;
//               macro tiles without any step are written as zeros directly.
//
// Two accumulators (2 x 256 of the 512 tensor-memory columns) let the epilogue of one macro tile overlap the
// multiplies of the next.  Two options serve the callers: macro tiles without steps can be left alone (C was cleared
// beforehand, or holds a partial result), and the products can be added to C instead of replacing it (the second and
// third pass of the split-precision mode).  Every wait on an mbarrier is bounded in time; when one runs out the
// block sets the error word, drains its copies and multiplies, frees its tensor memory and returns.
#include <cstddef>

#include "tc_utils.cuh"

namespace spamm {

// A stage of the ring holds SPS slots; a slot holds the operands of ONE k of one macro tile (8 KiB of A, 16 KiB of B)
// and up to GSTEPS steps of that k (steps of the same k differ only in which rows and columns take part, so they
// share the slab copies; their row sets are nested, so a k has at most 4 steps).  Both the producer and the
// issuing thread pay a fixed price per stage (barrier wait, arrive or commit), so several k share a stage: with one
// k per stage the lattice workload takes 30 ms instead of 22.
#ifndef SPAMM_SPS
#define SPAMM_SPS 2
#endif
constexpr int SPS = SPAMM_SPS;
constexpr int STAGE_BYTES = SPS * (A_SLAB_BYTES + B_SLAB_BYTES);   // 24 KiB per step
#ifndef SPAMM_STAGES
#define SPAMM_STAGES (8 / SPAMM_SPS)
#endif
constexpr int STAGES = SPAMM_STAGES;
constexpr int GSTEPS = 4;                                    // steps of one k that share a stage slot (more: next slot)
constexpr int GM_THREADS = 320;                            // producer, MMA, 4 epilogue warps, 4 filler warps
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t ACC_COLS = MT_C * TILE;                  // 256
constexpr int MAX_OPS = SPS * GSTEPS * 4;                   // a step has at most 4 runs of adjacent columns
constexpr int SMEM_CTRL_BYTES = 640 + STAGES * MAX_OPS * 16;
constexpr int SCHED = 4;                                    // depth of the ring of scheduled macro tiles
constexpr int GM_SMEM_BYTES = STAGES * STAGE_BYTES + SMEM_CTRL_BYTES + 4 * EPI_WARP_BYTES + 128;

struct Ctrl {
    unsigned long long full[STAGES];
    unsigned long long empty[STAGES];
    unsigned long long tmem_full[2];
    unsigned long long tmem_empty[2];
    unsigned long long drain;
    unsigned long long sched_full[SCHED];
    unsigned long long sched_empty[SCHED];
    int32_t filler_claim[2][4];
    uint32_t filler_base[2];
    int32_t tile_slot[SCHED];
    int32_t tile_cnt[SCHED];
    alignas(16) uint4 ops[STAGES][MAX_OPS];                     // per stage: the multiplies to issue, ready-made
    uint32_t n_ops[STAGES];
    uint32_t stage_last[STAGES];                               // this stage ends its macro tile
    uint32_t tmem_base;
    uint32_t abort_flag;
};
static_assert(sizeof(Ctrl) <= SMEM_CTRL_BYTES, "control block too large");

// Writes one macro tile of C as zeros with `nthreads` threads (a multiple of 64); `t` is the caller's index among them.
__device__ __forceinline__ void zero_fill_macro_tile(float *__restrict__ c, int64_t ldc, int mi, int mj, int rows_total,
                                                     int cols_total, int t, int nthreads)
{
    const int col = mj * (MT_C * TILE) + (t & 63) * 4;
    if (col >= cols_total) return;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    const int rows_per_pass = nthreads >> 6;
    const int row0 = mi * (MT_R * TILE) + (t >> 6);
#pragma unroll 4
    for (int rr = 0; rr < MT_R * TILE; rr += rows_per_pass) {
        const int row = row0 + rr;
        if (row < rows_total) __stcs(reinterpret_cast<float4 *>(c + (int64_t)row * ldc + col), z);
    }
}

enum {
    ERR_WAIT_EMPTY = 1, ERR_WAIT_FULL = 2, ERR_WAIT_TMEM_EMPTY = 3, ERR_WAIT_TMEM_FULL = 4, ERR_WAIT_DRAIN = 5,
    ERR_WAIT_SCHED_EMPTY = 6, ERR_WAIT_SCHED_FULL = 7
};

__global__ void __launch_bounds__(GM_THREADS, 1)
gated_multiply_kernel(const uint8_t *__restrict__ half_a, const uint8_t *__restrict__ half_b,
                      const uint32_t *__restrict__ steps, const int32_t *__restrict__ step_counts,
                      const int32_t *__restrict__ order, const int32_t *__restrict__ busy_list,
                      spamm_list_scalars *__restrict__ sc, int row_tiles, int k_tiles, int n_tiles,
                      float *__restrict__ c, int64_t ldc, int pairs_launched, int mode)
{
    const bool c_zeroed = (mode & GM_C_ZEROED) != 0;        // leave macro tiles without steps alone
    const bool accumulate = (mode & GM_ACCUMULATE) != 0;    // add to C
    const float acc_scale = (mode & GM_LOW_OPERAND) ? 1.0f / SPLIT_LOW_SCALE : 1.0f;
    extern __shared__ uint8_t smem_raw[];
    // stage data first (128-byte aligned), control block after it
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    Ctrl *ctrl = reinterpret_cast<Ctrl *>(smem + STAGES * STAGE_BYTES);
    volatile uint32_t *abort_flag = &ctrl->abort_flag;
    int32_t *err = &sc->error;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mi_n = (row_tiles + MT_R - 1) / MT_R;
    const int mj_n = (n_tiles + MT_C - 1) / MT_C;
    const unsigned int n_mt = (unsigned int)(mi_n * mj_n);
    const int64_t cap = (int64_t)STEP_CAP_PER_K * k_tiles;
    const int rows_total = row_tiles * TILE;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(smem_u32(&ctrl->full[s]), 1);
            mbar_init(smem_u32(&ctrl->empty[s]), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(smem_u32(&ctrl->tmem_full[b]), 1);
            mbar_init(smem_u32(&ctrl->tmem_empty[b]), 128);
        }
        for (int d = 0; d < SCHED; d++) {
            mbar_init(smem_u32(&ctrl->sched_full[d]), 1);
            mbar_init(smem_u32(&ctrl->sched_empty[d]), 5);   // the MMA thread + one lane of each epilogue warp
        }
        mbar_init(smem_u32(&ctrl->drain), 1);
        ctrl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&ctrl->tmem_base)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctrl->tmem_base;

    if (warp >= 2) {
        // clear both accumulators: every multiply accumulates
        const uint32_t q = (uint32_t)(warp & 3);
        for (uint32_t col = 0; col < TMEM_COLS; col += 32) tmem_st32_zero(tmem_base + ((q * 32u) << 16) + col);
        tmem_wait_st();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    // Dense macro tiles that have a dense vertical neighbour belong to the paired (two-SM) kernel, which runs first
    // on the stream whenever at least half of the macro tiles are dense; this kernel leaves them alone.  When the
    // gated two-SM kernel ran instead, it took every pair of macro-tile rows, and only the last row of an odd count
    // is left for this one.
    const bool gated_pairs = pairs_launched == GM_PAIRS_GATED && mi_n >= 2;
    const bool pair_active = gated_pairs || (pairs_launched == GM_PAIRS_DENSE && mi_n >= 2 && sc->dense_count * 2u >= n_mt);
    auto pair_owned = [&](int mt, int raw_count) -> bool {
        if (gated_pairs) return mt / mj_n < (mi_n & ~1);
        if (!pair_active || !step_list_dense(raw_count)) return false;
        const int mi = mt / mj_n, partner = mi ^ 1;
        return partner < mi_n && step_list_dense(step_counts[partner * mj_n + (mt % mj_n)]);
    };
    const bool nothing_left = pair_active && sc->pair_done == n_mt;

    if (warp == 0) {
        // ------------------------------------------------------------------ scheduler + producer
        // Work queue: macro tiles that have steps come first (they take several times longer than a macro tile
        // that is only written as zeros, so starting them first keeps the tail short), then all others in the
        // given order.  When most macro tiles have steps the first phase is skipped and the given order, which is
        // chosen for operand reuse in L2, is used for everything.
        const unsigned int busy_n = sc->busy_count;
        const bool use_busy = busy_n * 4u <= n_mt;
        // zero-only macro tiles are claimed four at a time; so are macro tiles with short lists when there are many per
        // SM (a claim is a chain of three dependent reads before the first copy can be issued; long lists keep the
        // one-by-one order, which is the one chosen for operand reuse in L2)
        const bool short_lists = sc->survivors < 256ull * n_mt && n_mt >= 16u * gridDim.x;
        const unsigned int chunk = (use_busy || short_lists) ? 4u : 1u;
        int phase = use_busy ? 1 : 2;
        int cand_mt = -1, cand_cnt = 0;                    // per lane: candidates of the claimed chunk
        uint32_t pending = 0;                              // lanes whose candidate is still to be scheduled
        uint32_t slot = 0, sidx = 0;
        bool ok = true;
        while (ok) {
            int mt = -1, cnt = 0;
            if (nothing_left) {
                // every macro tile was multiplied by the paired kernel: publish the end marker and stop
            } else if (phase == 1) {
                unsigned int ti = 0;
                if (lane == 0) ti = atomicAdd(&sc->queue_busy, 1u);
                ti = __shfl_sync(0xffffffffu, ti, 0);
                if (ti >= busy_n) {
                    phase = 2;
                    continue;
                }
                mt = busy_list[ti];
                cnt = step_counts[mt];
                if (pair_owned(mt, cnt)) continue;
                cnt = step_count_of(cnt);
            } else {
                // with C cleared beforehand only macro tiles that have steps are written: none are left in this phase
                // when the first phase has handled them
                bool exhausted = c_zeroed && use_busy;
                while (!pending && !exhausted) {
                    unsigned int p0 = 0;
                    if (lane == 0) p0 = atomicAdd(&sc->queue_all, chunk);
                    p0 = __shfl_sync(0xffffffffu, p0, 0);
                    if (p0 >= n_mt) {
                        exhausted = true;
                        break;
                    }
                    cand_mt = -1;
                    if ((unsigned int)lane < chunk && p0 + lane < n_mt) {
                        cand_mt = order ? order[p0 + lane] : (int)(p0 + lane);
                        const int raw = step_counts[cand_mt];
                        cand_cnt = step_count_of(raw);
                        if (use_busy && cand_cnt > 0) cand_mt = -1;     // already handled in the first phase
                        else if (c_zeroed && cand_cnt == 0) cand_mt = -1;   // already zero
                        else if (pair_owned(cand_mt, raw)) cand_mt = -1;
                    }
                    pending = __ballot_sync(0xffffffffu, cand_mt >= 0);
                }
                if (!exhausted) {
                    const int src = __ffs(pending) - 1;
                    pending &= pending - 1;
                    mt = __shfl_sync(0xffffffffu, cand_mt, src);
                    cnt = __shfl_sync(0xffffffffu, cand_cnt, src);
                }
            }
            if (lane == 0) {
                const uint32_t d = sidx % SCHED, ph = (sidx / SCHED) & 1u;
                ok = wait_bounded(smem_u32(&ctrl->sched_empty[d]), ph ^ 1u, abort_flag, err, ERR_WAIT_SCHED_EMPTY);
                if (ok) {
                    ctrl->tile_slot[d] = mt;
                    ctrl->tile_cnt[d] = cnt;
                    mbar_arrive(smem_u32(&ctrl->sched_full[d]));
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            sidx++;
            if (mt < 0 || !ok) break;
            if (cnt == 0) continue;

            const int mi = mt / mj_n, mj = mt % mj_n;
            const uint32_t *list = steps + (int64_t)mt * cap;
            const uint8_t *a_base = half_a + (int64_t)mi * k_tiles * A_SLAB_BYTES;
            const uint8_t *b_base = half_b + (int64_t)mj * B_SLAB_BYTES;
            // The whole warp assembles stages, 32 steps at a time, one step per lane: consecutive steps with the same
            // k form a slot (they share one copy of the A slab and one of the B columns they span), SPS slots a
            // stage.  Slot boundaries, the slots' unions of rows and columns and their copy extents come from
            // ballots and shuffles; the first lane of a slot issues the slot's copies, every lane writes the
            // multiplies of its own step into the stage's list; lane 0 waits for the stage to be free before and
            // arrives on its barrier after.
            uint32_t cur = (lane < cnt) ? __ldg(list + lane) : 0u;
            uint32_t nxt = (32 + lane < cnt) ? __ldg(list + 32 + lane) : 0u;
            for (int base = 0; base < cnt && ok;) {
                const int n_here = min(32, cnt - base);
                const bool more = base + 32 < cnt;
                const bool valid = lane < n_here;
                const uint32_t k = step_k(cur);
                const uint32_t k_prev = __shfl_up_sync(0xffffffffu, k, 1);
                const uint32_t k_heads = __ballot_sync(0xffffffffu, valid && (lane == 0 || k != k_prev));
                // position inside the run of equal k; a run longer than GSTEPS goes on in a further slot
                const int run_start = 31 - __clz(k_heads & (0xffffffffu >> (31 - lane)));
                const bool head = valid && (((lane - run_start) % GSTEPS) == 0);
                uint32_t heads = __ballot_sync(0xffffffffu, head);
                int used = n_here;
                if (more) {
                    // the last slot may go on in the next batch: leave it (and one more, to fill whole stages) for then
                    int n_sl = __popc(heads);
                    int drop = (n_sl >= 2) ? 1 : 0;
                    if (drop && ((n_sl - drop) % SPS) != 0 && n_sl - drop > 1) drop++;
                    for (int x = 0; x < drop; x++) {
                        const int hl = 31 - __clz(heads);
                        used = hl;
                        heads &= ~(1u << hl);
                    }
                }
                const bool last_batch = !more || base + used >= cnt;
                const int n_slots = __popc(heads);
                const int slot_idx = __popc(heads & (0xffffffffu >> (31 - lane))) - 1;      // of this lane's step
                // steps of this lane's slot, gathered into its first lane
                const uint32_t ends = (heads | (used < 32 ? (0xffffffffu << used) : 0u));
                uint32_t w1 = __shfl_down_sync(0xffffffffu, cur, 1);
                uint32_t w2 = __shfl_down_sync(0xffffffffu, cur, 2);
                uint32_t w3 = __shfl_down_sync(0xffffffffu, cur, 3);
                // number of steps in a slot that starts here: distance to the next slot start (or the end of the batch)
                const uint32_t after = (lane < 31) ? (ends >> (lane + 1)) : 0u;
                const int dist = after ? __ffs(after) : (32 - lane);
                if (dist < 2) w1 = 0u;
                if (dist < 3) w2 = 0u;
                if (dist < 4) w3 = 0u;
                const bool is_head = (heads >> lane) & 1u;
                const uint32_t all = cur | w1 | w2 | w3;
                const uint32_t rows_u = step_rows(all), cols_u = step_cols(all);
                const uint32_t a_bytes = (__popc(rows_u) == 1) ? TILE_BYTES : A_SLAB_BYTES;
                const uint32_t b_first = (uint32_t)(__ffs(cols_u) - 1);
                const uint32_t b_len = (uint32_t)(32 - __clz(cols_u)) - b_first;
                const int n_stages = (n_slots + SPS - 1) / SPS;
                // two slots of one stage whose k are neighbours and that need whole slabs of A: the slabs are
                // neighbours in memory too, and the first slot's lane fetches both with one copy
                const int next_head = (lane + dist) & 31;
                const uint32_t k_nh = __shfl_sync(0xffffffffu, k, next_head);
                const uint32_t ab_nh = __shfl_sync(0xffffffffu, a_bytes, next_head);
                const bool merge_next = SPS == 2 && is_head && (slot_idx % SPS) == 0 && slot_idx + 1 < n_slots &&
                                        a_bytes == A_SLAB_BYTES && ab_nh == A_SLAB_BYTES && k_nh == k + 1u;
                const uint32_t before = heads & ((1u << lane) - 1u);
                const int prev_head = before ? (31 - __clz(before)) : 0;
                const bool merged_prev = __shfl_sync(0xffffffffu, merge_next ? 1 : 0, prev_head) != 0 && is_head &&
                                         (slot_idx % SPS) == 1;
                // every lane turns its step into the multiplies it stands for: one per run of adjacent columns
                const bool in_use = lane < used;
                const uint32_t my_rows = step_rows(cur), my_cols = in_use ? step_cols(cur) : 0u;
                const int n_runs = __popc(my_cols & ~(my_cols << 1));
                int incl = n_runs;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const int tt = __shfl_up_sync(0xffffffffu, incl, d);
                    if (lane >= d) incl += tt;
                }
                const int my_stage = slot_idx / SPS;
                const uint32_t stage_heads = __ballot_sync(0xffffffffu, is_head && (slot_idx % SPS) == 0);
                const int st_first = 31 - __clz(stage_heads & (0xffffffffu >> (31 - lane)));
                const uint32_t st_ends = stage_heads | (used < 32 ? (0xffffffffu << used) : 0u);
                const uint32_t st_after = (lane < 31) ? (st_ends >> (lane + 1)) : 0u;
                const int st_last = st_after ? (lane + __ffs(st_after) - 1) : 31;
                const int excl_first = __shfl_sync(0xffffffffu, incl - n_runs, st_first & 31);
                const int incl_last = __shfl_sync(0xffffffffu, incl, st_last & 31);
                const int my_pos = incl - n_runs - excl_first;
                const int stage_total = incl_last - excl_first;      // meaningful in the first lane of a stage
                for (int j = 0; j < n_stages && ok; j++) {
                    const uint32_t s = slot % STAGES, ph = (slot / STAGES) & 1u;
                    if (lane == 0) ok = wait_bounded(smem_u32(&ctrl->empty[s]), ph ^ 1u, abort_flag, err, ERR_WAIT_EMPTY);
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                    const uint32_t bar = smem_u32(&ctrl->full[s]);
                    if (in_use && my_stage == j) {
                        const int t = slot_idx % SPS;
                        const uint32_t a_stage = smem_u32(smem + s * STAGE_BYTES);
                        const uint32_t b_stage = a_stage + SPS * A_SLAB_BYTES;
                        const uint32_t a_addr = a_stage + t * A_SLAB_BYTES, b_addr = b_stage + t * B_SLAB_BYTES;
                        if (is_head) {
                            const uint8_t *a_src = a_base + (int64_t)k * A_SLAB_BYTES;
                            const uint8_t *b_src = b_base + (int64_t)k * mj_n * B_SLAB_BYTES;
                            mbar_expect_tx(bar, (merged_prev ? 0u : a_bytes) + (merge_next ? A_SLAB_BYTES : 0u) +
                                                    b_len * TILE_BYTES);
                            if (merged_prev) {
                            } else if (a_bytes == A_SLAB_BYTES) {
                                bulk_g2s(a_addr, a_src, merge_next ? 2 * A_SLAB_BYTES : A_SLAB_BYTES, bar);
                            } else {
                                const uint32_t q = (uint32_t)(__ffs(rows_u) - 1);
                                bulk_g2s(a_addr + q * TILE_BYTES, a_src + q * TILE_BYTES, TILE_BYTES, bar);
                            }
                            bulk_g2s(b_addr + b_first * TILE_BYTES, b_src + b_first * TILE_BYTES, b_len * TILE_BYTES, bar);
                        }
                        uint32_t rest = my_cols;
                        int pos = my_pos;
                        while (rest) {
                            const int c0 = __ffs(rest) - 1;
                            const int len = __ffs(~(rest >> c0)) - 1;
                            const uint32_t n = (uint32_t)len * TILE;
                            const uint32_t idesc = (1u << 4) | ((n >> 3) << 17) | ((128u >> 4) << 24);
                            ctrl->ops[s][pos++] = make_uint4(idesc, (b_addr + (uint32_t)c0 * TILE_BYTES) >> 4,
                                                             (uint32_t)c0 * TILE, my_rows | ((a_addr >> 4) << 4));
                            rest &= ~(((1u << len) - 1u) << c0);
                        }
                        if (is_head && t == 0) {
                            ctrl->n_ops[s] = (uint32_t)stage_total;
                            ctrl->stage_last[s] = (last_batch && j == n_stages - 1) ? 1u : 0u;
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar);
                    slot++;
                }
                // the next 32 steps start `used` further on: part of them is already here
                base += used;
                const uint32_t from_cur = __shfl_sync(0xffffffffu, cur, (lane + used) & 31);
                const uint32_t from_nxt = __shfl_sync(0xffffffffu, nxt, (lane + used) & 31);
                cur = (lane + used < 32) ? from_cur : from_nxt;
                nxt = (base + 32 + lane < cnt) ? __ldg(list + base + 32 + lane) : 0u;
                if (used == 32) { /* cur is the old nxt entirely: handled by the select above */ }
            }
        }
        if (lane == 0 && *abort_flag) {
            // make sure every copy this block issued has landed before the block can exit
            const uint32_t first = slot > STAGES ? slot - STAGES : 0;
            for (uint32_t sl = first; sl < slot; sl++) {
                const uint32_t s = sl % STAGES, ph = (sl / STAGES) & 1u;
                const unsigned long long t0 = global_ns();
                while (!mbar_try_wait(smem_u32(&ctrl->full[s]), ph) && global_ns() - t0 < WAIT_LIMIT_NS) {}
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ tensor-core issue
        // Every lane runs the loop (waits, addresses, descriptors are then the same in all lanes of the warp, which
        // measurably shortens the issue path); lane 0 alone issues the multiplies, commits and arrives.
        {
            uint32_t slot = 0, acc_iter = 0;
            bool ok = true;
            // descriptor without the start address: adding (address >> 4) completes it, +16 is the second K=16 half
            const uint64_t desc0 = smem_desc(0);
            for (uint32_t sidx = 0; ok; sidx++) {
                const uint32_t d = sidx % SCHED, sph = (sidx / SCHED) & 1u;
                ok = wait_bounded(smem_u32(&ctrl->sched_full[d]), sph, abort_flag, err, ERR_WAIT_SCHED_FULL);
                if (!ok) break;
                const int mt = ctrl->tile_slot[d];
                const int cnt = ctrl->tile_cnt[d];
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ctrl->sched_empty[d]));
                if (mt < 0) break;
                if (cnt == 0) continue;
                const uint32_t buf = acc_iter & 1u;
                ok = wait_bounded(smem_u32(&ctrl->tmem_empty[buf]), ((acc_iter >> 1) & 1u) ^ 1u, abort_flag, err,
                                  ERR_WAIT_TMEM_EMPTY);
                if (!ok) break;
                tc_fence_after();
                const uint32_t dbase = tmem_base + buf * ACC_COLS;
                for (bool last = false; !last;) {
                    const uint32_t s = slot % STAGES, ph = (slot / STAGES) & 1u;
                    ok = wait_bounded(smem_u32(&ctrl->full[s]), ph, abort_flag, err, ERR_WAIT_FULL);
                    if (!ok) break;
                    tc_fence_after();
                    last = ctrl->stage_last[s] != 0u;
                    const uint32_t n_ops = ctrl->n_ops[s];
                    __syncwarp();       // every lane has read the stage's control words before lane 0 can release it
                    {
                        // every lane follows the list of multiplies (the values are the same in all lanes); lane 0 issues
                        uint4 op = ctrl->ops[s][0];
#pragma unroll 1
                        for (uint32_t i = 0; i < n_ops; i++) {
                            const uint4 nx = ctrl->ops[s][min(i + 1u, (uint32_t)MAX_OPS - 1u)];
                            const uint32_t rows = op.w & 0xfu;
                            const uint64_t da = desc0 + (uint64_t)(op.w >> 4), db = desc0 + (uint64_t)op.y;
                            const uint32_t dcol = dbase + op.z;
                            const uint32_t m0 = (rows & 1u) ? 0u : 0xffffffffu, m1 = (rows & 2u) ? 0u : 0xffffffffu;
                            const uint32_t m2 = (rows & 4u) ? 0u : 0xffffffffu, m3 = (rows & 8u) ? 0u : 0xffffffffu;
                            if (lane == 0) {
                                umma_f16(dcol, da, db, op.x, m0, m1, m2, m3);
                                umma_f16(dcol, da + 16u, db + 16u, op.x, m0, m1, m2, m3);
                            }
                            op = nx;
                        }
                        if (lane == 0) umma_commit(smem_u32(&ctrl->empty[s]));
                    }
                    __syncwarp();
                    slot++;
                }
                if (!ok) break;
                if (lane == 0) umma_commit(smem_u32(&ctrl->tmem_full[buf]));
                acc_iter++;
            }
            if (*abort_flag && lane == 0) {
                // wait for the multiplies already issued before tensor memory is freed
                umma_commit(smem_u32(&ctrl->drain));
                const unsigned long long t0 = global_ns();
                while (!mbar_try_wait(smem_u32(&ctrl->drain), 0) && global_ns() - t0 < WAIT_LIMIT_NS) {}
            }
        }
        __syncwarp();
    } else if (warp >= 6) {
        // ------------------------------------------------------------------ fillers (4 warps)
        // While the pipeline above works through the macro tiles that have steps, these warps already write the
        // macro tiles that are all zeros, so the memory system is busy from the start.  Every two warps form a
        // group of 64 threads that claims four macro tiles at a time from the same counter the scheduler uses for
        // its second phase; the next claim is issued before the current tiles are written.
        const unsigned int busy_n = sc->busy_count;
        if (busy_n * 4u <= n_mt && !nothing_left && !c_zeroed) {
            const int pair_lane = threadIdx.x & 63;          // index inside the group of two warps
            const uint32_t bar_id = 1u + (uint32_t)((warp - 6) >> 1);
            volatile int32_t *claim = &ctrl->filler_claim[(warp - 6) >> 1][0];
            auto claim_chunk = [&]() {
                // first four threads of the group: one candidate each
                if (pair_lane == 0) ctrl->filler_base[(warp - 6) >> 1] = atomicAdd(&sc->queue_all, 4u);
                asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");
                const unsigned int p0 = ctrl->filler_base[(warp - 6) >> 1];
                if (pair_lane < 4) {
                    int m = -1;
                    if (p0 + pair_lane < n_mt) {
                        m = order ? order[p0 + pair_lane] : (int)(p0 + pair_lane);
                        if (step_count_of(step_counts[m]) > 0) m = -1;      // handled by the pipeline
                    }
                    claim[pair_lane] = m;
                }
                asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");
                return p0 < n_mt;
            };
            bool more = claim_chunk();
            while (more) {
                int m[4];
#pragma unroll
                for (int i = 0; i < 4; i++) m[i] = claim[i];
                asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");   // everyone has read the claim
                more = claim_chunk();
#pragma unroll
                for (int i = 0; i < 4; i++)
                    if (m[i] >= 0)
                        zero_fill_macro_tile(c, ldc, m[i] / mj_n, m[i] % mj_n, rows_total, n_tiles * TILE, pair_lane,
                                             64);
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (4 warps)
        const uint32_t q = (uint32_t)(warp & 3);
        const int e = threadIdx.x - 64;
        uint8_t *epi_tile = smem + STAGES * STAGE_BYTES + SMEM_CTRL_BYTES + (warp - 2) * EPI_WARP_BYTES;
        uint32_t acc_iter = 0;
        bool ok = true;
        for (uint32_t sidx = 0; ok; sidx++) {
            const uint32_t d = sidx % SCHED, sph = (sidx / SCHED) & 1u;
            ok = wait_bounded(smem_u32(&ctrl->sched_full[d]), sph, abort_flag, err, ERR_WAIT_SCHED_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const int mt = ctrl->tile_slot[d];
            const int cnt = ctrl->tile_cnt[d];
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctrl->sched_empty[d]));
            if (mt < 0) break;
            const int mi = mt / mj_n, mj = mt % mj_n;
            if (cnt == 0) {
                zero_fill_macro_tile(c, ldc, mi, mj, rows_total, n_tiles * TILE, e, 128);
                continue;
            }
            const uint32_t buf = acc_iter & 1u;
            ok = wait_bounded(smem_u32(&ctrl->tmem_full[buf]), (acc_iter >> 1) & 1u, abort_flag, err,
                              ERR_WAIT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int row = mi * (MT_R * TILE) + (int)q * TILE + lane;
            const bool row_ok = row < rows_total;
            // first row of this warp's 32-row block of C, first column of the macro tile
            float *cblock = c + (int64_t)(row - lane) * ldc + (int64_t)mj * (MT_C * TILE);
            // two register sets: the load of the next block of 32 columns is under way while the current one is stored
            const uint32_t tacc = tmem_base + ((q * 32u) << 16) + buf * ACC_COLS;
            uint32_t v0[32], v1[32];
            tmem_ld32(tacc, v0);
#pragma unroll 1
            for (int cc = 0; cc < MT_C; cc += 2) {
                tmem_wait_ld();
                tmem_ld32(tacc + (uint32_t)(cc + 1) * TILE, v1);
                tmem_st32_zero(tacc + (uint32_t)cc * TILE);
                if (row_ok && mj * MT_C + cc < n_tiles)
                    store_block_coalesced(epi_tile, v0, cblock + cc * TILE, ldc, lane, accumulate, acc_scale);
                tmem_wait_ld();
                if (cc + 2 < MT_C) tmem_ld32(tacc + (uint32_t)(cc + 2) * TILE, v0);
                tmem_st32_zero(tacc + (uint32_t)(cc + 1) * TILE);
                if (row_ok && mj * MT_C + cc + 1 < n_tiles)
                    store_block_coalesced(epi_tile, v1, cblock + (cc + 1) * TILE, ldc, lane, accumulate, acc_scale);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(smem_u32(&ctrl->tmem_empty[buf]));
            acc_iter++;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                     : "memory");
    }
}

// Loads this file's kernels onto the current device now (kernels are loaded lazily, at their first launch, and such
// a load can wait for kernels that are running; a kernel of one GPU that waits for a peer must not find the peer stuck
// in the load of a kernel it needs).
int preload_multiply()
{
    cudaFuncAttributes a;
    SPAMM_CUDA_TRY(cudaFuncGetAttributes(&a, gated_multiply_kernel));
    return SPAMM_OK;
}

}  // namespace spamm

extern "C" int spamm_gated_multiply_dev(const void *d_half_a, const void *d_half_b, const uint32_t *d_steps,
                                        const int32_t *d_step_counts, const int32_t *d_order,
                                        const int32_t *d_busy_list, spamm_list_scalars *d_scalars, int row_tiles,
                                        int k_tiles, int n_tiles, float *d_c, int64_t ldc, void *stream)
{
    return spamm::gated_multiply_launch(d_half_a, d_half_b, d_steps, d_step_counts, d_order, d_busy_list, d_scalars,
                                        row_tiles, k_tiles, n_tiles, d_c, ldc, true, spamm::GM_PAIRS_DENSE, 0,
                                        (cudaStream_t)stream);
}

int spamm::gated_multiply_launch(const void *d_half_a, const void *d_half_b, const uint32_t *d_steps,
                                 const int32_t *d_step_counts, const int32_t *d_order, const int32_t *d_busy_list,
                                 spamm_list_scalars *d_scalars, int row_tiles, int k_tiles, int n_tiles, float *d_c,
                                 int64_t ldc, bool reset_queues, int pairs, int mode, cudaStream_t stream,
                                 const GpairArgs *gpair)
{
    using namespace spamm;
    // adding to C only makes sense where C is not overwritten with zeros, and never through the paired kernel
    if (mode < 0 || mode > (GM_C_ZEROED | GM_ACCUMULATE | GM_LOW_OPERAND) ||
        pairs < GM_PAIRS_NONE || pairs > GM_PAIRS_GATED || (pairs == GM_PAIRS_GATED && !gpair) ||
        ((mode & GM_ACCUMULATE) && (!(mode & GM_C_ZEROED) || pairs == GM_PAIRS_DENSE)) ||
        ((mode & GM_LOW_OPERAND) && !(mode & GM_ACCUMULATE)))
        return SPAMM_ERR_INVALID;
    if (!d_half_a || !d_half_b || !d_steps || !d_step_counts || !d_busy_list || !d_scalars || !d_c || row_tiles < 0 ||
        k_tiles < 0 || n_tiles < 0 || ldc < (int64_t)n_tiles * TILE || (ldc & 3) ||
        (reinterpret_cast<uintptr_t>(d_c) & 15) || (reinterpret_cast<uintptr_t>(d_half_a) & 15) ||
        (reinterpret_cast<uintptr_t>(d_half_b) & 15) || (reinterpret_cast<uintptr_t>(d_scalars) & 7))
        return SPAMM_ERR_INVALID;
    const int64_t n_mt = (int64_t)ceil_div(row_tiles, MT_R) * ceil_div(n_tiles, MT_C);
    if (n_mt == 0) return SPAMM_OK;
    if (n_mt > 0x3fffffffLL) return SPAMM_ERR_UNSUPPORTED;

    // per device, once: the kernel's shared-memory limit and the SM count (a process may drive several GPUs in turn)
    static int sm_count_of[64] = {};
    int dev = 0;
    SPAMM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SPAMM_ERR_UNSUPPORTED;
    if (sm_count_of[dev] == 0) {
        int major = 0, sms = 0;
        SPAMM_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        SPAMM_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        if (major != 10) return SPAMM_ERR_UNSUPPORTED;
        SPAMM_CUDA_TRY(cudaFuncSetAttribute(gated_multiply_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            GM_SMEM_BYTES));
        sm_count_of[dev] = sms;
    }
    const int sm_count = sm_count_of[dev];
    // the two work counters and the count of macro tiles the two-SM kernel wrote start from zero at every launch
    // (unless the packing kernel just reset them): a second multiply over the same lists must not see the first one's
    static_assert(offsetof(spamm_list_scalars, pair_done) == offsetof(spamm_list_scalars, queue_busy) + 8,
                  "queue_busy, queue_all, pair_done are cleared as one block");
    if (reset_queues) SPAMM_CUDA_TRY(cudaMemsetAsync(&d_scalars->queue_busy, 0, 3 * sizeof(unsigned int), stream));
    // dense macro tiles with a dense vertical neighbour go to pairs of SMs first (a no-op below half dense);
    // a caller that knows the lists are sparse can save the launch
    if (pairs == GM_PAIRS_DENSE) {
        int st = gated_multiply_pair_launch(d_half_a, d_half_b, d_step_counts, d_scalars, row_tiles, k_tiles, n_tiles,
                                            d_c, ldc, stream);
        if (st) return st;
    } else if (pairs == GM_PAIRS_GATED) {
        int st = gated_multiply_gpair_launch(d_half_a, d_half_b, gpair->norm_a, gpair->norm_b, gpair->tau, gpair->chunk_max,
                                             d_step_counts, gpair->scratch, gpair->build, d_scalars, row_tiles, k_tiles,
                                             n_tiles, d_c, ldc, mode, stream);
        if (st) return st;
        // an even number of macro-tile rows: nothing is left for the one-SM kernel
        if (ceil_div(row_tiles, MT_R) >= 2 && ceil_div(row_tiles, MT_R) % 2 == 0) return SPAMM_OK;
    }
    const int grid = (int)(n_mt < sm_count ? n_mt : sm_count);
    gated_multiply_kernel<<<grid, GM_THREADS, GM_SMEM_BYTES, stream>>>(
        static_cast<const uint8_t *>(d_half_a), static_cast<const uint8_t *>(d_half_b), d_steps, d_step_counts,
        d_order, d_busy_list, d_scalars, row_tiles, k_tiles, n_tiles, d_c, ldc, pairs, mode);
    SPAMM_CUDA_TRY(cudaGetLastError());
    return SPAMM_OK;
}
