// Skip-list builder.
//
// The reference builds, inside every multiply block, the list of k whose norm product passes the threshold
// (cuSpAMM.cu:302-334): a bitmap, an O(k^2) serial compaction and a tree count, with a strided walk down a
// column of B's norm map.  Here one warp owns a macro tile of 4 x 8 C tiles (the shape one tensor-core
// instruction group covers), each lane takes one k of a chunk of 32, evaluates the 32 products
// nA(i,k) * nB(k,j) in float (one rounded multiply, then >=, exactly the reference's test at cuSpAMM.cu:305-306),
// and the lists are compacted in ascending k with a warp prefix sum.  Per-tile list lengths come from
// ballots + popcounts.
//
// Output form: a "step" names one k, a set of tile rows and a set of tile columns whose every pair survives.
// For one k the rows selected in a column form nested sets (the float product is monotone in either factor),
// so grouping columns by equal row set loses nothing: the steps of a k are disjoint and cover the survivors.
//
// Pruning: a first small kernel takes, per group of 4 tile rows of A (8 tile columns of B) and chunk of 32 k, the
// largest norm.  Rounded float multiplication is monotone in each factor, so when the product of the two largest
// norms of a chunk is below the threshold, every product of the chunk is: the builder skips the chunk without
// reading it, and the result is still exact.
//
// By-products for the next two kernels: the list of distinct tiles of A and of B that some step names (what has to
// be converted to half) and the list of macro tiles that have at least one step (scheduled first by the multiply).
#include <cstddef>

#include "common.cuh"

namespace spamm {

// Waits until every sender's arrival flag has reached wait.epoch, at most wait.limit_ns; on expiry sets *wait.error
// and goes on (the host then reports the step as failed).  Called by whole blocks.
__device__ __forceinline__ void peer_wait(const PeerWait &wait)
{
    if (!wait.flags) return;
    if ((int)threadIdx.x < wait.n) {
        unsigned long long t0;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        for (;;) {
            unsigned int f;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(f) : "l"(wait.flags + threadIdx.x) : "memory");
            if ((int)(f - wait.epoch) >= 0) break;
            unsigned long long t1;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > wait.limit_ns) {
                atomicExch(wait.error, 1);
                break;
            }
        }
    }
    __syncthreads();
}

__global__ void peer_wait_selftest_kernel(PeerWait wait) { peer_wait(wait); }

// amax[mi][kc] = max |nA| over tile rows 4mi..4mi+3 and k in chunk kc; bmax[kc][mj] = max |nB| over k in chunk kc and
// tile columns 8mj..8mj+7.  One warp per output value.
__global__ void __launch_bounds__(256)
chunk_max_kernel(const float *__restrict__ norm_a, const float *__restrict__ norm_b, int row_tiles, int k_tiles,
                 int n_tiles, float *__restrict__ amax, float *__restrict__ bmax, uint4 *__restrict__ clear,
                 size_t clear_vecs, int keep_scalars, PeerWait wait)
{
    // optional: B's norm map is assembled by the other GPUs writing their shares into it; wait (at most 2 s) until
    // every sender's flag has reached this step's number
    peer_wait(wait);
    // optional: zero the counters and need flags the list builder (the next kernel) starts from.  The region begins
    // with `keep_scalars` sets of counters whose error and overflow words survive: a wait that ran out in an earlier
    // step must still be there when the host next looks (spamm_sync clears the two after reporting them).
    const size_t head_bytes = (size_t)keep_scalars * sizeof(spamm_list_scalars);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < clear_vecs; i += (size_t)gridDim.x * blockDim.x) {
        if (i * 16 >= head_bytes) {
            clear[i] = make_uint4(0u, 0u, 0u, 0u);
        } else {
            uint32_t *w = reinterpret_cast<uint32_t *>(clear + i);
#pragma unroll
            for (int x = 0; x < 4; x++) {
                const size_t off = (i * 16 + 4 * x) % sizeof(spamm_list_scalars);
                if (i * 16 + 4 * x >= head_bytes ||
                    (off != offsetof(spamm_list_scalars, overflow) && off != offsetof(spamm_list_scalars, error)))
                    w[x] = 0u;
            }
        }
    }
    const int lane = threadIdx.x & 31;
    const int mi_n = (row_tiles + MT_R - 1) / MT_R;
    const int mj_n = (n_tiles + MT_C - 1) / MT_C;
    const int kc_n = (k_tiles + 31) / 32;
    const int w = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int n_a = mi_n * kc_n, n_b = kc_n * mj_n;
    if (w >= n_a + n_b) return;
    float m = 0.0f;
    bool odd = false;    // an infinite or NaN norm in the chunk
    if (w < n_a) {
        const int mi = w / kc_n, kc = w % kc_n;
        const int k = kc * 32 + lane;
        if (k < k_tiles) {
#pragma unroll
            for (int r = 0; r < MT_R; r++) {
                const int row = mi * MT_R + r;
                if (row < row_tiles) {
                    const float v = fabsf(norm_a[(int64_t)row * k_tiles + k]);
                    odd |= !(v <= 3.0e38f);
                    m = fmaxf(m, v);
                }
            }
        }
    } else {
        const int kc = (w - n_a) / mj_n, mj = (w - n_a) % mj_n;
        // column c = lane & 7, four k per pass
#pragma unroll
        for (int p = 0; p < 8; p++) {
            const int k = kc * 32 + p * 4 + (lane >> 3);
            const int colt = mj * MT_C + (lane & 7);
            if (k < k_tiles && colt < n_tiles) {
                const float v = fabsf(norm_b[(int64_t)k * n_tiles + colt]);
                odd |= !(v <= 3.0e38f);
                m = fmaxf(m, v);
            }
        }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    // a chunk with a non-finite norm is never skipped: NaN makes the builder's "product < tau" test false
    if (__any_sync(0xffffffffu, odd)) m = __int_as_float(0x7fc00000);
    if (lane == 0) {
        if (w < n_a) amax[w] = m;
        else bmax[w - n_a] = m;
    }
}

// Sets bits of two flag bytes and returns, for each, the bits that were not set before.  Both words are read before
// either is looked at and both atomics are issued before either result is used: the two round trips overlap.
__device__ __forceinline__ void or_flag_bytes(uint8_t *base_a, int64_t idx_a, uint32_t bits_a, uint8_t *base_b,
                                              int64_t idx_b, uint32_t bits_b, uint32_t *new_a, uint32_t *new_b)
{
    const uintptr_t addr_a = reinterpret_cast<uintptr_t>(base_a) + (uintptr_t)idx_a;
    const uintptr_t addr_b = reinterpret_cast<uintptr_t>(base_b) + (uintptr_t)idx_b;
    unsigned int *wa = reinterpret_cast<unsigned int *>(addr_a & ~uintptr_t(3));
    unsigned int *wb = reinterpret_cast<unsigned int *>(addr_b & ~uintptr_t(3));
    const unsigned int sha = 8 * (unsigned)(addr_a & 3), shb = 8 * (unsigned)(addr_b & 3);
    const unsigned int va = bits_a << sha, vb = bits_b << shb;
    const unsigned int seen_a = *reinterpret_cast<volatile unsigned int *>(wa);
    const unsigned int seen_b = *reinterpret_cast<volatile unsigned int *>(wb);
    const bool do_a = (seen_a & va) != va, do_b = (seen_b & vb) != vb;
    unsigned int old_a = va, old_b = vb;
    if (do_a) old_a = atomicOr(wa, va);
    if (do_b) old_b = atomicOr(wb, vb);
    *new_a = ((va & ~old_a) >> sha) & 0xffu;
    *new_b = ((vb & ~old_b) >> shb) & 0xffu;
}

__global__ void __launch_bounds__(128)
build_lists_kernel(const float *__restrict__ norm_a, const float *__restrict__ norm_b, int row_tiles, int k_tiles,
                   int n_tiles, float tau, const float *__restrict__ amax, const float *__restrict__ bmax,
                   uint32_t *__restrict__ steps, int32_t *__restrict__ step_counts, int32_t *__restrict__ counts,
                   uint8_t *__restrict__ need_a, uint8_t *__restrict__ need_b, uint32_t *__restrict__ tile_list,
                   int32_t *__restrict__ busy_list, spamm_list_scalars *__restrict__ sc)
{
    const int lane = threadIdx.x & 31;
    const int mi_n = (row_tiles + MT_R - 1) / MT_R;
    const int mj_n = (n_tiles + MT_C - 1) / MT_C;
    const int kc_n = (k_tiles + 31) / 32;
    const int mt = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (mt >= mi_n * mj_n) return;
    const int mi = mt / mj_n, mj = mt % mj_n;
    const int64_t cap = (int64_t)STEP_CAP_PER_K * k_tiles;
    uint32_t *out = steps + (int64_t)mt * cap;

    int n_out = 0;       // warp-uniform
    int my_count = 0;    // lane b counts survivors of pair b = column*4 + row
    int full_k = 0;      // warp-uniform: number of k whose 32 products all survive

    // pairs (row r, column c) of this macro tile that exist, bit c*4 + r
    uint32_t valid_bits = 0;
#pragma unroll
    for (int c = 0; c < MT_C; c++)
#pragma unroll
        for (int r = 0; r < MT_R; r++)
            if (mi * MT_R + r < row_tiles && mj * MT_C + c < n_tiles) valid_bits |= 1u << (c * 4 + r);
    const bool b_vec = ((n_tiles & 3) == 0) && (mj * MT_C + MT_C <= n_tiles) &&
                       ((reinterpret_cast<uintptr_t>(norm_b) & 15) == 0);

    for (int g0 = 0; g0 < kc_n; g0 += 32) {
        // which of the next 32 chunks can hold a survivor at all
        bool alive = false;
        if (g0 + lane < kc_n) {
            const float pm = __fmul_rn(amax[(int64_t)mi * kc_n + g0 + lane], bmax[(int64_t)(g0 + lane) * mj_n + mj]);
            alive = !(pm < tau);
        }
        uint32_t chunks = __ballot_sync(0xffffffffu, alive);
        while (chunks) {
            const int kb = (g0 + __ffs(chunks) - 1) * 32;
            chunks &= chunks - 1;
            const int k = kb + lane;
            uint32_t mask = 0;
            if (k < k_tiles) {
                float a[MT_R], b[MT_C];
#pragma unroll
                for (int r = 0; r < MT_R; r++) {
                    const int row = mi * MT_R + r;
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
                    for (int c = 0; c < MT_C; c++) b[c] = (mj * MT_C + c < n_tiles) ? __ldg(brow + c) : 0.0f;
                }
#pragma unroll
                for (int c = 0; c < MT_C; c++) {
#pragma unroll
                    for (int r = 0; r < MT_R; r++) {
                        const float prod = __fmul_rn(a[r], b[c]);
                        if (prod >= tau) mask |= 1u << (c * 4 + r);
                    }
                }
                mask &= valid_bits;
            }
            if (!__any_sync(0xffffffffu, mask != 0)) continue;
            full_k += __popc(__ballot_sync(0xffffffffu, mask == 0xffffffffu));
            // per-tile list lengths
#pragma unroll
            for (int bit = 0; bit < 32; bit++) {
                const uint32_t v = __ballot_sync(0xffffffffu, (mask >> bit) & 1u);
                if (lane == bit) my_count += __popc(v);
            }
            // steps of this lane's k: columns grouped by equal row set
            uint32_t st[MT_C];
            int n = 0;
            uint32_t done = 0, rows_any = 0, cols_any = 0;
#pragma unroll
            for (int c = 0; c < MT_C; c++) {
                const uint32_t nib = (mask >> (4 * c)) & 0xfu;
                uint32_t val = 0;
                if (nib != 0 && !((done >> c) & 1u)) {
                    uint32_t cols = 0;
#pragma unroll
                    for (int c2 = 0; c2 < MT_C; c2++)
                        if (((mask >> (4 * c2)) & 0xfu) == nib) cols |= 1u << c2;
                    done |= cols;
                    val = step_pack((uint32_t)k, nib, cols);
                    rows_any |= nib;
                    cols_any |= cols;
                }
                st[c] = val;
                n += (val != 0);
            }
            // tiles named for the first time go to the conversion list
            uint32_t new_a = 0, new_b = 0;
            if (rows_any)
                or_flag_bytes(need_a, (int64_t)mi * k_tiles + k, rows_any, need_b, (int64_t)k * mj_n + mj, cols_any, &new_a,
                              &new_b);
            const int n_new = __popc(new_a) + __popc(new_b);
            // two warp prefix sums at once: steps (low 16 bits) and new tiles (high 16 bits); both are <= 12 per lane
            uint32_t incl = (uint32_t)n | ((uint32_t)n_new << 16);
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const uint32_t t = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += t;
            }
            const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
            const int total_steps = (int)(total & 0xffffu), total_new = (int)(total >> 16);
            int pos = n_out + (int)(incl & 0xffffu) - n;
            if ((int64_t)n_out + total_steps <= cap) {
#pragma unroll
                for (int c = 0; c < MT_C; c++) {
                    if (st[c] != 0) out[pos++] = st[c];
                }
                n_out += total_steps;
            } else if (lane == 0) {
                atomicExch(&sc->overflow, 1);
            }
            if (total_new) {
                unsigned int base = 0;
                if (lane == 0) base = atomicAdd(&sc->tile_count, (unsigned int)total_new);
                base = __shfl_sync(0xffffffffu, base, 0);
                unsigned int at = base + (incl >> 16) - (unsigned int)n_new;
                const uint32_t a_slab = (uint32_t)(mi * k_tiles + k), b_slab = (uint32_t)(k * mj_n + mj);
                while (new_a) {
                    const int q = __ffs(new_a) - 1;
                    new_a &= new_a - 1;
                    tile_list[at++] = (a_slab << 3) | (uint32_t)q;
                }
                while (new_b) {
                    const int c = __ffs(new_b) - 1;
                    new_b &= new_b - 1;
                    tile_list[at++] = 0x80000000u | (b_slab << 3) | (uint32_t)c;
                }
            }
        }
    }
    if (lane == 0) {
        // dense: every k is there and each is one step naming all rows and columns
        const bool dense = k_tiles > 0 && full_k == k_tiles && n_out == k_tiles;
        step_counts[mt] = n_out | (dense ? SPAMM_STEPS_DENSE : 0);
        if (n_out > 0) busy_list[atomicAdd(&sc->busy_count, 1u)] = mt;
        if (dense) atomicAdd(&sc->dense_count, 1u);
    }
    {
        const int r = lane & 3, c = lane >> 2;
        const int row = mi * MT_R + r, colt = mj * MT_C + c;
        if (row < row_tiles && colt < n_tiles) counts[(int64_t)row * n_tiles + colt] = my_count;
    }
    unsigned int s = (unsigned int)my_count;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
    if (lane == 0 && s) atomicAdd(&sc->survivors, (unsigned long long)s);
}

// Loads this file's kernels onto the current device now (kernels are loaded lazily, at their first launch, and such
// a load can wait for kernels that are running; a kernel of one GPU that waits for a peer must not find the peer stuck
// in the load of a kernel it needs).
int preload_lists()
{
    cudaFuncAttributes a;
    SPAMM_CUDA_TRY(cudaFuncGetAttributes(&a, peer_wait_selftest_kernel));
    SPAMM_CUDA_TRY(cudaFuncGetAttributes(&a, chunk_max_kernel));
    SPAMM_CUDA_TRY(cudaFuncGetAttributes(&a, build_lists_kernel));
    return SPAMM_OK;
}

}  // namespace spamm

extern "C" size_t spamm_build_lists_scratch_bytes(int row_tiles, int k_tiles, int n_tiles)
{
    using namespace spamm;
    if (row_tiles < 0 || k_tiles < 0 || n_tiles < 0) return 0;
    const size_t kc_n = (size_t)(k_tiles + 31) / 32;
    return sizeof(float) * kc_n * ((size_t)ceil_div(row_tiles, MT_R) + ceil_div(n_tiles, MT_C)) + 16;
}

int spamm::peer_wait_selftest_launch(const PeerWait &w, cudaStream_t stream)
{
    peer_wait_selftest_kernel<<<1, 32, 0, stream>>>(w);
    SPAMM_CUDA_TRY(cudaGetLastError());
    return SPAMM_OK;
}

int spamm::build_lists_launch(const float *d_norm_a, const float *d_norm_b, int row_tiles, int k_tiles, int n_tiles,
                              float tau, void *d_scratch, uint32_t *d_steps, int32_t *d_step_counts,
                              int32_t *d_counts, uint8_t *d_need_a, uint8_t *d_need_b, uint32_t *d_tile_list,
                              int32_t *d_busy_list, spamm_list_scalars *d_scalars, void *d_clear, size_t clear_bytes,
                              int keep_scalars, const PeerWait *wait, cudaStream_t stream)
{
    using namespace spamm;
    if (!d_norm_a || !d_norm_b || !d_scratch || !d_steps || !d_step_counts || !d_counts || !d_need_a || !d_need_b ||
        !d_tile_list || !d_busy_list || !d_scalars || row_tiles < 0 || k_tiles < 0 || n_tiles < 0 || k_tiles > 65535)
        return SPAMM_ERR_INVALID;
    if ((reinterpret_cast<uintptr_t>(d_scratch) & 3) || (reinterpret_cast<uintptr_t>(d_scalars) & 7) ||
        (reinterpret_cast<uintptr_t>(d_clear) & 15) || (clear_bytes & 15))
        return SPAMM_ERR_INVALID;
    const int mi_n = ceil_div(row_tiles, MT_R), mj_n = ceil_div(n_tiles, MT_C), kc_n = ceil_div(k_tiles, 32);
    const int64_t mts = (int64_t)mi_n * mj_n;
    if (mts == 0) return SPAMM_OK;
    const int64_t blocks = (mts + 3) / 4;
    if (blocks > 0x7fffffffLL || (int64_t)mi_n * k_tiles >= (1LL << 28) || (int64_t)k_tiles * mj_n >= (1LL << 28))
        return SPAMM_ERR_UNSUPPORTED;
    float *amax = static_cast<float *>(d_scratch);
    float *bmax = amax + (size_t)mi_n * kc_n;
    const int64_t warps = (int64_t)kc_n * (mi_n + mj_n);
    int64_t cm_blocks = (warps + 7) / 8;
    if (cm_blocks < 1) cm_blocks = 1;
    PeerWait w{};
    if (wait) w = *wait;
    chunk_max_kernel<<<(unsigned)cm_blocks, 256, 0, stream>>>(d_norm_a, d_norm_b, row_tiles, k_tiles, n_tiles, amax,
                                                             bmax, static_cast<uint4 *>(d_clear),
                                                             d_clear ? clear_bytes / 16 : 0, keep_scalars, w);
    build_lists_kernel<<<(unsigned)blocks, 128, 0, stream>>>(
        d_norm_a, d_norm_b, row_tiles, k_tiles, n_tiles, tau, amax, bmax, d_steps, d_step_counts, d_counts, d_need_a,
        d_need_b, d_tile_list, d_busy_list, d_scalars);
    SPAMM_CUDA_TRY(cudaGetLastError());
    return SPAMM_OK;
}

extern "C" int spamm_build_lists_dev(const float *d_norm_a, const float *d_norm_b, int row_tiles, int k_tiles,
                                     int n_tiles, float tau, void *d_scratch, uint32_t *d_steps,
                                     int32_t *d_step_counts, int32_t *d_counts, uint8_t *d_need_a, uint8_t *d_need_b,
                                     uint32_t *d_tile_list, int32_t *d_busy_list, spamm_list_scalars *d_scalars,
                                     void *stream)
{
    return spamm::build_lists_launch(d_norm_a, d_norm_b, row_tiles, k_tiles, n_tiles, tau, d_scratch, d_steps,
                                     d_step_counts, d_counts, d_need_a, d_need_b, d_tile_list, d_busy_list, d_scalars,
                                     nullptr, 0, 0, nullptr, (cudaStream_t)stream);
}
