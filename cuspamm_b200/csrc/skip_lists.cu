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
#include "common.cuh"

namespace spamm {

__device__ __forceinline__ void or_flag_byte(uint8_t *base, int64_t idx, uint32_t bits)
{
    unsigned int *w = reinterpret_cast<unsigned int *>(base + (idx & ~int64_t(3)));
    const unsigned int v = bits << (8 * (unsigned)(idx & 3));
    if ((*reinterpret_cast<volatile unsigned int *>(w) & v) != v) atomicOr(w, v);
}

__global__ void __launch_bounds__(128)
build_lists_kernel(const float *__restrict__ norm_a, const float *__restrict__ norm_b, int row_tiles, int k_tiles,
                   int n_tiles, float tau, uint32_t *__restrict__ steps, int32_t *__restrict__ step_counts,
                   int32_t *__restrict__ counts, unsigned long long *__restrict__ survivors,
                   uint8_t *__restrict__ need_a, uint8_t *__restrict__ need_b, int32_t *__restrict__ overflow)
{
    const int lane = threadIdx.x & 31;
    const int mi_n = (row_tiles + MT_R - 1) / MT_R;
    const int mj_n = (n_tiles + MT_C - 1) / MT_C;
    const int mt = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (mt >= mi_n * mj_n) return;
    const int mi = mt / mj_n, mj = mt % mj_n;
    const int64_t cap = (int64_t)STEP_CAP_PER_K * k_tiles;
    uint32_t *out = steps + (int64_t)mt * cap;

    int n_out = 0;       // warp-uniform
    int my_count = 0;    // lane b counts survivors of pair b = column*4 + row

    for (int kb = 0; kb < k_tiles; kb += 32) {
        const int k = kb + lane;
        const bool k_ok = k < k_tiles;
        uint32_t mask = 0;
        if (k_ok) {
            float a[MT_R];
#pragma unroll
            for (int r = 0; r < MT_R; r++) {
                const int row = mi * MT_R + r;
                a[r] = (row < row_tiles) ? norm_a[(int64_t)row * k_tiles + k] : 0.0f;
            }
#pragma unroll
            for (int c = 0; c < MT_C; c++) {
                const int colt = mj * MT_C + c;
                if (colt < n_tiles) {
                    const float b = norm_b[(int64_t)k * n_tiles + colt];
#pragma unroll
                    for (int r = 0; r < MT_R; r++) {
                        if (mi * MT_R + r < row_tiles) {
                            const float prod = __fmul_rn(a[r], b);
                            if (prod >= tau) mask |= 1u << (c * 4 + r);
                        }
                    }
                }
            }
        }
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
        int incl = n;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += t;
        }
        const int total = __shfl_sync(0xffffffffu, incl, 31);
        int pos = n_out + incl - n;
        if ((int64_t)n_out + total <= cap) {
#pragma unroll
            for (int c = 0; c < MT_C; c++) {
                if (st[c] != 0) out[pos++] = st[c];
            }
            n_out += total;
        } else if (lane == 0) {
            atomicExch(overflow, 1);
        }
        if (rows_any) {
            or_flag_byte(need_a, (int64_t)mi * k_tiles + k, rows_any);
            or_flag_byte(need_b, (int64_t)k * mj_n + mj, cols_any);
        }
    }
    if (lane == 0) step_counts[mt] = n_out;
    {
        const int r = lane & 3, c = lane >> 2;
        const int row = mi * MT_R + r, colt = mj * MT_C + c;
        if (row < row_tiles && colt < n_tiles) counts[(int64_t)row * n_tiles + colt] = my_count;
    }
    unsigned int s = (unsigned int)my_count;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
    if (lane == 0 && s) atomicAdd(survivors, (unsigned long long)s);
}

}  // namespace spamm

extern "C" int spamm_build_lists_dev(const float *d_norm_a, const float *d_norm_b, int row_tiles, int k_tiles,
                                     int n_tiles, float tau, uint32_t *d_steps, int32_t *d_step_counts,
                                     int32_t *d_counts, unsigned long long *d_survivors, uint8_t *d_need_a,
                                     uint8_t *d_need_b, int32_t *d_overflow, void *stream)
{
    using namespace spamm;
    if (!d_norm_a || !d_norm_b || !d_steps || !d_step_counts || !d_counts || !d_survivors || !d_need_a ||
        !d_need_b || !d_overflow || row_tiles < 0 || k_tiles < 0 || n_tiles < 0 || k_tiles > 65535)
        return SPAMM_ERR_INVALID;
    if ((reinterpret_cast<uintptr_t>(d_need_a) & 3) || (reinterpret_cast<uintptr_t>(d_need_b) & 3))
        return SPAMM_ERR_INVALID;
    const int64_t mts = (int64_t)ceil_div(row_tiles, MT_R) * ceil_div(n_tiles, MT_C);
    if (mts == 0) return SPAMM_OK;
    const int64_t blocks = (mts + 3) / 4;
    if (blocks > 0x7fffffffLL) return SPAMM_ERR_UNSUPPORTED;
    build_lists_kernel<<<(unsigned)blocks, 128, 0, (cudaStream_t)stream>>>(
        d_norm_a, d_norm_b, row_tiles, k_tiles, n_tiles, tau, d_steps, d_step_counts, d_counts, d_survivors,
        d_need_a, d_need_b, d_overflow);
    SPAMM_CUDA_TRY(cudaGetLastError());
    return SPAMM_OK;
}
