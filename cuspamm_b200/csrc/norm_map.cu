// Tile Frobenius-norm map: an HBM streaming kernel.
//
// Stands in for unroll_get_Fnorm_pri (reference cuSpAMM.cu:21-71) and, because the contract is float norms of
// the float data, for unroll_get_Fnorm_FP16 (cuSpAMM.cu:74-123).  The reference runs one 128-thread block per
// 2-4 KB tile; here one warp sweeps a strip of four adjacent tiles (32 rows x 128 columns = 16 KB) with one
// 128-bit load per lane and row, so every row of the strip is one fully used 512-byte request, and the 32 loads
// of a lane are independent of each other.
//
// Reduction order (the CPU checker uses the same, which makes the maps bit-equal):
//   lane g (0..7) of a tile owns columns 4g..4g+3; rows 0..31 in order, the four columns left to right,
//   acc = fma(x, x, acc) from +0; then acc_g + acc_{g^4}, then + the partner g^2, then + the partner g^1;
//   norm = sqrt (round to nearest).  Additions of two partners are commutative, so all eight lanes hold the
//   same bits after each step.
#include "common.cuh"

namespace spamm {

// One strip of four tiles per warp; `strip` counts strips of this matrix in row-major order.  Returns true in the
// lanes that hold a finished tile norm (*value) and its index in the map (*index).
__device__ __forceinline__ bool norm_strip_value(const float *__restrict__ x, int tile_rows, int tile_cols, int64_t ld,
                                                 int64_t strip, float *value, int64_t *index)
{
    const int lane = threadIdx.x & 31;
    const int strips_per_row = (tile_cols + 3) >> 2;
    if (strip >= (int64_t)tile_rows * strips_per_row) return false;
    const int tr = (int)(strip / strips_per_row);
    const int ts = (int)(strip % strips_per_row);
    const int col = ts * 128 + lane * 4;
    const bool in_range = col < tile_cols * TILE;
    const float *p = x + (int64_t)tr * TILE * ld + col;

    float acc = 0.0f;
#pragma unroll
    for (int r0 = 0; r0 < TILE; r0 += 8) {
        float4 v[8];
#pragma unroll
        for (int r = 0; r < 8; r++) {
            v[r] = in_range ? __ldcs(reinterpret_cast<const float4 *>(p + (int64_t)(r0 + r) * ld))
                            : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int r = 0; r < 8; r++) {
            acc = __fmaf_rn(v[r].x, v[r].x, acc);
            acc = __fmaf_rn(v[r].y, v[r].y, acc);
            acc = __fmaf_rn(v[r].z, v[r].z, acc);
            acc = __fmaf_rn(v[r].w, v[r].w, acc);
        }
    }
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));
    *value = __fsqrt_rn(acc);
    *index = (int64_t)tr * tile_cols + ts * 4 + (lane >> 3);
    return in_range && (lane & 7) == 0;
}

__device__ __forceinline__ void norm_strip(const float *__restrict__ x, int tile_rows, int tile_cols, int64_t ld,
                                           float *__restrict__ map, int64_t strip)
{
    float v;
    int64_t i;
    if (norm_strip_value(x, tile_rows, tile_cols, ld, strip, &v, &i)) map[i] = v;
}

__global__ void __launch_bounds__(256)
norm_map_kernel(const float *__restrict__ x, int tile_rows, int tile_cols, int64_t ld, float *__restrict__ map)
{
    norm_strip(x, tile_rows, tile_cols, ld, map, (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5));
}

// Two matrices in one launch (the A rows and B of one SpAMM step): blocks [0, blocks_a) work on the first.
__global__ void __launch_bounds__(256)
norm_map_pair_kernel(const float *__restrict__ xa, int tile_rows_a, int tile_cols_a, int64_t lda,
                     float *__restrict__ map_a, unsigned int blocks_a, const float *__restrict__ xb, int tile_rows_b,
                     int tile_cols_b, int64_t ldb, float *__restrict__ map_b)
{
    if (blockIdx.x < blocks_a)
        norm_strip(xa, tile_rows_a, tile_cols_a, lda, map_a, (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5));
    else
        norm_strip(xb, tile_rows_b, tile_cols_b, ldb, map_b,
                   (int64_t)(blockIdx.x - blocks_a) * 8 + (threadIdx.x >> 5));
}

// All-gather of B's norm-map shares without a collective call: after the norm kernel has written this GPU's share
// into its own map, one block per destination GPU copies the share into that GPU's map (peer-mapped memory, plain
// 128-bit stores over NVLink), fences system-wide and raises this GPU's flag there: "share of `rank` for step
// `epoch` has arrived".  The reader (the list builder's first kernel) waits for all flags with a time limit.
__global__ void __launch_bounds__(256)
push_share_kernel(const float4 *__restrict__ src, int64_t vecs, int64_t map_offset_vecs, PeerTargets t, int self,
                  unsigned int epoch)
{
    const int d = blockIdx.x;                       // destination GPU
    if (d != self) {
        float4 *dst = reinterpret_cast<float4 *>(t.map[d]) + map_offset_vecs;
        for (int64_t i = threadIdx.x; i < vecs; i += blockDim.x) dst[i] = src[i];
    }
    __syncthreads();                                // orders the block's stores before the fence below
    if (threadIdx.x == 0) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(t.flags[d] + self), "r"(epoch) : "memory");
    }
}

int norm_map_push_launch(const float *d_x, int rows, int cols, int64_t ld, int64_t map_offset, const PeerTargets &t,
                         int rank, unsigned int epoch, cudaStream_t stream)
{
    if (!d_x || rows <= 0 || cols <= 0 || rows % TILE || cols % TILE || (ld & 3) || t.n <= 0 || t.n > MAX_PEERS ||
        rank < 0 || rank >= t.n)
        return SPAMM_ERR_INVALID;
    const int tile_rows = rows / TILE, tile_cols = cols / TILE;
    const int64_t share = (int64_t)tile_rows * tile_cols;          // floats in this GPU's share of the map
    float *local = t.map[rank] + map_offset;
    if ((share & 3) || (map_offset & 3) || (reinterpret_cast<uintptr_t>(local) & 15)) return SPAMM_ERR_UNSUPPORTED;
    int st = spamm_norm_map_dev(d_x, rows, cols, ld, local, stream);
    if (st) return st;
    push_share_kernel<<<t.n, 256, 0, stream>>>(reinterpret_cast<const float4 *>(local), share / 4, map_offset / 4, t,
                                              rank, epoch);
    SPAMM_CUDA_TRY(cudaGetLastError());
    return SPAMM_OK;
}

}  // namespace spamm

extern "C" int spamm_norm_map_dev(const float *d_x, int rows, int cols, int64_t ld, float *d_map, void *stream)
{
    using namespace spamm;
    if (!d_x || !d_map || rows < 0 || cols < 0 || rows % TILE || cols % TILE || ld < cols || (ld & 3) ||
        (reinterpret_cast<uintptr_t>(d_x) & 15))
        return SPAMM_ERR_INVALID;
    if (rows == 0 || cols == 0) return SPAMM_OK;
    const int tile_rows = rows / TILE, tile_cols = cols / TILE;
    const int64_t strips = (int64_t)tile_rows * ((tile_cols + 3) / 4);
    const int64_t blocks = (strips + 7) / 8;
    if (blocks > 0x7fffffffLL) return SPAMM_ERR_UNSUPPORTED;
    norm_map_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(d_x, tile_rows, tile_cols, ld, d_map);
    SPAMM_CUDA_TRY(cudaGetLastError());
    return SPAMM_OK;
}

extern "C" int spamm_norm_map_pair_dev(const float *d_xa, int rows_a, int cols_a, int64_t lda, float *d_map_a,
                                       const float *d_xb, int rows_b, int cols_b, int64_t ldb, float *d_map_b,
                                       void *stream)
{
    using namespace spamm;
    if (!d_xa || !d_map_a || !d_xb || !d_map_b || rows_a < 0 || cols_a < 0 || rows_b < 0 || cols_b < 0 ||
        rows_a % TILE || cols_a % TILE || rows_b % TILE || cols_b % TILE || lda < cols_a || ldb < cols_b ||
        (lda & 3) || (ldb & 3) || (reinterpret_cast<uintptr_t>(d_xa) & 15) || (reinterpret_cast<uintptr_t>(d_xb) & 15))
        return SPAMM_ERR_INVALID;
    const int tra = rows_a / TILE, tca = cols_a / TILE, trb = rows_b / TILE, tcb = cols_b / TILE;
    const int64_t blocks_a = ((int64_t)tra * ((tca + 3) / 4) + 7) / 8;
    const int64_t blocks_b = ((int64_t)trb * ((tcb + 3) / 4) + 7) / 8;
    if (blocks_a + blocks_b == 0) return SPAMM_OK;
    if (blocks_a + blocks_b > 0x7fffffffLL) return SPAMM_ERR_UNSUPPORTED;
    norm_map_pair_kernel<<<(unsigned)(blocks_a + blocks_b), 256, 0, (cudaStream_t)stream>>>(
        d_xa, tra, tca, lda, d_map_a, (unsigned)blocks_a, d_xb, trb, tcb, ldb, d_map_b);
    SPAMM_CUDA_TRY(cudaGetLastError());
    return SPAMM_OK;
}
