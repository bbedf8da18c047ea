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

// ---------------------------------------------------------------------------------------------------------------
// Norm map and half conversion of EVERY tile in one pass (for workloads where most tiles survive the threshold: the
// separate conversion kernel would read most of the matrices a second time).  The sums are formed exactly as in
// norm_strip_value, so the maps are the same bits; while a batch of 8 rows is in registers it is also rounded to
// half and stored in the packed tile layout (see pack_half.cu).
//   A (element (row, kk) of a tile at (row/8)*512 + (kk/8)*128 + (row%8)*16 + (kk%8)*2): a lane owns 4 consecutive kk
//   of every row = 8 bytes; neighbouring lanes swap halves of two rows so that each stores 16 bytes and every pair
//   of lanes fills a 32-byte sector.
//   B (stored transposed: element (col, kk=row)): the 8 rows of a batch are the 8 kk of one 16-byte unit for each
//   of the lane's 4 columns, and those 4 units are adjacent: 64 contiguous bytes per lane and batch.
__device__ __forceinline__ unsigned int half2_bits(float a, float b)
{
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<unsigned int *>(&h);
}

template <bool IS_B>
__device__ __forceinline__ void norm_pack_strip(const float *__restrict__ x, int tile_rows, int tile_cols, int64_t ld,
                                                float *__restrict__ map, int64_t strip, uint8_t *__restrict__ half,
                                                int slabs_per_row)
{
    const int lane = threadIdx.x & 31;
    const int strips_per_row = (tile_cols + 3) >> 2;
    if (strip >= (int64_t)tile_rows * strips_per_row) return;
    const int tr = (int)(strip / strips_per_row);
    const int ts = (int)(strip % strips_per_row);
    const int col = ts * 128 + lane * 4;
    const bool in_range = col < tile_cols * TILE;
    const float *p = x + (int64_t)tr * TILE * ld + col;
    const int tc = ts * 4 + (lane >> 3);       // tile column of this lane
    const int g = lane & 7;
    // start of this lane's packed tile
    uint8_t *dst;
    if (IS_B)   // slabs [k = tr][column group], 8 tiles each
        dst = half + ((int64_t)tr * slabs_per_row + (tc >> 3)) * B_SLAB_BYTES + (tc & 7) * TILE_BYTES;
    else        // slabs [row group][k = tc], 4 tiles each
        dst = half + ((int64_t)(tr >> 2) * slabs_per_row + tc) * A_SLAB_BYTES + (tr & 3) * TILE_BYTES;

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
        if (IS_B) {
            if (in_range) {
                uint8_t *d = dst + (g >> 1) * 512 + (r0 >> 3) * 128 + (g & 1) * 64;
                uint4 u;
                u = make_uint4(half2_bits(v[0].x, v[1].x), half2_bits(v[2].x, v[3].x), half2_bits(v[4].x, v[5].x),
                               half2_bits(v[6].x, v[7].x));
                *reinterpret_cast<uint4 *>(d) = u;
                u = make_uint4(half2_bits(v[0].y, v[1].y), half2_bits(v[2].y, v[3].y), half2_bits(v[4].y, v[5].y),
                               half2_bits(v[6].y, v[7].y));
                *reinterpret_cast<uint4 *>(d + 16) = u;
                u = make_uint4(half2_bits(v[0].z, v[1].z), half2_bits(v[2].z, v[3].z), half2_bits(v[4].z, v[5].z),
                               half2_bits(v[6].z, v[7].z));
                *reinterpret_cast<uint4 *>(d + 32) = u;
                u = make_uint4(half2_bits(v[0].w, v[1].w), half2_bits(v[2].w, v[3].w), half2_bits(v[4].w, v[5].w),
                               half2_bits(v[6].w, v[7].w));
                *reinterpret_cast<uint4 *>(d + 48) = u;
            }
        } else {
            const bool odd = (g & 1) != 0;
#pragma unroll
            for (int r = 0; r < 8; r += 2) {
                // rows r (kept by the even lane) and r+1 (kept by the odd lane): each lane gives away the other row
                const unsigned int e0 = half2_bits(v[r].x, v[r].y), e1 = half2_bits(v[r].z, v[r].w);
                const unsigned int o0 = half2_bits(v[r + 1].x, v[r + 1].y), o1 = half2_bits(v[r + 1].z, v[r + 1].w);
                const unsigned int s0 = __shfl_xor_sync(0xffffffffu, odd ? e0 : o0, 1);
                const unsigned int s1 = __shfl_xor_sync(0xffffffffu, odd ? e1 : o1, 1);
                if (in_range) {
                    const int row = r0 + r + (odd ? 1 : 0);
                    const uint4 u = odd ? make_uint4(s0, s1, o0, o1) : make_uint4(e0, e1, s0, s1);
                    *reinterpret_cast<uint4 *>(dst + (row >> 3) * 512 + (g >> 1) * 128 + (row & 7) * 16) = u;
                }
            }
        }
    }
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));
    if (in_range && g == 0) map[(int64_t)tr * tile_cols + tc] = __fsqrt_rn(acc);
}

__global__ void __launch_bounds__(256)
norm_pack_pair_kernel(const float *__restrict__ xa, int tile_rows_a, int tile_cols_a, int64_t lda,
                      float *__restrict__ map_a, uint8_t *__restrict__ half_a, unsigned int blocks_a,
                      const float *__restrict__ xb, int tile_rows_b, int tile_cols_b, int64_t ldb,
                      float *__restrict__ map_b, uint8_t *__restrict__ half_b)
{
    if (blockIdx.x < blocks_a)
        norm_pack_strip<false>(xa, tile_rows_a, tile_cols_a, lda, map_a, (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5),
                               half_a, tile_cols_a);
    else
        norm_pack_strip<true>(xb, tile_rows_b, tile_cols_b, ldb, map_b,
                              (int64_t)(blockIdx.x - blocks_a) * 8 + (threadIdx.x >> 5), half_b,
                              (tile_cols_b + MT_C - 1) / MT_C);
}

int norm_pack_pair_launch(const float *d_xa, int rows_a, int cols_a, int64_t lda, float *d_map_a, void *d_half_a,
                          const float *d_xb, int rows_b, int cols_b, int64_t ldb, float *d_map_b, void *d_half_b,
                          cudaStream_t stream)
{
    if (!d_xa || !d_map_a || !d_xb || !d_map_b || !d_half_a || !d_half_b || rows_a <= 0 || cols_a <= 0 ||
        rows_b <= 0 || cols_b <= 0 || rows_a % TILE || cols_a % TILE || rows_b % TILE || cols_b % TILE ||
        lda < cols_a || ldb < cols_b || (lda & 3) || (ldb & 3) || (reinterpret_cast<uintptr_t>(d_xa) & 15) ||
        (reinterpret_cast<uintptr_t>(d_xb) & 15) || (reinterpret_cast<uintptr_t>(d_half_a) & 15) ||
        (reinterpret_cast<uintptr_t>(d_half_b) & 15))
        return SPAMM_ERR_INVALID;
    const int tra = rows_a / TILE, tca = cols_a / TILE, trb = rows_b / TILE, tcb = cols_b / TILE;
    const int64_t blocks_a = ((int64_t)tra * ((tca + 3) / 4) + 7) / 8;
    const int64_t blocks_b = ((int64_t)trb * ((tcb + 3) / 4) + 7) / 8;
    if (blocks_a + blocks_b > 0x7fffffffLL) return SPAMM_ERR_UNSUPPORTED;
    norm_pack_pair_kernel<<<(unsigned)(blocks_a + blocks_b), 256, 0, stream>>>(
        d_xa, tra, tca, lda, d_map_a, static_cast<uint8_t *>(d_half_a), (unsigned)blocks_a, d_xb, trb, tcb, ldb,
        d_map_b, static_cast<uint8_t *>(d_half_b));
    SPAMM_CUDA_TRY(cudaGetLastError());
    return SPAMM_OK;
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
        constexpr int U = 8;                        // eight loads in flight per thread
        for (int64_t i0 = threadIdx.x; i0 < vecs; i0 += (int64_t)blockDim.x * U) {
            float4 v[U];
#pragma unroll
            for (int u = 0; u < U; u++)
                if (i0 + (int64_t)u * blockDim.x < vecs) v[u] = src[i0 + (int64_t)u * blockDim.x];
#pragma unroll
            for (int u = 0; u < U; u++)
                if (i0 + (int64_t)u * blockDim.x < vecs) dst[i0 + (int64_t)u * blockDim.x] = v[u];
        }
    }
    __syncthreads();                                // orders the block's stores before the fence below
    if (threadIdx.x == 0) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(t.flags[d] + self), "r"(epoch) : "memory");
    }
}

// The norm maps of a GPU's rows of A and of its share of B's tile rows in ONE launch that also delivers the share: the
// blocks of the share come first in the grid; each of them, when its values are written, counts itself in, and the one
// that finds itself last copies the whole share into every other GPU's map (peer stores) and raises the flags.  The
// rest of the grid is still reading A meanwhile, so the exchange costs neither a launch nor time on the stream.
__global__ void __launch_bounds__(256)
norm_map_pair_push_kernel(const float *__restrict__ xb, int tile_rows_b, int tile_cols_b, int64_t ldb,
                          float *__restrict__ share, unsigned int blocks_b, const float *__restrict__ xa,
                          int tile_rows_a, int tile_cols_a, int64_t lda, float *__restrict__ map_a, int64_t share_vecs,
                          int64_t map_offset_vecs, PeerTargets t, int self, unsigned int epoch,
                          unsigned int *__restrict__ counter)
{
    if (blockIdx.x >= blocks_b) {
        norm_strip(xa, tile_rows_a, tile_cols_a, lda, map_a, (int64_t)(blockIdx.x - blocks_b) * 8 + (threadIdx.x >> 5));
        return;
    }
    norm_strip(xb, tile_rows_b, tile_cols_b, ldb, share, (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5));
    __shared__ unsigned int ticket;
    __syncthreads();                                // every warp of the block has written its norms
    if (threadIdx.x == 0) {
        __threadfence();                            // ... and they are visible before the block counts itself in
        ticket = atomicAdd(counter, 1u);
    }
    __syncthreads();
    if (ticket != blocks_b - 1) return;
    __threadfence();                                // the last block: everybody else's norms are visible to it
    // one block moves the whole share: eight loads in flight per thread, each value stored to every peer, so the
    // copy is bound by the stores over NVLink and not by one L2 round trip per 16 bytes
    const float4 *src = reinterpret_cast<const float4 *>(share);
    constexpr int PUSH_UNROLL = 8;
    for (int64_t i0 = threadIdx.x; i0 < share_vecs; i0 += (int64_t)blockDim.x * PUSH_UNROLL) {
        float4 v[PUSH_UNROLL];
#pragma unroll
        for (int u = 0; u < PUSH_UNROLL; u++) {
            const int64_t i = i0 + (int64_t)u * blockDim.x;
            if (i < share_vecs) v[u] = __ldcg(src + i);
        }
        for (int d = 0; d < t.n; d++) {
            if (d == self) continue;
            float4 *dst = reinterpret_cast<float4 *>(t.map[d]) + map_offset_vecs;
#pragma unroll
            for (int u = 0; u < PUSH_UNROLL; u++) {
                const int64_t i = i0 + (int64_t)u * blockDim.x;
                if (i < share_vecs) dst[i] = v[u];
            }
        }
    }
    __syncthreads();                                // orders the block's stores before the fence below
    if (threadIdx.x == 0) {
        *counter = 0u;                              // for the next step (stream order)
        __threadfence_system();
        for (int d = 0; d < t.n; d++)
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(t.flags[d] + self), "r"(epoch) : "memory");
    }
}

int norm_map_pair_push_launch(const float *d_xa, int rows_a, int cols_a, int64_t lda, float *d_map_a, const float *d_xb,
                              int rows_b, int cols_b, int64_t ldb, float *d_local_share, int64_t map_offset,
                              const PeerTargets &t, int rank, unsigned int epoch, unsigned int *d_counter,
                              cudaStream_t stream)
{
    if (!d_xa || !d_map_a || !d_xb || !d_local_share || !d_counter || rows_a < 0 || cols_a <= 0 || rows_b <= 0 ||
        cols_b <= 0 || rows_a % TILE || cols_a % TILE || rows_b % TILE || cols_b % TILE || lda < cols_a || ldb < cols_b ||
        (lda & 3) || (ldb & 3) || (reinterpret_cast<uintptr_t>(d_xa) & 15) || (reinterpret_cast<uintptr_t>(d_xb) & 15) ||
        t.n <= 0 || t.n > MAX_PEERS || rank < 0 || rank >= t.n)
        return SPAMM_ERR_INVALID;
    const int tra = rows_a / TILE, tca = cols_a / TILE, trb = rows_b / TILE, tcb = cols_b / TILE;
    const int64_t share = (int64_t)trb * tcb;
    if ((share & 3) || (map_offset & 3) || (reinterpret_cast<uintptr_t>(d_local_share) & 15) ||
        d_local_share != t.map[rank] + map_offset)
        return SPAMM_ERR_UNSUPPORTED;
    const int64_t blocks_a = ((int64_t)tra * ((tca + 3) / 4) + 7) / 8;
    const int64_t blocks_b = ((int64_t)trb * ((tcb + 3) / 4) + 7) / 8;
    if (blocks_a + blocks_b > 0x7fffffffLL) return SPAMM_ERR_UNSUPPORTED;
    norm_map_pair_push_kernel<<<(unsigned)(blocks_a + blocks_b), 256, 0, stream>>>(
        d_xb, trb, tcb, ldb, d_local_share, (unsigned)blocks_b, d_xa, tra, tca, lda, d_map_a, share / 4, map_offset / 4, t,
        rank, epoch, d_counter);
    SPAMM_CUDA_TRY(cudaGetLastError());
    return SPAMM_OK;
}

int push_share_launch(const float *d_local_share, int64_t share, int64_t map_offset, const PeerTargets &t, int rank,
                      unsigned int epoch, cudaStream_t stream)
{
    if (!d_local_share || share <= 0 || t.n <= 0 || t.n > MAX_PEERS || rank < 0 || rank >= t.n) return SPAMM_ERR_INVALID;
    if ((share & 3) || (map_offset & 3) || (reinterpret_cast<uintptr_t>(d_local_share) & 15) ||
        d_local_share != t.map[rank] + map_offset)
        return SPAMM_ERR_UNSUPPORTED;
    push_share_kernel<<<t.n, 256, 0, stream>>>(reinterpret_cast<const float4 *>(d_local_share), share / 4,
                                              map_offset / 4, t, rank, epoch);
    SPAMM_CUDA_TRY(cudaGetLastError());
    return SPAMM_OK;
}

// Loads this file's kernels onto the current device now (kernels are loaded lazily, at their first launch, and such
// a load can wait for kernels that are running; a kernel of one GPU that waits for a peer must not find the peer stuck
// in the load of a kernel it needs).
int preload_norm()
{
    cudaFuncAttributes a;
    SPAMM_CUDA_TRY(cudaFuncGetAttributes(&a, norm_map_kernel));
    SPAMM_CUDA_TRY(cudaFuncGetAttributes(&a, norm_map_pair_kernel));
    SPAMM_CUDA_TRY(cudaFuncGetAttributes(&a, norm_pack_pair_kernel));
    SPAMM_CUDA_TRY(cudaFuncGetAttributes(&a, push_share_kernel));
    SPAMM_CUDA_TRY(cudaFuncGetAttributes(&a, norm_map_pair_push_kernel));
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
