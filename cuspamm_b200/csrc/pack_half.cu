// float -> half conversion of the tiles that some skip list names, into the packed tile layout the tensor-core
// kernel loads with plain bulk copies.
//
// The reference converts whole matrices to half on the host when it generates them (tool.cu:418); with float
// host matrices as the interface the conversion has to happen on the GPU, and only the tiles that survive the
// threshold are ever read by the multiply, so only those are converted (a tile of A is needed iff some list of
// its tile row names its k; the list builder appends every such tile once to a work list, which this kernel walks
// with one warp per tile).
//
// Packed tile (2 KiB): element (o, kk) at byte (o/8)*512 + (kk/8)*128 + (o%8)*16 + (kk%8)*2, i.e. 8x8 "core
// matrices" of 128 contiguous bytes, the K-major no-swizzle operand layout of tcgen05.mma.  For A, o is the row
// and kk the column of the tile; for B, o is the column and kk the row (B is stored transposed inside a tile),
// so both operands are K-major.
#include "common.cuh"

namespace spamm {

// The part of x that its half rounding leaves over (exact in float), scaled by 2^11 before it is itself rounded to
// half: the residual is at most half a unit in the last place of the high part, i.e. 2^-11 of it, so the scaled value
// has the magnitude of the high part (never above 2^15) and keeps its bits where the unscaled one would fall into
// half's subnormal range (inputs below 1e-4) or vanish (below 6e-8).  The multiply's adding passes scale back.
__device__ __forceinline__ float half_residual(float x)
{
    return (x - __half2float(__float2half_rn(x))) * SPLIT_LOW_SCALE;
}

__device__ __forceinline__ uint4 pack8(const float *f)
{
    __half2 h0 = __floats2half2_rn(f[0], f[1]);
    __half2 h1 = __floats2half2_rn(f[2], f[3]);
    __half2 h2 = __floats2half2_rn(f[4], f[5]);
    __half2 h3 = __floats2half2_rn(f[6], f[7]);
    uint4 u;
    u.x = *reinterpret_cast<unsigned int *>(&h0);
    u.y = *reinterpret_cast<unsigned int *>(&h1);
    u.z = *reinterpret_cast<unsigned int *>(&h2);
    u.w = *reinterpret_cast<unsigned int *>(&h3);
    return u;
}

__global__ void __launch_bounds__(256)
pack_half_kernel(const float *__restrict__ a, const float *__restrict__ b, int k_tiles, int n_tiles,
                 const uint32_t *__restrict__ tile_list, spamm_list_scalars *__restrict__ sc,
                 uint8_t *__restrict__ half_a, uint8_t *__restrict__ half_b, uint8_t *__restrict__ low_a,
                 uint8_t *__restrict__ low_b, int reset_queues)
{
    // low_a / low_b (both or neither): second set of packed tiles holding half(x - half(x)), same layout and
    // slab order, for the split-precision mode
    // optional: the multiply kernel (next on the stream) starts its three work counters from zero
    if (reset_queues && blockIdx.x == 0 && threadIdx.x < 3) (&sc->queue_busy)[threadIdx.x] = 0u;   // queue_busy, queue_all, pair_done
    __shared__ float tr[8][TILE][TILE + 1];
    __shared__ unsigned int blk_cnt[2];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x < 2) blk_cnt[threadIdx.x] = 0;
    __syncthreads();

    const int mj_n = (n_tiles + MT_C - 1) / MT_C;
    const int64_t K = (int64_t)k_tiles * TILE, N = (int64_t)n_tiles * TILE;
    const unsigned int n_list = sc->tile_count;
    unsigned int cnt_a = 0, cnt_b = 0;

    // one warp per listed tile
    for (unsigned int t = sc->tile_begin + blockIdx.x * 8 + warp; t < n_list; t += gridDim.x * 8) {
        const uint32_t id = tile_list[t];
        const int sub = (int)(id & 7u);
        const int64_t slab = (int64_t)((id & 0x7fffffffu) >> 3);
        if (!(id & 0x80000000u)) {
            const int mi = (int)(slab / k_tiles), k = (int)(slab % k_tiles);
            const float *src = a + ((int64_t)(mi * MT_R + sub) * TILE) * K + (int64_t)k * TILE;
            uint8_t *dst = half_a + slab * A_SLAB_BYTES + sub * TILE_BYTES;
#pragma unroll
            for (int it = 0; it < 4; it++) {
                const int row = it * 8 + (lane >> 2), kg = lane & 3;
                const float4 lo = *reinterpret_cast<const float4 *>(src + (int64_t)row * K + kg * 8);
                const float4 hi = *reinterpret_cast<const float4 *>(src + (int64_t)row * K + kg * 8 + 4);
                const float f[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                const int off = (row >> 3) * 512 + kg * 128 + (row & 7) * 16;
                *reinterpret_cast<uint4 *>(dst + off) = pack8(f);
                if (low_a) {
                    float g[8];
#pragma unroll
                    for (int x = 0; x < 8; x++) g[x] = half_residual(f[x]);
                    *reinterpret_cast<uint4 *>(low_a + slab * A_SLAB_BYTES + sub * TILE_BYTES + off) = pack8(g);
                }
            }
            cnt_a++;
        } else {
            const int k = (int)(slab / mj_n), mj = (int)(slab % mj_n);
            const float *src = b + ((int64_t)k * TILE) * N + (int64_t)(mj * MT_C + sub) * TILE;
            uint8_t *dst = half_b + slab * B_SLAB_BYTES + sub * TILE_BYTES;
            __syncwarp();
#pragma unroll 8
            for (int kk = 0; kk < TILE; kk++) tr[warp][kk][lane] = src[(int64_t)kk * N + lane];
            __syncwarp();
#pragma unroll
            for (int kg = 0; kg < 4; kg++) {
                float f[8];
#pragma unroll
                for (int x = 0; x < 8; x++) f[x] = tr[warp][kg * 8 + x][lane];
                const int off = (lane >> 3) * 512 + kg * 128 + (lane & 7) * 16;
                *reinterpret_cast<uint4 *>(dst + off) = pack8(f);
                if (low_b) {
                    float g[8];
#pragma unroll
                    for (int x = 0; x < 8; x++) g[x] = half_residual(f[x]);
                    *reinterpret_cast<uint4 *>(low_b + slab * B_SLAB_BYTES + sub * TILE_BYTES + off) = pack8(g);
                }
            }
            cnt_b++;
        }
    }
    if (lane == 0) {
        if (cnt_a) atomicAdd(&blk_cnt[0], cnt_a);
        if (cnt_b) atomicAdd(&blk_cnt[1], cnt_b);
    }
    __syncthreads();
    if (threadIdx.x == 0 && blk_cnt[0]) atomicAdd(&sc->packed_a, blk_cnt[0]);
    if (threadIdx.x == 1 && blk_cnt[1]) atomicAdd(&sc->packed_b, blk_cnt[1]);
}

// Loads this file's kernels onto the current device now (kernels are loaded lazily, at their first launch, and such
// a load can wait for kernels that are running; a kernel of one GPU that waits for a peer must not find the peer stuck
// in the load of a kernel it needs).
int preload_pack()
{
    cudaFuncAttributes a;
    SPAMM_CUDA_TRY(cudaFuncGetAttributes(&a, pack_half_kernel));
    return SPAMM_OK;
}

}  // namespace spamm

extern "C" int spamm_pack_half_dev(const float *d_a, const float *d_b, int row_tiles, int k_tiles, int n_tiles,
                                   const uint32_t *d_tile_list, spamm_list_scalars *d_scalars, void *d_half_a,
                                   void *d_half_b, void *stream)
{
    return spamm::pack_half_launch(d_a, d_b, row_tiles, k_tiles, n_tiles, d_tile_list, d_scalars, d_half_a, d_half_b,
                                   nullptr, nullptr, false, (cudaStream_t)stream);
}

int spamm::pack_half_launch(const float *d_a, const float *d_b, int row_tiles, int k_tiles, int n_tiles,
                            const uint32_t *d_tile_list, spamm_list_scalars *d_scalars, void *d_half_a, void *d_half_b,
                            void *d_low_a, void *d_low_b, bool reset_queues, cudaStream_t stream)
{
    using namespace spamm;
    if (!d_a || !d_b || !d_tile_list || !d_scalars || !d_half_a || !d_half_b || row_tiles < 0 || k_tiles < 0 ||
        n_tiles < 0)
        return SPAMM_ERR_INVALID;
    if ((reinterpret_cast<uintptr_t>(d_a) & 15) || (reinterpret_cast<uintptr_t>(d_b) & 15) ||
        (reinterpret_cast<uintptr_t>(d_half_a) & 15) || (reinterpret_cast<uintptr_t>(d_half_b) & 15) ||
        (reinterpret_cast<uintptr_t>(d_low_a) & 15) || (reinterpret_cast<uintptr_t>(d_low_b) & 15) ||
        ((d_low_a == nullptr) != (d_low_b == nullptr)))
        return SPAMM_ERR_INVALID;
    const int64_t total = ((int64_t)ceil_div(row_tiles, MT_R) * MT_R + (int64_t)ceil_div(n_tiles, MT_C) * MT_C) * k_tiles;
    if (total == 0) return SPAMM_OK;
    // the number of listed tiles is known only on the device: a fixed grid strides over the list
    int64_t blocks = (total + 7) / 8;
    const int64_t max_blocks = 148 * 8;
    if (blocks > max_blocks) blocks = max_blocks;
    pack_half_kernel<<<(unsigned)blocks, 256, 0, stream>>>(
        d_a, d_b, k_tiles, n_tiles, d_tile_list, d_scalars, static_cast<uint8_t *>(d_half_a),
        static_cast<uint8_t *>(d_half_b), static_cast<uint8_t *>(d_low_a), static_cast<uint8_t *>(d_low_b),
        reset_queues ? 1 : 0);
    SPAMM_CUDA_TRY(cudaGetLastError());
    return SPAMM_OK;
}
