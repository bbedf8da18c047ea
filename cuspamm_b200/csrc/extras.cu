// Valid-product counter and threshold tuner on the GPU.
//
// The reference counts the tile products that pass the threshold with a triple host loop (countValid,
// tool.cu:493-529) and tunes the threshold to a target valid ratio by bisection over that loop (tuneValidRate,
// tool.cu:438-490, constants main.h:35-38).  Here the count is a kernel over the two norm maps: one block takes one
// tile row of A's map and 256 tile columns of B's, every thread walks k for its column (coalesced reads of B's
// map, broadcast reads of A's), and the block writes ONE partial count and ONE partial sum of products to a
// scratch array; a second, single-block kernel adds the partials in index order, so the result does not depend
// on scheduling.
#include "common.cuh"

namespace spamm {

constexpr int CV_THREADS = 256;

struct CountPartial {
    unsigned long long count;
    double sum;
};

__global__ void __launch_bounds__(CV_THREADS)
count_valid_kernel(const float *__restrict__ norm_a, const float *__restrict__ norm_b, int row_tiles, int k_tiles,
                   int n_tiles, float tau, CountPartial *__restrict__ partials)
{
    const int spans = (n_tiles + CV_THREADS - 1) / CV_THREADS;
    const int row = blockIdx.x / spans;
    const int col = (blockIdx.x % spans) * CV_THREADS + threadIdx.x;
    unsigned int cnt = 0;
    double sum = 0.0;
    if (col < n_tiles) {
        const float *a = norm_a + (int64_t)row * k_tiles;
        for (int k = 0; k < k_tiles; k++) {
            const float prod = __fmul_rn(a[k], norm_b[(int64_t)k * n_tiles + col]);
            cnt += (prod >= tau) ? 1u : 0u;
            sum += (double)prod;
        }
    }
    __shared__ unsigned int s_cnt[CV_THREADS / 32];
    __shared__ double s_sum[CV_THREADS / 32];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        cnt += __shfl_xor_sync(0xffffffffu, cnt, d);
        sum += __shfl_xor_sync(0xffffffffu, sum, d);
    }
    if ((threadIdx.x & 31) == 0) {
        s_cnt[threadIdx.x >> 5] = cnt;
        s_sum[threadIdx.x >> 5] = sum;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long c = 0;
        double s = 0.0;
        for (int w = 0; w < CV_THREADS / 32; w++) {
            c += s_cnt[w];
            s += s_sum[w];
        }
        partials[blockIdx.x].count = c;
        partials[blockIdx.x].sum = s;
    }
}

__global__ void __launch_bounds__(CV_THREADS)
count_valid_finish_kernel(const CountPartial *__restrict__ partials, int n, unsigned long long *__restrict__ count,
                          double *__restrict__ sum)
{
    __shared__ unsigned long long s_cnt[CV_THREADS];
    __shared__ double s_sum[CV_THREADS];
    unsigned long long c = 0;
    double s = 0.0;
    // thread t adds partials t, t+256, ... in order; then thread 0 adds the 256 thread sums in order
    for (int i = threadIdx.x; i < n; i += CV_THREADS) {
        c += partials[i].count;
        s += partials[i].sum;
    }
    s_cnt[threadIdx.x] = c;
    s_sum[threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        c = 0;
        s = 0.0;
        for (int t = 0; t < CV_THREADS; t++) {
            c += s_cnt[t];
            s += s_sum[t];
        }
        *count = c;
        if (sum) *sum = s;
    }
}

static int64_t count_valid_blocks(int row_tiles, int n_tiles)
{
    return (int64_t)row_tiles * ((n_tiles + CV_THREADS - 1) / CV_THREADS);
}

static int launch_count_valid(const float *d_norm_a, const float *d_norm_b, int row_tiles, int k_tiles, int n_tiles,
                              float tau, CountPartial *d_partials, unsigned long long *d_count, double *d_sum,
                              cudaStream_t stream)
{
    const int64_t blocks = count_valid_blocks(row_tiles, n_tiles);
    if (blocks > 0)
        count_valid_kernel<<<(unsigned)blocks, CV_THREADS, 0, stream>>>(d_norm_a, d_norm_b, row_tiles, k_tiles,
                                                                         n_tiles, tau, d_partials);
    count_valid_finish_kernel<<<1, CV_THREADS, 0, stream>>>(d_partials, (int)blocks, d_count, d_sum);
    SPAMM_CUDA_TRY(cudaGetLastError());
    return SPAMM_OK;
}

}  // namespace spamm

using namespace spamm;

extern "C" size_t spamm_count_valid_scratch_bytes(int row_tiles, int n_tiles)
{
    if (row_tiles < 0 || n_tiles < 0) return 0;
    const int64_t blocks = count_valid_blocks(row_tiles, n_tiles);
    return (size_t)(blocks > 0 ? blocks : 1) * sizeof(CountPartial);
}

extern "C" int spamm_count_valid_dev(const float *d_norm_a, const float *d_norm_b, int row_tiles, int k_tiles,
                                     int n_tiles, float tau, void *d_scratch, size_t scratch_bytes,
                                     unsigned long long *d_count, double *d_sum, void *stream)
{
    if (!d_norm_a || !d_norm_b || !d_scratch || !d_count || row_tiles < 0 || k_tiles < 0 || n_tiles < 0)
        return SPAMM_ERR_INVALID;
    if (count_valid_blocks(row_tiles, n_tiles) > 0x7fffffffLL) return SPAMM_ERR_UNSUPPORTED;
    if (scratch_bytes < spamm_count_valid_scratch_bytes(row_tiles, n_tiles) ||
        (reinterpret_cast<uintptr_t>(d_scratch) & 15))
        return SPAMM_ERR_INVALID;
    return launch_count_valid(d_norm_a, d_norm_b, row_tiles, k_tiles, n_tiles, tau,
                              static_cast<CountPartial *>(d_scratch), d_count, d_sum, (cudaStream_t)stream);
}
