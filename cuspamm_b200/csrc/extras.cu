// Valid-product counter and threshold tuner on the GPU.
//
// The reference counts the tile products that pass the threshold with a triple host loop (countValid,
// tool.cu:493-529) and tunes the threshold to a target valid ratio by bisection over that loop (tuneValidRate,
// tool.cu:438-490, constants main.h:35-38).  Here the count is a kernel over the two norm maps: one block takes one
// tile row of A's map and 256 tile columns of B's, every thread walks k for its column (coalesced reads of B's
// map, broadcast reads of A's), and the block writes ONE partial count and ONE partial sum of products to a
// scratch array; a second, single-block kernel adds the partials in index order, so the result does not depend
// on scheduling.
#include <cstdio>

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

// ------------------------------------------------------------------------------------------------------------------
// Error norms against a reference product: the three Frobenius norms the reference prints with COUNTERRTRANS
// (tool.cu:6-24, called from check_simple_gpu, tool.cu:227-280): ||ref - C||_F, ||ref||_F, ||C||_F.  Sums of squares
// in double, block partials first and one block adding them in index order, so the result is reproducible.
namespace spamm {

struct ErrPartial {
    double diff, ref, own;
};

__global__ void __launch_bounds__(256)
error_norms_kernel(const float4 *__restrict__ ref, const float4 *__restrict__ own, size_t vecs,
                   ErrPartial *__restrict__ partials)
{
    double d = 0.0, r = 0.0, o = 0.0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += (size_t)gridDim.x * blockDim.x) {
        const float4 a = ref[i], b = own[i];
        const float e0 = a.x - b.x, e1 = a.y - b.y, e2 = a.z - b.z, e3 = a.w - b.w;
        d += (double)e0 * e0 + (double)e1 * e1 + (double)e2 * e2 + (double)e3 * e3;
        r += (double)a.x * a.x + (double)a.y * a.y + (double)a.z * a.z + (double)a.w * a.w;
        o += (double)b.x * b.x + (double)b.y * b.y + (double)b.z * b.z + (double)b.w * b.w;
    }
    __shared__ double sd[256], sr[256], so[256];
    sd[threadIdx.x] = d; sr[threadIdx.x] = r; so[threadIdx.x] = o;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if ((int)threadIdx.x < s) {
            sd[threadIdx.x] += sd[threadIdx.x + s];
            sr[threadIdx.x] += sr[threadIdx.x + s];
            so[threadIdx.x] += so[threadIdx.x + s];
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) partials[blockIdx.x] = ErrPartial{sd[0], sr[0], so[0]};
}

__global__ void error_norms_finish_kernel(const ErrPartial *__restrict__ partials, int n, double *__restrict__ out)
{
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        double d = 0.0, r = 0.0, o = 0.0;
        for (int i = 0; i < n; i++) {
            d += partials[i].diff;
            r += partials[i].ref;
            o += partials[i].own;
        }
        out[0] = sqrt(d);
        out[1] = sqrt(r);
        out[2] = sqrt(o);
    }
}

constexpr int ERR_BLOCKS = 148 * 4;

}  // namespace spamm

extern "C" size_t spamm_error_norms_scratch_bytes(void) { return sizeof(ErrPartial) * ERR_BLOCKS; }

extern "C" int spamm_error_norms_dev(const float *d_ref, const float *d_own, size_t elements, void *d_scratch,
                                     size_t scratch_bytes, double *d_out3, void *stream)
{
    if (!d_ref || !d_own || !d_scratch || !d_out3 || (elements & 3) || scratch_bytes < spamm_error_norms_scratch_bytes() ||
        (reinterpret_cast<uintptr_t>(d_ref) & 15) || (reinterpret_cast<uintptr_t>(d_own) & 15) ||
        (reinterpret_cast<uintptr_t>(d_scratch) & 7))
        return SPAMM_ERR_INVALID;
    error_norms_kernel<<<ERR_BLOCKS, 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const float4 *>(d_ref), reinterpret_cast<const float4 *>(d_own), elements / 4,
        static_cast<ErrPartial *>(d_scratch));
    error_norms_finish_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(static_cast<ErrPartial *>(d_scratch), ERR_BLOCKS,
                                                                 d_out3);
    SPAMM_CUDA_TRY(cudaGetLastError());
    return SPAMM_OK;
}

// ------------------------------------------------------------------------------------------------------------------
// The same count for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc when they need a count: a process whose framework has already
// taken all of HBM into its own caching pool, so that a raw allocation fails or fragments the pool; a serving loop
// that must not stall, since cudaMalloc and cudaFree synchronise the whole device; a plugin that is handed its
// buffers by its host and is forbidden to create more.  They still own the inputs (the two norm maps) and the
// outputs (the count and the sum); what they cannot supply is the work space for the per-block partial sums.  That
// work space lives here, in device memory that is part of the loaded library image: one fixed array per GPU, held
// from the moment the library is loaded on that GPU until the process exits.
namespace spamm {

constexpr int CV_STATIC_MAX_BLOCKS = 8192;   // 8192 partials x 16 B = 128 KiB per GPU

static __device__ __align__(256) unsigned char g_count_valid_scratch[CV_STATIC_MAX_BLOCKS * sizeof(CountPartial)];

// Device address of the array above, per CUDA device.  In host code the array's name is only a handle of the
// runtime, not an address a kernel can use, so the address is asked for once per device with that device current.
constexpr int CV_MAX_DEVICES = 64;
static CountPartial *g_cv_scratch_addr[CV_MAX_DEVICES] = {};

static int static_scratch_for_current_device(CountPartial **out)
{
    int dev = 0;
    SPAMM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= CV_MAX_DEVICES) {
        record_error_text("spamm_count_valid_static: device ordinal beyond 63");
        return SPAMM_ERR_UNSUPPORTED;
    }
    if (!g_cv_scratch_addr[dev]) {
        void *ptr = nullptr;
        SPAMM_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_count_valid_scratch));
        if (!ptr) {
            record_error_text("spamm_count_valid_static: the scratch array has no device address");
            return SPAMM_ERR_CUDA;
        }
        g_cv_scratch_addr[dev] = static_cast<CountPartial *>(ptr);
    }
    *out = g_cv_scratch_addr[dev];
    return SPAMM_OK;
}

}  // namespace spamm

extern "C" int spamm_count_valid_static_max_blocks(void) { return CV_STATIC_MAX_BLOCKS; }

extern "C" int spamm_count_valid_static(const float *d_norm_a, const float *d_norm_b, int row_tiles, int k_tiles,
                                        int n_tiles, float tau, unsigned long long *d_count, double *d_sum,
                                        void *stream)
{
    if (!d_norm_a || !d_norm_b || !d_count || row_tiles < 0 || k_tiles < 0 || n_tiles < 0) return SPAMM_ERR_INVALID;
    const int64_t blocks = count_valid_blocks(row_tiles, n_tiles);
    if (blocks > CV_STATIC_MAX_BLOCKS) {
        static thread_local char msg[224];
        snprintf(msg, sizeof(msg),
                 "spamm_count_valid_static: %lld partial sums needed (row_tiles * ceil(n_tiles/256)), the built-in "
                 "array holds %d; use spamm_count_valid_dev with caller scratch",
                 (long long)blocks, CV_STATIC_MAX_BLOCKS);
        record_error_text(msg);
        return SPAMM_ERR_UNSUPPORTED;
    }
    CountPartial *scratch = nullptr;
    int st = static_scratch_for_current_device(&scratch);
    if (st) return st;
    // Nothing in the array has to start at zero: every block of the first kernel overwrites its own slot and the
    // second kernel reads only the slots written by this call.
    return launch_count_valid(d_norm_a, d_norm_b, row_tiles, k_tiles, n_tiles, tau, scratch, d_count, d_sum,
                              (cudaStream_t)stream);
}
