// The plan object behind the C ABI (one GPU, one block of C tile rows), shared by the files that implement the
// plan-level entry points: plan.cu (single plan) and group.cu (several plans driven by one process).
#pragma once
#include <cstddef>

#include "common.cuh"

namespace spamm {

// The kernels' counters live at the head of the buffer that is cleared before every list build: one set for the
// whole block of rows, or one per chunk of rows when spamm_multiply pipelines the copies with the kernels.
using DeviceScalars = spamm_list_scalars;
constexpr int MAX_CHUNKS = 64;
constexpr size_t CHUNK_TARGET_BYTES = size_t(64) << 20;    // most rows of A copied per pipeline step
constexpr size_t CHUNK_MIN_BYTES = size_t(16) << 20;       // least

// Makes `dev` the current device for the lifetime of the object and restores the previous one.
struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev)
    {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) ok = cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard()
    {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

}  // namespace spamm

struct spamm_plan {
    int M = 0, K = 0, N = 0;            // padded to multiples of 32 (main.h:54-56): the sizes every kernel works on
    int in_M = 0, in_K = 0, in_N = 0;   // the caller's sizes: leading dimensions and extents of the host matrices
    int row_begin = 0, row_tiles = 0;   // in tiles
    int k_tiles = 0, n_tiles = 0, mi_n = 0, mj_n = 0;
    int device = 0;
    cudaStream_t stream = nullptr;
    float *d_a = nullptr, *d_b = nullptr, *d_c = nullptr;
    float *d_norm_a = nullptr, *d_norm_b = nullptr;
    int32_t *d_counts = nullptr, *d_step_counts = nullptr;
    uint32_t *d_steps = nullptr;
    uint8_t *d_half_a = nullptr, *d_half_b = nullptr;
    uint8_t *d_low_a = nullptr, *d_low_b = nullptr;     // split precision: packed half(x - half(x)), allocated on demand
    int precision = SPAMM_PRECISION_HALF;
    int32_t *d_order = nullptr;         // macro-tile visiting order of the multiply kernel
    int32_t *d_busy = nullptr;          // macro tiles that have steps
    uint32_t *d_tile_list = nullptr;    // tiles to convert to half
    void *d_list_scratch = nullptr;     // chunk maxima of the list builder
    uint8_t *d_cleared = nullptr;       // [spamm::DeviceScalars | need_a | need_b], cleared per list build
    size_t cleared_bytes = 0, need_a_off = 0, need_b_off = 0;
    spamm::DeviceScalars *h_scalars = nullptr; // pinned
    void *d_cv_scratch = nullptr;       // partial sums of the valid-product counter
    size_t cv_scratch_bytes = 0;
    void *d_err_scratch = nullptr;      // block partials + 3 doubles of spamm_error_norms
    unsigned long long *d_cv_count = nullptr;   // [count, sum(double)] on the device
    unsigned long long *h_cv = nullptr;         // pinned mirror of the two
    cudaEvent_t ev[8] = {};
    cudaStream_t stream_d2h = nullptr;  // second stream: copies C chunks out while the next chunk is computed
    cudaEvent_t ev_chunk[spamm::MAX_CHUNKS] = {};
    cudaStream_t stream_h2d = nullptr;  // third stream: uploads of the pipelined spamm_multiply, back to back
    cudaEvent_t ev_up[spamm::MAX_CHUNKS + 2] = {};      // [c]: rows of chunk c are on the GPU; [spamm::MAX_CHUNKS]: B is; [+1]: entry fence
    cudaEvent_t ev_zero[2] = {};        // fork / join of the early clearing of C on the second stream
    int zero_hint = -1;                 // last counters read: did at most a quarter of the macro tiles have steps
    bool c_zero_pending = false;        // C is being cleared on the second stream; the multiply writes busy tiles only
    int chunk_tiles = 0;                // tile rows per chunk of the pipelined spamm_multiply (multiple of 4)
    int n_chunks = 1;
    int32_t *d_order_chunk = nullptr, *d_order_last = nullptr;   // macro-tile orders for a full / the last chunk

    int active_scalars = 1;             // how many sets of counters the last operation used (one per chunk)
    bool queues_clean = false;          // the multiply's two work counters are zero (cleared by the list build or the packing kernel)
    void *d_gpair = nullptr;            // records of the gated two-SM multiply kernel, allocated when it is first chosen
    bool gpair_valid = false;           // they belong to the current lists
    float last_tau = 0.0f;              // threshold of the current lists
    int multiply_mode = 0;              // SPAMM_MULTIPLY_*: which multiply kernels may run, see spamm_plan_set_multiply_mode
    int gpair_hint = -1;                // last counters read: long lists in most macro tiles (-1: unknown)
    int dense_hint = -1;                // last counters read: were at least half of the macro tiles dense (-1: unknown)
    int pack_mode = SPAMM_PACK_AUTO;    // which tiles are converted to half, see spamm_plan_set_pack_mode
    int pack_all_hint = -1;             // last counters read: did the lists name at least half of all tiles (-1: unknown)
    bool packed_all = false;            // the last spamm_norms converted every tile: spamm_pack has nothing to do
    // peer exchange of B's norm-map shares (one process per GPU, see spamm_peer_attach)
    float *d_norm_b_buf[2] = {nullptr, nullptr};   // B's map, double buffered by step parity; d_norm_b is the current
    unsigned int *d_peer_flags = nullptr;          // [spamm::MAX_PEERS] arrival flags + [1] block counter of the push kernel
    int *d_peer_error = nullptr;
    int *h_peer_error = nullptr;                   // pinned
    int peer_world = 0, peer_rank = 0;
    unsigned int peer_epoch = 0;
    bool peer_wait_pending = false;
    void *peer_mapped[spamm::MAX_PEERS][3] = {};          // what cudaIpcOpenMemHandle returned, per peer
    float *peer_norm_b[spamm::MAX_PEERS][2] = {};
    unsigned int *peer_flags[spamm::MAX_PEERS] = {};      // every peer's arrival flags, as mapped into this process
    bool have_norms = false, have_lists = false, have_pack = false;
    int64_t launches = 0;
    bool multiply_chunked = false;      // which form the last plan_multiply_issue took

    spamm::DeviceScalars *scalars() const { return reinterpret_cast<spamm::DeviceScalars *>(d_cleared); }
    // rows of the caller's A (and C) that fall into this plan's block: the last block may end inside the padding
    int rows_in() const
    {
        const int64_t left = (int64_t)in_M - (int64_t)row_begin * spamm::TILE;
        const int64_t mine = (int64_t)row_tiles * spamm::TILE;
        return (int)(left < 0 ? 0 : (left < mine ? left : mine));
    }
    bool padded() const { return in_M != M || in_K != K || in_N != N; }
    uint8_t *need_a() const { return d_cleared + need_a_off; }
    uint8_t *need_b() const { return d_cleared + need_b_off; }
    size_t bytes_a() const { return sizeof(float) * (size_t)row_tiles * spamm::TILE * K; }
    size_t bytes_b() const { return sizeof(float) * (size_t)K * N; }
    size_t bytes_c() const { return sizeof(float) * (size_t)row_tiles * spamm::TILE * N; }
    size_t bytes_norm_a() const { return sizeof(float) * (size_t)row_tiles * k_tiles; }
    size_t bytes_norm_b() const { return sizeof(float) * (size_t)k_tiles * n_tiles; }
    size_t bytes_counts() const { return sizeof(int32_t) * (size_t)row_tiles * n_tiles; }
    size_t n_mt() const { return (size_t)mi_n * mj_n; }
    size_t step_cap() const { return (size_t)spamm::STEP_CAP_PER_K * k_tiles; }
    size_t bytes_steps() const { return sizeof(uint32_t) * n_mt() * step_cap(); }
    size_t bytes_step_counts() const { return sizeof(int32_t) * n_mt(); }
    size_t bytes_half_a() const { return (size_t)mi_n * k_tiles * spamm::A_SLAB_BYTES; }
    size_t bytes_half_b() const { return (size_t)k_tiles * mj_n * spamm::B_SLAB_BYTES; }
};


namespace spamm {

// Direct form of spamm_peer_attach for plans of ONE process whose devices have peer access to each other enabled:
// plan `rank` of `world` learns the addresses of every plan's two norm maps of B and arrival flags.
int plan_attach_direct(spamm_plan *p, int world, int rank, spamm_plan *const *all);
// spamm_multiply in two halves, so that one host thread can keep several devices busy: `issue` queues the uploads, the
// kernels and the downloads (b == nullptr: B is resident, complete once `b_ready`, which may be null, has occurred),
// `finish` waits, reads the counters and fills the statistics.
int plan_multiply_issue(spamm_plan *p, const float *a_rows, const float *b, float *c_rows, float tau,
                        cudaEvent_t b_ready);
int plan_multiply_finish(spamm_plan *p, spamm_stats *stats);
// rows x cols floats between two matrices with their own leading dimensions, either direction; one flat copy when
// both are packed the same way
int copy_matrix(float *dst, size_t dst_ld, const float *src, size_t src_ld, size_t rows, size_t cols,
                cudaMemcpyKind kind, cudaStream_t stream);

}  // namespace spamm
