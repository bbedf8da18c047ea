// Shared constants and small helpers of the SpAMM kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include "../../include/spamm.h"

namespace spamm {

constexpr int TILE = SPAMM_TILE;                 // 32, LoNum of the reference (main.h:32)
constexpr int MT_R = SPAMM_MT_ROWS;              // C tiles per macro tile, vertically
constexpr int MT_C = SPAMM_MT_COLS;              // C tiles per macro tile, horizontally
constexpr int TILE_BYTES = TILE * TILE * 2;      // one packed half tile
constexpr int A_SLAB_BYTES = MT_R * TILE_BYTES;  // 8 KiB: 128 rows x 32 k
constexpr int B_SLAB_BYTES = MT_C * TILE_BYTES;  // 16 KiB: 256 columns x 32 k
constexpr int STEP_CAP_PER_K = 8;                // a k yields at most 8 steps (one per tile column)

// step word: bits 0-15 k, 16-19 row mask, 20-27 column mask
__host__ __device__ inline uint32_t step_pack(uint32_t k, uint32_t rows, uint32_t cols) {
    return (k & 0xffffu) | ((rows & 0xfu) << 16) | ((cols & 0xffu) << 20);
}
__host__ __device__ inline uint32_t step_k(uint32_t s) { return s & 0xffffu; }
__host__ __device__ inline uint32_t step_rows(uint32_t s) { return (s >> 16) & 0xfu; }
__host__ __device__ inline uint32_t step_cols(uint32_t s) { return (s >> 20) & 0xffu; }

__host__ __device__ inline int step_count_of(int32_t v) { return v & SPAMM_STEPS_MASK; }
__host__ __device__ inline bool step_list_dense(int32_t v) { return (v & SPAMM_STEPS_DENSE) != 0; }

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Records a CUDA error for spamm_last_cuda_error and maps it to a status.
int record_cuda_error(cudaError_t e, const char *what);
void record_error_text(const char *text);

// Peer-to-peer exchange of B's norm-map shares between the GPUs of one box (one process per GPU).
constexpr int MAX_PEERS = 8;
struct PeerTargets {
    float *map[MAX_PEERS];            // the norm map of B of every GPU (this one included), peer-mapped
    unsigned int *flags[MAX_PEERS];   // every GPU's arrival flags, one word per sender
    int n;
};
struct PeerWait {                     // what the list builder waits for before it reads B's map
    const unsigned int *flags;        // this GPU's arrival flags
    int n;                            // senders
    unsigned int epoch;               // value every flag must have reached
    int *error;                       // set when the wait runs out
    unsigned long long limit_ns;      // how long to wait
};
constexpr unsigned long long PEER_WAIT_LIMIT_NS = 2000000000ull;
int peer_wait_selftest_launch(const PeerWait &w, cudaStream_t stream);
// Stores `share` floats of this GPU's map of B (at d_local_share = t.map[rank] + map_offset) into every other GPU's map
// and raises this GPU's arrival flag, value `epoch`, on every GPU.
int push_share_launch(const float *d_local_share, int64_t share, int64_t map_offset, const PeerTargets &t, int rank,
                      unsigned int epoch, cudaStream_t stream);
// The norm maps of this GPU's rows of A and of its share of B's tile rows in one launch whose last block of the share
// also stores the share into every other GPU's map and raises the arrival flags (d_counter: one word, zero on entry).
int norm_map_pair_push_launch(const float *d_xa, int rows_a, int cols_a, int64_t lda, float *d_map_a, const float *d_xb,
                              int rows_b, int cols_b, int64_t ldb, float *d_local_share, int64_t map_offset,
                              const PeerTargets &t, int rank, unsigned int epoch, unsigned int *d_counter,
                              cudaStream_t stream);
// Both norm maps AND the half conversion of every tile of A and B in one launch (for mostly surviving workloads).
int norm_pack_pair_launch(const float *d_xa, int rows_a, int cols_a, int64_t lda, float *d_map_a, void *d_half_a,
                          const float *d_xb, int rows_b, int cols_b, int64_t ldb, float *d_map_b, void *d_half_b,
                          cudaStream_t stream);

// Internal launchers behind the extern "C" entry points, with the extras the plan uses to save launches:
//  - the list builder's first kernel can clear a region (counters + need flags) before the lists are built,
//  - the packing kernel can reset the multiply's two work counters, which the multiply launcher then leaves alone,
//  - the multiply can be told that C was cleared beforehand: it then writes only macro tiles that have steps.
int build_lists_launch(const float *d_norm_a, const float *d_norm_b, int row_tiles, int k_tiles, int n_tiles, float tau,
                       void *d_scratch, uint32_t *d_steps, int32_t *d_step_counts, int32_t *d_counts,
                       uint8_t *d_need_a, uint8_t *d_need_b, uint32_t *d_tile_list, int32_t *d_busy_list,
                       spamm_list_scalars *d_scalars, void *d_clear, size_t clear_bytes, int keep_scalars,
                       const PeerWait *wait, cudaStream_t stream);
int pack_half_launch(const float *d_a, const float *d_b, int row_tiles, int k_tiles, int n_tiles,
                     const uint32_t *d_tile_list, spamm_list_scalars *d_scalars, void *d_half_a, void *d_half_b,
                     void *d_low_a, void *d_low_b, bool reset_queues, cudaStream_t stream);
int gated_multiply_launch(const void *d_half_a, const void *d_half_b, const uint32_t *d_steps,
                          const int32_t *d_step_counts, const int32_t *d_order, const int32_t *d_busy_list,
                          spamm_list_scalars *d_scalars, int row_tiles, int k_tiles, int n_tiles, float *d_c,
                          int64_t ldc, bool reset_queues, int pairs, int mode, cudaStream_t stream,
                          const struct GpairArgs *gpair = nullptr);
// `pairs` of gated_multiply_launch: which kernel on pairs of SMs runs before the one-SM kernel
constexpr int GM_PAIRS_NONE = 0;    // none
constexpr int GM_PAIRS_DENSE = 1;   // dense macro tiles with dense neighbours (gated_multiply_pair.cu); a no-op below half dense
constexpr int GM_PAIRS_GATED = 2;   // every pair of macro-tile rows, gated (gated_multiply_gpair.cu)
// `mode` of gated_multiply_launch, a sum of:
constexpr int GM_C_ZEROED = 1;      // C was cleared beforehand (or holds a partial result): macro tiles without steps are left alone
constexpr int GM_ACCUMULATE = 2;    // the products are added to what C holds instead of replacing it
constexpr int GM_LOW_OPERAND = 4;   // with GM_ACCUMULATE: one operand is a scaled low part, the sum is scaled back first
// Split precision stores the low part of every element multiplied by this power of two (see pack_half.cu).
constexpr float SPLIT_LOW_SCALE = 2048.0f;

int gated_multiply_pair_launch(const void *d_half_a, const void *d_half_b, const int32_t *d_step_counts,
                               spamm_list_scalars *d_scalars, int row_tiles, int k_tiles, int n_tiles, float *d_c,
                               int64_t ldc, cudaStream_t stream);

// What the gated two-SM kernel needs beyond the lists: it derives its own per-pair records from the norm maps.
struct GpairArgs {
    const float *norm_a, *norm_b;   // the maps the lists were built from (norm_a: this block of rows)
    float tau;                      // and the threshold
    const void *chunk_max;          // the list builder's scratch (chunk maxima), still holding that build's values
    void *scratch;                  // gated_multiply_gpair_scratch_bytes(...) bytes, 16-byte aligned
    bool build;                     // the records are not there yet (first multiply on these lists)
};
size_t gated_multiply_gpair_scratch_bytes(int row_tiles, int k_tiles, int n_tiles);
int gated_multiply_gpair_launch(const void *d_half_a, const void *d_half_b, const float *d_norm_a, const float *d_norm_b,
                                float tau, const void *d_chunk_max, const int32_t *d_step_counts, void *d_scratch,
                                bool build_records, spamm_list_scalars *d_scalars, int row_tiles, int k_tiles,
                                int n_tiles, float *d_c, int64_t ldc, int mode, cudaStream_t stream);

// Per source file: load its kernels onto the current device now instead of at their first launch.
int preload_norm();
int preload_lists();
int preload_pack();
int preload_multiply();
int preload_multiply_pair();
int preload_multiply_gpair();

#define SPAMM_CUDA_TRY(call)                                                    \
    do {                                                                        \
        cudaError_t e__ = (call);                                               \
        if (e__ != cudaSuccess) return ::spamm::record_cuda_error(e__, #call);  \
    } while (0)

}  // namespace spamm
