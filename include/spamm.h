/*
 * spamm.h -- C ABI of libspamm.so, a B200 (sm_100a) engine for SpAMM
 * (Sparse Approximate Matrix Multiply) over 32x32 tiles:
 *
 *      C(i,j) = sum over k with  ||A(i,k)||_F * ||B(k,j)||_F >= tau  of  half(A(i,k)) * half(B(k,j))
 *
 * The reference benchmark (buaa-hipo/cuSpAMM) has no library interface: its boundary is a set of
 * compile-time constants plus four kernel launches issued by `main`.  Each entry point below names the
 * reference lines it stands in for (paths inside the reference project).
 *
 * Conventions
 *   - all matrices are row-major float with no gaps between rows (leading dimension = number of columns).  M, K, N
 *     need not be multiples of 32: the library pads them on the device, with zeros, to the next multiple, as the
 *     reference pads its sizes (main.h:54-56; it leaves the padding uninitialised, cuSpAMM.cu:410).  Host matrices
 *     keep the caller's sizes on the way in and out; norm maps, list lengths and device buffers have the padded ones;
 *   - a plan owns one GPU and one block of C tile rows [row_tile_begin, row_tile_begin+row_tile_count),
 *     which is the reference's per-device row split (cuSpAMM.cu:503,530 `main_row_offset`); one plan per
 *     process and GPU, a multi-GPU run is several plans;
 *   - every function returns a spamm_status (0 = success); nothing prints, exits or throws;
 *   - pointers named d_* are device pointers of the plan's GPU, all others are host pointers;
 *   - a plan is not thread-safe; calls on one plan are ordered on the plan's CUDA stream.  Different plans may be
 *     driven from different host threads: the only process-wide state are small per-device caches (SM counts, the
 *     address of the built-in scratch array) that every thread fills with the same values.
 */
#ifndef SPAMM_H
#define SPAMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SPAMM_TILE 32          /* LoNum, main.h:32 */
#define SPAMM_MT_ROWS 4        /* C tiles per macro tile, vertically (128 rows)  */
#define SPAMM_MT_COLS 8        /* C tiles per macro tile, horizontally (256 columns) */
#define SPAMM_STEPS_DENSE 0x40000000   /* flag bit in a macro tile's step count, see spamm_build_lists_dev */
#define SPAMM_STEPS_MASK  0x3fffffff

typedef enum spamm_status {
    SPAMM_OK = 0,
    SPAMM_ERR_INVALID = 1,      /* bad argument (null pointer, non-positive dimension, bad row block) */
    SPAMM_ERR_CUDA = 2,         /* a CUDA runtime call failed; see spamm_last_cuda_error */
    SPAMM_ERR_ALLOC = 3,        /* device or host allocation failed */
    SPAMM_ERR_DEVICE_WAIT = 4,  /* a bounded wait inside a kernel ran out; results are not valid */
    SPAMM_ERR_STATE = 5,        /* call out of order (e.g. multiply before build_lists) */
    SPAMM_ERR_UNSUPPORTED = 6,  /* not an sm_100 GPU, or a size beyond a documented limit */
    SPAMM_ERR_OVERFLOW = 7      /* a per-macro-tile step list did not fit (needs non-finite norms) */
} spamm_status;

typedef struct spamm_plan spamm_plan;

/* Per-call figures; times are CUDA-event milliseconds on the plan's stream. */
typedef struct spamm_stats {
    float ms_h2d;               /* host->device copies of A rows and B (spamm_multiply only) */
    float ms_norm;              /* both norm maps */
    float ms_lists;             /* skip-list build */
    float ms_pack;              /* float->half packing of the tiles some list names */
    float ms_multiply;          /* gated multiply, including writing every C tile */
    float ms_d2h;               /* device->host copy of the C rows (spamm_multiply only) */
    float ms_device_total;      /* norm + lists + pack + multiply, one event pair around all four */
    int64_t survivors;          /* S: tile products executed (== sum of the per-tile list lengths) */
    int64_t tile_products;      /* row_tile_count * (K/32) * (N/32) */
    int64_t steps;              /* entries of the macro-tile step lists the multiply kernel walked */
    int64_t packed_tiles_a;     /* A tiles converted to half this call */
    int64_t packed_tiles_b;     /* B tiles converted to half this call */
    double executed_flops;      /* 65536 * S */
} spamm_stats;

/*
 * Counters the list builder, the packing kernel and the multiply kernel keep in device memory (one per problem).
 * The caller of the kernel-level entry points clears the whole structure before spamm_build_lists_dev.
 */
typedef struct spamm_list_scalars {
    unsigned long long survivors;   /* S, written by the list builder */
    unsigned int tile_count;        /* end of this problem's entries in the list of tiles to convert to half */
    unsigned int tile_begin;        /* their beginning: set tile_begin = tile_count = n to append after n earlier entries */
    unsigned int busy_count;        /* entries of the list of macro tiles that have steps */
    unsigned int packed_a;          /* tiles of A converted by the packing kernel */
    unsigned int packed_b;          /* tiles of B converted by the packing kernel */
    unsigned int queue_busy;        /* work counters of the multiply kernels; every multiply call resets the three */
    unsigned int queue_all;
    unsigned int pair_done;         /* macro tiles the two-SM multiply kernel took care of in this call */
    unsigned int dense_count;       /* macro tiles whose list has every k with every row and column (list builder) */
    int32_t overflow;               /* non-zero: a step list did not fit; kept until spamm_sync has reported it */
    int32_t error;                  /* non-zero: a bounded wait of the multiply kernel ran out (which one); kept likewise */
} spamm_list_scalars;

/* Names for spamm_device_buffer. */
typedef enum spamm_buffer {
    SPAMM_BUF_A = 0,            /* float  [row_tile_count*32][K]   this plan's rows of A                      */
    SPAMM_BUF_B = 1,            /* float  [K][N]                                                               */
    SPAMM_BUF_C = 2,            /* float  [row_tile_count*32][N]   this plan's rows of C                      */
    SPAMM_BUF_NORM_A = 3,       /* float  [row_tile_count][K/32]                                               */
    SPAMM_BUF_NORM_B = 4,       /* float  [K/32][N/32]                                                         */
    SPAMM_BUF_COUNTS = 5,       /* int32  [row_tile_count][N/32]   list length of every C tile                 */
    SPAMM_BUF_STEPS = 6,        /* uint32 [macro tiles][step capacity]                                         */
    SPAMM_BUF_STEP_COUNTS = 7,  /* int32  [macro tiles]                                                        */
    SPAMM_BUF_HALF_A = 8,       /* packed half tiles of A (2 KiB each, see spamm_pack_half_dev)                */
    SPAMM_BUF_HALF_B = 9        /* packed half tiles of B                                                      */
} spamm_buffer;

/* ---------------------------------------------------------------- plan: the reference's `main` ---- */

/*
 * Replaces the compile-time configuration and per-device allocation of the reference:
 * inM/inK/inN (para.h:6-8), the row split over DEVICEDIM devices (para.h:9, cuSpAMM.cu:503,530) and
 * the cudaMallocManaged block (cuSpAMM.cu:433-451).  `device` is a CUDA ordinal.  Allocates every device
 * buffer the path needs; no later call allocates.  The row block is given in tiles of the padded M
 * (ceil(M/32) tile rows in all); a block that reaches into the padding simply holds fewer rows of the caller's A.
 */
int spamm_plan_create(spamm_plan **out, int M, int K, int N,
                      int row_tile_begin, int row_tile_count, int device);
int spamm_plan_destroy(spamm_plan *plan);

/*
 * Host->device copies (cuSpAMM.cu:449-450).  a_rows points at the FIRST ROW OF THIS PLAN'S BLOCK
 * (row_tile_begin*32 of the full matrix), leading dimension K (the caller's, unpadded), and holds the rows of the
 * caller's A that fall into the block; b is the whole of B (K x N, leading dimension N).  Either may be NULL
 * to leave that operand as it is.  Asynchronous on the plan's stream when the host memory is pinned.
 */
int spamm_upload(spamm_plan *plan, const float *a_rows, const float *b);

/*
 * The timed region of the reference (cuSpAMM.cu:458-546) in four steps, all asynchronous on the plan's
 * stream.  spamm_run issues the four in order.
 *   spamm_norms        both norm maps            (unroll_get_Fnorm_*, launches at cuSpAMM.cu:486,503)
 *   spamm_build_lists  skip lists for tau        (cuSpAMM.cu:302-334; tau is the float `Norm`, compared with >=)
 *   spamm_pack         half copies of the tiles that some list names (the reference converts every
 *                      element on the host at generation time, tool.cu:418)
 *   spamm_gated_multiply   C rows of this plan   (get_C_FP16_B32, cuSpAMM.cu:336-391)
 */
int spamm_norms(spamm_plan *plan);
int spamm_build_lists(spamm_plan *plan, float tau);
int spamm_pack(spamm_plan *plan);
int spamm_gated_multiply(spamm_plan *plan);
int spamm_run(spamm_plan *plan, float tau);
/* spamm_build_lists + spamm_pack + spamm_gated_multiply in one call (what follows the norm maps). */
int spamm_finish(spamm_plan *plan, float tau);

/*
 * spamm_norms with only tile rows [b_tile_begin, b_tile_begin+b_tile_count) of B's norm map computed here; the
 * caller fills the rest of SPAMM_BUF_NORM_B (e.g. an all-gather between the GPUs that each computed a share)
 * before spamm_build_lists.  The reference recomputes the whole map of B on every device (cuSpAMM.cu:486).
 */
int spamm_norms_share(spamm_plan *plan, int b_tile_begin, int b_tile_count);
/* The two halves of spamm_norms_share, so that the exchange of B's shares can run while A's map is computed. */
int spamm_norm_b_share(spamm_plan *plan, int b_tile_begin, int b_tile_count);
int spamm_norm_a(spamm_plan *plan);

/*
 * Exchange of B's norm-map shares without a collective call, for one process per GPU on one box.  Every process
 * exports three IPC handles of its plan (spamm_peer_handles: 3 x 64 bytes), gathers everybody's (any host-side
 * all-gather), and attaches them in rank order (spamm_peer_attach: world x 192 bytes, world <= 8).  From then on
 * spamm_norm_b_share_push computes this GPU's share of B's map and a second small kernel copies it into the map of
 * EVERY other GPU (plain 128-bit peer stores over NVLink), then raises a flag on every GPU; the next
 * spamm_build_lists waits, at most 2 s, until all shares of that step have arrived (SPAMM_ERR_DEVICE_WAIT from
 * spamm_sync otherwise).  B's map is double buffered by step, so a GPU may run one step ahead of the slowest.
 * Every process must make the same sequence of calls.  The reference recomputes all of B's map on every device
 * (cuSpAMM.cu:486).
 */
int spamm_peer_handles(spamm_plan *plan, void *out, size_t out_bytes);
int spamm_peer_attach(spamm_plan *plan, int world, int rank, const void *all_handles);
int spamm_norm_b_share_push(spamm_plan *plan, int b_tile_begin, int b_tile_count);
/*
 * One whole step of a GPU that shares the work on B's norm map with its peers (attached with spamm_peer_attach, or
 * plans of one spamm_group), in a single call: one launch computes the norm maps of this plan's rows of A and of tile
 * rows [b_tile_begin, b_tile_begin+b_tile_count) of B, a small kernel stores that share into every peer's map, then
 * lists (which wait for the peers' shares), packing and multiply follow as in spamm_finish.  Asynchronous.  This is
 * the per-device body of the reference's parallel region (cuSpAMM.cu:470-537) with B's map computed once instead of
 * once per device (cuSpAMM.cu:486).
 */
int spamm_run_shared(spamm_plan *plan, float tau, int b_tile_begin, int b_tile_count);
/* The first part of spamm_run_shared alone (the two norm maps and the store of the share); spamm_finish completes the step. */
int spamm_norms_shared(spamm_plan *plan, int b_tile_begin, int b_tile_count);
/*
 * Exercises the bounded device-side wait of the exchange on one GPU: a small kernel waits for arrival flags of
 * `senders` GPUs that nothing will ever set, gives up after limit_ms (1..5000) and reports it.  Returns
 * SPAMM_ERR_DEVICE_WAIT when the wait ran out as it should (the plan stays usable), SPAMM_OK if it did not.
 */
int spamm_peer_wait_selftest(spamm_plan *plan, int senders, unsigned int limit_ms);

/* Waits for the plan's stream, then reports a device-side wait that ran out (SPAMM_ERR_DEVICE_WAIT) or SPAMM_OK. */
int spamm_sync(spamm_plan *plan);

/* Device->host copy of this plan's rows of C (the caller's N columns, leading dimension N) into c_rows; blocking. */
int spamm_download_c(spamm_plan *plan, float *c_rows);

/*
 * One call for the whole driver loop body with float host matrices in and out: upload, norms, lists, pack,
 * multiply, download; blocking.
 * a_rows / c_rows are this plan's row block, b is all of B.  stats may be NULL.
 * Blocks of more than 16 MiB of A are processed in chunks of rows (16 to 64 MiB) so that the upload of the next chunk, the
 * kernels of the current one and the download of the previous one overlap (use pinned host memory for that); the
 * phases then interleave and only ms_device_total (the whole call, copies included), ms_h2d (B alone) and the
 * counts are reported.  After such a call spamm_gated_multiply needs a new spamm_build_lists.
 */
int spamm_multiply(spamm_plan *plan, const float *a_rows, const float *b, float *c_rows,
                   float tau, spamm_stats *stats);

/*
 * The two halves of spamm_multiply for callers that assemble B on the GPU themselves (several GPUs that each upload a
 * share of B over their own PCIe link and exchange the shares over NVLink; the reference copies all of B to every
 * device, cuSpAMM.cu:449-450).
 *   spamm_upload_b_rows        rows [row_begin, row_begin+rows) of B (leading dimension N) into the plan's copy of B,
 *                              asynchronous on the plan's stream;
 *   spamm_multiply_b_resident  spamm_multiply without the upload of B: the rows of A go up, the path runs and the
 *                              rows of C come down, pipelined in chunks as in spamm_multiply.  b_ready_event (a
 *                              cudaEvent_t, may be NULL) is an event after which B is complete in the plan's buffer;
 *                              the uploads of A do not wait for it, the first kernel that reads B does.
 */
int spamm_upload_b_rows(spamm_plan *plan, const float *b_rows, int row_begin, int rows);
int spamm_multiply_b_resident(spamm_plan *plan, const float *a_rows, float *c_rows, float tau, void *b_ready_event,
                              spamm_stats *stats);

/*
 * Tile rows per chunk of the pipelined spamm_multiply (a multiple of 4; at most 64 chunks).  The default is an eighth
 * of the block, between 16 and 64 MiB of A.  A value >= the plan's row_tile_count turns the pipelining off.
 */
int spamm_plan_set_chunk_tiles(spamm_plan *plan, int tiles);

/*
 * Precision of the tile products.
 *   SPAMM_PRECISION_HALF   (default) operands rounded to half, float accumulation: the reference's tensor-core build
 *                          (USINGHALF 1, cuSpAMM.cu:276-392).
 *   SPAMM_PRECISION_SPLIT  float-level accuracy on the tensor cores, in place of the reference's CUDA-core float
 *                          build (USINGHALF 0: cuSpAMM.cu:126-274).  Every operand element x is split as
 *                          hi = half(x), lo = half(2^11 * (x - hi)); the product is hi*hi + 2^-11 * (hi*lo + lo*hi),
 *                          three tensor-core passes over the same lists, float accumulation (lo*lo, about 2^-22 of
 *                          the result, is dropped).  The scaling keeps the low part out of half's subnormal range,
 *                          so the mode holds for elements down to about 3e-11 in magnitude (half alone: 6e-8).
 *                          Norm maps and lists are the same in both modes; the multiply takes about three times as
 *                          long.
 * Takes effect at the next spamm_pack; allocates a second set of packed-tile buffers the first time.
 */
enum { SPAMM_PRECISION_HALF = 0, SPAMM_PRECISION_SPLIT = 1 };
int spamm_plan_set_precision(spamm_plan *plan, int precision);

/*
 * Optional, for callers that issue the steps one by one (spamm_run and spamm_finish do this themselves): announces
 * that the rest of a whole step (lists, pack, multiply) follows.  If the counters read back by the last spamm_sync /
 * spamm_run_timed showed that at most a quarter of the 128 x 256 blocks of C received any product, all of C is
 * cleared now with a memset on the plan's second stream, beside the work of the main stream, and the next
 * spamm_gated_multiply writes only the blocks that receive products; otherwise nothing happens.  The result is
 * the same either way.  The reference writes every C tile from its multiply kernel (cuSpAMM.cu:381-390).
 */
int spamm_clear_c_early(spamm_plan *plan);

/*
 * Which tiles spamm_norms / spamm_pack convert to half.  The reference converts whole matrices on the host when it
 * generates them (tool.cu:418); here the conversion runs on the GPU inside the timed step:
 *   SPAMM_PACK_LISTED  only the tiles some skip list names, by spamm_pack (best when few products survive);
 *   SPAMM_PACK_ALL     every tile, by spamm_norms while it has the tile in registers (best when most survive:
 *                      the matrices are read once instead of twice); spamm_pack then launches nothing;
 *   SPAMM_PACK_AUTO    (default) LISTED, until counters read back by spamm_sync / spamm_run_timed show that the
 *                      lists named at least half of all tiles; then ALL, until they show otherwise.
 * Results are identical in every mode.
 */
enum { SPAMM_PACK_AUTO = 0, SPAMM_PACK_LISTED = 1, SPAMM_PACK_ALL = 2 };
int spamm_plan_set_pack_mode(spamm_plan *plan, int mode);

/*
 * Which multiply kernels spamm_gated_multiply may use.  Results are the same in every mode (up to the order of the float
 * additions inside the tensor cores).
 *   SPAMM_MULTIPLY_AUTO         (default) by the counters of the plan's previous step: mostly dense macro tiles go to
 *                               pairs of SMs ungated (four macro tiles per pair), everything else to the one-SM kernel;
 *   SPAMM_MULTIPLY_ONE_SM       the one-SM kernel only;
 *   SPAMM_MULTIPLY_GATED_PAIRS  the gated kernel on pairs of SMs for every pair of macro-tile rows: two vertically
 *                               adjacent macro tiles share the tiles of B they load, a third less traffic from L2
 *                               into the SMs.  Allocates 16 bytes per k and pair of macro tiles at first use.  Not
 *                               chosen automatically: as measured it is slower than the one-SM kernel.
 */
enum { SPAMM_MULTIPLY_AUTO = 0, SPAMM_MULTIPLY_ONE_SM = 1, SPAMM_MULTIPLY_GATED_PAIRS = 2 };
int spamm_plan_set_multiply_mode(spamm_plan *plan, int mode);

/* Same as spamm_run but records per-phase events; blocking.  Inputs must already be resident. */
int spamm_run_timed(spamm_plan *plan, float tau, spamm_stats *stats);

/* Readbacks used by the parity tests (blocking).  Sizes as in spamm_buffer. */
int spamm_get_norm_a(spamm_plan *plan, float *out);
int spamm_get_norm_b(spamm_plan *plan, float *out);
int spamm_get_counts(spamm_plan *plan, int32_t *out, int64_t *survivors);
/*
 * The skip lists the multiply kernel actually walks, expanded to the per-C-tile form of the reference
 * (sC_offset, cuSpAMM.cu:315-326): offsets has row_tile_count*(N/32)+1 entries, k_idx[offsets[t]..offsets[t+1])
 * are the surviving k of tile t (row-major tile order inside this plan's block), ascending.
 * Call once with k_idx == NULL to learn offsets (and the total in offsets[last]).
 */
int spamm_get_lists(spamm_plan *plan, int64_t *offsets, int32_t *k_idx);

/*
 * Number of tile products of this plan's block whose norm product is >= tau, and the sum of all norm products:
 * the reference's countValid (tool.cu:493-529) as two kernels over the norm maps.  Needs spamm_norms; blocking.
 */
int spamm_count_valid(spamm_plan *plan, float tau, int64_t *count, double *sum_of_products);
/*
 * The three Frobenius norms the reference's comparator prints (COUNTERRTRANS, tool.cu:6-24, used by
 * check_simple_gpu, tool.cu:227-280): out3 = { ||ref - C||, ||ref||, ||C|| } over this plan's rows of C, where
 * d_reference is a device matrix of the same shape (e.g. the dense product: the same plan run with tau = 0 and its
 * C copied aside, or a cuBLAS result).  Blocking.
 */
int spamm_error_norms(spamm_plan *plan, const float *d_reference, double out3[3]);
/*
 * Threshold for a wanted valid ratio: the reference's tuneValidRate (tool.cu:438-490) -- first guess the mean norm
 * product, then bisection until |ratio - expected_rate| < tolerance or max_iters passes (ExpectedRate 0.75,
 * TUNINGERROR 0.01, TUNINGTIME 20 in main.h:35-38) -- with every count done on the GPU.  Needs spamm_norms; blocking.
 * *tau is the value to pass to spamm_build_lists; *rate the ratio of the last count; *iters the passes used.
 */
int spamm_tune_tau(spamm_plan *plan, double expected_rate, int max_iters, double tolerance, float *tau,
                   double *rate, int *iters);

/* Raw access for callers that move data between GPUs themselves (NCCL broadcast of B and of its norm map). */
int spamm_device_buffer(spamm_plan *plan, int which, void **d_ptr, size_t *bytes);
/* The plan's cudaStream_t, as an opaque pointer. */
int spamm_stream(spamm_plan *plan, void **stream);
int spamm_plan_dims(spamm_plan *plan, int *M, int *K, int *N, int *row_tile_begin, int *row_tile_count);

/* ---------------------------------------------------------------- several GPUs, one process ------- */

/*
 * The reference drives DEVICEDIM GPUs from one process (para.h:9): per-device plans and full replicas of A and B
 * (cuSpAMM.cu:404-451), one host thread per device in the timed region (cuSpAMM.cu:470-537), every device computing
 * all of B's norm map (cuSpAMM.cu:486), no gather of C.  A spamm_group is that, for one host thread and with the
 * redundancy removed: device d owns C tile rows [d*T/G, (d+1)*T/G) (boundaries on multiples of 4 tile rows), only its
 * rows of A are uploaded to it, every device uploads 1/G of B over its own PCIe link and the shares are exchanged with
 * peer-to-peer copies over NVLink, every device computes 1/G of B's norm map per step and stores it into the other
 * devices' maps (plain peer stores; the list builder waits, at most 2 s, for all shares), and every device copies its
 * rows of C into its slice of the host result.  Needs peer access between all devices of the group
 * (SPAMM_ERR_UNSUPPORTED otherwise); n_devices 1..8; device_ids NULL means 0..n_devices-1.  K/32 need not divide
 * by n_devices (the shares of B then differ by one tile row).  Not thread-safe; one host thread drives all devices.
 */
typedef struct spamm_group spamm_group;
int spamm_group_create(spamm_group **out, int M, int K, int N, int n_devices, const int *device_ids);
int spamm_group_destroy(spamm_group *group);
int spamm_group_size(spamm_group *group);
/* Plan of device i of the group (owned by the group), for the read-backs above and for spamm_plan_dims. */
int spamm_group_plan(spamm_group *group, int i, spamm_plan **plan);
/* Host->device: the rows of A to their owners, B by shares + exchange.  Either may be NULL.  Asynchronous. */
int spamm_group_upload(spamm_group *group, const float *a, const float *b);
/* One step of the timed region on every device (spamm_run_shared per device; spamm_run for a group of one). */
int spamm_group_run(spamm_group *group, float tau);
/* Waits for every device; the first failure of any device is returned. */
int spamm_group_sync(spamm_group *group);
/* Device->host: every device's rows of C into c (M x N, leading dimension N); blocking. */
int spamm_group_download_c(spamm_group *group, float *c);
/* Sum of the devices' surviving products of the last step; blocking. */
int spamm_group_survivors(spamm_group *group, int64_t *survivors);
/*
 * Host matrices in and out on all devices: B by shares and exchange, then per device the pipelined upload of its rows
 * of A, the path, and the download of its rows of C (spamm_multiply_b_resident); blocking.  stats (may be NULL)
 * receives the sums of the counts and, as ms_device_total, the slowest device's time.
 */
int spamm_group_multiply(spamm_group *group, const float *a, const float *b, float *c, float tau, spamm_stats *stats);

/* ---------------------------------------------------------------- kernels on caller memory -------- */
/* `stream` is a cudaStream_t passed as void*; all launches are asynchronous. */

/*
 * Frobenius-norm map of a row-major float matrix (rows x cols, leading dimension ld elements):
 * d_map[(r/32)*(cols/32) + c/32] = sqrt(sum of squares of the tile).  Replaces unroll_get_Fnorm_pri
 * (cuSpAMM.cu:21-71) and, as the contract is float norms of float data, unroll_get_Fnorm_FP16 (cuSpAMM.cu:74-123).
 * d_x must be 16-byte aligned and ld a multiple of 4.
 */
int spamm_norm_map_dev(const float *d_x, int rows, int cols, int64_t ld, float *d_map, void *stream);
/* The same for two matrices in one launch (the A rows and B of one step). */
int spamm_norm_map_pair_dev(const float *d_xa, int rows_a, int cols_a, int64_t lda, float *d_map_a,
                            const float *d_xb, int rows_b, int cols_b, int64_t ldb, float *d_map_b, void *stream);

/*
 * Skip-list build (cuSpAMM.cu:302-334) for row_tiles x (N/32) C tiles.  For every macro tile of
 * SPAMM_MT_ROWS x SPAMM_MT_COLS C tiles it writes a list of steps, ascending in k; a step is
 *     bits 0-15  k,   bits 16-19  which of the 4 tile rows take part,   bits 20-27  which of the 8 tile columns,
 * and every (row, column) pair of a step is a surviving product, every surviving product is in exactly one step.
 * The norm maps must be non-negative (they are norms).
 *   d_scratch      work space of spamm_build_lists_scratch_bytes(...) bytes (chunk maxima used for pruning)
 *   d_steps        8*(K/32) words per macro tile, macro tiles in row-major order
 *   d_step_counts  [macro tiles] number of steps written, in bits 0-29; bit 30 (SPAMM_STEPS_DENSE) is set when the
 *                  list holds every k and every step names all 4 rows and 8 columns (a dense macro tile)
 *   d_counts       [row_tiles][N/32] per-tile list lengths
 *   d_need_a/_b    one byte per A slab of 4 tiles / B slab of 8 tiles, a bit per tile that some step names;
 *                  zero on entry, or the flags an earlier call on other rows of A left (tiles of B that are flagged
 *                  already are not listed again); the arrays are accessed in aligned 4-byte words, so keep them
 *                  padded to a multiple of 4 bytes
 *   d_tile_list    every named tile once: bit 31 = tile of B, bits 3-30 = slab index, bits 0-2 = tile in the slab;
 *                  room for (4*ceil(row_tiles/4) + 8*ceil(n_tiles/8)) * (K/32) entries
 *   d_busy_list    the macro tiles with at least one step, in no particular order; room for all macro tiles
 *   d_scalars      zero on entry; receives S, the two list lengths and the overflow flag
 */
size_t spamm_build_lists_scratch_bytes(int row_tiles, int k_tiles, int n_tiles);
int spamm_build_lists_dev(const float *d_norm_a, const float *d_norm_b, int row_tiles, int k_tiles, int n_tiles,
                          float tau, void *d_scratch, uint32_t *d_steps, int32_t *d_step_counts, int32_t *d_counts,
                          uint8_t *d_need_a, uint8_t *d_need_b, uint32_t *d_tile_list, int32_t *d_busy_list,
                          spamm_list_scalars *d_scalars, void *stream);

/*
 * float -> half (round to nearest even, as __float2half at tool.cu:418) of the listed 32x32 tiles into the
 * packed layout the multiply kernel loads: every tile is 2 KiB,
 *     byte offset of element (o, kk) = (o/8)*512 + (kk/8)*128 + (o%8)*16 + (kk%8)*2,
 * o = row of an A tile / column of a B tile, kk = the index that is summed over.  A tiles are grouped
 * 4 (rows) to a slab, slabs ordered [row group][k]; B tiles 8 (columns) to a slab, slabs ordered [k][column group].
 * d_tile_list and d_scalars->tile_begin / tile_count come from spamm_build_lists_dev.
 */
int spamm_pack_half_dev(const float *d_a, const float *d_b, int row_tiles, int k_tiles, int n_tiles,
                        const uint32_t *d_tile_list, spamm_list_scalars *d_scalars, void *d_half_a, void *d_half_b,
                        void *stream);

/*
 * Gated multiply (get_C_FP16_B32, cuSpAMM.cu:336-391): walks the step lists, multiplies on the tensor cores
 * (half inputs, float accumulation) and writes every C tile of the block, zeros where a list is empty.
 * Two kernels are launched: when at least half of the macro tiles are dense, vertically adjacent dense ones are
 * multiplied by pairs of SMs (one 256 x 256 tensor-core tile per pair); everything else goes through the
 * one-SM kernel.
 * d_order (may be NULL = row-major) is a permutation of the macro-tile indices: the order in which the resident
 * blocks take macro tiles from the work queue; spamm_macro_tile_order fills one that keeps concurrently processed
 * macro tiles close together in both directions, so that they share operand tiles in L2.  When few macro tiles
 * have steps, those (d_busy_list) are taken first.
 * d_scalars->error is set non-zero if a bounded device wait ran out.
 */
int spamm_gated_multiply_dev(const void *d_half_a, const void *d_half_b, const uint32_t *d_steps,
                             const int32_t *d_step_counts, const int32_t *d_order, const int32_t *d_busy_list,
                             spamm_list_scalars *d_scalars, int row_tiles, int k_tiles, int n_tiles, float *d_c,
                             int64_t ldc, void *stream);
/* Host helper: writes the macro-tile order described above into order[ceil(row_tiles/4)*ceil(n_tiles/8)]. */
int spamm_macro_tile_order(int row_tiles, int n_tiles, int32_t *order);

/*
 * countValid (tool.cu:493-529) on caller memory: *d_count = #{(i,k,j): nA(i,k)*nB(k,j) >= tau}, *d_sum (may be
 * NULL) = the sum of all products in double.  d_scratch is work space of at least
 * spamm_count_valid_scratch_bytes(row_tiles, n_tiles) bytes, 16-byte aligned; its contents are overwritten.
 */
size_t spamm_count_valid_scratch_bytes(int row_tiles, int n_tiles);
int spamm_count_valid_dev(const float *d_norm_a, const float *d_norm_b, int row_tiles, int k_tiles, int n_tiles,
                          float tau, void *d_scratch, size_t scratch_bytes, unsigned long long *d_count,
                          double *d_sum, void *stream);

/* The error norms on caller memory; d_scratch holds spamm_error_norms_scratch_bytes() bytes, d_out3 three doubles. */
size_t spamm_error_norms_scratch_bytes(void);
int spamm_error_norms_dev(const float *d_ref, const float *d_own, size_t elements, void *d_scratch,
                          size_t scratch_bytes, double *d_out3, void *stream);

/*
 * spamm_count_valid_dev without caller scratch and without any allocation.  No counterpart in the reference: it
 * exists for hosts that cannot call cudaMalloc at this point (all of HBM already sits in their framework's own
 * pool; a serving loop that must not hit the device-wide synchronisation of cudaMalloc/cudaFree; a plugin that
 * may only use the buffers it is handed).  The caller still passes the norm maps and the two outputs; the
 * per-block partial sums go to a fixed 128 KiB array inside the library image, which every GPU that loads the
 * library holds until the process exits.
 * Limit: row_tiles * ceil(n_tiles/256) <= spamm_count_valid_static_max_blocks() (8192; a square N=32768 problem
 * needs 4096).  Larger problems are refused with SPAMM_ERR_UNSUPPORTED and a message in spamm_last_cuda_error.
 * The first call on a GPU looks up the array's device address (with that GPU current); make that first call
 * outside any stream capture.  All calls on one GPU share the array and it keeps the previous call's contents
 * (nothing in it needs clearing): two calls that overlap on the GPU -- different streams, or different host
 * threads -- race on it and must be ordered by the caller.
 */
int spamm_count_valid_static(const float *d_norm_a, const float *d_norm_b, int row_tiles, int k_tiles, int n_tiles,
                             float tau, unsigned long long *d_count, double *d_sum, void *stream);
int spamm_count_valid_static_max_blocks(void);

/* ---------------------------------------------------------------- generators and misc ------------- */

/*
 * Input generators of the reference (host side, float out):
 *   spamm_gen_decay_exp  a_ij = c * v^|i-j|          (getDecayMatrixExp, tool.cu:409-422)
 *   spamm_gen_decay_alg  a_ij = c / (|i-j|^v + 1)    (getDecayMatrixAlg, tool.cu:426-436)
 *   spamm_gen_ones       a_ij = 1                    (getNormMatrix, tool.cu:370-406: every tile norm is 32)
 * and seeded variants used by the benchmark configurations (sign or magnitude drawn from a counter-based
 * hash of (seed, i, j), so any block of rows can be generated independently):
 *   spamm_gen_signed_exp    a_ij = s_ij * exp(-lambda*|i-j|),  s_ij = +-1
 *   spamm_gen_uniform_alg   a_ij = u_ij / (|i-j|^2 + 1),       u_ij uniform in [-1,1)
 *   spamm_gen_uniform       a_ij = u_ij,                       u_ij uniform in [-1,1)
 *   spamm_gen_lattice       a_ij = u * exp(-|r_i - r_j|), points on an L^3 cubic grid in lexicographic order,
 *                           u uniform in [0.5,1) with a random sign, symmetric (hash of (min(i,j), max(i,j)))
 * Rows [row_begin, row_begin+rows) of an (.. x cols) matrix are written to `out` (leading dimension cols).
 */
int spamm_gen_decay_exp(float *out, float c, float v, int64_t row_begin, int64_t rows, int64_t cols);
int spamm_gen_decay_alg(float *out, float c, float v, int64_t row_begin, int64_t rows, int64_t cols);
int spamm_gen_ones(float *out, int64_t row_begin, int64_t rows, int64_t cols);
int spamm_gen_signed_exp(float *out, double lambda, uint64_t seed, int64_t row_begin, int64_t rows, int64_t cols);
int spamm_gen_uniform_alg(float *out, uint64_t seed, int64_t row_begin, int64_t rows, int64_t cols);
int spamm_gen_uniform(float *out, uint64_t seed, int64_t row_begin, int64_t rows, int64_t cols);
int spamm_gen_lattice(float *out, int L, uint64_t seed, int64_t row_begin, int64_t rows);

const char *spamm_status_string(int status);
/* Text of the last CUDA error seen by this thread inside the library ("" if none). */
const char *spamm_last_cuda_error(void);
/* Launches counted since the plan was created (kernels of this library only). */
int64_t spamm_kernel_launches(spamm_plan *plan);

#ifdef __cplusplus
}
#endif
#endif /* SPAMM_H */
