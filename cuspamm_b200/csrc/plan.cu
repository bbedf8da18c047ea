// Host side of the C ABI: the plan object that replaces the reference's `main` (cuSpAMM.cu:395-556) --
// configuration, per-device buffers, the timed loop body and its event timing.
#include <cmath>
#include <cstddef>
#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "plan.cuh"

namespace spamm {

static thread_local std::string g_last_cuda_error;

int record_cuda_error(cudaError_t e, const char *what)
{
    g_last_cuda_error = std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
    if (e == cudaErrorMemoryAllocation) return SPAMM_ERR_ALLOC;
    return SPAMM_ERR_CUDA;
}

// Stores a detail message for spamm_last_cuda_error when the failing call is not a CUDA runtime call.
void record_error_text(const char *text) { g_last_cuda_error = text; }

int copy_matrix(float *dst, size_t dst_ld, const float *src, size_t src_ld, size_t rows, size_t cols,
                cudaMemcpyKind kind, cudaStream_t stream)
{
    if (rows == 0 || cols == 0) return SPAMM_OK;
    if (dst_ld == cols && src_ld == cols)
        SPAMM_CUDA_TRY(cudaMemcpyAsync(dst, src, sizeof(float) * rows * cols, kind, stream));
    else
        SPAMM_CUDA_TRY(cudaMemcpy2DAsync(dst, sizeof(float) * dst_ld, src, sizeof(float) * src_ld, sizeof(float) * cols,
                                         rows, kind, stream));
    return SPAMM_OK;
}

int plan_attach_direct(spamm_plan *p, int world, int rank, spamm_plan *const *all)
{
    if (!p || !all || world < 2 || world > MAX_PEERS || rank < 0 || rank >= world) return SPAMM_ERR_INVALID;
    if (p->peer_world) return SPAMM_ERR_STATE;
    for (int r = 0; r < world; r++) {
        if (!all[r] || all[r]->k_tiles != p->k_tiles || all[r]->n_tiles != p->n_tiles) return SPAMM_ERR_INVALID;
        p->peer_norm_b[r][0] = all[r]->d_norm_b_buf[0];
        p->peer_norm_b[r][1] = all[r]->d_norm_b_buf[1];
        p->peer_flags[r] = all[r]->d_peer_flags;
    }
    p->peer_world = world;
    p->peer_rank = rank;
    return SPAMM_OK;
}

}  // namespace spamm

using namespace spamm;

namespace {

template <typename T>
int dev_alloc(T **p, size_t bytes)
{
    *p = nullptr;
    if (bytes == 0) bytes = 16;
    cudaError_t e = cudaMalloc(reinterpret_cast<void **>(p), bytes);
    if (e != cudaSuccess) {
        record_cuda_error(e, "cudaMalloc");
        return SPAMM_ERR_ALLOC;
    }
    return SPAMM_OK;
}

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Zeroes the counters and need flags the list builder starts from, except the error and overflow words of every set
// of counters: those stay until read_scalars has shown them to the host.
int clear_list_state(spamm_plan *p, cudaStream_t stream)
{
    const size_t head = sizeof(DeviceScalars) * MAX_CHUNKS;
    SPAMM_CUDA_TRY(cudaMemset2DAsync(p->d_cleared, sizeof(DeviceScalars), 0, offsetof(DeviceScalars, overflow),
                                     MAX_CHUNKS, stream));
    SPAMM_CUDA_TRY(cudaMemsetAsync(p->d_cleared + head, 0, p->cleared_bytes - head, stream));
    return SPAMM_OK;
}

int read_scalars(spamm_plan *p)
{
    SPAMM_CUDA_TRY(cudaMemcpyAsync(p->h_scalars, p->scalars(), sizeof(DeviceScalars) * MAX_CHUNKS,
                                   cudaMemcpyDeviceToHost, p->stream));
    // the error and overflow words are sticky on the device (a list build does not clear them, so a failure in an
    // earlier step of a queue of steps is still there); now that the host has them, they start afresh
    SPAMM_CUDA_TRY(cudaMemset2DAsync(&p->scalars()->overflow, sizeof(DeviceScalars), 0, 2 * sizeof(int32_t), MAX_CHUNKS,
                                     p->stream));
    if (p->peer_world > 1) {
        SPAMM_CUDA_TRY(cudaMemcpyAsync(p->h_peer_error, p->d_peer_error, sizeof(int), cudaMemcpyDeviceToHost,
                                       p->stream));
        SPAMM_CUDA_TRY(cudaMemsetAsync(p->d_peer_error, 0, sizeof(int), p->stream));
    }
    SPAMM_CUDA_TRY(cudaStreamSynchronize(p->stream));
    // remember whether these lists were mostly dense: the next multiply launches the paired kernel only then
    // (a wrong guess costs speed, never correctness: the one-SM kernel is told whether the paired one ran)
    unsigned long long dense = 0;
    for (int c = 0; c < p->active_scalars; c++) dense += p->h_scalars[c].dense_count;
    p->dense_hint = (dense * 2 >= p->n_mt() && p->n_mt() > 0) ? 1 : 0;
    // and whether they were long lists in most macro tiles (at least 1024 surviving products per macro tile that has
    // any, i.e. 32 full steps' worth): the traffic from L2 into the SMs then bounds the multiply, and the gated kernel
    // on pairs of SMs, which shares the tiles of B between two macro tiles, is the faster one
    {
        unsigned long long busy = 0, surv = 0;
        for (int c = 0; c < p->active_scalars; c++) {
            busy += p->h_scalars[c].busy_count;
            surv += p->h_scalars[c].survivors;
        }
        p->gpair_hint = (p->have_lists && busy * 2 >= p->n_mt() && busy > 0 && surv >= 1024ull * busy) ? 1 : 0;
    }
    // and whether few macro tiles had steps: the next step then clears C with a memset on the second stream while
    // the lists are built and the tiles converted (kernels that leave the memory system idle), and its multiply
    // writes only the macro tiles that have steps
    if (p->have_lists && p->active_scalars == 1)
        p->zero_hint = ((unsigned long long)p->h_scalars[0].busy_count * 4ull <= p->n_mt()) ? 1 : 0;
    // and whether they named most of the operand tiles: the next spamm_norms then converts all tiles while it has
    // them in registers instead of leaving the named ones to a second pass over the matrices
    if (p->have_lists && p->active_scalars == 1) {
        const unsigned long long named = p->h_scalars[0].tile_count - p->h_scalars[0].tile_begin;
        const unsigned long long all = (unsigned long long)p->row_tiles * p->k_tiles +
                                       (unsigned long long)p->k_tiles * p->n_tiles;
        p->pack_all_hint = (all > 0 && named * 2 >= all) ? 1 : 0;
    }
    return SPAMM_OK;
}

int status_from_scalars(const spamm_plan *p)
{
    if (p->peer_world > 1 && *p->h_peer_error) return SPAMM_ERR_DEVICE_WAIT;
    for (int c = 0; c < MAX_CHUNKS; c++) {     // every set: an earlier call may have used more sets than the last
        if (p->h_scalars[c].error) return SPAMM_ERR_DEVICE_WAIT;
        if (p->h_scalars[c].overflow) return SPAMM_ERR_OVERFLOW;
    }
    return SPAMM_OK;
}

int64_t total_survivors(const spamm_plan *p)
{
    int64_t s = 0;
    for (int c = 0; c < p->active_scalars; c++) s += (int64_t)p->h_scalars[c].survivors;
    return s;
}

}  // namespace

extern "C" {
static int build_lists_impl(spamm_plan *p, float tau, bool whole_step);
}

// Which kernel on pairs of SMs runs before the one-SM multiply kernel (a wrong guess costs speed, never correctness).
static int pairs_choice(const spamm_plan *p)
{
    if (p->multiply_mode == SPAMM_MULTIPLY_ONE_SM) return GM_PAIRS_NONE;
    if (p->multiply_mode == SPAMM_MULTIPLY_GATED_PAIRS) return GM_PAIRS_GATED;
    // The gated kernel on pairs of SMs is never chosen automatically: measured on long half-full lists (a lattice
    // density matrix, N = 32768) it moves a third fewer bytes but keeps fewer of them in flight (its ring slots are
    // sized for the largest k, and a stage passes through both blocks before it is free again), 48 ms against 37.5 ms.
    return p->dense_hint != 0 ? GM_PAIRS_DENSE : GM_PAIRS_NONE;      // unknown yet: the dense kernel checks by itself
}

// The gated two-SM kernel's records live in a buffer of their own (16 bytes per k and pair of macro tiles), allocated
// the first time that kernel is chosen.  Fills `args` for a multiply over tile rows [t0, t0+tiles) of the plan's block
// (t0 a multiple of 8); returns GM_PAIRS_NONE in *pairs when the buffer cannot be had, so that the caller falls back.
static void gpair_args_for(spamm_plan *p, int t0, const float *norm_a, GpairArgs *args, int *pairs)
{
    if (*pairs != GM_PAIRS_GATED) return;
    if (!p->d_gpair) {
        const size_t bytes = gated_multiply_gpair_scratch_bytes(p->row_tiles, p->k_tiles, p->n_tiles) + 16 * MAX_CHUNKS;
        if (t0 % (2 * MT_R) || cudaMalloc(&p->d_gpair, bytes ? bytes : 16) != cudaSuccess) {
            cudaGetLastError();
            p->d_gpair = nullptr;
            *pairs = GM_PAIRS_NONE;
            return;
        }
    }
    if (t0 % (2 * MT_R)) {
        *pairs = GM_PAIRS_NONE;
        return;
    }
    // every pair of macro-tile rows before t0 has its records and counts before this block's
    const size_t units_before = (size_t)(t0 / (2 * MT_R)) * p->mj_n;
    args->norm_a = norm_a;
    args->norm_b = p->d_norm_b;
    args->tau = p->last_tau;
    args->chunk_max = p->d_list_scratch;
    args->scratch = static_cast<char *>(p->d_gpair) + units_before * ((size_t)p->k_tiles * 16 + 16);
    args->build = true;
}

// (Re)builds the macro-tile orders for the chunk shapes of the pipelined spamm_multiply.
static int setup_chunk_orders(spamm_plan *p)
{
    cudaFree(p->d_order_chunk);
    cudaFree(p->d_order_last);
    p->d_order_chunk = p->d_order_last = nullptr;
    if (p->n_chunks <= 1) return SPAMM_OK;
    const int last_tiles = p->row_tiles - (p->n_chunks - 1) * p->chunk_tiles;
    const size_t n_full = (size_t)ceil_div(p->chunk_tiles, MT_R) * p->mj_n;
    const size_t n_last = (size_t)ceil_div(last_tiles, MT_R) * p->mj_n;
    std::vector<int32_t> o(n_full > n_last ? n_full : n_last);
    int st;
    if ((st = dev_alloc(&p->d_order_chunk, sizeof(int32_t) * n_full))) return st;
    if ((st = dev_alloc(&p->d_order_last, sizeof(int32_t) * n_last))) return st;
    spamm_macro_tile_order(p->chunk_tiles, p->n_tiles, o.data());
    SPAMM_CUDA_TRY(cudaMemcpy(p->d_order_chunk, o.data(), sizeof(int32_t) * n_full, cudaMemcpyHostToDevice));
    spamm_macro_tile_order(last_tiles, p->n_tiles, o.data());
    SPAMM_CUDA_TRY(cudaMemcpy(p->d_order_last, o.data(), sizeof(int32_t) * n_last, cudaMemcpyHostToDevice));
    return SPAMM_OK;
}

extern "C" {

int spamm_plan_set_precision(spamm_plan *p, int precision)
{
    if (!p || (precision != SPAMM_PRECISION_HALF && precision != SPAMM_PRECISION_SPLIT)) return SPAMM_ERR_INVALID;
    DeviceGuard guard(p->device);
    if (precision == SPAMM_PRECISION_SPLIT && (!p->d_low_a || !p->d_low_b)) {
        int st;
        if (!p->d_low_a && (st = dev_alloc(&p->d_low_a, p->bytes_half_a()))) return st;
        if (!p->d_low_b && (st = dev_alloc(&p->d_low_b, p->bytes_half_b()))) {
            cudaFree(p->d_low_a);       // both or neither: a later call starts over
            p->d_low_a = nullptr;
            return st;
        }
    }
    if (precision != p->precision) {
        p->have_pack = false;       // the packed tiles belong to the other mode
        p->packed_all = false;      // the norm pass converts high parts only: spamm_pack must run
    }
    p->precision = precision;
    return SPAMM_OK;
}

int spamm_plan_set_multiply_mode(spamm_plan *p, int mode)
{
    if (!p || (mode != SPAMM_MULTIPLY_AUTO && mode != SPAMM_MULTIPLY_ONE_SM && mode != SPAMM_MULTIPLY_GATED_PAIRS))
        return SPAMM_ERR_INVALID;
    p->multiply_mode = mode;
    return SPAMM_OK;
}

int spamm_plan_set_pack_mode(spamm_plan *p, int mode)
{
    if (!p || (mode != SPAMM_PACK_AUTO && mode != SPAMM_PACK_LISTED && mode != SPAMM_PACK_ALL)) return SPAMM_ERR_INVALID;
    p->pack_mode = mode;
    return SPAMM_OK;
}

int spamm_plan_set_chunk_tiles(spamm_plan *p, int tiles)
{
    if (!p || tiles <= 0 || tiles % MT_R) return SPAMM_ERR_INVALID;
    if (p->row_tiles > 0 && ceil_div(p->row_tiles, tiles) > MAX_CHUNKS) return SPAMM_ERR_INVALID;
    DeviceGuard guard(p->device);
    SPAMM_CUDA_TRY(cudaStreamSynchronize(p->stream));
    p->chunk_tiles = tiles;
    p->n_chunks = p->row_tiles > 0 ? ceil_div(p->row_tiles, tiles) : 1;
    return setup_chunk_orders(p);
}

int spamm_plan_create(spamm_plan **out, int M, int K, int N, int row_tile_begin, int row_tile_count, int device)
{
    if (!out) return SPAMM_ERR_INVALID;
    *out = nullptr;
    if (M <= 0 || K <= 0 || N <= 0 || M > INT32_MAX - TILE || K > INT32_MAX - TILE || N > INT32_MAX - TILE)
        return SPAMM_ERR_INVALID;
    // sizes that are not multiples of 32 are padded with zeros on the device (the reference pads, main.h:54-56, and
    // leaves the padding uninitialised, cuSpAMM.cu:410); zero tiles have norm 0 and zero rows add nothing
    const int in_M = M, in_K = K, in_N = N;
    M = (M + TILE - 1) / TILE * TILE;
    K = (K + TILE - 1) / TILE * TILE;
    N = (N + TILE - 1) / TILE * TILE;
    if (row_tile_begin < 0 || row_tile_count < 0 || row_tile_begin + (int64_t)row_tile_count > M / TILE)
        return SPAMM_ERR_INVALID;
    if (K / TILE > 65535) return SPAMM_ERR_UNSUPPORTED;
    int ndev = 0;
    SPAMM_CUDA_TRY(cudaGetDeviceCount(&ndev));
    if (device < 0 || device >= ndev) return SPAMM_ERR_INVALID;
    DeviceGuard guard(device);
    if (!guard.ok) return record_cuda_error(cudaGetLastError(), "cudaSetDevice");
    int cc_major = 0;
    SPAMM_CUDA_TRY(cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, device));
    if (cc_major != 10) return SPAMM_ERR_UNSUPPORTED;

    {
        // every kernel of the path is loaded onto this device before any of them runs (see preload_norm)
        int st;
        if ((st = preload_norm()) || (st = preload_lists()) || (st = preload_pack()) || (st = preload_multiply()) ||
            (st = preload_multiply_pair()) || (st = preload_multiply_gpair()))
            return st;
    }
    spamm_plan *p = new (std::nothrow) spamm_plan();
    if (!p) return SPAMM_ERR_ALLOC;
    p->M = M; p->K = K; p->N = N;
    p->in_M = in_M; p->in_K = in_K; p->in_N = in_N;
    p->row_begin = row_tile_begin; p->row_tiles = row_tile_count;
    p->k_tiles = K / TILE; p->n_tiles = N / TILE;
    p->mi_n = ceil_div(p->row_tiles, MT_R); p->mj_n = ceil_div(p->n_tiles, MT_C);
    p->device = device;

    int st = SPAMM_OK;
    auto fail = [&](int code) {
        spamm_plan_destroy(p);
        return code;
    };
    {
        // The main stream gets a priority above the second one: when C is cleared on the second stream beside the
        // list build, the blocks of the (small) list kernels must not queue behind those of the memset.
        int least = 0, greatest = 0;
        if (cudaDeviceGetStreamPriorityRange(&least, &greatest) != cudaSuccess) least = greatest = 0;
        const int main_priority = greatest < least ? least - 1 : least;
        if (cudaStreamCreateWithPriority(&p->stream, cudaStreamNonBlocking, main_priority) != cudaSuccess ||
            cudaStreamCreateWithPriority(&p->stream_d2h, cudaStreamNonBlocking, least) != cudaSuccess ||
            cudaStreamCreateWithPriority(&p->stream_h2d, cudaStreamNonBlocking, least) != cudaSuccess)
            return fail(record_cuda_error(cudaGetLastError(), "cudaStreamCreate"));
    }
    for (auto &e : p->ev_chunk)
        if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess)
            return fail(record_cuda_error(cudaGetLastError(), "cudaEventCreate"));
    for (auto &e : p->ev_zero)
        if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess)
            return fail(record_cuda_error(cudaGetLastError(), "cudaEventCreate"));
    for (auto &e : p->ev_up)
        if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess)
            return fail(record_cuda_error(cudaGetLastError(), "cudaEventCreate"));
    {
        // chunking of the pipelined path: an eighth of the block's rows of A per chunk, between 16 and 64 MiB (a block
        // of at most 16 MiB goes in one piece), whole macro-tile rows, at most 64 chunks
        const size_t row_bytes = sizeof(float) * (size_t)TILE * K;
        size_t target = p->bytes_a() / 8;
        if (target < CHUNK_MIN_BYTES) target = CHUNK_MIN_BYTES;
        if (target > CHUNK_TARGET_BYTES) target = CHUNK_TARGET_BYTES;
        int ct = (int)((target + row_bytes - 1) / row_bytes);
        ct = (ct + 2 * MT_R - 1) / (2 * MT_R) * (2 * MT_R);      // whole pairs of macro-tile rows
        while (p->row_tiles > 0 && ceil_div(p->row_tiles, ct) > MAX_CHUNKS) ct += 2 * MT_R;
        p->chunk_tiles = ct;
        p->n_chunks = p->row_tiles > 0 ? ceil_div(p->row_tiles, ct) : 1;
    }
    for (auto &e : p->ev)
        if (cudaEventCreate(&e) != cudaSuccess) return fail(record_cuda_error(cudaGetLastError(), "cudaEventCreate"));
    if ((st = dev_alloc(&p->d_a, p->bytes_a()))) return fail(st);
    if ((st = dev_alloc(&p->d_b, p->bytes_b()))) return fail(st);
    if ((st = dev_alloc(&p->d_c, p->bytes_c()))) return fail(st);
    if (p->padded()) {
        // uploads write the caller's extent only: the padding is cleared once, here, and stays zero
        if (cudaMemset(p->d_a, 0, p->bytes_a()) != cudaSuccess || cudaMemset(p->d_b, 0, p->bytes_b()) != cudaSuccess)
            return fail(record_cuda_error(cudaGetLastError(), "cudaMemset(padding)"));
    }
    if ((st = dev_alloc(&p->d_norm_a, p->bytes_norm_a()))) return fail(st);
    if ((st = dev_alloc(&p->d_norm_b_buf[0], p->bytes_norm_b()))) return fail(st);
    if ((st = dev_alloc(&p->d_norm_b_buf[1], p->bytes_norm_b()))) return fail(st);
    p->d_norm_b = p->d_norm_b_buf[0];
    if ((st = dev_alloc(&p->d_peer_flags, sizeof(unsigned int) * (MAX_PEERS + 8)))) return fail(st);
    if ((st = dev_alloc(&p->d_peer_error, sizeof(int)))) return fail(st);
    if (cudaMemset(p->d_peer_flags, 0, sizeof(unsigned int) * (MAX_PEERS + 8)) != cudaSuccess ||
        cudaMemset(p->d_peer_error, 0, sizeof(int)) != cudaSuccess ||
        cudaMallocHost(reinterpret_cast<void **>(&p->h_peer_error), sizeof(int)) != cudaSuccess)
        return fail(record_cuda_error(cudaGetLastError(), "peer exchange buffers"));
    *p->h_peer_error = 0;
    if ((st = dev_alloc(&p->d_counts, p->bytes_counts()))) return fail(st);
    if ((st = dev_alloc(&p->d_step_counts, p->bytes_step_counts()))) return fail(st);
    if ((st = dev_alloc(&p->d_steps, p->bytes_steps()))) return fail(st);
    if ((st = dev_alloc(&p->d_half_a, p->bytes_half_a()))) return fail(st);
    if ((st = dev_alloc(&p->d_half_b, p->bytes_half_b()))) return fail(st);
    if ((st = dev_alloc(&p->d_order, p->bytes_step_counts()))) return fail(st);
    if ((st = dev_alloc(&p->d_busy, p->bytes_step_counts()))) return fail(st);
    if ((st = dev_alloc(&p->d_tile_list,
                        sizeof(uint32_t) * ((size_t)p->mi_n * MT_R + (size_t)p->mj_n * MT_C) * p->k_tiles)))
        return fail(st);
    if ((st = dev_alloc(&p->d_list_scratch, spamm_build_lists_scratch_bytes(p->row_tiles, p->k_tiles, p->n_tiles))))
        return fail(st);
    if (p->n_mt()) {
        std::vector<int32_t> order(p->n_mt());
        spamm_macro_tile_order(p->row_tiles, p->n_tiles, order.data());
        if (cudaMemcpy(p->d_order, order.data(), p->bytes_step_counts(), cudaMemcpyHostToDevice) != cudaSuccess)
            return fail(record_cuda_error(cudaGetLastError(), "cudaMemcpy(order)"));
    }
    if ((st = setup_chunk_orders(p))) return fail(st);
    p->need_a_off = round_up(sizeof(DeviceScalars) * MAX_CHUNKS, 16);
    p->need_b_off = p->need_a_off + round_up((size_t)p->mi_n * p->k_tiles, 16);
    p->cleared_bytes = p->need_b_off + round_up((size_t)p->k_tiles * p->mj_n, 16);
    if ((st = dev_alloc(&p->d_cleared, p->cleared_bytes))) return fail(st);
    p->cv_scratch_bytes = spamm_count_valid_scratch_bytes(p->row_tiles, p->n_tiles);
    if ((st = dev_alloc(&p->d_cv_scratch, p->cv_scratch_bytes))) return fail(st);
    if ((st = dev_alloc(&p->d_cv_count, 16))) return fail(st);
    if ((st = dev_alloc(&p->d_err_scratch, spamm_error_norms_scratch_bytes() + 32))) return fail(st);
    if (cudaMallocHost(reinterpret_cast<void **>(&p->h_scalars), sizeof(DeviceScalars) * MAX_CHUNKS) != cudaSuccess)
        return fail(record_cuda_error(cudaGetLastError(), "cudaMallocHost"));
    if (cudaMallocHost(reinterpret_cast<void **>(&p->h_cv), 16) != cudaSuccess)
        return fail(record_cuda_error(cudaGetLastError(), "cudaMallocHost"));
    memset(p->h_scalars, 0, sizeof(DeviceScalars) * MAX_CHUNKS);
    if (p->cleared_bytes < sizeof(DeviceScalars) * MAX_CHUNKS + 16 ||
        cudaMemsetAsync(p->d_cleared, 0, p->cleared_bytes, p->stream) != cudaSuccess ||
        cudaStreamSynchronize(p->stream) != cudaSuccess)
        return fail(record_cuda_error(cudaGetLastError(), "cudaMemsetAsync"));
    *out = p;
    return SPAMM_OK;
}

int spamm_plan_destroy(spamm_plan *p)
{
    if (!p) return SPAMM_OK;
    DeviceGuard guard(p->device);
    if (p->stream) cudaStreamSynchronize(p->stream);
    cudaFree(p->d_a); cudaFree(p->d_b); cudaFree(p->d_c);
    for (int r = 0; r < MAX_PEERS; r++)
        for (int i = 0; i < 3; i++)
            if (p->peer_mapped[r][i]) cudaIpcCloseMemHandle(p->peer_mapped[r][i]);
    cudaFree(p->d_norm_a); cudaFree(p->d_norm_b_buf[0]); cudaFree(p->d_norm_b_buf[1]);
    cudaFree(p->d_peer_flags); cudaFree(p->d_peer_error);
    if (p->h_peer_error) cudaFreeHost(p->h_peer_error);
    cudaFree(p->d_counts); cudaFree(p->d_step_counts); cudaFree(p->d_steps);
    cudaFree(p->d_half_a); cudaFree(p->d_half_b); cudaFree(p->d_cleared); cudaFree(p->d_order);
    cudaFree(p->d_low_a); cudaFree(p->d_low_b); cudaFree(p->d_gpair);
    cudaFree(p->d_busy); cudaFree(p->d_tile_list); cudaFree(p->d_list_scratch);
    cudaFree(p->d_cv_scratch); cudaFree(p->d_cv_count); cudaFree(p->d_err_scratch);
    if (p->h_scalars) cudaFreeHost(p->h_scalars);
    if (p->h_cv) cudaFreeHost(p->h_cv);
    for (auto &e : p->ev)
        if (e) cudaEventDestroy(e);
    for (auto &e : p->ev_chunk)
        if (e) cudaEventDestroy(e);
    for (auto &e : p->ev_zero)
        if (e) cudaEventDestroy(e);
    for (auto &e : p->ev_up)
        if (e) cudaEventDestroy(e);
    cudaFree(p->d_order_chunk); cudaFree(p->d_order_last);
    if (p->stream_d2h) cudaStreamDestroy(p->stream_d2h);
    if (p->stream_h2d) cudaStreamDestroy(p->stream_h2d);
    if (p->stream) cudaStreamDestroy(p->stream);
    delete p;
    return SPAMM_OK;
}

int spamm_upload(spamm_plan *p, const float *a_rows, const float *b)
{
    if (!p) return SPAMM_ERR_INVALID;
    DeviceGuard guard(p->device);
    int st;
    if (a_rows && (st = copy_matrix(p->d_a, p->K, a_rows, p->in_K, p->rows_in(), p->in_K, cudaMemcpyHostToDevice,
                                    p->stream)))
        return st;
    if (b && (st = copy_matrix(p->d_b, p->N, b, p->in_N, p->in_K, p->in_N, cudaMemcpyHostToDevice, p->stream)))
        return st;
    if (a_rows || b) p->have_norms = p->have_lists = p->have_pack = false;
    return SPAMM_OK;
}

int spamm_norm_b_share(spamm_plan *p, int b_tile_begin, int b_tile_count)
{
    if (!p || b_tile_begin < 0 || b_tile_count < 0 || b_tile_begin + (int64_t)b_tile_count > p->k_tiles)
        return SPAMM_ERR_INVALID;
    DeviceGuard guard(p->device);
    if (b_tile_count) {
        int st = spamm_norm_map_dev(p->d_b + (size_t)b_tile_begin * TILE * p->N, b_tile_count * TILE, p->N, p->N,
                                    p->d_norm_b + (size_t)b_tile_begin * p->n_tiles, p->stream);
        if (st) return st;
        p->launches++;
    }
    p->have_lists = p->have_pack = false;
    p->packed_all = false;
    return SPAMM_OK;
}

int spamm_norm_a(spamm_plan *p)
{
    if (!p) return SPAMM_ERR_INVALID;
    DeviceGuard guard(p->device);
    if (p->row_tiles) {
        int st = spamm_norm_map_dev(p->d_a, p->row_tiles * TILE, p->K, p->K, p->d_norm_a, p->stream);
        if (st) return st;
        p->launches++;
    }
    p->have_norms = true;       // the caller answers for B's map (spamm_norm_b_share + its exchange)
    p->have_lists = p->have_pack = false;
    p->packed_all = false;
    return SPAMM_OK;
}

int spamm_norms_share(spamm_plan *p, int b_tile_begin, int b_tile_count)
{
    int st = spamm_norm_b_share(p, b_tile_begin, b_tile_count);
    if (st) return st;
    return spamm_norm_a(p);
}

int spamm_peer_handles(spamm_plan *p, void *out, size_t out_bytes)
{
    if (!p || !out || out_bytes < 3 * sizeof(cudaIpcMemHandle_t)) return SPAMM_ERR_INVALID;
    DeviceGuard guard(p->device);
    cudaIpcMemHandle_t *h = static_cast<cudaIpcMemHandle_t *>(out);
    SPAMM_CUDA_TRY(cudaIpcGetMemHandle(&h[0], p->d_norm_b_buf[0]));
    SPAMM_CUDA_TRY(cudaIpcGetMemHandle(&h[1], p->d_norm_b_buf[1]));
    SPAMM_CUDA_TRY(cudaIpcGetMemHandle(&h[2], p->d_peer_flags));
    return SPAMM_OK;
}

int spamm_peer_attach(spamm_plan *p, int world, int rank, const void *all_handles)
{
    if (!p || !all_handles || world < 2 || world > MAX_PEERS || rank < 0 || rank >= world) return SPAMM_ERR_INVALID;
    if (p->peer_world) return SPAMM_ERR_STATE;
    DeviceGuard guard(p->device);
    const cudaIpcMemHandle_t *h = static_cast<const cudaIpcMemHandle_t *>(all_handles);
    for (int r = 0; r < world; r++) {
        if (r == rank) {
            p->peer_norm_b[r][0] = p->d_norm_b_buf[0];
            p->peer_norm_b[r][1] = p->d_norm_b_buf[1];
            p->peer_flags[r] = p->d_peer_flags;
            continue;
        }
        for (int i = 0; i < 3; i++) {
            cudaError_t e = cudaIpcOpenMemHandle(&p->peer_mapped[r][i], h[r * 3 + i], cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) {
                // leave nothing half attached: close what was opened so far, so that a retry starts clean
                p->peer_mapped[r][i] = nullptr;
                for (int rr = 0; rr <= r; rr++)
                    for (int ii = 0; ii < 3; ii++)
                        if (p->peer_mapped[rr][ii]) {
                            cudaIpcCloseMemHandle(p->peer_mapped[rr][ii]);
                            p->peer_mapped[rr][ii] = nullptr;
                        }
                return record_cuda_error(e, "cudaIpcOpenMemHandle");
            }
        }
        p->peer_norm_b[r][0] = static_cast<float *>(p->peer_mapped[r][0]);
        p->peer_norm_b[r][1] = static_cast<float *>(p->peer_mapped[r][1]);
        p->peer_flags[r] = static_cast<unsigned int *>(p->peer_mapped[r][2]);
    }
    p->peer_world = world;
    p->peer_rank = rank;
    return SPAMM_OK;
}

int spamm_peer_wait_selftest(spamm_plan *p, int senders, unsigned int limit_ms)
{
    if (!p || senders < 1 || senders > MAX_PEERS || limit_ms == 0 || limit_ms > 5000) return SPAMM_ERR_INVALID;
    DeviceGuard guard(p->device);
    // wait for a step number no sender has announced: the wait must run out after limit_ms and say so
    PeerWait w{p->d_peer_flags, senders, p->peer_epoch + 0x40000000u, p->d_peer_error, (unsigned long long)limit_ms * 1000000ull};
    int st = peer_wait_selftest_launch(w, p->stream);
    if (st) return st;
    SPAMM_CUDA_TRY(cudaMemcpyAsync(p->h_peer_error, p->d_peer_error, sizeof(int), cudaMemcpyDeviceToHost, p->stream));
    SPAMM_CUDA_TRY(cudaMemsetAsync(p->d_peer_error, 0, sizeof(int), p->stream));      // leave the plan usable
    SPAMM_CUDA_TRY(cudaStreamSynchronize(p->stream));
    const int expired = *p->h_peer_error;
    *p->h_peer_error = 0;
    return expired ? SPAMM_ERR_DEVICE_WAIT : SPAMM_OK;
}

// Norm map of this GPU's share of B (and, with `with_a`, of its rows of A in the same launch), then the small kernel
// that stores the share into every other GPU's map and raises the arrival flags.
static int norm_share_and_push(spamm_plan *p, int b_tile_begin, int b_tile_count, bool with_a)
{
    if (!p || b_tile_begin < 0 || b_tile_count <= 0 || b_tile_begin + (int64_t)b_tile_count > p->k_tiles)
        return SPAMM_ERR_INVALID;
    if (p->peer_world < 2) return SPAMM_ERR_STATE;
    DeviceGuard guard(p->device);
    // A new step: its shares go to the other buffer of every GPU, so a GPU that is still building the previous
    // step's lists is not disturbed; nobody can be two steps ahead, because every step waits for all flags.
    p->peer_epoch++;
    const int buf = (int)(p->peer_epoch & 1u);
    p->d_norm_b = p->d_norm_b_buf[buf];
    PeerTargets t{};
    t.n = p->peer_world;
    for (int r = 0; r < p->peer_world; r++) {
        t.map[r] = p->peer_norm_b[r][buf];
        t.flags[r] = p->peer_flags[r];
    }
    const float *b_share = p->d_b + (size_t)b_tile_begin * TILE * p->N;
    const int64_t map_offset = (int64_t)b_tile_begin * p->n_tiles;
    int st;
    if (with_a && p->row_tiles) {
        // one launch: the share's blocks first, the last of them to finish delivers the share while the rest of the
        // grid still reads A
        st = norm_map_pair_push_launch(p->d_a, p->row_tiles * TILE, p->K, p->K, p->d_norm_a, b_share, b_tile_count * TILE,
                                       p->N, p->N, p->d_norm_b + map_offset, map_offset, t, p->peer_rank, p->peer_epoch,
                                       p->d_peer_flags + MAX_PEERS, p->stream);
        if (st) return st;
        p->launches += 1;
    } else {
        st = spamm_norm_map_dev(b_share, b_tile_count * TILE, p->N, p->N, p->d_norm_b + map_offset, p->stream);
        if (st) return st;
        if ((st = push_share_launch(p->d_norm_b + map_offset, (int64_t)b_tile_count * p->n_tiles, map_offset, t,
                                    p->peer_rank, p->peer_epoch, p->stream)))
            return st;
        p->launches += 2;
    }
    p->peer_wait_pending = true;
    p->have_lists = p->have_pack = false;
    p->packed_all = false;
    if (with_a) p->have_norms = true;
    return SPAMM_OK;
}

int spamm_norm_b_share_push(spamm_plan *p, int b_tile_begin, int b_tile_count)
{
    return norm_share_and_push(p, b_tile_begin, b_tile_count, false);
}

int spamm_norms_shared(spamm_plan *p, int b_tile_begin, int b_tile_count)
{
    return norm_share_and_push(p, b_tile_begin, b_tile_count, true);
}

int spamm_run_shared(spamm_plan *p, float tau, int b_tile_begin, int b_tile_count)
{
    int st = norm_share_and_push(p, b_tile_begin, b_tile_count, true);
    if (st) return st;
    return spamm_finish(p, tau);
}

int spamm_norms(spamm_plan *p)
{
    if (!p) return SPAMM_ERR_INVALID;
    if (p->row_tiles == 0) return spamm_norms_share(p, 0, p->k_tiles);
    DeviceGuard guard(p->device);
    // both maps in one launch; with the conversion of every tile to half when most tiles are going to be needed
    const bool all = p->precision == SPAMM_PRECISION_HALF &&
                     (p->pack_mode == SPAMM_PACK_ALL || (p->pack_mode == SPAMM_PACK_AUTO && p->pack_all_hint == 1));
    int st = all ? norm_pack_pair_launch(p->d_a, p->row_tiles * TILE, p->K, p->K, p->d_norm_a, p->d_half_a, p->d_b,
                                         p->K, p->N, p->N, p->d_norm_b, p->d_half_b, p->stream)
                 : spamm_norm_map_pair_dev(p->d_a, p->row_tiles * TILE, p->K, p->K, p->d_norm_a, p->d_b, p->K, p->N,
                                           p->N, p->d_norm_b, p->stream);
    if (st) return st;
    p->packed_all = all;
    p->launches++;
    p->have_norms = true;
    p->have_lists = p->have_pack = false;
    return SPAMM_OK;
}

int spamm_finish(spamm_plan *p, float tau)
{
    int st;
    if ((st = build_lists_impl(p, tau, true))) return st;
    if ((st = spamm_pack(p))) return st;
    return spamm_gated_multiply(p);
}

int spamm_clear_c_early(spamm_plan *p)
{
    if (!p) return SPAMM_ERR_INVALID;
    if (!p->row_tiles || p->zero_hint != 1 || p->c_zero_pending) return SPAMM_OK;
    DeviceGuard guard(p->device);
    // few macro tiles are expected to have steps: clear all of C now, on the second stream, beside whatever the
    // main stream does until the multiply (exchange of norm maps, list build, conversion)
    SPAMM_CUDA_TRY(cudaEventRecord(p->ev_zero[0], p->stream));
    SPAMM_CUDA_TRY(cudaStreamWaitEvent(p->stream_d2h, p->ev_zero[0], 0));
    SPAMM_CUDA_TRY(cudaMemsetAsync(p->d_c, 0, p->bytes_c(), p->stream_d2h));
    SPAMM_CUDA_TRY(cudaEventRecord(p->ev_zero[1], p->stream_d2h));
    p->c_zero_pending = true;
    return SPAMM_OK;
}

int spamm_build_lists(spamm_plan *p, float tau)
{
    return build_lists_impl(p, tau, false);       // on its own it leaves C alone
}

// `whole_step`: the packing and the multiply follow at once, so C may be cleared early (see zero_hint).
static int build_lists_impl(spamm_plan *p, float tau, bool whole_step)
{
    if (!p) return SPAMM_ERR_INVALID;
    if (!p->have_norms) return SPAMM_ERR_STATE;
    DeviceGuard guard(p->device);
    p->active_scalars = 1;
    p->last_tau = tau;
    p->gpair_valid = false;
    PeerWait wait{p->d_peer_flags, p->peer_world, p->peer_epoch, p->d_peer_error, PEER_WAIT_LIMIT_NS};
    if (whole_step) {
        int st = spamm_clear_c_early(p);
        if (st) return st;
    }
    if (p->row_tiles) {
        // the builder's first kernel clears the counters and need flags: no separate memset on the stream
        int st = build_lists_launch(p->d_norm_a, p->d_norm_b, p->row_tiles, p->k_tiles, p->n_tiles, tau,
                                    p->d_list_scratch, p->d_steps, p->d_step_counts, p->d_counts, p->need_a(),
                                    p->need_b(), p->d_tile_list, p->d_busy, p->scalars(), p->d_cleared,
                                    p->cleared_bytes, MAX_CHUNKS, p->peer_wait_pending ? &wait : nullptr, p->stream);
        p->peer_wait_pending = false;
        if (st) return st;
        p->launches += 2;
        p->queues_clean = true;     // the clear covers the multiply's two work counters
    } else {
        int st = clear_list_state(p, p->stream);
        if (st) return st;
    }
    p->have_lists = true;
    p->have_pack = false;
    return SPAMM_OK;
}

int spamm_pack(spamm_plan *p)
{
    if (!p) return SPAMM_ERR_INVALID;
    if (!p->have_lists) return SPAMM_ERR_STATE;
    DeviceGuard guard(p->device);
    if (p->row_tiles && !p->packed_all) {
        const bool split = p->precision == SPAMM_PRECISION_SPLIT;
        int st = pack_half_launch(p->d_a, p->d_b, p->row_tiles, p->k_tiles, p->n_tiles, p->d_tile_list, p->scalars(),
                                  p->d_half_a, p->d_half_b, split ? p->d_low_a : nullptr, split ? p->d_low_b : nullptr,
                                  true, p->stream);
        if (st) return st;
        p->launches++;
        p->queues_clean = true;
    }
    p->have_pack = true;
    return SPAMM_OK;
}

int spamm_gated_multiply(spamm_plan *p)
{
    if (!p) return SPAMM_ERR_INVALID;
    if (!p->have_pack) return SPAMM_ERR_STATE;
    DeviceGuard guard(p->device);
    if (p->row_tiles) {
        const bool zeroed = p->c_zero_pending;
        if (zeroed) SPAMM_CUDA_TRY(cudaStreamWaitEvent(p->stream, p->ev_zero[1], 0));
        p->c_zero_pending = false;      // consumed: a second multiply on the same lists writes all of C itself
        int pairs = pairs_choice(p);
        GpairArgs gp{};
        gpair_args_for(p, 0, p->d_norm_a, &gp, &pairs);
        gp.build = !p->gpair_valid;
        int st = gated_multiply_launch(p->d_half_a, p->d_half_b, p->d_steps, p->d_step_counts, p->d_order, p->d_busy,
                                       p->scalars(), p->row_tiles, p->k_tiles, p->n_tiles, p->d_c, p->N,
                                       !p->queues_clean, pairs, zeroed ? GM_C_ZEROED : 0, p->stream, &gp);
        if (pairs == GM_PAIRS_GATED) p->gpair_valid = true;
        gp.build = false;
        p->queues_clean = false;
        if (st) return st;
        p->launches++;
        if (p->precision == SPAMM_PRECISION_SPLIT) {
            // x = hi + lo per operand: hi*hi is in C; hi*lo and lo*hi are added by two more passes over the same
            // lists (lo*lo, 2^-22 of the result, is dropped)
            for (int pass = 0; pass < 2; pass++) {
                st = gated_multiply_launch(pass == 0 ? p->d_half_a : p->d_low_a, pass == 0 ? p->d_low_b : p->d_half_b,
                                           p->d_steps, p->d_step_counts, p->d_order, p->d_busy, p->scalars(),
                                           p->row_tiles, p->k_tiles, p->n_tiles, p->d_c, p->N, true,
                                           pairs == GM_PAIRS_GATED ? GM_PAIRS_GATED : GM_PAIRS_NONE,
                                           GM_C_ZEROED | GM_ACCUMULATE | GM_LOW_OPERAND, p->stream, &gp);
                if (st) return st;
                p->launches++;
            }
        }
    }
    return SPAMM_OK;
}

int spamm_run(spamm_plan *p, float tau)
{
    int st;
    if ((st = spamm_norms(p))) return st;
    if ((st = build_lists_impl(p, tau, true))) return st;
    if ((st = spamm_pack(p))) return st;
    return spamm_gated_multiply(p);
}

int spamm_sync(spamm_plan *p)
{
    if (!p) return SPAMM_ERR_INVALID;
    DeviceGuard guard(p->device);
    int st = read_scalars(p);
    if (st) return st;
    return status_from_scalars(p);
}

int spamm_download_c(spamm_plan *p, float *c_rows)
{
    if (!p || !c_rows) return SPAMM_ERR_INVALID;
    DeviceGuard guard(p->device);
    int st = copy_matrix(c_rows, p->in_N, p->d_c, p->N, p->rows_in(), p->in_N, cudaMemcpyDeviceToHost, p->stream);
    if (st) return st;
    SPAMM_CUDA_TRY(cudaStreamSynchronize(p->stream));
    return SPAMM_OK;
}

static void fill_stats(spamm_plan *p, spamm_stats *s)
{
    s->survivors = total_survivors(p);
    s->tile_products = (int64_t)p->row_tiles * p->k_tiles * p->n_tiles;
    s->packed_tiles_a = s->packed_tiles_b = 0;
    for (int c = 0; c < p->active_scalars; c++) {
        s->packed_tiles_a += (int64_t)p->h_scalars[c].packed_a;
        s->packed_tiles_b += (int64_t)p->h_scalars[c].packed_b;
    }
    if (p->packed_all) {            // converted by the norm pass: every tile, listed or not
        s->packed_tiles_a = (int64_t)p->row_tiles * p->k_tiles;
        s->packed_tiles_b = (int64_t)p->k_tiles * p->n_tiles;
    }
    s->executed_flops = 65536.0 * (double)s->survivors;
}

static int64_t sum_step_counts(spamm_plan *p, int *status)
{
    std::vector<int32_t> sc(p->n_mt());
    *status = SPAMM_OK;
    if (sc.empty()) return 0;
    cudaError_t e = cudaMemcpyAsync(sc.data(), p->d_step_counts, p->bytes_step_counts(), cudaMemcpyDeviceToHost,
                                    p->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(p->stream);
    if (e != cudaSuccess) {
        *status = record_cuda_error(e, "cudaMemcpyAsync(step counts)");
        return 0;
    }
    int64_t t = 0;
    for (int32_t v : sc) t += step_count_of(v);
    return t;
}

// Records ev[0..4] around the four phases.
static int run_with_events(spamm_plan *p, float tau)
{
    int st;
    SPAMM_CUDA_TRY(cudaEventRecord(p->ev[0], p->stream));
    if ((st = spamm_norms(p))) return st;
    SPAMM_CUDA_TRY(cudaEventRecord(p->ev[1], p->stream));
    if ((st = build_lists_impl(p, tau, true))) return st;
    SPAMM_CUDA_TRY(cudaEventRecord(p->ev[2], p->stream));
    if ((st = spamm_pack(p))) return st;
    SPAMM_CUDA_TRY(cudaEventRecord(p->ev[3], p->stream));
    if ((st = spamm_gated_multiply(p))) return st;
    SPAMM_CUDA_TRY(cudaEventRecord(p->ev[4], p->stream));
    return SPAMM_OK;
}

static int phase_times(spamm_plan *p, spamm_stats *s)
{
    SPAMM_CUDA_TRY(cudaEventElapsedTime(&s->ms_norm, p->ev[0], p->ev[1]));
    SPAMM_CUDA_TRY(cudaEventElapsedTime(&s->ms_lists, p->ev[1], p->ev[2]));
    SPAMM_CUDA_TRY(cudaEventElapsedTime(&s->ms_pack, p->ev[2], p->ev[3]));
    SPAMM_CUDA_TRY(cudaEventElapsedTime(&s->ms_multiply, p->ev[3], p->ev[4]));
    SPAMM_CUDA_TRY(cudaEventElapsedTime(&s->ms_device_total, p->ev[0], p->ev[4]));
    return SPAMM_OK;
}

int spamm_run_timed(spamm_plan *p, float tau, spamm_stats *stats)
{
    if (!p) return SPAMM_ERR_INVALID;
    DeviceGuard guard(p->device);
    int st = run_with_events(p, tau);
    if (st) return st;
    if ((st = read_scalars(p))) return st;
    if (stats) {
        memset(stats, 0, sizeof(*stats));
        if ((st = phase_times(p, stats))) return st;
        fill_stats(p, stats);
        stats->steps = sum_step_counts(p, &st);
        if (st) return st;
    }
    return status_from_scalars(p);
}

// One chunk of tile rows [t0, t0+tiles) of the plan's block through norm -> lists -> pack -> multiply, with its own
// set of counters.  Everything the chunk writes lands where the whole-block path would have put it.
static int run_chunk(spamm_plan *p, int chunk, int t0, int tiles, float tau, const int32_t *d_order,
                     cudaStream_t stream, bool do_norm)
{
    const size_t mi0 = (size_t)t0 / MT_R;                 // chunks start on macro-tile rows
    const size_t mt0 = mi0 * p->mj_n;
    DeviceScalars *sc = p->scalars() + chunk;
    float *a = p->d_a + (size_t)t0 * TILE * p->K;
    float *norm_a = p->d_norm_a + (size_t)t0 * p->k_tiles;
    int st;
    if (do_norm && (st = spamm_norm_map_dev(a, tiles * TILE, p->K, p->K, norm_a, stream))) return st;
    if (chunk > 0) {
        // the tile list is shared: this chunk's entries follow the previous chunk's
        SPAMM_CUDA_TRY(cudaMemcpyAsync(&sc->tile_count, &(sc - 1)->tile_count, sizeof(unsigned int),
                                       cudaMemcpyDeviceToDevice, stream));
        SPAMM_CUDA_TRY(cudaMemcpyAsync(&sc->tile_begin, &(sc - 1)->tile_count, sizeof(unsigned int),
                                       cudaMemcpyDeviceToDevice, stream));
    }
    if ((st = spamm_build_lists_dev(norm_a, p->d_norm_b, tiles, p->k_tiles, p->n_tiles, tau, p->d_list_scratch,
                                    p->d_steps + mt0 * p->step_cap(), p->d_step_counts + mt0,
                                    p->d_counts + (size_t)t0 * p->n_tiles, p->need_a() + mi0 * p->k_tiles, p->need_b(),
                                    p->d_tile_list, p->d_busy + mt0, sc, stream)))
        return st;
    uint8_t *half_a = p->d_half_a + mi0 * p->k_tiles * A_SLAB_BYTES;
    const bool split = p->precision == SPAMM_PRECISION_SPLIT;
    uint8_t *low_a = split ? p->d_low_a + mi0 * p->k_tiles * A_SLAB_BYTES : nullptr;
    if ((st = pack_half_launch(a, p->d_b, tiles, p->k_tiles, p->n_tiles, p->d_tile_list, sc, half_a, p->d_half_b, low_a,
                               split ? p->d_low_b : nullptr, true, stream)))
        return st;
    int pairs = pairs_choice(p);
    GpairArgs gp{};
    p->last_tau = tau;
    gpair_args_for(p, t0, norm_a, &gp, &pairs);
    if ((st = gated_multiply_launch(half_a, p->d_half_b, p->d_steps + mt0 * p->step_cap(), p->d_step_counts + mt0,
                                    d_order, p->d_busy + mt0, sc, tiles, p->k_tiles, p->n_tiles,
                                    p->d_c + (size_t)t0 * TILE * p->N, p->N, false, pairs, 0, stream, &gp)))
        return st;
    gp.build = false;
    p->gpair_valid = false;         // these records are a chunk's, not the whole block's
    for (int pass = 0; split && pass < 2; pass++) {
        if ((st = gated_multiply_launch(pass == 0 ? half_a : low_a, pass == 0 ? p->d_low_b : p->d_half_b,
                                        p->d_steps + mt0 * p->step_cap(), p->d_step_counts + mt0, d_order,
                                        p->d_busy + mt0, sc, tiles, p->k_tiles, p->n_tiles,
                                        p->d_c + (size_t)t0 * TILE * p->N, p->N, true,
                                        pairs == GM_PAIRS_GATED ? GM_PAIRS_GATED : GM_PAIRS_NONE,
                                        GM_C_ZEROED | GM_ACCUMULATE | GM_LOW_OPERAND, stream, &gp)))
            return st;
        p->launches++;
    }
    p->launches += do_norm ? 5 : 4;
    return SPAMM_OK;
}

int spamm_upload_b_rows(spamm_plan *p, const float *b_rows, int row_begin, int rows)
{
    if (!p || !b_rows || row_begin < 0 || rows < 0 || row_begin + (int64_t)rows > p->in_K) return SPAMM_ERR_INVALID;
    DeviceGuard guard(p->device);
    int st = copy_matrix(p->d_b + (size_t)row_begin * p->N, p->N, b_rows, p->in_N, rows, p->in_N, cudaMemcpyHostToDevice,
                         p->stream);
    if (st) return st;
    p->have_norms = p->have_lists = p->have_pack = false;
    return SPAMM_OK;
}

static int multiply_impl(spamm_plan *p, const float *a_rows, const float *b, float *c_rows, float tau,
                         cudaEvent_t b_ready, spamm_stats *stats)
{
    int st = plan_multiply_issue(p, a_rows, b, c_rows, tau, b_ready);
    if (st) return st;
    return plan_multiply_finish(p, stats);
}

int spamm_multiply(spamm_plan *p, const float *a_rows, const float *b, float *c_rows, float tau, spamm_stats *stats)
{
    if (!p || !a_rows || !b || !c_rows) return SPAMM_ERR_INVALID;
    return multiply_impl(p, a_rows, b, c_rows, tau, nullptr, stats);
}

int spamm_multiply_b_resident(spamm_plan *p, const float *a_rows, float *c_rows, float tau, void *b_ready_event,
                              spamm_stats *stats)
{
    if (!p || !a_rows || !c_rows) return SPAMM_ERR_INVALID;
    return multiply_impl(p, a_rows, nullptr, c_rows, tau, static_cast<cudaEvent_t>(b_ready_event), stats);
}

}  // extern "C"

// The asynchronous part of spamm_multiply: everything is queued, nothing is waited for.
// b == nullptr: B is in the plan's buffer already, or will be once `b_ready` (may be null) has completed.
int spamm::plan_multiply_issue(spamm_plan *p, const float *a_rows, const float *b, float *c_rows, float tau,
                               cudaEvent_t b_ready)
{
    DeviceGuard guard(p->device);
    int st;
    p->multiply_chunked = !(p->n_chunks <= 1 || p->row_tiles == 0);
    if (!p->multiply_chunked) {
        // small problem: one pass, phase by phase
        SPAMM_CUDA_TRY(cudaEventRecord(p->ev[5], p->stream));
        if (b_ready) SPAMM_CUDA_TRY(cudaStreamWaitEvent(p->stream, b_ready, 0));
        if ((st = spamm_upload(p, a_rows, b))) return st;
        if ((st = run_with_events(p, tau))) return st;
        if ((st = copy_matrix(c_rows, p->in_N, p->d_c, p->N, p->rows_in(), p->in_N, cudaMemcpyDeviceToHost, p->stream)))
            return st;
        SPAMM_CUDA_TRY(cudaEventRecord(p->ev[6], p->stream));
        return SPAMM_OK;
    }

    // Large problem: the copies dominate (PCIe), so they are overlapped with each other and with the kernels.
    // B goes up first (every C row needs all of it); then the rows of A go up chunk by chunk, each chunk runs the
    // whole path on the main stream, and its rows of C go down on a second stream while the next chunk goes up.
    p->packed_all = false;
    if (p->c_zero_pending) {
        // an early clearing of C announced for a step that never came: it must have ended before chunks write C
        SPAMM_CUDA_TRY(cudaStreamWaitEvent(p->stream, p->ev_zero[1], 0));
        p->c_zero_pending = false;
    }
    SPAMM_CUDA_TRY(cudaEventRecord(p->ev[5], p->stream));
    if ((st = clear_list_state(p, p->stream))) return st;
    // All uploads go back to back on their own stream (they start after everything already queued on the main
    // stream, which may still read the old matrices); the main stream waits for B, then for each chunk of rows.
    SPAMM_CUDA_TRY(cudaEventRecord(p->ev_up[MAX_CHUNKS + 1], p->stream));
    SPAMM_CUDA_TRY(cudaStreamWaitEvent(p->stream_h2d, p->ev_up[MAX_CHUNKS + 1], 0));
    if (b && (st = copy_matrix(p->d_b, p->N, b, p->in_N, p->in_K, p->in_N, cudaMemcpyHostToDevice, p->stream_h2d)))
        return st;
    SPAMM_CUDA_TRY(cudaEventRecord(p->ev_up[MAX_CHUNKS], p->stream_h2d));
    const int rows_in = p->rows_in();
    // rows of the caller's matrices inside a chunk of tile rows (the last chunk may reach into the padding)
    auto rows_of = [&](int t0, int tiles) {
        const int lo = t0 * TILE, hi = (t0 + tiles) * TILE;
        return (size_t)(rows_in <= lo ? 0 : (rows_in < hi ? rows_in : hi) - lo);
    };
    for (int c = 0; c < p->n_chunks; c++) {
        const int t0 = c * p->chunk_tiles;
        const int tiles = (c == p->n_chunks - 1) ? p->row_tiles - t0 : p->chunk_tiles;
        if ((st = copy_matrix(p->d_a + (size_t)t0 * TILE * p->K, p->K, a_rows + (size_t)t0 * TILE * p->in_K, p->in_K,
                              rows_of(t0, tiles), p->in_K, cudaMemcpyHostToDevice, p->stream_h2d)))
            return st;
        SPAMM_CUDA_TRY(cudaEventRecord(p->ev_up[c], p->stream_h2d));
    }
    SPAMM_CUDA_TRY(cudaStreamWaitEvent(p->stream, p->ev_up[MAX_CHUNKS], 0));
    if (b_ready) SPAMM_CUDA_TRY(cudaStreamWaitEvent(p->stream, b_ready, 0));   // somebody else is still writing B
    SPAMM_CUDA_TRY(cudaEventRecord(p->ev[0], p->stream));
    if ((st = spamm_norm_map_dev(p->d_b, p->K, p->N, p->N, p->d_norm_b, p->stream))) return st;
    p->launches++;
    p->active_scalars = p->n_chunks;
    for (int c = 0; c < p->n_chunks; c++) {
        const int t0 = c * p->chunk_tiles;
        const int tiles = (c == p->n_chunks - 1) ? p->row_tiles - t0 : p->chunk_tiles;
        const size_t c_off = (size_t)t0 * TILE * p->N;
        SPAMM_CUDA_TRY(cudaStreamWaitEvent(p->stream, p->ev_up[c], 0));
        if ((st = run_chunk(p, c, t0, tiles, tau, c == p->n_chunks - 1 ? p->d_order_last : p->d_order_chunk,
                            p->stream, true)))
            return st;
        SPAMM_CUDA_TRY(cudaEventRecord(p->ev_chunk[c], p->stream));
        SPAMM_CUDA_TRY(cudaStreamWaitEvent(p->stream_d2h, p->ev_chunk[c], 0));
        if ((st = copy_matrix(c_rows + (size_t)t0 * TILE * p->in_N, p->in_N, p->d_c + c_off, p->N, rows_of(t0, tiles),
                              p->in_N, cudaMemcpyDeviceToHost, p->stream_d2h)))
            return st;
    }
    // the main stream ends when the last rows of C have arrived
    SPAMM_CUDA_TRY(cudaEventRecord(p->ev[7], p->stream_d2h));
    SPAMM_CUDA_TRY(cudaStreamWaitEvent(p->stream, p->ev[7], 0));
    SPAMM_CUDA_TRY(cudaEventRecord(p->ev[6], p->stream));
    p->have_norms = p->have_lists = true;
    p->have_pack = false;       // the per-chunk work lists are not those of a whole-block multiply
    return SPAMM_OK;
}

// The blocking part: waits for what plan_multiply_issue queued, reads the counters, fills the statistics.
int spamm::plan_multiply_finish(spamm_plan *p, spamm_stats *stats)
{
    DeviceGuard guard(p->device);
    int st;
    if ((st = read_scalars(p))) return st;
    if (stats) {
        memset(stats, 0, sizeof(*stats));
        if (!p->multiply_chunked) {
            if ((st = phase_times(p, stats))) return st;
            SPAMM_CUDA_TRY(cudaEventElapsedTime(&stats->ms_h2d, p->ev[5], p->ev[0]));
            SPAMM_CUDA_TRY(cudaEventElapsedTime(&stats->ms_d2h, p->ev[4], p->ev[6]));
        } else {
            // the phases interleave with the copies: only the whole call is timed (spamm_run_timed gives phases)
            SPAMM_CUDA_TRY(cudaEventElapsedTime(&stats->ms_device_total, p->ev[5], p->ev[6]));
            SPAMM_CUDA_TRY(cudaEventElapsedTime(&stats->ms_h2d, p->ev[5], p->ev[0]));
        }
        fill_stats(p, stats);
        stats->steps = sum_step_counts(p, &st);
        if (st) return st;
    }
    return status_from_scalars(p);
}

extern "C" {

int spamm_get_norm_a(spamm_plan *p, float *out)
{
    if (!p || !out) return SPAMM_ERR_INVALID;
    if (!p->have_norms) return SPAMM_ERR_STATE;
    DeviceGuard guard(p->device);
    SPAMM_CUDA_TRY(cudaMemcpyAsync(out, p->d_norm_a, p->bytes_norm_a(), cudaMemcpyDeviceToHost, p->stream));
    SPAMM_CUDA_TRY(cudaStreamSynchronize(p->stream));
    return SPAMM_OK;
}

int spamm_get_norm_b(spamm_plan *p, float *out)
{
    if (!p || !out) return SPAMM_ERR_INVALID;
    if (!p->have_norms) return SPAMM_ERR_STATE;
    DeviceGuard guard(p->device);
    SPAMM_CUDA_TRY(cudaMemcpyAsync(out, p->d_norm_b, p->bytes_norm_b(), cudaMemcpyDeviceToHost, p->stream));
    SPAMM_CUDA_TRY(cudaStreamSynchronize(p->stream));
    return SPAMM_OK;
}

int spamm_get_counts(spamm_plan *p, int32_t *out, int64_t *survivors)
{
    if (!p) return SPAMM_ERR_INVALID;
    if (!p->have_lists) return SPAMM_ERR_STATE;
    DeviceGuard guard(p->device);
    if (out && p->row_tiles)
        SPAMM_CUDA_TRY(cudaMemcpyAsync(out, p->d_counts, p->bytes_counts(), cudaMemcpyDeviceToHost, p->stream));
    int st = read_scalars(p);
    if (st) return st;
    if (survivors) *survivors = total_survivors(p);
    return status_from_scalars(p);
}

int spamm_get_lists(spamm_plan *p, int64_t *offsets, int32_t *k_idx)
{
    if (!p || !offsets) return SPAMM_ERR_INVALID;
    if (!p->have_lists) return SPAMM_ERR_STATE;
    DeviceGuard guard(p->device);
    const size_t n_mt = p->n_mt();
    const size_t tiles = (size_t)p->row_tiles * p->n_tiles;
    std::vector<int32_t> sc(n_mt);
    if (n_mt) {
        SPAMM_CUDA_TRY(cudaMemcpyAsync(sc.data(), p->d_step_counts, p->bytes_step_counts(), cudaMemcpyDeviceToHost,
                                       p->stream));
        SPAMM_CUDA_TRY(cudaStreamSynchronize(p->stream));
    }
    std::vector<size_t> first(n_mt + 1, 0);
    for (int32_t &v : sc) v = step_count_of(v);
    for (size_t m = 0; m < n_mt; m++) first[m + 1] = first[m] + (size_t)sc[m];
    std::vector<uint32_t> steps(first[n_mt]);
    for (size_t m = 0; m < n_mt; m++) {
        if (sc[m] > 0)
            SPAMM_CUDA_TRY(cudaMemcpyAsync(steps.data() + first[m], p->d_steps + m * p->step_cap(),
                                           sizeof(uint32_t) * (size_t)sc[m], cudaMemcpyDeviceToHost, p->stream));
    }
    SPAMM_CUDA_TRY(cudaStreamSynchronize(p->stream));
    // pass 1: list lengths
    std::vector<int64_t> len(tiles, 0);
    for (size_t m = 0; m < n_mt; m++) {
        const int mi = (int)(m / p->mj_n), mj = (int)(m % p->mj_n);
        for (size_t i = first[m]; i < first[m + 1]; i++) {
            const uint32_t w = steps[i];
            for (int r = 0; r < MT_R; r++) {
                if (!((step_rows(w) >> r) & 1u)) continue;
                for (int c = 0; c < MT_C; c++)
                    if ((step_cols(w) >> c) & 1u) len[(size_t)(mi * MT_R + r) * p->n_tiles + (mj * MT_C + c)]++;
            }
        }
    }
    offsets[0] = 0;
    for (size_t t = 0; t < tiles; t++) offsets[t + 1] = offsets[t] + len[t];
    if (!k_idx) return SPAMM_OK;
    std::vector<int64_t> cur(offsets, offsets + tiles);
    for (size_t m = 0; m < n_mt; m++) {
        const int mi = (int)(m / p->mj_n), mj = (int)(m % p->mj_n);
        for (size_t i = first[m]; i < first[m + 1]; i++) {
            const uint32_t w = steps[i];
            for (int r = 0; r < MT_R; r++) {
                if (!((step_rows(w) >> r) & 1u)) continue;
                for (int c = 0; c < MT_C; c++)
                    if ((step_cols(w) >> c) & 1u)
                        k_idx[cur[(size_t)(mi * MT_R + r) * p->n_tiles + (mj * MT_C + c)]++] = (int32_t)step_k(w);
            }
        }
    }
    return SPAMM_OK;
}

int spamm_macro_tile_order(int row_tiles, int n_tiles, int32_t *order)
{
    if (row_tiles < 0 || n_tiles < 0 || !order) return SPAMM_ERR_INVALID;
    const int mi_n = ceil_div(row_tiles, MT_R), mj_n = ceil_div(n_tiles, MT_C);
    // Bands of 16 macro-tile rows, walked column by column: about 148 consecutive entries (one per SM) then cover
    // 16 rows x 9 columns, so a wave of blocks reads 16 slabs of A and 9 of B per k instead of 2 and 64.
    const int band = 16;
    size_t n = 0;
    for (int i0 = 0; i0 < mi_n; i0 += band)
        for (int j = 0; j < mj_n; j++)
            for (int i = i0; i < i0 + band && i < mi_n; i++) order[n++] = i * mj_n + j;
    return SPAMM_OK;
}

int spamm_error_norms(spamm_plan *p, const float *d_reference, double out3[3])
{
    if (!p || !d_reference || !out3) return SPAMM_ERR_INVALID;
    DeviceGuard guard(p->device);
    out3[0] = out3[1] = out3[2] = 0.0;
    if (p->row_tiles == 0) return SPAMM_OK;
    const size_t part = spamm_error_norms_scratch_bytes();
    double *d_out = reinterpret_cast<double *>(static_cast<char *>(p->d_err_scratch) + part);
    int st = spamm_error_norms_dev(d_reference, p->d_c, (size_t)p->row_tiles * TILE * p->N, p->d_err_scratch, part, d_out,
                                   p->stream);
    if (st) return st;
    p->launches += 2;
    SPAMM_CUDA_TRY(cudaMemcpyAsync(out3, d_out, 3 * sizeof(double), cudaMemcpyDeviceToHost, p->stream));
    SPAMM_CUDA_TRY(cudaStreamSynchronize(p->stream));
    return SPAMM_OK;
}

int spamm_count_valid(spamm_plan *p, float tau, int64_t *count, double *sum_of_products)
{
    if (!p || !count) return SPAMM_ERR_INVALID;
    if (!p->have_norms) return SPAMM_ERR_STATE;
    DeviceGuard guard(p->device);
    int st = spamm_count_valid_dev(p->d_norm_a, p->d_norm_b, p->row_tiles, p->k_tiles, p->n_tiles, tau,
                                   p->d_cv_scratch, p->cv_scratch_bytes, p->d_cv_count,
                                   reinterpret_cast<double *>(p->d_cv_count + 1), p->stream);
    if (st) return st;
    p->launches += 2;
    SPAMM_CUDA_TRY(cudaMemcpyAsync(p->h_cv, p->d_cv_count, 16, cudaMemcpyDeviceToHost, p->stream));
    SPAMM_CUDA_TRY(cudaStreamSynchronize(p->stream));
    *count = (int64_t)p->h_cv[0];
    if (sum_of_products) memcpy(sum_of_products, &p->h_cv[1], sizeof(double));
    return SPAMM_OK;
}

// smallest float that is >= x: "float product >= x" in double is the same test as "float product >= this"
static float float_at_least(double x)
{
    float f = (float)x;
    if ((double)f < x) f = nextafterf(f, INFINITY);
    return f;
}

int spamm_tune_tau(spamm_plan *p, double expected_rate, int max_iters, double tolerance, float *tau, double *rate,
                   int *iters)
{
    if (!p || !tau || max_iters <= 0 || !(tolerance > 0)) return SPAMM_ERR_INVALID;
    if (!p->have_norms) return SPAMM_ERR_STATE;
    const double total = (double)p->row_tiles * p->k_tiles * p->n_tiles;
    double norm = 0.0, up = 0.0, down = 0.0, valid_rate = 0.0;
    int it = 0;
    for (; it < max_iters; it++) {
        int64_t count = 0;
        double ave = 0.0;
        int st = spamm_count_valid(p, float_at_least(norm), &count, &ave);
        if (st) return st;
        valid_rate = total > 0 ? (double)((float)count / (float)total) : 0.0;
        if (fabs(valid_rate - expected_rate) < tolerance) break;
        if (it == 0) {
            norm = total > 0 ? ave / total : 0.0;
            up = norm;
            continue;
        }
        if (valid_rate > expected_rate) {
            if (up == norm) up *= 2;
            down = norm;
            norm = (norm + up) / 2;
        } else {
            up = norm;
            norm = (norm + down) / 2;
        }
    }
    *tau = (float)norm;
    if (rate) *rate = valid_rate;
    if (iters) *iters = it;
    return SPAMM_OK;
}

int spamm_device_buffer(spamm_plan *p, int which, void **d_ptr, size_t *bytes)
{
    if (!p || !d_ptr || !bytes) return SPAMM_ERR_INVALID;
    switch (which) {
    case SPAMM_BUF_A: *d_ptr = p->d_a; *bytes = p->bytes_a(); break;
    case SPAMM_BUF_B: *d_ptr = p->d_b; *bytes = p->bytes_b(); break;
    case SPAMM_BUF_C: *d_ptr = p->d_c; *bytes = p->bytes_c(); break;
    case SPAMM_BUF_NORM_A: *d_ptr = p->d_norm_a; *bytes = p->bytes_norm_a(); break;
    case SPAMM_BUF_NORM_B: *d_ptr = p->d_norm_b; *bytes = p->bytes_norm_b(); break;
    case SPAMM_BUF_COUNTS: *d_ptr = p->d_counts; *bytes = p->bytes_counts(); break;
    case SPAMM_BUF_STEPS: *d_ptr = p->d_steps; *bytes = p->bytes_steps(); break;
    case SPAMM_BUF_STEP_COUNTS: *d_ptr = p->d_step_counts; *bytes = p->bytes_step_counts(); break;
    case SPAMM_BUF_HALF_A: *d_ptr = p->d_half_a; *bytes = p->bytes_half_a(); break;
    case SPAMM_BUF_HALF_B: *d_ptr = p->d_half_b; *bytes = p->bytes_half_b(); break;
    default: return SPAMM_ERR_INVALID;
    }
    return SPAMM_OK;
}

int spamm_stream(spamm_plan *p, void **stream)
{
    if (!p || !stream) return SPAMM_ERR_INVALID;
    *stream = p->stream;
    return SPAMM_OK;
}

int spamm_plan_dims(spamm_plan *p, int *M, int *K, int *N, int *row_tile_begin, int *row_tile_count)
{
    if (!p) return SPAMM_ERR_INVALID;
    if (M) *M = p->in_M;
    if (K) *K = p->in_K;
    if (N) *N = p->in_N;
    if (row_tile_begin) *row_tile_begin = p->row_begin;
    if (row_tile_count) *row_tile_count = p->row_tiles;
    return SPAMM_OK;
}

const char *spamm_status_string(int status)
{
    switch (status) {
    case SPAMM_OK: return "ok";
    case SPAMM_ERR_INVALID: return "invalid argument";
    case SPAMM_ERR_CUDA: return "CUDA runtime error";
    case SPAMM_ERR_ALLOC: return "allocation failed";
    case SPAMM_ERR_DEVICE_WAIT: return "a bounded wait inside a kernel ran out";
    case SPAMM_ERR_STATE: return "call out of order";
    case SPAMM_ERR_UNSUPPORTED: return "unsupported device or size";
    case SPAMM_ERR_OVERFLOW: return "step list overflow";
    default: return "unknown status";
    }
}

const char *spamm_last_cuda_error(void) { return g_last_cuda_error.c_str(); }

int64_t spamm_kernel_launches(spamm_plan *p) { return p ? p->launches : 0; }

}  // extern "C"
