// Several GPUs driven by one process and one host thread: the reference's DEVICEDIM form (para.h:9; per-device plans and
// replicas cuSpAMM.cu:404-451; the parallel region cuSpAMM.cu:470-537) without its redundancy.  Every device owns a
// block of C tile rows (cuSpAMM.cu:503,530), uploads only its rows of A and 1/G of B, receives the other shares of B
// over NVLink (peer copies), computes 1/G of B's norm map per step and stores it into its peers' maps.
#include <cstring>
#include <new>
#include <vector>

#include "plan.cuh"

using namespace spamm;

struct spamm_group {
    int n = 0;
    int M = 0, K = 0, N = 0;                 // the caller's sizes
    std::vector<int> device;
    std::vector<spamm_plan *> plan;
    std::vector<int> b_begin, b_count;       // every device's share of B's tile rows
    bool shared_norms = false;               // the shares of B's norm map are exchanged (else every device computes all)
    std::vector<cudaStream_t> xfer;          // per device: the stream its incoming shares of B arrive on
    std::vector<cudaEvent_t> ev_share;       // per device: its own share of B is in its memory
    std::vector<cudaEvent_t> ev_b_ready;     // per device: all of B is
    std::vector<cudaEvent_t> ev_t0, ev_t1;   // per device: around spamm_group_multiply
};

namespace {

// C tile rows per device: equal blocks on multiples of 4 tile rows (one macro tile) when there are enough rows, the
// remainder to the first devices; the reference gives device d rows [d*T/G, (d+1)*T/G) (cuSpAMM.cu:503,530).
void split_rows(int row_tiles, int n, std::vector<int> &begin, std::vector<int> &count)
{
    const int unit = row_tiles >= MT_R * n ? MT_R : 1;
    const int units = row_tiles / unit;
    begin.assign(n, 0);
    count.assign(n, 0);
    int b = 0;
    for (int d = 0; d < n; d++) {
        int c = (units / n + (d < units % n ? 1 : 0)) * unit;
        if (d == n - 1) c = row_tiles - b;
        begin[d] = b;
        count[d] = c;
        b += c;
    }
}

// Uploads B by shares (device d copies tile rows b_begin[d].. of B from the host) and queues the peer copies that
// complete B on every device; ev_b_ready[d] marks the end on device d.
int upload_b(spamm_group *g, const float *b)
{
    int st;
    for (int d = 0; d < g->n; d++) {
        spamm_plan *p = g->plan[d];
        const int r0 = g->b_begin[d] * TILE;
        int rows = g->b_count[d] * TILE;
        if (r0 + rows > g->K) rows = g->K > r0 ? g->K - r0 : 0;        // the last share may end inside the padding
        DeviceGuard guard(p->device);
        if (rows && (st = spamm_upload_b_rows(p, b + (size_t)r0 * g->N, r0, rows))) return st;
        SPAMM_CUDA_TRY(cudaEventRecord(g->ev_share[d], p->stream));
    }
    for (int q = 0; q < g->n; q++) {
        spamm_plan *dst = g->plan[q];
        DeviceGuard guard(dst->device);
        // what is still queued on the destination may read the old B
        SPAMM_CUDA_TRY(cudaEventRecord(g->ev_b_ready[q], dst->stream));
        SPAMM_CUDA_TRY(cudaStreamWaitEvent(g->xfer[q], g->ev_b_ready[q], 0));
        for (int i = 1; i < g->n; i++) {
            const int d = (q + i) % g->n;                                // every destination starts with another source
            spamm_plan *src = g->plan[d];
            const size_t off = (size_t)g->b_begin[d] * TILE * src->N;
            const size_t bytes = sizeof(float) * (size_t)g->b_count[d] * TILE * src->N;
            if (!bytes) continue;
            SPAMM_CUDA_TRY(cudaStreamWaitEvent(g->xfer[q], g->ev_share[d], 0));
            SPAMM_CUDA_TRY(cudaMemcpyPeerAsync(dst->d_b + off, dst->device, src->d_b + off, src->device, bytes, g->xfer[q]));
        }
        SPAMM_CUDA_TRY(cudaEventRecord(g->ev_b_ready[q], g->xfer[q]));
        dst->have_norms = dst->have_lists = dst->have_pack = false;
    }
    return SPAMM_OK;
}

}  // namespace

extern "C" {

int spamm_group_destroy(spamm_group *g)
{
    if (!g) return SPAMM_OK;
    for (int d = 0; d < (int)g->plan.size(); d++) {
        DeviceGuard guard(g->device[d]);
        if (d < (int)g->xfer.size() && g->xfer[d]) {
            cudaStreamSynchronize(g->xfer[d]);
            cudaStreamDestroy(g->xfer[d]);
        }
        for (auto *v : {&g->ev_share, &g->ev_b_ready, &g->ev_t0, &g->ev_t1})
            if (d < (int)v->size() && (*v)[d]) cudaEventDestroy((*v)[d]);
    }
    for (spamm_plan *p : g->plan) spamm_plan_destroy(p);
    delete g;
    return SPAMM_OK;
}

int spamm_group_create(spamm_group **out, int M, int K, int N, int n_devices, const int *device_ids)
{
    if (!out) return SPAMM_ERR_INVALID;
    *out = nullptr;
    if (M <= 0 || K <= 0 || N <= 0 || n_devices < 1 || n_devices > MAX_PEERS) return SPAMM_ERR_INVALID;
    for (int d = 0; d < n_devices; d++)
        for (int e = 0; device_ids && e < d; e++)
            if (device_ids[d] == device_ids[e]) return SPAMM_ERR_INVALID;
    int ndev = 0;
    SPAMM_CUDA_TRY(cudaGetDeviceCount(&ndev));
    spamm_group *g = new (std::nothrow) spamm_group();
    if (!g) return SPAMM_ERR_ALLOC;
    g->n = n_devices;
    g->M = M; g->K = K; g->N = N;
    for (int d = 0; d < n_devices; d++) g->device.push_back(device_ids ? device_ids[d] : d);
    auto fail = [&](int code) {
        spamm_group_destroy(g);
        return code;
    };
    for (int dev : g->device)
        if (dev < 0 || dev >= ndev) return fail(SPAMM_ERR_INVALID);
    // every device reads and writes the others' norm maps and copies of B directly
    for (int a = 0; a < n_devices; a++) {
        DeviceGuard guard(g->device[a]);
        for (int b = 0; b < n_devices; b++) {
            if (a == b) continue;
            int can = 0;
            SPAMM_CUDA_TRY(cudaDeviceCanAccessPeer(&can, g->device[a], g->device[b]));
            if (!can) {
                record_error_text("spamm_group_create: no peer access between two devices of the group");
                return fail(SPAMM_ERR_UNSUPPORTED);
            }
            cudaError_t e = cudaDeviceEnablePeerAccess(g->device[b], 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();      // not an error: clear it
            else if (e != cudaSuccess) return fail(record_cuda_error(e, "cudaDeviceEnablePeerAccess"));
        }
    }
    const int row_tiles = (M + TILE - 1) / TILE, k_tiles = (K + TILE - 1) / TILE, n_tiles = (N + TILE - 1) / TILE;
    std::vector<int> begin, count;
    split_rows(row_tiles, n_devices, begin, count);
    g->plan.assign(n_devices, nullptr);
    for (int d = 0; d < n_devices; d++) {
        int st = spamm_plan_create(&g->plan[d], M, K, N, begin[d], count[d], g->device[d]);
        if (st) return fail(st);
    }
    // shares of B's tile rows: as even as they come; a share's piece of the norm map must be a whole number of
    // 16-byte vectors at a 16-byte offset for the peer stores, otherwise every device computes the whole map
    g->b_begin.assign(n_devices, 0);
    g->b_count.assign(n_devices, 0);
    g->shared_norms = n_devices > 1;
    for (int d = 0, b = 0; d < n_devices; d++) {
        g->b_begin[d] = b;
        g->b_count[d] = k_tiles / n_devices + (d < k_tiles % n_devices ? 1 : 0);
        b += g->b_count[d];
        if (g->b_count[d] == 0 || ((int64_t)g->b_begin[d] * n_tiles) % 4 || ((int64_t)g->b_count[d] * n_tiles) % 4)
            g->shared_norms = false;
    }
    g->xfer.assign(n_devices, nullptr);
    g->ev_share.assign(n_devices, nullptr);
    g->ev_b_ready.assign(n_devices, nullptr);
    g->ev_t0.assign(n_devices, nullptr);
    g->ev_t1.assign(n_devices, nullptr);
    for (int d = 0; d < n_devices; d++) {
        DeviceGuard guard(g->device[d]);
        if (cudaStreamCreateWithFlags(&g->xfer[d], cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&g->ev_share[d], cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&g->ev_b_ready[d], cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreate(&g->ev_t0[d]) != cudaSuccess || cudaEventCreate(&g->ev_t1[d]) != cudaSuccess)
            return fail(record_cuda_error(cudaGetLastError(), "group streams and events"));
    }
    if (g->shared_norms)
        for (int d = 0; d < n_devices; d++) {
            int st = plan_attach_direct(g->plan[d], n_devices, d, g->plan.data());
            if (st) return fail(st);
        }
    *out = g;
    return SPAMM_OK;
}

int spamm_group_size(spamm_group *g) { return g ? g->n : 0; }

int spamm_group_plan(spamm_group *g, int i, spamm_plan **plan)
{
    if (!g || !plan || i < 0 || i >= g->n) return SPAMM_ERR_INVALID;
    *plan = g->plan[i];
    return SPAMM_OK;
}

int spamm_group_upload(spamm_group *g, const float *a, const float *b)
{
    if (!g) return SPAMM_ERR_INVALID;
    int st;
    if (a)
        for (int d = 0; d < g->n; d++) {
            spamm_plan *p = g->plan[d];
            if ((st = spamm_upload(p, a + (size_t)p->row_begin * TILE * g->K, nullptr))) return st;
        }
    if (b) {
        if ((st = upload_b(g, b))) return st;
        // later work on a device's own stream starts when its B is complete
        for (int d = 0; d < g->n; d++) {
            DeviceGuard guard(g->device[d]);
            SPAMM_CUDA_TRY(cudaStreamWaitEvent(g->plan[d]->stream, g->ev_b_ready[d], 0));
        }
    }
    return SPAMM_OK;
}

int spamm_group_run(spamm_group *g, float tau)
{
    if (!g) return SPAMM_ERR_INVALID;
    for (int d = 0; d < g->n; d++) {
        int st = g->shared_norms ? spamm_run_shared(g->plan[d], tau, g->b_begin[d], g->b_count[d])
                                 : spamm_run(g->plan[d], tau);
        if (st) return st;
    }
    return SPAMM_OK;
}

int spamm_group_sync(spamm_group *g)
{
    if (!g) return SPAMM_ERR_INVALID;
    int first = SPAMM_OK;
    for (int d = 0; d < g->n; d++) {
        const int st = spamm_sync(g->plan[d]);
        if (st && !first) first = st;
    }
    return first;
}

int spamm_group_download_c(spamm_group *g, float *c)
{
    if (!g || !c) return SPAMM_ERR_INVALID;
    int st;
    for (int d = 0; d < g->n; d++) {
        spamm_plan *p = g->plan[d];
        DeviceGuard guard(p->device);
        if ((st = copy_matrix(c + (size_t)p->row_begin * TILE * g->N, g->N, p->d_c, p->N, p->rows_in(), g->N,
                              cudaMemcpyDeviceToHost, p->stream)))
            return st;
    }
    for (int d = 0; d < g->n; d++) {
        DeviceGuard guard(g->device[d]);
        SPAMM_CUDA_TRY(cudaStreamSynchronize(g->plan[d]->stream));
    }
    return SPAMM_OK;
}

int spamm_group_survivors(spamm_group *g, int64_t *survivors)
{
    if (!g || !survivors) return SPAMM_ERR_INVALID;
    *survivors = 0;
    for (int d = 0; d < g->n; d++) {
        int64_t s = 0;
        const int st = spamm_get_counts(g->plan[d], nullptr, &s);
        if (st) return st;
        *survivors += s;
    }
    return SPAMM_OK;
}

int spamm_group_multiply(spamm_group *g, const float *a, const float *b, float *c, float tau, spamm_stats *stats)
{
    if (!g || !a || !b || !c) return SPAMM_ERR_INVALID;
    int st;
    for (int d = 0; d < g->n; d++) {
        DeviceGuard guard(g->device[d]);
        SPAMM_CUDA_TRY(cudaEventRecord(g->ev_t0[d], g->plan[d]->stream));
    }
    if ((st = upload_b(g, b))) return st;
    // every device: its rows of A go up while the shares of B still travel; the first kernel that reads B waits
    for (int d = 0; d < g->n; d++) {
        spamm_plan *p = g->plan[d];
        if ((st = plan_multiply_issue(p, a + (size_t)p->row_begin * TILE * g->K, nullptr,
                                      c + (size_t)p->row_begin * TILE * g->N, tau, g->ev_b_ready[d])))
            return st;
        DeviceGuard guard(p->device);
        SPAMM_CUDA_TRY(cudaEventRecord(g->ev_t1[d], p->stream));
    }
    if (stats) memset(stats, 0, sizeof(*stats));
    int first = SPAMM_OK;
    for (int d = 0; d < g->n; d++) {
        spamm_stats s;
        st = plan_multiply_finish(g->plan[d], &s);
        if (st && !first) first = st;
        if (stats) {
            stats->survivors += s.survivors;
            stats->tile_products += s.tile_products;
            stats->steps += s.steps;
            stats->packed_tiles_a += s.packed_tiles_a;
            stats->packed_tiles_b += s.packed_tiles_b;
            stats->executed_flops += s.executed_flops;
            float ms = 0.f;
            DeviceGuard guard(g->device[d]);
            if (cudaEventElapsedTime(&ms, g->ev_t0[d], g->ev_t1[d]) == cudaSuccess && ms > stats->ms_device_total)
                stats->ms_device_total = ms;
        }
    }
    return first;
}

}  // extern "C"
