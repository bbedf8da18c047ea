// Small wrappers around the sm_100a instructions the multiply kernels are made of: mbarriers with bounded waits,
// bulk async copies, tcgen05 (tensor memory allocation, MMA, commit, load/store), shared-memory descriptors.
#pragma once
#include "common.cuh"

namespace spamm {

constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull; // 2 s

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// raises the barrier's pending byte count without arriving (any thread; the arrival that ends the phase comes later)
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Waits for the phase of `bar` with the given parity to complete, at most WAIT_LIMIT_NS.
static __device__ __noinline__ bool wait_slow(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag, int32_t *err,
                                       int code)
{
    // a try_wait suspends the thread for a while by itself: most waits end in one of these, before the (slow to read)
    // global timer is needed at all
    if (mbar_try_wait(bar, parity) || mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (global_ns() - t0 > WAIT_LIMIT_NS) {
            *abort_flag = 1;
            atomicCAS(err, 0, code);
            return false;
        }
    }
}
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                             int32_t *err, int code)
{
    if (mbar_try_wait(bar, parity)) return true;
    return wait_slow(bar, parity, abort_flag, err, code);
}

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(bar)
                 : "memory");
}

// K-major, no swizzle: 8-row groups 512 B apart (SBO), the two 8-element k chunks of a K=16 step 128 B apart (LBO).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr)
{
    const uint32_t lo = ((addr & 0x3ffffu) >> 4) | ((128u >> 4) << 16);
    const uint32_t hi = (512u >> 4) | (1u << 14);
    return ((uint64_t)hi << 32) | lo;
}

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t m0, uint32_t m1, uint32_t m2, uint32_t m3)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, 1, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%4, %5, %6, %7}, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(m0), "r"(m1), "r"(m2), "r"(m3)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t *v)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32_zero(uint32_t taddr)
{
    const uint32_t z = 0;
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, "
        "%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr),
        "r"(z)
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }


// Epilogue store of one 32 x 32 block of C.  tcgen05.ld leaves every thread with the 32 values of ONE row; storing
// them directly makes each warp instruction touch 32 different lines.  Going through a per-warp shared-memory tile
// (rows 144 bytes apart: conflict-free for 128-bit accesses both ways) lets every store instruction write four
// complete 128-byte rows.
constexpr int EPI_ROW_BYTES = 144;
constexpr int EPI_WARP_BYTES = 32 * EPI_ROW_BYTES;          // 4608 bytes per epilogue warp

// With `add` the block, times `scale` (a power of two), is added to what C holds.  The old values are all requested
// before anything else happens: issued one by one between the stores (the compiler cannot move a load of C above a
// store to C) they cost a round trip to L2 or DRAM each, eight per block.
template <bool add>
__device__ __forceinline__ void store_block_coalesced_impl(uint8_t *warp_tile, const uint32_t *v, float *c_block,
                                                           int64_t ldc, int lane, float scale)
{
    const int sub = lane >> 3, part = lane & 7;               // four rows per instruction, eight lanes per row
    float4 old[8];
    if (add) {
#pragma unroll
        for (int i = 0; i < 8; i++)
            old[i] = __ldcs(reinterpret_cast<const float4 *>(c_block + (int64_t)(4 * i + sub) * ldc + part * 4));
    }
    uint4 *mine = reinterpret_cast<uint4 *>(warp_tile + lane * EPI_ROW_BYTES);
#pragma unroll
    for (int x = 0; x < 8; x++) mine[x] = make_uint4(v[4 * x], v[4 * x + 1], v[4 * x + 2], v[4 * x + 3]);
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int r = 4 * i + sub;
        float4 o = *reinterpret_cast<const float4 *>(warp_tile + r * EPI_ROW_BYTES + part * 16);
        float4 *dst = reinterpret_cast<float4 *>(c_block + (int64_t)r * ldc + part * 4);
        if (add) {
            o.x = __fmaf_rn(o.x, scale, old[i].x);
            o.y = __fmaf_rn(o.y, scale, old[i].y);
            o.z = __fmaf_rn(o.z, scale, old[i].z);
            o.w = __fmaf_rn(o.w, scale, old[i].w);
        }
        __stcs(dst, o);
    }
    __syncwarp();
}
__device__ __forceinline__ void store_block_coalesced(uint8_t *warp_tile, const uint32_t *v, float *c_block,
                                                      int64_t ldc, int lane, bool add = false, float scale = 1.0f)
{
    if (add) store_block_coalesced_impl<true>(warp_tile, v, c_block, ldc, lane, scale);
    else store_block_coalesced_impl<false>(warp_tile, v, c_block, ldc, lane, scale);
}

}  // namespace spamm
