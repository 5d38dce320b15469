// Inline-PTX helpers for the sm_100a kernels that drive the tensor cores and the cluster network directly:
// mbarriers with bounded waits, tcgen05 (MMA from shared-memory descriptors, tensor-memory loads, commit),
// st.async into a cluster peer's shared memory, and the tagged 64-bit words blocks exchange through L2.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b2 {
namespace ptx {

typedef unsigned long long u64;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier ----------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// arrive on the barrier at the same offset in another block of the cluster (address from mapa)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t remote_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
// "I have finished READING the buffer this barrier guards" to a peer: no earlier write of this thread has to become
// visible with it, so the arrival is relaxed (a release would wait for every global store still in flight)
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t remote_bar) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
// try_wait suspends the thread until the phase completes or a time limit passes (the hint, in nanoseconds, asks for a
// longer one than the default): a waiting warp then leaves the issue slots to the warps that work
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(20000u)
        : "memory");
    return ok != 0;
}
// the same with cluster-scope acquire: the data a peer delivered before it completed the phase is visible
__device__ __forceinline__ bool mbar_try_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(20000u)
        : "memory");
    return ok != 0;
}
// Bounded wait: false when the cycle budget ran out or *give_up (a flag in this block's shared memory that a
// thread sets when its own wait ran out) became non-zero.
template <bool CLUSTER>
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int *give_up, long long budget) {
    if (CLUSTER ? mbar_try_cluster(bar, parity) : mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (CLUSTER ? mbar_try_cluster(bar, parity) : mbar_try(bar, parity)) return true;
        if (*give_up || clock64() - t0 > budget) return false;
    }
}

// ---- cluster ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 16 bytes into a peer's shared memory; the bytes are counted on the peer's transaction barrier
__device__ __forceinline__ void st_async_v4(uint32_t raddr, uint32_t x, uint32_t y, uint32_t z, uint32_t w, uint32_t rbar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(raddr),
                 "r"(x), "r"(y), "r"(z), "r"(w), "r"(rbar)
                 : "memory");
}

// ---- proxies and tcgen05 ----------------------------------------------------------------------------------
// generic-proxy writes to shared memory become visible to the tensor core (async proxy)
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor (version 1) of a K-major tile stored as rows of 128 bytes with the 128-byte
// swizzle (16-byte chunk index XOR row%8): 8-row groups lie `sbo` bytes apart; the leading-dimension offset is
// not used by swizzled K-major tiles.
__device__ __forceinline__ u64 desc_kmajor_sw128(uint32_t addr, uint32_t sbo_bytes) {
    u64 d = 0;
    d |= (u64)((addr >> 4) & 0x3FFF);
    d |= (u64)(1) << 16;                               // 16 bytes >> 4
    d |= (u64)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= 1ULL << 46;
    d |= 2ULL << 61;                                   // SWIZZLE_128B
    return d;
}
// The same for a K-major tile without swizzle: 8 rows x 16 bytes form a contiguous 128-byte core matrix; core matrices
// that follow each other along K lie `lbo` bytes apart, 8-row groups `sbo` bytes apart.
__device__ __forceinline__ u64 desc_kmajor_nosw(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    u64 d = 0;
    d |= (u64)((addr >> 4) & 0x3FFF);
    d |= (u64)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (u64)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= 1ULL << 46;
    return d;
}
// instruction descriptor of kind::f16 with fp16 operands, both K-major, fp32 accumulation
__device__ __forceinline__ uint32_t idesc_f16(int M, int N) {
    return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, u64 adesc, u64 bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// the barrier gets one arrival once every MMA this thread has issued so far is complete
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}
// 16 consecutive columns of this thread's tensor-memory lane
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// generic-proxy view of global memory (after an acquire) ordered before bulk copies issued by this thread
__device__ __forceinline__ void fence_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
// bulk copy global -> shared (16-byte aligned, size a multiple of 16); completion counts bytes on the mbarrier
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}
// bulk copy from this block's shared memory into a cluster peer's (addresses from mapa); bytes counted on the peer's barrier
__device__ __forceinline__ void bulk_s2c(uint32_t remote_dst, uint32_t src, uint32_t bytes, uint32_t remote_bar) {
    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(remote_dst),
                 "r"(src), "r"(bytes), "r"(remote_bar)
                 : "memory");
}
// step counters blocks publish to each other: release after the data, acquire before reading it
__device__ __forceinline__ void st_release_u32(unsigned *p, unsigned v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// 16 bytes from L2 (never from a stale L1 line)
__device__ __forceinline__ float4 ld_l2_f4(const float *p) {
    float4 v;
    asm volatile("ld.relaxed.gpu.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

// ---- exchange through L2 ----------------------------------------------------------------------------------
// One naturally aligned 64-bit word carries {tag : payload}: a reader that sees the tag it waits for has the
// payload of the same store.  Relaxed, gpu scope: no fence, no atomics.
__device__ __forceinline__ void st_tagged(u64 *p, unsigned tag, unsigned payload) {
    const u64 x = ((u64)tag << 32) | (u64)payload;
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(x) : "memory");
}
__device__ __forceinline__ void ld_tagged2(const u64 *p, u64 &a, u64 &b) {
    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ int ld_relaxed_s32(const int *p) {
    int x;
    asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(x) : "l"(p) : "memory");
    return x;
}
// named barrier that also ORs a predicate over its threads: all of them learn whether any gave up a wait
__device__ __forceinline__ bool bar_named_or(int id, int threads, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 q, %3, 0;\n\t"
        "bar.red.or.pred p, %1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"(id), "r"(threads), "r"((uint32_t)pred)
        : "memory");
    return r != 0;
}
__device__ __forceinline__ void bar_named(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }

}  // namespace ptx
}  // namespace b2
