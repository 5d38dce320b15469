// fp32-accurate GEMM on the 5th-generation tensor cores (tcgen05, sm_100a): every operand is split into a
// high and a low part and three products are accumulated.  Two arithmetic modes share one kernel:
//   * fp16 parts with a per-operand power-of-two scale (kind::f16, the default of split_operand): x*S = hi + lo*2^-11
//     with 2^13 <= max|x|*S < 2^14, hi = rn_f16(x*S), lo = rn_f16((x*S - hi)*2^11).  22 significand bits for every
//     element down to 2^-28 of the operand's largest; the tensor pipe runs at twice the tf32 rate and the hi/lo
//     copies take 4 bytes per element.  The cross terms are accumulated apart (they carry the factor 2^-11).
//   * tf32 parts (kind::tf32), kept for the per-timestep recurrence whose operands are written in that form.
//
// Stands where the reference calls helpers::Matrix::assignProduct/addProduct -> cublasSgemm
// (helpers/Matrix.cu:354-377, helpers/cublas.cu:52-84 of the reference) for the large products of
// the training path: input projection, error back-projection and the weight-gradient
// contractions (layers/LstmLayer.cu:1756-1775, 2298-2334 and the per-weight loop :490-572;
// layers/FeedForwardLayer.cu:1080,1690,1719).
//
// Numerics.  Every operand is split once into its two parts; the kernel accumulates a_lo*b_hi + a_hi*b_lo
// (cross terms, an accumulator of their own) and a_hi*b_hi in fp32 in tensor memory.  The dropped lo*lo
// term and the rounding of lo are below 2^-21 of |a||b|.
//
// Kernel.  One 128 x 128 output tile per block, K in slabs of one 128-byte swizzle row (64 halves or
// 32 floats).  Warp 0 (one lane) feeds a 3-stage shared-memory ring with TMA (cp.async.bulk.tensor.2d,
// SWIZZLE_128B, no multicast); warps 1 and 10 (one lane each) issue the tcgen05.mma of the main product and
// of the cross terms (M=128, N=128, K=16 resp. 8; 12 per slab) on shared-memory descriptors and release
// slots with tcgen05.commit; warps 2-9 (two per tensor-memory lane quarter, half of the tile's columns each)
// drain the double-buffered main accumulator from TMEM with tcgen05.ld every SEG slabs, add the
// segments in registers and finally write C.  Operands may be K-major (k
// contiguous) or MN-major (m resp. n contiguous); MN-major tiles are fetched as column blocks one
// swizzle row wide so that they land in the canonical MN-major SWIZZLE_128B layout.  Optional split-K over
// gridDim.z into scratch (summed by a second kernel in a fixed order).
//
// Every mbarrier wait is bounded by a cycle budget; on expiry the block records
// B2_ERR_STEP_TIMEOUT in *status, leaves its loops, releases its tensor memory and returns.
#include <cuda.h>

#include <cuda_fp16.h>
#include <cstring>
#include "common.cuh"

namespace b2 {
namespace {

constexpr int BM = 128, STAGES = 3;   // the tile's N extent is a template parameter: 128, or 64 for narrow products
constexpr int TILE_BYTES = BM * 128;                    // 16 KiB: one operand part (hi or lo) of one stage: 128 rows of one swizzle row
constexpr int STAGE_BYTES = 4 * TILE_BYTES;             // A_hi, A_lo, B_hi, B_lo
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024; // + slack to align the ring to 1024 B
constexpr int NTHREADS = 352;   // warp 0 TMA, 1 and 10 MMA issue, 2-9 epilogue
constexpr int TC_MAX_BATCH = 8;
// what differs between the two arithmetic modes
template <bool F16>
struct Mode {
    static constexpr int BK = F16 ? 64 : 32;            // contraction positions per slab: one 128-byte swizzle row
    static constexpr int SEG = 4;                       // slabs per drained accumulator segment: 16 main MMAs (256 resp. 128 positions)
    static constexpr int MNBOX = F16 ? 64 : 32;         // MN-major operands arrive as column blocks one swizzle row wide
    static constexpr int MNBOX_BYTES = BK * 128;        // ... of BK rows each
};
constexpr float LO_UNSCALE = 1.0f / 2048.0f;
// exponent e of the operand scale S = 2^e from the bit pattern of the operand's largest finite |x|: 2^13 <= max * S < 2^14
__host__ __device__ __forceinline__ int f16_scale_exp(unsigned maxbits) {
    if (maxbits == 0u) return 0;
    int e = 13 - ((int)(maxbits >> 23) - 127);          // subnormal maxima (exponent field 0) end at the clamp
    return e < -100 ? -100 : (e > 100 ? 100 : e);
}
constexpr int TMEM_COLS = 512;                          // 2 x 128 main accumulator + 2 x 128 cross terms
constexpr long long WAIT_CYCLES = 4000000000LL;         // about two seconds

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
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
// bounded wait; false when the budget ran out
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try(bar, parity)) return true;
        if (clock64() - t0 > WAIT_CYCLES) return false;
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"((unsigned long long)map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}
// shared-memory matrix descriptor (version 1).  layout type 2 = SWIZZLE_128B (K-major tiles),
// 1 = SWIZZLE_128B with 32-byte atoms, the only swizzled layout the tensor core accepts for
// MN-major 32-bit operands
__device__ __forceinline__ unsigned long long make_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                        unsigned long long layout_type) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr >> 4) & 0x3FFF);
    d |= (unsigned long long)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (unsigned long long)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= 1ULL << 46;
    d |= layout_type << 61;
    return d;
}
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, unsigned long long adesc, unsigned long long bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, unsigned long long adesc, unsigned long long bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

struct TcArgs {
    float *C;
    long ldc;          // column-major C: element (m, n) at n*ldc + m
    int M, N, K;
    int kchunk;        // K range handled per gridDim.z slice (multiple of BK)
    const unsigned *a_max, *b_max;   // fp16 mode: bit patterns of the operands' largest |x| (their scales follow from them)
    int a_kmajor, b_kmajor;
    int accumulate;
    float *ws;         // split-K partials [z][N][M] when gridDim.z > 1
    int *status;
    // Batched use (nbatch > 0): blockIdx.z = batch * splits + split.  A batch shifts the tensor-map
    // coordinates of both operands and the output pointer; split z of batch b writes (never
    // accumulates) to C + c_off[b] + z * c_split_stride with leading dimension ldc.
    int nbatch, splits;
    int a_off_inner[TC_MAX_BATCH], a_off_outer[TC_MAX_BATCH];
    int b_off_inner[TC_MAX_BATCH], b_off_outer[TC_MAX_BATCH];
    long long c_off[TC_MAX_BATCH];
    long long c_split_stride;
    // The contraction index may run over segments of kseg_len consecutive positions that lie
    // kseg_stride apart in both operands (the four gate blocks of one direction); 0 = contiguous.
    int kseg_len, kseg_stride;
    // work items of the persistent tile loop: tiles_m x tiles_n output tiles x nz splits / batches
    int tiles_m, tiles_n, nz;
};

template <int BN, bool F16>
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_split3_kernel(const __grid_constant__ CUtensorMap mapAhi, const __grid_constant__ CUtensorMap mapAlo,
                   const __grid_constant__ CUtensorMap mapBhi, const __grid_constant__ CUtensorMap mapBlo, TcArgs a) {
    extern __shared__ unsigned char smem_raw[];
    constexpr int BK = Mode<F16>::BK, SEG = Mode<F16>::SEG, MNBOX = Mode<F16>::MNBOX, MNBOX_BYTES = Mode<F16>::MNBOX_BYTES;
    __shared__ __align__(8) unsigned long long bars[2 * STAGES + 8];
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int fail_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;   // SWIZZLE_128B atoms need 1024-byte alignment
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * (uint32_t)s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (uint32_t)(STAGES + s); };
    // the main (hi*hi) accumulator is double-buffered in tensor memory and drained every SEG slabs;
    // the cross-term accumulator is double-buffered over tiles
    auto big_full = [&](int b) { return bar0 + 8u * (uint32_t)(2 * STAGES + b); };
    auto big_empty = [&](int b) { return bar0 + 8u * (uint32_t)(2 * STAGES + 2 + b); };
    auto x_empty = [&](int b) { return bar0 + 8u * (uint32_t)(2 * STAGES + 4 + b); };
    auto x_full = [&](int b) { return bar0 + 8u * (uint32_t)(2 * STAGES + 6 + b); };

    // Persistent over work items (m tile fastest, then n tile, then split / batch): barriers and tensor
    // memory are set up once per block, and the epilogue of one tile (global stores from registers)
    // overlaps the MMAs of the next.
    const int items = a.tiles_m * a.tiles_n * a.nz;
    const int nkb_full = (a.kchunk + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 2); }   // both issuers release a slot
        for (int b = 0; b < 2; ++b) {
            mbar_init(big_full(b), 1); mbar_init(big_empty(b), 8); mbar_init(x_empty(b), 8); mbar_init(x_full(b), 1);
        }
        fail_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void *)&tmem_base_s)), "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int kbg = 0;   // k-blocks issued by this block so far (ring position)
            bool ok = true;
            for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
                if (fail_s) break;
                const int m0 = (item % a.tiles_m) * BM, n0 = ((item / a.tiles_m) % a.tiles_n) * BN;
                const int z = item / (a.tiles_m * a.tiles_n);
                const int zsplit = a.nbatch ? z % a.splits : z, batch = a.nbatch ? z / a.splits : 0;
                const int a_in = a.nbatch ? a.a_off_inner[batch] : 0, a_out = a.nbatch ? a.a_off_outer[batch] : 0;
                const int b_in = a.nbatch ? a.b_off_inner[batch] : 0, b_out = a.nbatch ? a.b_off_outer[batch] : 0;
                const int kbeg = zsplit * a.kchunk;
                const int nkb = min(nkb_full, (a.K - kbeg + BK - 1) / BK);
                for (int kb = 0; kb < nkb; ++kb, ++kbg) {
                    const int s = kbg % STAGES;
                    const uint32_t ph = (uint32_t)(kbg / STAGES) & 1u;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u)) { fail_s = 1; ok = false; break; }
                    const uint32_t base = ring + (uint32_t)s * STAGE_BYTES;
                    int k0 = kbeg + kb * BK;
                    if (a.kseg_len) k0 = (k0 / a.kseg_len) * a.kseg_stride + k0 % a.kseg_len;   // segmented contraction index
                    mbar_expect_tx(full_bar(s), 2 * TILE_BYTES + 2 * BN * 128);
                    // the contraction index is the inner coordinate of a K-major operand, the outer one otherwise
                    if (a.a_kmajor) {
                        tma_load_2d(base, &mapAhi, k0 + a_in, m0 + a_out, full_bar(s));
                        tma_load_2d(base + TILE_BYTES, &mapAlo, k0 + a_in, m0 + a_out, full_bar(s));
                    } else {
#pragma unroll
                        for (int b = 0; b < BM / MNBOX; ++b) {
                            tma_load_2d(base + b * MNBOX_BYTES, &mapAhi, m0 + MNBOX * b + a_in, k0 + a_out, full_bar(s));
                            tma_load_2d(base + TILE_BYTES + b * MNBOX_BYTES, &mapAlo, m0 + MNBOX * b + a_in, k0 + a_out, full_bar(s));
                        }
                    }
                    if (a.b_kmajor) {
                        tma_load_2d(base + 2 * TILE_BYTES, &mapBhi, k0 + b_in, n0 + b_out, full_bar(s));
                        tma_load_2d(base + 3 * TILE_BYTES, &mapBlo, k0 + b_in, n0 + b_out, full_bar(s));
                    } else {
#pragma unroll
                        for (int b = 0; b < BN / MNBOX; ++b) {
                            tma_load_2d(base + 2 * TILE_BYTES + b * MNBOX_BYTES, &mapBhi, n0 + MNBOX * b + b_in, k0 + b_out, full_bar(s));
                            tma_load_2d(base + 3 * TILE_BYTES + b * MNBOX_BYTES, &mapBlo, n0 + MNBOX * b + b_in, k0 + b_out, full_bar(s));
                        }
                    }
                }
            }
        }
    } else if (warp == 1 || warp == 10) {
        // ---------------- MMA issuers: warp 1 the main products (hi*hi), warp 10 the cross terms ----------------
        // One thread spends about 85 cycles on issuing an MMA of this shape, more than the tensor core needs to run
        // it; two issuers with accumulators of their own keep the pipe busy and the summation order fixed.
        if (lane == 0) {
            const bool cross = (warp == 10);
            // instruction descriptor: D=f32, A=B=tf32 (format 2) or f16 (format 0), M=128, N=BN, majors per operand
            const uint32_t fmt = F16 ? 0u : 2u;
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((a.a_kmajor ? 0u : 1u) << 15) |
                                   ((a.b_kmajor ? 0u : 1u) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            // K-major: rows of 128 B, 8-row groups 1024 B apart (SBO); one MMA advances 32 B inside the row.
            // MN-major, tf32: [k][32 floats] blocks; 32-wide column blocks 4096 B apart (LBO), groups of 4 k-rows
            // 512 B apart (SBO); one MMA (K=8) advances two such groups = 1024 B.
            // MN-major, fp16: [k][64 halves] blocks, 64-wide column blocks 8192 B apart (LBO), groups of 8 k-rows
            // 1024 B apart (SBO); one MMA (K=16) advances two such groups = 2048 B.
            const uint32_t mn_sbo = F16 ? 1024u : 512u, mn_step = F16 ? 2048u : 1024u;
            const unsigned long long mn_lt = F16 ? 2ULL : 1ULL;
            const uint32_t a_lbo = a.a_kmajor ? 16u : (uint32_t)MNBOX_BYTES, b_lbo = a.b_kmajor ? 16u : (uint32_t)MNBOX_BYTES;
            const uint32_t a_sbo = a.a_kmajor ? 1024u : mn_sbo, b_sbo = a.b_kmajor ? 1024u : mn_sbo;
            const unsigned long long a_lt = a.a_kmajor ? 2ULL : mn_lt, b_lt = a.b_kmajor ? 2ULL : mn_lt;
            const uint32_t a_step = a.a_kmajor ? 32u : mn_step, b_step = a.b_kmajor ? 32u : mn_step;
            // Tensor-memory accumulation rounds toward zero, so a long chain drifts linearly with its
            // length.  Two measures keep fp32 accuracy: the cross terms (2^-11 of the main term) get an
            // accumulator of their own, and the main accumulator is handed to the epilogue warps every
            // SEG slabs, which add the segments in registers with round-to-nearest.
            bool ok = true;
            int kbg = 0, gseg = 0, it = 0;
            for (int item = blockIdx.x; item < items && ok; item += gridDim.x, ++it) {
                if (fail_s) break;
                const int z = item / (a.tiles_m * a.tiles_n);
                const int zsplit = a.nbatch ? z % a.splits : z;
                const int kbeg = zsplit * a.kchunk;
                const int nkb = min(nkb_full, (a.K - kbeg + BK - 1) / BK);
                const int xb = it & 1;
                const uint32_t t_small = tmem_base + (uint32_t)(2 * BN + xb * BN);
                // the cross-term accumulator of two tiles ago must have been read
                if (cross && !mbar_wait(x_empty(xb), ((uint32_t)(it >> 1) & 1u) ^ 1u)) { fail_s = 1; ok = false; break; }
                const int nseg = (nkb + SEG - 1) / SEG;
                for (int seg = 0; seg < nseg && ok; ++seg, ++gseg) {
                    const int buf = gseg & 1;
                    const uint32_t use = (uint32_t)(gseg >> 1);
                    if (!cross && !mbar_wait(big_empty(buf), (use & 1u) ^ 1u)) { fail_s = 1; ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t t_big = tmem_base + (uint32_t)buf * BN;
                    const int kb_end = min(nkb, (seg + 1) * SEG);
                    for (int kb = seg * SEG; kb < kb_end; ++kb, ++kbg) {
                        const int s = kbg % STAGES;
                        const uint32_t ph = (uint32_t)(kbg / STAGES) & 1u;
                        if (!mbar_wait(full_bar(s), ph)) { fail_s = 1; ok = false; break; }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t base = ring + (uint32_t)s * STAGE_BYTES;
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const unsigned long long ahi = make_desc(base + kk * a_step, a_lbo, a_sbo, a_lt);
                            const unsigned long long bhi = make_desc(base + 2 * TILE_BYTES + kk * b_step, b_lbo, b_sbo, b_lt);
                            if (cross) {
                                const unsigned long long alo = make_desc(base + TILE_BYTES + kk * a_step, a_lbo, a_sbo, a_lt);
                                const unsigned long long blo = make_desc(base + 3 * TILE_BYTES + kk * b_step, b_lbo, b_sbo, b_lt);
                                if (F16) {
                                    mma_f16(t_small, alo, bhi, idesc, (kb | kk) ? 1u : 0u);
                                    mma_f16(t_small, ahi, blo, idesc, 1u);
                                } else {
                                    mma_tf32(t_small, alo, bhi, idesc, (kb | kk) ? 1u : 0u);
                                    mma_tf32(t_small, ahi, blo, idesc, 1u);
                                }
                            } else {
                                if (F16) mma_f16(t_big, ahi, bhi, idesc, (kb != seg * SEG || kk) ? 1u : 0u);
                                else mma_tf32(t_big, ahi, bhi, idesc, (kb != seg * SEG || kk) ? 1u : 0u);
                            }
                        }
                        mma_commit(empty_bar(s));   // slot is free once both issuers' MMAs have read it
                    }
                    if (!cross) mma_commit(big_full(buf));   // the main products of this segment are complete
                }
                if (cross && ok) mma_commit(x_full(xb));     // the cross terms of this tile are complete
            }
        }
    } else {
        // ---------------- epilogue: drain segments from TMEM, sum in registers, write C ----------------
        // Eight warps: a warp may read the tensor-memory lane quarter (warp id mod 4); warps 2-5 take the first half of the
        // tile's columns, warps 6-9 the second, so that draining a segment and storing a tile take half as long.
        const int q = warp & 3;             // TMEM lane quarter this warp may read
        constexpr int HN = BN / 2;          // columns per warp
        const int cbase = ((warp - 2) >> 2) * HN;
        const uint32_t lane_base = tmem_base + ((uint32_t)(32 * q) << 16);
        bool ok = true;
        int gseg = 0, it = 0;
        for (int item = blockIdx.x; item < items && ok; item += gridDim.x, ++it) {
            if (fail_s) break;
            const int m0 = (item % a.tiles_m) * BM, n0 = ((item / a.tiles_m) % a.tiles_n) * BN;
            const int z = item / (a.tiles_m * a.tiles_n);
            const int zsplit = a.nbatch ? z % a.splits : z, batch = a.nbatch ? z / a.splits : 0;
            const int kbeg = zsplit * a.kchunk;
            const int nkb = min(nkb_full, (a.K - kbeg + BK - 1) / BK);
            const int xb = it & 1;
            float acc[HN];
#pragma unroll
            for (int j = 0; j < HN; ++j) acc[j] = 0.0f;
            const int nseg = (nkb + SEG - 1) / SEG;
            for (int seg = 0; seg < nseg; ++seg, ++gseg) {
                const int buf = gseg & 1;
                const uint32_t use = (uint32_t)(gseg >> 1);
                ok = __all_sync(0xffffffffu, mbar_wait(big_full(buf), use & 1u));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int c0 = 0; c0 < HN; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld32(lane_base + (uint32_t)(buf * BN + cbase + c0), r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[c0 + j] += __uint_as_float(r[j]);
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(big_empty(buf)) : "memory");
            }
            if (!ok) {
                if (lane == 0) fail_s = 1;
                break;
            }
            // the cross terms; after this read tensor memory is free for the tile after next, and the stores
            // below run under the next tile's MMAs
            ok = __all_sync(0xffffffffu, mbar_wait(x_full(xb), (uint32_t)(it >> 1) & 1u));
            if (!ok) {
                if (lane == 0) fail_s = 1;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int c0 = 0; c0 < HN; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(lane_base + (uint32_t)(2 * BN + xb * BN + cbase + c0), r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[c0 + j] += F16 ? __uint_as_float(r[j]) * LO_UNSCALE : __uint_as_float(r[j]);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(x_empty(xb)) : "memory");

            // fp16 mode: undo the operand scales (two exact factors: their product may leave the fp32 range)
            float inv_a = 1.0f, inv_b = 1.0f;
            if (F16) { inv_a = ldexpf(1.0f, -f16_scale_exp(*a.a_max)); inv_b = ldexpf(1.0f, -f16_scale_exp(*a.b_max)); }
            const int m = m0 + 32 * q + lane;
            const bool batched = a.nbatch > 0;
            const bool split = !batched && a.nz > 1;
            float *dst = batched ? a.C + a.c_off[batch] + (long long)zsplit * a.c_split_stride
                                 : (split ? a.ws + (size_t)z * (size_t)a.M * a.N : a.C);
            const long ld = split ? (long)a.M : a.ldc;
            if (m < a.M) {
#pragma unroll
                for (int j = 0; j < HN; ++j) {
                    const int n = n0 + cbase + j;
                    if (n < a.N) {
                        float *p = dst + (size_t)n * ld + m;
                        float v = F16 ? acc[j] * inv_a * inv_b : acc[j];
                        if (!split && !batched && a.accumulate) v += *p;
                        *p = v;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (fail_s && threadIdx.x == 0) atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT);
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

__global__ void tc_splitk_reduce_kernel(float *__restrict__ C, long ldc, const float *__restrict__ ws, int M, int N,
                                        int splits, int accumulate) {
    size_t total = (size_t)M * N;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float s = 0.0f;
        for (int z = 0; z < splits; ++z) s += ws[(size_t)z * total + i];
        size_t m = i % M, n = i / M;
        float *p = C + n * ldc + m;
        *p = accumulate ? *p + s : s;
    }
}

// sums the K-split partials of a batched launch: batch b, split z at ws[(b*splits + z)*M*N ...] (leading
// dimension M) -> C + c_off[b] (leading dimension ldc), fixed order
struct BatchOffsets { long long c_off[TC_MAX_BATCH]; };
__global__ void tc_batched_reduce_kernel(float *__restrict__ C, BatchOffsets off, long ldc, const float *__restrict__ ws, int M,
                                         int N, int splits, int nbatch) {
    const size_t per = (size_t)M * N, total = per * nbatch;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int b = (int)(i / per);
        const size_t e = i % per;
        const float *p = ws + (size_t)b * splits * per + e;
        float s = 0.0f;
        for (int z = 0; z < splits; ++z) s += p[(size_t)z * per];
        C[off.c_off[b] + (long long)(e / M) * ldc + (long long)(e % M)] = s;
    }
}

// hi = rn_tf32(x), lo = rn_tf32(x - hi); dense destination [outer][ldp], zero padded to ldp
__global__ void split_tf32_kernel(const float *__restrict__ src, long s_outer, int outer, int inner, float *__restrict__ hi,
                                  float *__restrict__ lo, long ldp) {
    const size_t total = (size_t)outer * ldp;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t o = i / ldp;
        const int c = (int)(i % ldp);
        float x = c < inner ? src[o * s_outer + c] : 0.0f;
        uint32_t h, l;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
        float rem = x - __uint_as_float(h);
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(rem));
        hi[i] = __uint_as_float(h);
        lo[i] = __uint_as_float(l);
    }
}

// the same for rows that are whole float4 groups (inner, the source stride and all bases multiples of 4)
__device__ __forceinline__ void split4(const float4 x, float4 &h, float4 &l) {
    const float in[4] = {x.x, x.y, x.z, x.w};
    float hh[4], ll[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t a, b;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(a) : "f"(in[i]));
        const float rem = in[i] - __uint_as_float(a);
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(b) : "f"(rem));
        hh[i] = __uint_as_float(a);
        ll[i] = __uint_as_float(b);
    }
    h = make_float4(hh[0], hh[1], hh[2], hh[3]);
    l = make_float4(ll[0], ll[1], ll[2], ll[3]);
}
__global__ void __launch_bounds__(256) split_tf32_vec4_kernel(const float *__restrict__ src, long s_outer, int outer, int inner4,
                                                              float4 *__restrict__ hi, float4 *__restrict__ lo) {
    const size_t total = (size_t)outer * inner4;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    // two independent groups per iteration keep more loads in flight
    for (; i + stride < total; i += 2 * stride) {
        const size_t j = i + stride;
        const float4 x0 = __ldg((const float4 *)(src + (i / inner4) * s_outer) + (i % inner4));
        const float4 x1 = __ldg((const float4 *)(src + (j / inner4) * s_outer) + (j % inner4));
        float4 h0, l0, h1, l1;
        split4(x0, h0, l0);
        split4(x1, h1, l1);
        hi[i] = h0; lo[i] = l0;
        hi[j] = h1; lo[j] = l1;
    }
    if (i < total) {
        const float4 x0 = __ldg((const float4 *)(src + (i / inner4) * s_outer) + (i % inner4));
        float4 h0, l0;
        split4(x0, h0, l0);
        hi[i] = h0; lo[i] = l0;
    }
}

// ---- fp16 parts.  The largest finite |x| of the operand first (bit pattern, atomicMax), then the split with the scale that follows from it.
__global__ void __launch_bounds__(256) absmax_kernel(const float *__restrict__ src, long s_outer, int outer, int inner, int vec4,
                                                     unsigned *maxbits) {
    unsigned m = 0u;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    if (vec4) {
        const int inner4 = inner / 4;
        const size_t total = (size_t)outer * inner4;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
            const float4 x = __ldg((const float4 *)(src + (i / inner4) * s_outer) + (i % inner4));
            const unsigned b0 = __float_as_uint(fabsf(x.x)), b1 = __float_as_uint(fabsf(x.y));
            const unsigned b2 = __float_as_uint(fabsf(x.z)), b3 = __float_as_uint(fabsf(x.w));
            if (b0 < 0x7f800000u) m = max(m, b0);   // NaN / Inf do not set the scale
            if (b1 < 0x7f800000u) m = max(m, b1);
            if (b2 < 0x7f800000u) m = max(m, b2);
            if (b3 < 0x7f800000u) m = max(m, b3);
        }
    } else {
        const size_t total = (size_t)outer * inner;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
            const unsigned b = __float_as_uint(fabsf(src[(i / inner) * s_outer + (i % inner)]));
            if (b < 0x7f800000u) m = max(m, b);
        }
    }
    for (int o = 16; o; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    __shared__ unsigned wm[8];
    if ((threadIdx.x & 31) == 0) wm[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) m = max(m, wm[w]);
        if (m) atomicMax(maxbits, m);
    }
}
__global__ void set_word_kernel(unsigned *dst, unsigned v) { *dst = v; }
inline unsigned float_bits(float f) { unsigned u; memcpy(&u, &f, sizeof u); return u; }
// x*S = hi + lo * 2^-11; both parts as fp16 bit patterns
__device__ __forceinline__ void split_f16_one(float x, float S, unsigned short &h, unsigned short &l) {
    const float xs = x * S;
    const __half hh = __float2half_rn(xs);
    const __half ll = __float2half_rn((xs - __half2float(hh)) * 2048.0f);
    h = __half_as_ushort(hh);
    l = __half_as_ushort(ll);
}
// dense destination [outer][ldp] halves, zero padded to ldp
__global__ void split_f16_kernel(const float *__restrict__ src, long s_outer, int outer, int inner, unsigned short *__restrict__ hi,
                                 unsigned short *__restrict__ lo, long ldp, const unsigned *__restrict__ maxbits) {
    const float S = ldexpf(1.0f, f16_scale_exp(*maxbits));
    const size_t total = (size_t)outer * ldp;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t o = i / ldp;
        const int c = (int)(i % ldp);
        const float x = c < inner ? src[o * s_outer + c] : 0.0f;
        split_f16_one(x, S, hi[i], lo[i]);
    }
}
// rows that are whole groups of 8 (inner == ldp, a multiple of 8; bases and the source stride 16-byte aligned)
__global__ void __launch_bounds__(256) split_f16_vec8_kernel(const float *__restrict__ src, long s_outer, int outer, int inner8,
                                                             uint4 *__restrict__ hi, uint4 *__restrict__ lo,
                                                             const unsigned *__restrict__ maxbits) {
    const float S = ldexpf(1.0f, f16_scale_exp(*maxbits));
    const size_t total = (size_t)outer * inner8;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const float4 *p = (const float4 *)(src + (i / inner8) * s_outer) + 2 * (i % inner8);
        const float4 x0 = __ldg(p), x1 = __ldg(p + 1);
        const float in[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
        unsigned short h[8], l[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) split_f16_one(in[e], S, h[e], l[e]);
        hi[i] = make_uint4(h[0] | ((unsigned)h[1] << 16), h[2] | ((unsigned)h[3] << 16), h[4] | ((unsigned)h[5] << 16),
                           h[6] | ((unsigned)h[7] << 16));
        lo[i] = make_uint4(l[0] | ((unsigned)l[1] << 16), l[2] | ((unsigned)l[3] << 16), l[4] | ((unsigned)l[5] << 16),
                           l[6] | ((unsigned)l[7] << 16));
    }
}

typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                             const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;

int get_encode() {
    if (g_encode) return B2_OK;
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    B2_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (!fn || qres != cudaDriverEntryPointSuccess) {
        set_error("cuTensorMapEncodeTiled is not available from this driver");
        return B2_ERR_CUDA;
    }
    g_encode = (EncodeFn)fn;
    return B2_OK;
}

// 2-D tensor map over one part of a split operand: dim0 = contiguous extent `inner`, dim1 = `outer` rows `ld` elements
// apart.  The box is one swizzle row wide; a K-major box has `rows` rows of the tile, an MN-major one BK rows.
int make_map(CUtensorMap *map, const float *base, long inner, long outer, long ld, int rows, bool kmajor, bool f16) {
    const int bk = f16 ? Mode<true>::BK : Mode<false>::BK, mnbox = f16 ? Mode<true>::MNBOX : Mode<false>::MNBOX;
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)ld * (f16 ? 2 : 4)};
    cuuint32_t box[2] = {(cuuint32_t)(kmajor ? bk : mnbox), (cuuint32_t)(kmajor ? rows : bk)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)base, dims,
                          strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          (kmajor || f16) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed (%d) for inner %ld outer %ld ld %ld", (int)r, inner, outer, ld);
        return B2_ERR_CUDA;
    }
    return B2_OK;
}

// one block per SM (the kernel loops over its share of the tiles), fewer when there is less work
int persistent_grid(int items) {
    const int sms = sm_count();
    return items < sms ? items : sms;
}

int set_kernel_attributes() {
    B2_TRY(set_max_dynamic_smem((const void *)gemm_split3_kernel<64, false>, SMEM_BYTES));
    B2_TRY(set_max_dynamic_smem((const void *)gemm_split3_kernel<128, false>, SMEM_BYTES));
    B2_TRY(set_max_dynamic_smem((const void *)gemm_split3_kernel<64, true>, SMEM_BYTES));
    B2_TRY(set_max_dynamic_smem((const void *)gemm_split3_kernel<128, true>, SMEM_BYTES));
    return B2_OK;
}

int launch_kernel(int bn, bool f16, int grid, const CUtensorMap &mAh, const CUtensorMap &mAl, const CUtensorMap &mBh,
                  const CUtensorMap &mBl, const TcArgs &a, cudaStream_t st) {
    if (f16) {
        if (bn == 64) gemm_split3_kernel<64, true><<<grid, NTHREADS, SMEM_BYTES, st>>>(mAh, mAl, mBh, mBl, a);
        else gemm_split3_kernel<128, true><<<grid, NTHREADS, SMEM_BYTES, st>>>(mAh, mAl, mBh, mBl, a);
    } else {
        if (bn == 64) gemm_split3_kernel<64, false><<<grid, NTHREADS, SMEM_BYTES, st>>>(mAh, mAl, mBh, mBl, a);
        else gemm_split3_kernel<128, false><<<grid, NTHREADS, SMEM_BYTES, st>>>(mAh, mAl, mBh, mBl, a);
    }
    count_launch();
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

}  // namespace

int split_tf32(const float *src, long s_outer, int outer, int inner, float *hi, float *lo, long ldp, cudaStream_t st) {
    size_t total = (size_t)outer * ldp;
    if (!total) return B2_OK;
    if ((inner % 4) == 0 && ldp == inner && (s_outer % 4) == 0 && ((uintptr_t)src % 16) == 0 && ((uintptr_t)hi % 16) == 0 &&
        ((uintptr_t)lo % 16) == 0) {
        const size_t groups = total / 4;
        size_t blocks = (groups + 511) / 512;
        if (blocks > (size_t)sm_count() * 8) blocks = (size_t)sm_count() * 8;
        if (blocks < 1) blocks = 1;
        split_tf32_vec4_kernel<<<(int)blocks, 256, 0, st>>>(src, s_outer, outer, inner / 4, (float4 *)hi, (float4 *)lo);
        count_launch();
        B2_CUDA(cudaGetLastError());
        return B2_OK;
    }
    size_t blocks = (total + 255) / 256;
    if (blocks > (size_t)sm_count() * 16) blocks = (size_t)sm_count() * 16;
    split_tf32_kernel<<<(int)blocks, 256, 0, st>>>(src, s_outer, outer, inner, hi, lo, ldp);
    count_launch();
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

// fp16 parts of a strided matrix view: hi / lo hold [outer][ldp] halves (ldp a multiple of 8), maxbits one word that
// receives the bit pattern of the largest finite |x| (the scale follows from it, on the device)
int split_f16(const float *src, long s_outer, int outer, int inner, void *hi, void *lo, long ldp, unsigned *maxbits,
              cudaStream_t st, float bound) {
    const size_t total = (size_t)outer * ldp;
    if (!total) return B2_OK;
    const bool v4 = (inner % 4) == 0 && (s_outer % 4) == 0 && ((uintptr_t)src % 16) == 0;
    if (bound > 0.0f) {
        // the caller knows that no entry exceeds `bound`: the scale follows from it, the pass over the operand is saved
        set_word_kernel<<<1, 1, 0, st>>>(maxbits, float_bits(bound));
        count_launch();
        B2_CUDA(cudaGetLastError());
    } else {
        B2_CUDA(cudaMemsetAsync(maxbits, 0, sizeof(unsigned), st));
        const size_t work = v4 ? (size_t)outer * (inner / 4) : (size_t)outer * inner;
        size_t blocks = (work + 1023) / 1024;
        if (blocks > (size_t)sm_count() * 8) blocks = (size_t)sm_count() * 8;
        if (blocks < 1) blocks = 1;
        absmax_kernel<<<(int)blocks, 256, 0, st>>>(src, s_outer, outer, inner, v4 ? 1 : 0, maxbits);
        count_launch();
        B2_CUDA(cudaGetLastError());
    }
    if (v4 && (inner % 8) == 0 && ldp == inner && ((uintptr_t)hi % 16) == 0 && ((uintptr_t)lo % 16) == 0) {
        const size_t groups = total / 8;
        size_t blocks = (groups + 255) / 256;
        if (blocks > (size_t)sm_count() * 16) blocks = (size_t)sm_count() * 16;
        split_f16_vec8_kernel<<<(int)blocks, 256, 0, st>>>(src, s_outer, outer, inner / 8, (uint4 *)hi, (uint4 *)lo, maxbits);
    } else {
        size_t blocks = (total + 255) / 256;
        if (blocks > (size_t)sm_count() * 16) blocks = (size_t)sm_count() * 16;
        split_f16_kernel<<<(int)blocks, 256, 0, st>>>(src, s_outer, outer, inner, (unsigned short *)hi, (unsigned short *)lo, ldp,
                                                      maxbits);
    }
    count_launch();
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

bool gemm_tc_supported(const SplitOperand &A, const SplitOperand &B, int m, int n, int k) {
    if (m < 1 || n < 1 || k < 1 || A.f16 != B.f16) return false;
    auto ok = [](const SplitOperand &o) {
        return o.hi && o.lo && (o.ld % (o.f16 ? 8 : 4)) == 0 && ((uintptr_t)o.hi % 16) == 0 && ((uintptr_t)o.lo % 16) == 0 &&
               (!o.f16 || o.maxbits);
    };
    return ok(A) && ok(B);
}


// C(m x n) (+)= A' B' from pre-split operands.  K-major A: rows m, `ld` floats apart, k contiguous;
// MN-major A: rows k, m contiguous.  Likewise B with n.
int gemm_tc(float *C, long ldc, const SplitOperand &A, const SplitOperand &B, int m, int n, int k, bool accumulate, float *ws,
            size_t ws_floats, int *status, cudaStream_t st) {
    B2_TRY(get_encode());
    B2_TRY(set_kernel_attributes());
    if (!gemm_tc_supported(A, B, m, n, k)) { set_error("gemm_tc: operand parts missing, misaligned or of different kinds"); return B2_ERR_BAD_ARG; }
    const bool f16 = A.f16;
    const int BK = f16 ? Mode<true>::BK : Mode<false>::BK;
    const int BN = n <= 64 ? 64 : 128;
    CUtensorMap mAh, mAl, mBh, mBl;
    B2_TRY(make_map(&mAh, A.hi, A.kmajor ? k : m, A.kmajor ? m : k, A.ld, BM, A.kmajor, f16));
    B2_TRY(make_map(&mAl, A.lo, A.kmajor ? k : m, A.kmajor ? m : k, A.ld, BM, A.kmajor, f16));
    B2_TRY(make_map(&mBh, B.hi, B.kmajor ? k : n, B.kmajor ? n : k, B.ld, BN, B.kmajor, f16));
    B2_TRY(make_map(&mBl, B.lo, B.kmajor ? k : n, B.kmajor ? n : k, B.ld, BN, B.kmajor, f16));
    dim3 grid((m + BM - 1) / BM, (n + BN - 1) / BN, 1);
    const int tiles = grid.x * grid.y;
    // Split K to fill the SMs when there are few output tiles; the partial sums are added with
    // fp32 FADD in a fixed order.
    int splits = 1;
    if (ws && k >= 1024) {
        // Model of the persistent kernel: every block runs ceil(items / SMs) tiles of k/splits slabs
        // (about 0.4 us per slab and 3 us per tile), then the partial sums cost a pass over
        // splits * m * n floats.  Pick the split count with the smallest estimate.
        const int sms = persistent_grid(1 << 30);
        const size_t per = (size_t)m * n;
        int maxs = (k + 255) / 256;
        if (maxs > 64) maxs = 64;
        if ((size_t)maxs * per > ws_floats) maxs = (int)(ws_floats / per);
        double best = 0.0;
        for (int sp = 1; sp <= maxs; ++sp) {
            const int items = tiles * sp;
            const int waves = (items + sms - 1) / sms;
            const double slabs = (double)((k + sp - 1) / sp + BK - 1) / BK;
            double t = waves * (0.4 * slabs + 3.0);
            if (sp > 1) t += 4.0 + (double)sp * per * 8.0 / 5.0e6;   // write + read of the partials at ~5 TB/s, in us
            if (sp == 1 || t < best) { best = t; splits = sp; }
        }
    }
    int kchunk = (k + splits - 1) / splits;
    kchunk = (kchunk + BK - 1) / BK * BK;
    splits = (k + kchunk - 1) / kchunk;
    grid.z = splits;
    TcArgs a;
    a.C = C; a.ldc = ldc; a.M = m; a.N = n; a.K = k; a.kchunk = kchunk;
    a.a_kmajor = A.kmajor ? 1 : 0; a.b_kmajor = B.kmajor ? 1 : 0;
    a.accumulate = accumulate ? 1 : 0; a.ws = ws; a.status = status;
    a.a_max = A.maxbits; a.b_max = B.maxbits;
    a.nbatch = 0; a.splits = splits; a.c_split_stride = 0; a.kseg_len = 0; a.kseg_stride = 0;
    a.tiles_m = (int)grid.x; a.tiles_n = (int)grid.y; a.nz = splits;
    B2_TRY(launch_kernel(BN, f16, persistent_grid(a.tiles_m * a.tiles_n * a.nz), mAh, mAl, mBh, mBl, a, st));
    if (splits > 1) {
        size_t total = (size_t)m * n;
        int blocks = (int)((total + 255) / 256);
        if (blocks > sm_count() * 8) blocks = sm_count() * 8;
        tc_splitk_reduce_kernel<<<blocks, 256, 0, st>>>(C, ldc, ws, m, n, splits, accumulate ? 1 : 0);
        count_launch();
        B2_CUDA(cudaGetLastError());
    }
    return B2_OK;
}

// ---- planned, batched launches: the tensor maps are encoded once and reused for many launches that
// differ only in coordinate offsets (one launch per timestep of the tensor-core recurrence)
struct TcPlan {
    int bn;   // N extent of the tile: 64 or 128
    bool f16;
    CUtensorMap mAh, mAl, mBh, mBl;
    TcArgs args;
    dim3 grid;
};

int tc_plan_create(TcPlan **out, const SplitOperand &A, long a_inner, long a_outer, const SplitOperand &B, long b_inner,
                   long b_outer, int m, int n, int k, int splits, int kseg_len, int kseg_stride, long ldc) {
    B2_TRY(get_encode());
    B2_TRY(set_kernel_attributes());
    if (!gemm_tc_supported(A, B, m, n, k)) { set_error("tc_plan_create: operand parts missing, misaligned or of different kinds"); return B2_ERR_BAD_ARG; }
    const bool f16 = A.f16;
    const int BK = f16 ? Mode<true>::BK : Mode<false>::BK;
    const int BN = n <= 64 ? 64 : 128;
    // a segmented contraction index needs whole slabs per split; a contiguous one may be ragged (the
    // tensor maps fill the overhang with zeros as long as one operand's extent ends at k)
    if (splits < 1 || (kseg_len && ((k % (splits * BK)) != 0 || (kseg_len % BK) != 0))) {
        set_error("tc_plan_create: k=%d must divide into %d splits of whole %d-slabs (segment %d)", k, splits, BK, kseg_len);
        return B2_ERR_BAD_SHAPE;
    }
    TcPlan *p = new TcPlan;
    p->bn = BN;
    p->f16 = f16;
    int rc = make_map(&p->mAh, A.hi, a_inner, a_outer, A.ld, BM, A.kmajor, f16);
    if (rc == B2_OK) rc = make_map(&p->mAl, A.lo, a_inner, a_outer, A.ld, BM, A.kmajor, f16);
    if (rc == B2_OK) rc = make_map(&p->mBh, B.hi, b_inner, b_outer, B.ld, BN, B.kmajor, f16);
    if (rc == B2_OK) rc = make_map(&p->mBl, B.lo, b_inner, b_outer, B.ld, BN, B.kmajor, f16);
    if (rc != B2_OK) { delete p; return rc; }
    TcArgs &a = p->args;
    a = TcArgs{};
    a.ldc = ldc; a.M = m; a.N = n; a.K = k;
    a.kchunk = ((k + splits - 1) / splits + BK - 1) / BK * BK;
    if ((long)a.kchunk * (splits - 1) >= k) {
        set_error("tc_plan_create: %d splits leave an empty split for k=%d", splits, k);
        delete p;
        return B2_ERR_BAD_SHAPE;
    }
    a.a_kmajor = A.kmajor ? 1 : 0; a.b_kmajor = B.kmajor ? 1 : 0;
    a.a_max = A.maxbits; a.b_max = B.maxbits;
    a.splits = splits; a.kseg_len = kseg_len; a.kseg_stride = kseg_stride;
    p->grid = dim3((m + BM - 1) / BM, (n + BN - 1) / BN, 1);
    *out = p;
    return B2_OK;
}

void tc_plan_destroy(TcPlan *p) { delete p; }

int tc_batched_reduce(float *C, const long long *c_off, int nbatch, long ldc, const float *ws, int m, int n, int splits,
                      cudaStream_t st) {
    if (nbatch < 1 || nbatch > TC_MAX_BATCH) { set_error("tc_batched_reduce: 1..%d batches", TC_MAX_BATCH); return B2_ERR_BAD_ARG; }
    BatchOffsets off;
    for (int b = 0; b < nbatch; ++b) off.c_off[b] = c_off[b];
    const size_t total = (size_t)m * n * nbatch;
    int blocks = (int)((total + 255) / 256);
    if (blocks > sm_count() * 8) blocks = sm_count() * 8;
    tc_batched_reduce_kernel<<<blocks, 256, 0, st>>>(C, off, ldc, ws, m, n, splits, nbatch);
    count_launch();
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

int tc_sm_count() { return persistent_grid(1 << 30); }

int tc_plan_launch(const TcPlan *p, float *C, const TcBatch *batches, int nbatch, long long c_split_stride, int *status,
                   cudaStream_t st) {
    if (nbatch < 1 || nbatch > TC_MAX_BATCH) { set_error("tc_plan_launch: 1..%d batches", TC_MAX_BATCH); return B2_ERR_BAD_ARG; }
    TcArgs a = p->args;
    a.C = C; a.status = status; a.nbatch = nbatch; a.c_split_stride = c_split_stride;
    for (int b = 0; b < nbatch; ++b) {
        a.a_off_inner[b] = batches[b].a_in; a.a_off_outer[b] = batches[b].a_out;
        a.b_off_inner[b] = batches[b].b_in; a.b_off_outer[b] = batches[b].b_out;
        a.c_off[b] = batches[b].c_off;
    }
    a.tiles_m = (int)p->grid.x; a.tiles_n = (int)p->grid.y; a.nz = nbatch * a.splits;
    return launch_kernel(p->bn, p->f16, persistent_grid(a.tiles_m * a.tiles_n * a.nz), p->mAh, p->mAl, p->mBh, p->mBl, a, st);
}

}  // namespace b2
