// Persistent tensor-core recurrence: ONE launch runs all timesteps of a (b)lstm layer's forward sweep (a second
// one the BPTT sweep) for any number of parallel sequences, with the recurrent weights RESIDENT in shared memory
// as tcgen05 operands for the whole sweep.
//
// Replaces the reference's loop of 4 cublasSgemm + 1 Thrust functor per timestep and direction
// (layers/LstmLayer.cu:1805-1858,1878-1927 forward with ComputeBlockOutputFn :57-185; :2115-2176,2195-2253
// backward with ComputeBlockErrorsFn :237-405 of the reference), and the launch pair per timestep of
// lstm_step_tc.cu, which re-reads the weights from L2 at every step.
//
// Numerics.  fp32 values enter the tensor cores as TWO fp16 terms: x = hi + lo * 2^-11 with hi = rn_f16(x * S),
// lo = rn_f16((x * S - hi) * 2^11).  S is a power of two: 1 for block outputs and gate deltas (both lie in
// [-1, 1]: h = tanh(c) * og, and the deltas are clipped by helpers::limitedError), and per direction
// 2^13 <= max|w| * S < 2^14 for the recurrent weights.  Three kind::f16 MMAs per product, a_hi*b_hi into a main
// accumulator and a_lo*b_hi + a_hi*b_lo into a cross-term accumulator, both fp32 in tensor memory; the result
// (main + cross * 2^-11) / S carries 22 mantissa bits of each operand, the same scheme as the large GEMMs
// (gemm_tc.cu).  An accumulator never takes more than 8 main-term MMAs
// (K = 128): tensor-memory accumulation truncates, so longer contractions are split over blocks and added by CUDA cores.
//
// Measured on B200: a tcgen05.mma costs its issuing thread about 85 cycles whatever M and N are (up to N = 128), so
// the instruction count per step is what matters.  The decomposition therefore spreads the 3 * (4*els/128) * (els/16)
// instructions of a step and direction evenly: els = 512 gives 16 row tiles x 4 contraction slices = 64 blocks per
// direction, 24 instructions per block and step, for up to 64 sequences at once.
//
//   forward : block (r, q) keeps W_rec rows {gate g, unit 32r + jj} x source units [128q, 128q + 128) (128 x 128,
//             hi + lo = 64 KB).  Per step it multiplies them with h[t-1] of its slice (operand B, N = 32 or 64
//             sequences), the four blocks of a row tile (a thread-block cluster) exchange quarters of the 128 x N
//             partial sums through distributed shared memory (st.async + transaction barrier) and each finishes 8
//             units: gate activations, peepholes, cell state, h.  h is published as fp16 hi/lo chunks, already in
//             the swizzled operand layout, into a per-slice image in global memory (L2), followed by one release
//             store of the step counter per block; a consumer's polling warp acquires the 16 counters of its slice
//             and fetches the whole operand with ONE bulk copy (cp.async.bulk) that completes on the MMA's barrier.
//   backward: the same weight tile, stored transposed, is operand A of  e[k] = sum_c W[c][k] delta[c]  with the
//             block's own row tile as the contraction range: the four blocks of a row tile compute 8 units' gate
//             deltas each, write them as fp16 hi / lo into their own operand buffer (stored WITHOUT swizzle, so that
//             a block's share is contiguous per gate) and hand them to each other through distributed shared memory
//             (bulk copies issued by a sender warp, or st.async from the cell warps where the latency is in the chain);
//             block (r, q) turns them into partial output errors of source units [128q, 128q + 128), publishes them
//             (fp32) with a release store of its step counter, and the block that owns a unit adds the 16 partials
//             in a fixed order (bitwise deterministic) and runs the error functor.
// Groups of sequences ("chunks" of N) are independent; a group of blocks works on several chunks in turn, so that
// the exchange of one chunk overlaps the tensor-core work of another.  Warps are specialised (poll / MMA issue /
// tensor-memory drain / cell math / publisher; backward also sender and reduce) and hand buffers to each other through
// mbarriers.  With few chunks per group a step is a chain of latencies, and the exchange through L2 uses
// self-validating words {step tag : payload} instead of counters and bulk copies (template parameter LL; make_plan
// chooses per sweep, every choice gives the same bits).
//
// Every wait is bounded (cycle budget of about two seconds, poll-round limit for the step counters): on expiry the
// thread records B2_ERR_STEP_TIMEOUT in the layer's status word and raises the block's give-up flag, every role
// leaves its loops, the cluster meets at its hardware barrier, tensor memory is released and the block returns.
#include <cuda_fp16.h>

#include <algorithm>
#include <atomic>
#include "common.cuh"
#include "ptx.cuh"

namespace b2 {
namespace {

using namespace ptx;

constexpr int MAXC = 16;                 // chunks a group of blocks works on at most
constexpr int KSL = 128;                 // contraction extent a block holds
constexpr int UPC = 8;                   // units a block finishes (32 units of a row tile / 4 blocks)
constexpr int KS = 4;                    // blocks of a row tile = cluster size
constexpr long long WAIT_CYCLES = 4000000000LL;
constexpr unsigned POLL_LIMIT = 1u << 22;
constexpr float LO_SCALE = 2048.0f, LO_UNSCALE = 1.0f / 2048.0f;
constexpr uint32_t A_HALF = 32768, A_BYTES = 65536;   // weight image: hi, lo of 128 rows x 128 fp16

// Warp roles.  Forward: warp 0 MMA issue, 1 poll + operand fetch, 2-5 drain, then the cell-math warps, the publisher, and
// a second MMA-issue warp.  Backward: warp 0 MMA issue, then the cell-math warps, 4 drain warps, 4 gather + reduce warps,
// the publisher, a second MMA-issue warp and the sender.  Two issuers: measured with a probe, 24 MMAs cost one issuing thread 1870
// cycles, two threads of different warps (12 each, accumulators of their own) 940.
// With several chunks per group the cell math bounds the throughput, so that variant gets twice the cell warps; with
// one chunk per group (LL) a step is a chain of latencies and fewer, fatter threads are as good.
__host__ __device__ constexpr int fwd_cell_warps(bool ll) { return ll ? 8 : 16; }
__host__ __device__ constexpr int bwd_cell_warps(bool ll) { return ll ? 4 : 8; }
__host__ __device__ constexpr int fwd_threads(bool ll) { return 32 * (8 + fwd_cell_warps(ll)); }
__host__ __device__ constexpr int bwd_threads(bool ll) { return 32 * (12 + bwd_cell_warps(ll)); }

// Optional timing trace (build with -DB2_PTC_TRACE): block 0 records clock64() at the hand-over points of its
// roles for the first chunk-steps of a launch; b2_debug_ptc_trace copies the records out.
#ifdef B2_PTC_TRACE
constexpr int TRACE_ITEMS = 96, TRACE_SLOTS = 8, TRACE_ROLES = 4;
__device__ long long g_ptc_trace[2][TRACE_ROLES][TRACE_ITEMS][TRACE_SLOTS];   // [forward / backward sweep]
#define PTC_TRACE(role, item, slot)                                                                  \
    do {                                                                                             \
        if (blockIdx.x == 0 && (item) < TRACE_ITEMS) g_ptc_trace[0][role][item][slot] = clock64();   \
    } while (0)
#define PTC_TRACE_B(role, item, slot)                                                                \
    do {                                                                                             \
        if (blockIdx.x == 0 && (item) < TRACE_ITEMS) g_ptc_trace[1][role][item][slot] = clock64();   \
    } while (0)
#else
#define PTC_TRACE(role, item, slot) do { } while (0)
#define PTC_TRACE_B(role, item, slot) do { } while (0)
#endif
#if defined(B2_PTC_TRACE) && defined(B2_PTC_TRACE_CELL)
#define PTC_TRACE_C(role, item, slot) PTC_TRACE(role, item, slot)
#else
#define PTC_TRACE_C(role, item, slot) do { } while (0)
#endif

struct PtcArgs {
    LstmShape sh;
    LstmBuffers bf;
    const float *w;
    float *y;              // forward: block outputs
    const float *dy;       // backward: output errors
    const uint4 *wimg;     // the blocks' weight images, 64 KB each, [direction][row tile][slice]
    const float *scale;    // [direction][2]: S, 1/S
    unsigned char *xh;     // forward exchange: operand images [direction][chunk][step parity][slice][hi/lo][2][NC][128 B]
    float *xe;             // backward exchange: [direction][chunk][step parity][row tile][NC][els]
    unsigned *flags;       // step counters [direction][chunk][block of the group]
    int *status;
    unsigned tag_base;
    int nslices;           // sequence slices per direction (chunks are dealt to the slices round robin)
    int nchunks;           // chunks of NC sequences in all
};

// The activations of the cell warps.  They are the longest stretch of instructions in a chunk-step, so they use the
// hardware approximations: ex2.approx on x * log2(e) (__expf: 2 + |1.17 x| ulp on e^-x, which the logistic function damps by
// y (1 - y) <= 1/4) and rcp.approx (1 ulp).  The result stays within 2 ulp of the correctly rounded logistic function,
// the same class as expf + IEEE division; the clamps are those of the reference's safeExp
// (helpers/NumericLimits / activation functions: exp arguments limited to +-88.72).
__device__ __forceinline__ float fast_logistic(float x) {
    const float lim = 88.722839f;
    if (x < lim) {
        if (x > -lim) return __fdividef(1.0f, 1.0f + __expf(-x));
        return 0.0f;
    }
    return 1.0f;
}
__device__ __forceinline__ float fast_tanh(float x) { return 2.0f * fast_logistic(2.0f * x) - 1.0f; }

__device__ __forceinline__ unsigned split_f16(float x) {   // hi in the low half, lo in the high half
    const __half h = __float2half_rn(x);
    const __half l = __float2half_rn((x - __half2float(h)) * LO_SCALE);
    return (unsigned)__half_as_ushort(h) | ((unsigned)__half_as_ushort(l) << 16);
}

// advances (s, cl) to the next chunk-step of the sweep: steps outermost, chunk cl only while s < Tc[cl]
__device__ __forceinline__ bool next_item(int &s, int &cl, int ncl, const int *Tc, int Tmax) {
    for (;;) {
        if (++cl >= ncl) { cl = 0; ++s; }
        if (s >= Tmax) return false;
        if (s < Tc[cl]) return true;
    }
}

// Lengths of the sequences of this work item's chunks (padding frames trail a sequence, as the data set writes
// them; frames below Tmin are real for every sequence slot), the chunks' longest lengths and their maximum.
template <int NC>
__device__ void find_lengths(const PtcArgs &a, int sl, int ncl, int *lens, int *Tc, int *Tmax_s, int nthreads) {
    const int P = a.sh.P, T = a.sh.T;
    for (int i = threadIdx.x; i < ncl * NC; i += nthreads) {
        const int cl = i / NC, n = i % NC;
        const int pg = (sl + cl * a.nslices) * NC + n;
        int len = 0;
        if (pg < P) {
            int lo = a.sh.Tmin, hi = T;
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (a.bf.pat[(size_t)mid * P + pg] == PAT_NONE) hi = mid; else lo = mid + 1;
            }
            len = lo;
        }
        lens[i] = len;
    }
    __syncthreads();
    if ((int)threadIdx.x < ncl) {
        int m = 0;
        for (int n = 0; n < NC; ++n) m = max(m, lens[threadIdx.x * NC + n]);
        Tc[threadIdx.x] = m;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int m = 0;
        for (int c = 0; c < ncl; ++c) m = max(m, Tc[c]);
        *Tmax_s = m;
    }
    __syncthreads();
}

template <int ELS, int NC>
struct Geo {
    static constexpr int RT = ELS / 32;            // row tiles per direction
    static constexpr int GROUP = RT * KS;          // blocks per group
    static_assert(ELS == 4 * KSL && RT == 16, "instantiated for 512 units per direction: 4 slices, 16 producers per slice");
    static_assert(NC == 32 || NC == 64, "chunks of 32 or 64 sequences");
    static constexpr uint32_t ZBLK = 4 * NC * UPC * 4;                  // one 4-gate x NC x 8-unit block of partial sums
    static constexpr uint32_t B_HL = 2 * NC * 128, B_BUF = 2 * B_HL;    // operand B: [hi/lo][2 column blocks][NC rows x 128 B]
    // forward
    static constexpr uint32_t F_B = A_BYTES, F_ZOWN = F_B + 2 * B_BUF, F_ZRECV = F_ZOWN + 2 * ZBLK;
    // staging of the tagged words of one operand (chunks of 32 sequences with several chunks per group: gather warps)
    static constexpr uint32_t F_STAGE = F_ZRECV + 2 * (KS - 1) * ZBLK;
    static constexpr uint32_t F_END = F_STAGE + (NC == 32 ? NC * 1024 : 0);
    // backward
    static constexpr uint32_t B_B = A_BYTES, B_ESUM = B_B + 2 * B_BUF;
    // what a cell hands to its own next step (forget gate, cell error, two gate deltas), for up to CARRY chunks per group
    static constexpr int CARRY = NC == 32 ? 8 : 4;
    static constexpr uint32_t B_CARRY = B_ESUM + 2 * NC * UPC * 4;
    static constexpr uint32_t B_END = B_CARRY + CARRY * 4 * NC * UPC * 4;
    static constexpr size_t fwd_smem() { return F_END + 1024; }
    static constexpr size_t bwd_smem() { return B_END + 1024; }
};

// copies this block's 64 KB weight image into shared memory (generic proxy) and hands it to the tensor core
__device__ __forceinline__ void load_weight_image(unsigned char *dst, const uint4 *src, int nthreads) {
    uint4 *d4 = reinterpret_cast<uint4 *>(dst);
    for (int i = threadIdx.x; i < (int)(A_BYTES / 16); i += nthreads) d4[i] = __ldg(src + i);
    fence_async_smem();
    __syncthreads();
}

// One warp waits until the 16 step counters flags[lane * stride] (lanes 16-31 repeat 0-15) have reached `want`; the
// counters only grow.  The acquire orders the producers' data, written before their release stores, before what
// this warp reads next.
__device__ __forceinline__ bool poll_flags(const unsigned *flags, int stride, unsigned want, int lane, volatile int *give_up,
                                           const int *status) {
    const unsigned *p = flags + (size_t)((lane & 15) * stride);
    for (unsigned round = 0;; ++round) {
        const bool ready = (int)(ld_acquire_u32(p) - want) >= 0;
        if (__all_sync(0xffffffffu, ready)) return true;
        if (round >= POLL_LIMIT || *give_up || ((round & 255u) == 255u && ld_relaxed_s32(status) != 0)) return false;
    }
}

// =====================================================================================================
// forward
// =====================================================================================================
template <int ELS, int NC, bool LL>
__global__ void __launch_bounds__(fwd_threads(LL), 1) lstm_fwd_ptc_kernel(PtcArgs a) {
    typedef Geo<ELS, NC> G;
    constexpr int CW = fwd_cell_warps(LL), FWD_THREADS = fwd_threads(LL);
    constexpr int RT = G::RT, CPT = NC / (4 * CW);   // a cell warp covers 8 units x 4 sequences
    static_assert(CPT >= 1, "more cell warps than cells");
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) u64 bars[17];
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int give_up_s;
    __shared__ int lens_s[MAXC * NC], Tc_s[MAXC], Tmax_s;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char *gbase = smem_raw + (sbase - smem_u32(smem_raw));
    const uint32_t bar0 = smem_u32(bars);
    auto rel_full = [&](int b) { return bar0 + 8u * (uint32_t)(12 + b); };  // cell warps have stored their part of h[t] -> publisher
    auto rel_free = [&](int b) { return bar0 + 8u * (uint32_t)(14 + b); };  // publisher -> cell warps
    auto b_full = [&](int b) { return bar0 + 8u * (uint32_t)b; };          // bulk copy of operand B -> MMA
    auto b_free = [&](int b) { return bar0 + 8u * (uint32_t)(2 + b); };    // MMA -> poll warp
    auto acc_full = [&](int b) { return bar0 + 8u * (uint32_t)(4 + b); };  // MMA -> drain warps
    auto acc_free = [&](int b) { return bar0 + 8u * (uint32_t)(6 + b); };  // drain warps -> MMA
    auto z_full = [&](int b) { return bar0 + 8u * (uint32_t)(8 + b); };    // own and the peers' partial sums are in -> cell warps
    auto z_free = [&](int b) { return bar0 + 8u * (uint32_t)(10 + b); };   // cell warps of the whole cluster have read them -> drain warps
    const uint32_t stage_bar = bar0 + 8u * 16u;                             // bulk copies of tagged words -> gather warps
    // Chunks of 32 sequences with several chunks per group: the operand of a chunk-step was published a whole chunk-step
    // earlier, so two otherwise idle warps collect it (bulk copies of the tagged words into a staging area, validation and
    // repacking from there) while the cell warps work on the other chunks.  With one chunk per group the cell warps collect
    // it themselves, word by word, right after publishing (lowest latency).
    const bool gw = LL && NC == 32 && (a.nchunks + a.nslices - 1) / a.nslices >= 2;

    const int P = a.sh.P, T = a.sh.T, ls = a.sh.ls, D = a.sh.D;
    const int grp = blockIdx.x / G::GROUP, ngroups = gridDim.x / G::GROUP;
    const int bidx = blockIdx.x % G::GROUP, r = bidx / KS;
    const int q = (int)cluster_ctarank();
    const LstmOffsets off = lstm_offsets(a.sh.pls, ls, ELS);

    if (tid == 0) {
        for (int b = 0; b < 2; ++b) {
            mbar_init(b_full(b), LL && !gw ? CW : 1); mbar_init(b_free(b), 2); mbar_init(acc_full(b), 2); mbar_init(acc_free(b), 4);
            mbar_init(z_full(b), 5);           // 4 drain warps + the arrival that announces the peers' bytes
            mbar_init(z_free(b), CW * KS);     // every cell warp of every block of the cluster
            mbar_init(rel_full(b), CW); mbar_init(rel_free(b), 1);
        }
        mbar_init(stage_bar, 1);
        give_up_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc(smem_u32(&tmem_base_s), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    // a peer's shared memory and barriers may be touched only once the peer runs
    cluster_sync_all();

    int m_g = 0, m_m = 0, m_d = 0, m_e = 0;   // running count of MMA items per role (buffer = count & 1)
    int m_p = 0;                             // running count of published chunk-steps (cell warps and publisher)
    uint32_t st_ph = 0;                      // phase of the staging barrier (gather warps)
    const int nwork = D * a.nslices;
    for (int wi = grp; wi < nwork; wi += ngroups) {
        const int d = wi % D, sl = wi / D;
        const int ncl = (a.nchunks - sl + a.nslices - 1) / a.nslices;
        load_weight_image(gbase, a.wimg + (size_t)((d * RT + r) * KS + q) * (A_BYTES / 16), FWD_THREADS);
        find_lengths<NC>(a, sl, ncl, lens_s, Tc_s, &Tmax_s, FWD_THREADS);
        const int Tmax = Tmax_s;
        const float invS = a.scale[2 * d + 1];
        const size_t dch = (size_t)d * a.nchunks;

        if (warp == 0 || warp == 7 + CW) {
            // ------------------------------------------------ MMA issue (two warps, half of the k-steps each) ------------------------------------------------
            if (lane == 0) {
                const int hh = warp == 0 ? 0 : 1;
                const uint32_t idesc = idesc_f16(128, NC);
                int s = 0, cl = -1;
                while (next_item(s, cl, ncl, Tc_s, Tmax)) {
                    if (s == 0) continue;
                    if (give_up_s) break;
                    const int buf = m_m & 1;
                    const uint32_t ph = (uint32_t)(m_m >> 1) & 1u;
                    const int ti = m_m;
                    (void)ti;
                    ++m_m;
                    if (hh == 0) PTC_TRACE(0, ti, 0);
                    if (!mbar_wait_bounded<false>(b_full(buf), ph, &give_up_s, WAIT_CYCLES) ||
                        !mbar_wait_bounded<false>(acc_free(buf), ph ^ 1u, &give_up_s, WAIT_CYCLES)) {
                        give_up_s = 1;
                        break;
                    }
                    if (hh == 0) PTC_TRACE(0, ti, 1);
                    if (LL) fence_async_smem();
                    tc_fence_after();
                    // accumulators of buffer buf: [main | cross] of issuer 0, then of issuer 1, 64 columns each
                    const uint32_t acc = tmem + (uint32_t)(buf * 256 + hh * 128);
                    const uint32_t bb = sbase + G::F_B + (uint32_t)buf * G::B_BUF;
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4) {
                        const int ks = 4 * hh + k4;
                        const uint32_t ao = (uint32_t)(ks >> 2) * 16384u + (uint32_t)(ks & 3) * 32u;
                        const uint32_t bo = (uint32_t)(ks >> 2) * (NC * 128u) + (uint32_t)(ks & 3) * 32u;
                        const u64 ahi = desc_kmajor_sw128(sbase + ao, 1024), alo = desc_kmajor_sw128(sbase + A_HALF + ao, 1024);
                        const u64 bhi = desc_kmajor_sw128(bb + bo, 1024), blo = desc_kmajor_sw128(bb + G::B_HL + bo, 1024);
                        mma_f16(acc + 64u, alo, bhi, idesc, k4 ? 1u : 0u);
                        mma_f16(acc + 64u, ahi, blo, idesc, 1u);
                        mma_f16(acc, ahi, bhi, idesc, k4 ? 1u : 0u);
                    }
                    mma_commit(b_free(buf));
                    mma_commit(acc_full(buf));
                    if (hh == 0) PTC_TRACE(0, ti, 2);
                }
            }
        } else if (gw && (warp == 1 || warp == 6 + CW)) {
            // ------------------------------------ gather warps: tagged words of h[t-1] -> operand B ------------------------------------
            if constexpr (LL && NC == 32) {
                const int gt = (warp == 1 ? 0 : 32) + lane;          // 64 gather threads
                int s = 0, cl = -1;
                while (next_item(s, cl, ncl, Tc_s, Tmax)) {
                    if (s == 0) continue;
                    if (give_up_s) break;
                    const int buf = m_g & 1;
                    const uint32_t ph = (uint32_t)(m_g >> 1) & 1u;
                    ++m_g;
                    const int ac = sl + cl * a.nslices;
                    // operand buffer buf: the MMAs of the chunk-step before last have read it (the gather threads go on together or not at all)
                    bool ok = mbar_wait_bounded<false>(b_free(buf), ph ^ 1u, &give_up_s, WAIT_CYCLES);
                    if (bar_named_or(1, 64, !ok)) { give_up_s = 1; atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT); break; }
                    const u64 *src = reinterpret_cast<const u64 *>(a.xh) + ((dch + ac) * 2 + ((s - 1) & 1)) * (size_t)(NC * ELS) + KSL * q;
                    const unsigned tag = a.tag_base + (unsigned)(s - 1);
                    const uint32_t bb = sbase + G::F_B + (uint32_t)buf * G::B_BUF;
                    const uint32_t stg = sbase + G::F_STAGE;
                    // Cheap wait first: one word per gather thread (of each of the 16 source blocks, the sequences their cell warps
                    // publish last) until it shows the step's tag; a round of bulk copies that comes too early costs far more.
                    {
                        const u64 *sw = src + (size_t)(NC - 1 - (gt >> 4)) * ELS + 8 * (gt & 15) + 6;
                        for (unsigned round = 0; ok; ++round) {
                            u64 w0, w1;
                            ld_tagged2(sw, w0, w1);
                            if ((unsigned)(w0 >> 32) == tag && (unsigned)(w1 >> 32) == tag) break;
                            if (round >= POLL_LIMIT || give_up_s || ((round & 1023u) == 1023u && ld_relaxed_s32(a.status) != 0)) ok = false;
                        }
                        if (bar_named_or(1, 64, !ok)) { give_up_s = 1; atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT); break; }
                    }
                    for (unsigned round = 0;; ++round) {
                        // one row of 128 words (this block's contraction slice of one sequence) per copy; then wait for all of them
                        if (gt == 0) mbar_expect_tx(stage_bar, NC * 1024u);
                        if (gt < NC) bulk_g2s(stg + (uint32_t)gt * 1024u, src + (size_t)gt * ELS, 1024u, stage_bar);
                        ok = mbar_wait_bounded<false>(stage_bar, st_ph, &give_up_s, WAIT_CYCLES);
                        st_ph ^= 1u;
                        bool all = ok;
                        if (ok) {
#pragma unroll 2
                            for (int i = 0; i < NC * 16 / 64; ++i) {
                                const int ci = gt + 64 * i, n = ci >> 4, kc = ci & 15;
                                const uint4 *sp = reinterpret_cast<const uint4 *>(gbase + G::F_STAGE + n * 1024 + kc * 64);
                                const uint4 w01 = sp[0], w23 = sp[1], w45 = sp[2], w67 = sp[3];   // {payload, tag} pairs
                                const bool valid = w01.y == tag && w01.w == tag && w23.y == tag && w23.w == tag && w45.y == tag &&
                                                   w45.w == tag && w67.y == tag && w67.w == tag;
                                if (!valid) { all = false; continue; }
                                const uint32_t pl[8] = {w01.x, w01.z, w23.x, w23.z, w45.x, w45.z, w67.x, w67.z};   // hi | lo << 16
                                uint32_t hi[4], lo[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    hi[e] = (pl[2 * e] & 0xffffu) | (pl[2 * e + 1] << 16);
                                    lo[e] = (pl[2 * e] >> 16) | (pl[2 * e + 1] & 0xffff0000u);
                                }
                                const uint32_t o = (uint32_t)(kc >> 3) * (NC * 128u) + (uint32_t)n * 128u + (uint32_t)(((kc & 7) ^ (n & 7)) * 16);
                                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(bb + o), "r"(hi[0]), "r"(hi[1]), "r"(hi[2]), "r"(hi[3]) : "memory");
                                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(bb + G::B_HL + o), "r"(lo[0]), "r"(lo[1]), "r"(lo[2]), "r"(lo[3]) : "memory");
                            }
                        }
                        // every gather thread is through the staging area; repeat while a word did not show the step's tag yet
                        if (!bar_named_or(1, 64, !all)) break;
                        if (!ok || round >= POLL_LIMIT || give_up_s || ((round & 255u) == 255u && ld_relaxed_s32(a.status) != 0)) ok = false;
                        if (bar_named_or(1, 64, !ok)) { ok = false; break; }
                    }
                    if (!ok) { give_up_s = 1; atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT); break; }
                    fence_async_smem();
                    bar_named(1, 64);
                    if (gt == 0) mbar_arrive(b_full(buf));
                }
            }
        } else if (warp == 1) {
            // ------------------------------------ wait for h[t-1] of this block's slice, fetch it as operand B ------------------------------------
            int s = 0, cl = -1;
            while (!LL && next_item(s, cl, ncl, Tc_s, Tmax)) {
                if (s == 0) continue;
                if (give_up_s) break;
                const int buf = m_g & 1;
                const uint32_t ph = (uint32_t)(m_g >> 1) & 1u;
                const int ti = m_g;
                (void)ti;
                ++m_g;
                if (lane == 0) PTC_TRACE(2, ti, 0);
                const int ac = sl + cl * a.nslices;
                bool ok = __all_sync(0xffffffffu, mbar_wait_bounded<false>(b_free(buf), ph ^ 1u, &give_up_s, WAIT_CYCLES));
                if (lane == 0) PTC_TRACE(2, ti, 1);
                // the 16 blocks that finish the units of slice q: row tiles 4q .. 4q+3, all four of each
                ok = ok && poll_flags(a.flags + (dch + ac) * G::GROUP + 16 * q, 1, a.tag_base + (unsigned)(s - 1), lane, &give_up_s, a.status);
                if (!ok) { give_up_s = 1; atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT); break; }
                if (lane == 0) {
                    PTC_TRACE(2, ti, 2);
                    fence_async_all();
                    mbar_expect_tx(b_full(buf), G::B_BUF);
                    bulk_g2s(sbase + G::F_B + (uint32_t)buf * G::B_BUF,
                             a.xh + ((dch + ac) * 2 + ((s - 1) & 1)) * (size_t)(KS * G::B_BUF) + (size_t)q * G::B_BUF, G::B_BUF, b_full(buf));
                }
                __syncwarp();
            }
        } else if (warp == 6 + CW) {
            // ------------------------------------ publisher: the block's step counter follows its h[t] ------------------------------------
            // The cell warps hand their stores over through a CTA-scope barrier; the release store at gpu scope is
            // cumulative over them.  Its fence waits for every global store of the block that is still in flight, which
            // is why it sits in a warp of its own and not in the cell warps' loop.
            int s = 0, cl = -1;
            while (!LL && next_item(s, cl, ncl, Tc_s, Tmax)) {
                if (s + 1 >= Tc_s[cl]) continue;
                if (give_up_s) break;
                const int pb = m_p & 1;
                const uint32_t pph = (uint32_t)(m_p >> 1) & 1u;
                const int ti = m_p;
                (void)ti;
                ++m_p;
                if (lane == 0) PTC_TRACE(2, ti, 4);
                const bool ok = mbar_wait_bounded<false>(rel_full(pb), pph, &give_up_s, WAIT_CYCLES);
                if (!__all_sync(0xffffffffu, ok)) { give_up_s = 1; atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT); break; }
                if (lane == 0) {
                    PTC_TRACE(2, ti, 5);
                    st_release_u32(a.flags + (dch + (size_t)(sl + cl * a.nslices)) * G::GROUP + bidx, a.tag_base + (unsigned)s);
                    mbar_arrive(rel_free(pb));
                    PTC_TRACE(2, ti, 6);
                }
                __syncwarp();
            }
        } else if (warp <= 5) {
            // ------------------------------------ drain tensor memory: quarters of the partial sums to their blocks ------------------------------------
            const int gate = warp & 3;                       // the tensor-memory lane quarter this warp may read = the gate
            const uint32_t lane_base = tmem + ((uint32_t)(32 * gate) << 16);
            // row (gate, lane): unit `lane` of the row tile is finished by block lane / 8 of the cluster
            const int tr = lane >> 3, tj = lane & 7;
            const int slot_r = q < tr ? q : q - 1;           // this block's position among the target's sources
            int s = 0, cl = -1;
            while (next_item(s, cl, ncl, Tc_s, Tmax)) {
                if (s == 0) continue;
                if (give_up_s) break;
                const int buf = m_d & 1;
                const uint32_t ph = (uint32_t)(m_d >> 1) & 1u;
                const int ti = m_d;
                (void)ti;
                ++m_d;
                if (warp == 2 && lane == 0) PTC_TRACE(3, ti, 0);
                // the partial sums of the item before last have been read, here and in the peers this warp writes to
                bool ok = mbar_wait_bounded<true>(z_free(buf), ph ^ 1u, &give_up_s, WAIT_CYCLES);
                if (warp == 2 && lane == 0) PTC_TRACE(3, ti, 3);
                if (warp == 2 && lane == 0) mbar_expect_tx(z_full(buf), (uint32_t)(KS - 1) * G::ZBLK);
                ok = ok && mbar_wait_bounded<false>(acc_full(buf), ph, &give_up_s, WAIT_CYCLES);
                if (!__all_sync(0xffffffffu, ok)) { give_up_s = 1; atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT); break; }
                if (warp == 2 && lane == 0) PTC_TRACE(3, ti, 1);
                tc_fence_after();
                float *zown = reinterpret_cast<float *>(gbase + G::F_ZOWN + (uint32_t)buf * G::ZBLK);
                const uint32_t la = sbase + G::F_ZRECV + (uint32_t)(buf * (KS - 1) + slot_r) * G::ZBLK;
                const uint32_t rbar = map_to_rank(z_full(buf), (uint32_t)tr);
#pragma unroll
                for (int col = 0; col < NC; col += 16) {
                    uint32_t mn[16], cx[16], mn1[16], cx1[16];
                    tmem_ld16(lane_base + (uint32_t)(buf * 256 + col), mn);
                    tmem_ld16(lane_base + (uint32_t)(buf * 256 + 64 + col), cx);
                    tmem_ld16(lane_base + (uint32_t)(buf * 256 + 128 + col), mn1);
                    tmem_ld16(lane_base + (uint32_t)(buf * 256 + 192 + col), cx1);
                    tmem_ld_wait();
                    float v[16];
#pragma unroll
                    for (int c = 0; c < 16; ++c)
                        v[c] = ((__uint_as_float(mn[c]) + __uint_as_float(mn1[c])) +
                                (__uint_as_float(cx[c]) + __uint_as_float(cx1[c])) * LO_UNSCALE) * invS;
#pragma unroll
                    for (int qd = 0; qd < 4; ++qd) {
                        const int o = ((gate * (NC / 4) + (col >> 2) + qd) * UPC + tj) * 4;   // floats
                        if (tr == q)
                            *reinterpret_cast<float4 *>(zown + o) = make_float4(v[4 * qd], v[4 * qd + 1], v[4 * qd + 2], v[4 * qd + 3]);
                        else
                            st_async_v4(map_to_rank(la + (uint32_t)o * 4u, (uint32_t)tr), __float_as_uint(v[4 * qd]),
                                        __float_as_uint(v[4 * qd + 1]), __float_as_uint(v[4 * qd + 2]), __float_as_uint(v[4 * qd + 3]), rbar);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) { mbar_arrive(acc_free(buf)); mbar_arrive(z_full(buf)); }
                if (warp == 2 && lane == 0) PTC_TRACE(3, ti, 2);
            }
        } else {
            // ------------------------------------ cell math (ComputeBlockOutputFn of the reference) ------------------------------------
            const int ct = tid - 192;
            const int jj = ct & 7, slot = ct >> 3;           // unit jj of this block, sequences slot*CPT .. +CPT
            const int j = 32 * r + q * UPC + jj;             // unit inside the direction
            const int u = d * ELS + j;
            float b4[4], pw[3];
#pragma unroll
            for (int g = 0; g < 4; ++g) b4[g] = a.sh.bias * __ldg(a.w + off.bias + (size_t)g * ls + u);
#pragma unroll
            for (int g = 0; g < 3; ++g) pw[g] = __ldg(a.w + off.peep + (size_t)g * ls + u);
            // where this block's 8 units sit inside the operand image of their slice
            const int qs = r >> 2;                                                     // the slice the units belong to
            const uint32_t img_cb = (uint32_t)((r & 3) >> 1) * (NC * 128u);            // column block
            const int img_kc = 4 * (r & 1) + q;                                        // 16-byte chunk inside the 128-byte row

            // Inputs of a chunk-step besides the recurrent sums: the projected inputs and the previous cell state.  With
            // several chunks per group they are requested one whole chunk-step ahead (second register set), so that
            // the loads have landed when the sums arrive; with one chunk the previous state is the one just computed.
            float pre[CPT][4], cpv[CPT], pre_n[LL ? 1 : CPT][4], cpv_n[LL ? 1 : CPT];
            auto fetch_into = [&](float (*pr)[4], float *cv, int s2, int cl2) {
                const int t = d ? Tc_s[cl2] - 1 - s2 : s2, prev = d ? t + 1 : t - 1;
                const int p0 = (sl + cl2 * a.nslices) * NC;
#pragma unroll
                for (int i = 0; i < CPT; ++i) {
                    const int n = slot * CPT + i, pg = p0 + n;
                    cv[i] = 0.0f;
#pragma unroll
                    for (int g = 0; g < 4; ++g) pr[i][g] = 0.0f;
                    if (pg < P && t < lens_s[cl2 * NC + n]) {
                        const float *ap = a.bf.acts + ((size_t)t * P + pg) * 4 * ls + u;
#pragma unroll
                        for (int g = 0; g < 4; ++g) pr[i][g] = ap[(size_t)g * ls];
                        if (s2 > 0) cv[i] = a.bf.cells[((size_t)prev * P + pg) * ls + u];
                    }
                }
            };
            auto fetch = [&](int s2, int cl2) { fetch_into(pre, cpv, s2, cl2); };
            // One chunk per group: nothing overlaps, the step is a chain of latencies.  h[t] then travels as self-validating
            // words {step tag : hi16 : lo16} that these warps collect into operand B themselves, right after they have
            // published their own part: no release fence at the producers, no counter round trip, no bulk-copy start-up.
            // sprev: the step whose h is collected; buf / ph: buffer and barrier phase of the chunk-step that consumes it.
            auto gather_ll = [&](int sprev, int ac, int buf, uint32_t ph) {
                static_assert(!LL || CW == 8, "the collecting code is laid out for 256 threads");
                constexpr int CH = NC * 16 / 256;   // 16-byte operand chunks (8 source units of one sequence) per thread
                bool okg = mbar_wait_bounded<false>(b_free(buf), ph ^ 1u, &give_up_s, WAIT_CYCLES);
                const u64 *src = reinterpret_cast<const u64 *>(a.xh) + ((dch + ac) * 2 + (sprev & 1)) * (size_t)(NC * ELS) + KSL * q;
                const unsigned tag = a.tag_base + (unsigned)sprev;
                const uint32_t bb = sbase + G::F_B + (uint32_t)buf * G::B_BUF;
                // first only this thread's first two words (little traffic while the producers are still busy) ...
                for (unsigned round = 0; okg; ++round) {
                    u64 w0, w1;
                    ld_tagged2(src + (size_t)(ct >> 4) * ELS + (ct & 15) * 8, w0, w1);
                    if ((unsigned)(w0 >> 32) == tag && (unsigned)(w1 >> 32) == tag) break;
                    if (round >= POLL_LIMIT || give_up_s || ((round & 1023u) == 1023u && ld_relaxed_s32(a.status) != 0)) okg = false;
                }
                // ... then everything, in rounds that re-read only what has not shown the tag yet
                unsigned done = 0;
                for (unsigned round = 0; okg && done != (1u << CH) - 1u; ++round) {
                    u64 wds[CH][8];
#pragma unroll
                    for (int c = 0; c < CH; ++c) {
                        if (done & (1u << c)) continue;
                        const int ci = ct + 256 * c;
                        const u64 *p = src + (size_t)(ci >> 4) * ELS + (ci & 15) * 8;
#pragma unroll
                        for (int e = 0; e < 4; ++e) ld_tagged2(p + 2 * e, wds[c][2 * e], wds[c][2 * e + 1]);
                    }
#pragma unroll
                    for (int c = 0; c < CH; ++c) {
                        if (done & (1u << c)) continue;
                        bool all = true;
#pragma unroll
                        for (int e = 0; e < 8; ++e) all = all && ((unsigned)(wds[c][e] >> 32) == tag);
                        if (!all) continue;
                        const int ci = ct + 256 * c, n = ci >> 4, kc = ci & 15;
                        uint32_t hi[4], lo[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const unsigned w0 = (unsigned)wds[c][2 * e], w1 = (unsigned)wds[c][2 * e + 1];   // payload: hi | lo << 16
                            hi[e] = (w0 & 0xffffu) | (w1 << 16);
                            lo[e] = (w0 >> 16) | (w1 & 0xffff0000u);
                        }
                        const uint32_t o = (uint32_t)(kc >> 3) * (NC * 128u) + (uint32_t)n * 128u + (uint32_t)(((kc & 7) ^ (n & 7)) * 16);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(bb + o), "r"(hi[0]), "r"(hi[1]), "r"(hi[2]), "r"(hi[3]) : "memory");
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(bb + G::B_HL + o), "r"(lo[0]), "r"(lo[1]), "r"(lo[2]), "r"(lo[3]) : "memory");
                        done |= 1u << c;
                    }
                    if (done != (1u << CH) - 1u &&
                        (round >= POLL_LIMIT || give_up_s || ((round & 1023u) == 1023u && ld_relaxed_s32(a.status) != 0)))
                        okg = false;
                }
                if (!__all_sync(0xffffffffu, okg)) { give_up_s = 1; atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT); return; }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(b_full(buf));
                
            };
            int s = 0, cl = -1;
            bool more = next_item(s, cl, ncl, Tc_s, Tmax);
            if (more) fetch(s, cl);
            while (more) {
                if (give_up_s) break;
                const int ac = sl + cl * a.nslices, p0 = ac * NC;
                const int t = d ? Tc_s[cl] - 1 - s : s;
                int s_n = s, cl_n = cl;
                bool more_n = false;
                if constexpr (!LL) {
                    more_n = next_item(s_n, cl_n, ncl, Tc_s, Tmax);
                    if (more_n) fetch_into(pre_n, cpv_n, s_n, cl_n);
                }
                float z[CPT][4];
#pragma unroll
                for (int i = 0; i < CPT; ++i)
#pragma unroll
                    for (int g = 0; g < 4; ++g) z[i][g] = 0.0f;
                const int ti = m_e;
                (void)ti;
                if (s > 0) {
                    const int buf = m_e & 1;
                    const uint32_t ph = (uint32_t)(m_e >> 1) & 1u;
                    ++m_e;
                    if (ct == 0) PTC_TRACE_C(1, ti, 0);
                    const bool ok = mbar_wait_bounded<true>(z_full(buf), ph, &give_up_s, WAIT_CYCLES);
                    if (!__all_sync(0xffffffffu, ok)) { give_up_s = 1; atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT); break; }
                    if (ct == 0) PTC_TRACE_C(1, ti, 1);
                    // partial sums of the contraction slices in slice order (own slice from zown, the others' as received)
                    const float *zown = reinterpret_cast<const float *>(gbase + G::F_ZOWN + (uint32_t)buf * G::ZBLK);
                    const float *zrecv = reinterpret_cast<const float *>(gbase + G::F_ZRECV + (uint32_t)(buf * (KS - 1)) * G::ZBLK);
#pragma unroll
                    for (int rs = 0; rs < KS; ++rs) {
                        const float *src = rs == q ? zown : zrecv + (size_t)(rs < q ? rs : rs - 1) * (G::ZBLK / 4);
#pragma unroll
                        for (int i = 0; i < CPT; ++i) {
                            const int n = slot * CPT + i;
#pragma unroll
                            for (int g = 0; g < 4; ++g) z[i][g] += src[((g * (NC / 4) + (n >> 2)) * UPC + jj) * 4 + (n & 3)];
                        }
                    }
                    // this warp is done with the buffers: tell the drain warps here (lane 0) and in the three peers
                    __syncwarp();
                    if (lane == 0) mbar_arrive(z_free(buf));
                    else if (lane < KS) mbar_arrive_cluster_relaxed(map_to_rank(z_free(buf), (uint32_t)((q + lane) & (KS - 1))));
                    if (ct == 0) PTC_TRACE_C(1, ti, 2);
                }
                const bool first = (s == 0), publish = (s + 1 < Tc_s[cl]);
                unsigned char *img = a.xh + ((dch + ac) * 2 + (s & 1)) * (size_t)(KS * G::B_BUF) + (size_t)qs * G::B_BUF + img_cb;
                float ni[CPT], ig[CPT], fg[CPT], og[CPT], cs[CPT], hh[CPT];
#pragma unroll
                for (int i = 0; i < CPT; ++i) {
                    const int n = slot * CPT + i, pg = p0 + n;
                    ni[i] = ig[i] = fg[i] = og[i] = cs[i] = hh[i] = 0.0f;
                    if (pg < P && t < lens_s[cl * NC + n]) {
                        float x0 = pre[i][0] + z[i][0] + b4[0], x1 = pre[i][1] + z[i][1] + b4[1];
                        float x2 = pre[i][2] + z[i][2] + b4[2], x3 = pre[i][3] + z[i][3] + b4[3];
                        const float cp = cpv[i];
                        if (!first) { x1 += cp * pw[0]; x2 += cp * pw[1]; }
                        ni[i] = fast_tanh(x0); ig[i] = fast_logistic(x1); fg[i] = fast_logistic(x2);
                        float c = ni[i] * ig[i];
                        if (!first) c += cp * fg[i];
                        og[i] = fast_logistic(x3 + c * pw[2]);
                        cs[i] = c;
                        hh[i] = fast_tanh(c) * og[i];
                    }
                    if (publish && LL) {
                        st_tagged(reinterpret_cast<u64 *>(a.xh) + ((dch + ac) * 2 + (s & 1)) * (size_t)(NC * ELS) + (size_t)n * ELS + j,
                                  a.tag_base + (unsigned)s, split_f16(hh[i]));
                    } else if (publish) {
                        // the 8 units of sequence n sit in 8 adjacent lanes: pack their fp16 hi (lo) parts into one 16-byte chunk
                        const unsigned x = split_f16(hh[i]);
                        const unsigned y1 = __shfl_down_sync(0xffffffffu, x, 1);
                        const unsigned hp = (x & 0xffffu) | (y1 << 16), lp = (x >> 16) | (y1 & 0xffff0000u);
                        const unsigned h1 = __shfl_down_sync(0xffffffffu, hp, 2), h2 = __shfl_down_sync(0xffffffffu, hp, 4);
                        const unsigned h3 = __shfl_down_sync(0xffffffffu, hp, 6);
                        const unsigned l1 = __shfl_down_sync(0xffffffffu, lp, 2), l2 = __shfl_down_sync(0xffffffffu, lp, 4);
                        const unsigned l3 = __shfl_down_sync(0xffffffffu, lp, 6);
                        if (jj == 0) {
                            unsigned char *dst = img + (size_t)n * 128 + (size_t)((img_kc ^ (n & 7)) * 16);
                            *reinterpret_cast<uint4 *>(dst) = make_uint4(hp, h1, h2, h3);
                            *reinterpret_cast<uint4 *>(dst + G::B_HL) = make_uint4(lp, l1, l2, l3);
                        }
                    }
                }
                if (ct == 0 && s > 0) PTC_TRACE_C(1, ti, 6);
                if (publish && !LL) {
                    // this warp's part of h[t] is on its way: hand it to the publisher; the layer's own state is stored afterwards
                    const int pb = m_p & 1;
                    const uint32_t pph = (uint32_t)(m_p >> 1) & 1u;
                    ++m_p;
                    __syncwarp();
                    if (lane == 0) {
                        if (!mbar_wait_bounded<false>(rel_free(pb), pph ^ 1u, &give_up_s, WAIT_CYCLES)) give_up_s = 1;
                        mbar_arrive(rel_full(pb));
                    }
                }
                if (ct == 0 && s > 0) PTC_TRACE_C(1, ti, 3);
                if constexpr (LL) {
                    // Collect the operand of the NEXT chunk-step now (h of that chunk's previous step), store afterwards.  With one
                    // chunk per group that is what this step has just published, and the wait for the other blocks is part of the
                    // chain; with two chunks it was published a whole chunk-step ago and is there already.
                    int s_g = s, cl_g = cl;
                    if (!gw && next_item(s_g, cl_g, ncl, Tc_s, Tmax) && s_g > 0) {
                        gather_ll(s_g - 1, sl + cl_g * a.nslices, m_e & 1, (uint32_t)(m_e >> 1) & 1u);
                        if (give_up_s) break;
                    }
                    if (ct == 0 && s > 0) PTC_TRACE_C(1, ti, 5);
                }
#pragma unroll
                for (int i = 0; i < CPT; ++i) {
                    const int n = slot * CPT + i, pg = p0 + n;
                    if (pg < P) {
                        const size_t f = (size_t)t * P + pg;
                        float *ap = a.bf.acts + f * 4 * ls + u;
                        ap[0] = ni[i]; ap[ls] = ig[i]; ap[2 * (size_t)ls] = fg[i]; ap[3 * (size_t)ls] = og[i];   // zeros on padding
                        a.bf.cells[f * ls + u] = cs[i];
                        a.y[f * ls + u] = hh[i];
                    }
                }
                if (ct == 0 && s > 0) PTC_TRACE_C(1, ti, 7);
                if constexpr (LL) {
                    more = next_item(s, cl, ncl, Tc_s, Tmax);
                    if (more) fetch(s, cl);
                } else {
                    const bool same_chunk = (cl_n == cl);   // one chunk in this group: its previous cell state is cs[]
                    s = s_n; cl = cl_n; more = more_n;
#pragma unroll
                    for (int i = 0; i < CPT; ++i) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) pre[i][g] = pre_n[i][g];
                        cpv[i] = same_chunk ? cs[i] : cpv_n[i];
                    }
                }
                if (ct == 0 && s > 1) PTC_TRACE_C(1, ti, 4);
            }
            // frames beyond a chunk's longest sequence are padding for all its sequences: outputs are zero there
            for (int c2 = 0; c2 < ncl; ++c2) {
                const int p0 = (sl + c2 * a.nslices) * NC;
                for (int i = slot; i < (T - Tc_s[c2]) * NC; i += 4 * CW) {
                    const int t = Tc_s[c2] + i / NC, pg = p0 + i % NC;
                    if (pg < P) a.y[((size_t)t * P + pg) * ls + u] = 0.0f;
                }
            }
        }
        __syncthreads();   // every role is through this work item (the weight image may be replaced)
        if (give_up_s) break;
    }
    tc_fence_before();
    __syncthreads();
    if (give_up_s && tid == 0) atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT);
    // nobody leaves while a peer may still write into its shared memory
    cluster_sync_all();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

// =====================================================================================================
// backward
// =====================================================================================================
template <int ELS, int NC, bool LL>
__global__ void __launch_bounds__(bwd_threads(LL), 1) lstm_bwd_ptc_kernel(PtcArgs a) {
    typedef Geo<ELS, NC> G;
    constexpr int CW = bwd_cell_warps(LL), BWD_THREADS = bwd_threads(LL), CT = 32 * CW;
    constexpr int RT = G::RT, CPT = NC / (4 * CW);   // a cell warp covers 8 units x 4 sequences
    static_assert(CPT >= 1, "more cell warps than cells");
    // one chunk of 32 sequences per group: the cell warps send their part of operand B to the peers themselves (below)
    constexpr bool SELF_SEND = LL && NC == 32;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) u64 bars[18];
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int give_up_s;
    __shared__ int lens_s[MAXC * NC], Tc_s[MAXC], Tmax_s;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char *gbase = smem_raw + (sbase - smem_u32(smem_raw));
    const uint32_t bar0 = smem_u32(bars);
    auto rel_full = [&](int b) { return bar0 + 8u * (uint32_t)(12 + b); };  // drain warps have stored their partial errors -> publisher
    auto rel_free = [&](int b) { return bar0 + 8u * (uint32_t)(14 + b); };  // publisher -> drain warps
    auto b_full = [&](int b) { return bar0 + 8u * (uint32_t)b; };          // cell warps of the cluster -> MMA
    auto b_free = [&](int b) { return bar0 + 8u * (uint32_t)(2 + b); };    // MMAs of the whole cluster done -> cell warps
    auto acc_full = [&](int b) { return bar0 + 8u * (uint32_t)(4 + b); };  // MMA -> drain
    auto acc_free = [&](int b) { return bar0 + 8u * (uint32_t)(6 + b); };  // drain -> MMA
    auto e_full = [&](int b) { return bar0 + 8u * (uint32_t)(8 + b); };    // reduce warps -> cell warps
    auto e_free = [&](int b) { return bar0 + 8u * (uint32_t)(10 + b); };   // cell warps -> reduce warps
    auto s_full = [&](int b) { return bar0 + 8u * (uint32_t)(16 + b); };   // cell warps have written the block's share of operand B -> sender

    const int P = a.sh.P, T = a.sh.T, ls = a.sh.ls, D = a.sh.D;
    const int grp = blockIdx.x / G::GROUP, ngroups = gridDim.x / G::GROUP;
    const int bidx = blockIdx.x % G::GROUP, r = bidx / KS;
    const int q = (int)cluster_ctarank();
    const LstmOffsets off = lstm_offsets(a.sh.pls, ls, ELS);

    if (tid == 0) {
        for (int b = 0; b < 2; ++b) {
            mbar_init(b_full(b), SELF_SEND ? CW : 1);   // every cell warp announces its part, or the sender warp does
            mbar_init(b_free(b), KS + 1);        // two local MMA issuers + the other three blocks' drains
            mbar_init(acc_full(b), 2); mbar_init(acc_free(b), 4);
            mbar_init(e_full(b), 4); mbar_init(e_free(b), CW);
            mbar_init(rel_full(b), 4); mbar_init(rel_free(b), 1);
            mbar_init(s_full(b), CW);
        }
        give_up_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc(smem_u32(&tmem_base_s), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    cluster_sync_all();

    // producer side (cell -> MMA -> drain) counts the chunk-steps whose deltas somebody consumes (s + 1 < Tc);
    // consumer side (reduce -> cell) counts the chunk-steps that receive a recurrent error (s >= 1)
    int mp_m = 0, mp_c = 0, mp_d = 0, mc_r = 0, mc_c = 0, mp_p = 0, mp_s = 0;
    const int nwork = D * a.nslices;
    for (int wi = grp; wi < nwork; wi += ngroups) {
        const int d = wi % D, sl = wi / D;
        const int ncl = (a.nchunks - sl + a.nslices - 1) / a.nslices;
        load_weight_image(gbase, a.wimg + (size_t)((d * RT + r) * KS + q) * (A_BYTES / 16), BWD_THREADS);
        find_lengths<NC>(a, sl, ncl, lens_s, Tc_s, &Tmax_s, BWD_THREADS);
        const int Tmax = Tmax_s;
        const float invS = a.scale[2 * d + 1];
        const size_t dch = (size_t)d * a.nchunks;

        if (warp == 0 || warp == CW + 10) {
            // ------------------------------------------------ MMA issue (two warps, half of the k-steps each) ------------------------------------------------
            if (lane == 0) {
                const int hh = warp == 0 ? 0 : 1;
                const uint32_t idesc = idesc_f16(128, NC);
                int s = 0, cl = -1;
                while (next_item(s, cl, ncl, Tc_s, Tmax)) {
                    if (s + 1 >= Tc_s[cl]) continue;
                    if (give_up_s) break;
                    const int buf = mp_m & 1;
                    const uint32_t ph = (uint32_t)(mp_m >> 1) & 1u;
                    const int ti = mp_m;
                    (void)ti;
                    ++mp_m;
                    if (hh == 0) PTC_TRACE_B(0, ti, 0);
                    if (!mbar_wait_bounded<true>(b_full(buf), ph, &give_up_s, WAIT_CYCLES) ||
                        !mbar_wait_bounded<false>(acc_free(buf), ph ^ 1u, &give_up_s, WAIT_CYCLES)) {
                        give_up_s = 1;
                        break;
                    }
                    if (hh == 0) PTC_TRACE_B(0, ti, 1);
                    fence_async_smem();
                    tc_fence_after();
                    const uint32_t acc = tmem + (uint32_t)(buf * 256 + hh * 128);
                    const uint32_t bb = sbase + G::B_B + (uint32_t)buf * G::B_BUF;
                    // Operand B (the row tile's gate deltas) is stored WITHOUT swizzle: for every 16-byte chunk along the
                    // contraction (8 gate rows = the 8 units of one block and gate) the core matrices of all sequences
                    // are contiguous, so that a block hands its share to a peer with one bulk copy per gate.
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4) {
                        const int ks = 4 * hh + k4;
                        const uint32_t ao = (uint32_t)(ks >> 2) * 16384u + (uint32_t)(ks & 3) * 32u;
                        const uint32_t bo = (uint32_t)ks * 2u * (NC * 16u);
                        const u64 ahi = desc_kmajor_sw128(sbase + ao, 1024), alo = desc_kmajor_sw128(sbase + A_HALF + ao, 1024);
                        const u64 bhi = desc_kmajor_nosw(bb + bo, NC * 16u, 128), blo = desc_kmajor_nosw(bb + G::B_HL + bo, NC * 16u, 128);
                        mma_f16(acc + 64u, alo, bhi, idesc, k4 ? 1u : 0u);
                        mma_f16(acc + 64u, ahi, blo, idesc, 1u);
                        mma_f16(acc, ahi, bhi, idesc, k4 ? 1u : 0u);
                    }
                    mma_commit(b_free(buf));
                    mma_commit(acc_full(buf));
                    if (hh == 0) PTC_TRACE_B(0, ti, 2);
                }
            }
        } else if (warp <= CW) {
            // ------------------------------------------------ cell math: the error functor ------------------------------------------------
            const int et = tid - 32;
            const int jj = et & 7, slot = et >> 3;           // unit jj of this block, sequences slot*CPT .. +CPT
            const int j = 32 * r + q * UPC + jj;
            const int u = d * ELS + j;
            const float p_ig = __ldg(a.w + off.peep + u), p_fg = __ldg(a.w + off.peep + (size_t)ls + u);
            const float p_og = __ldg(a.w + off.peep + 2 * (size_t)ls + u);
            const float *esum = reinterpret_cast<const float *>(gbase + G::B_ESUM);
            // A cell's forget-gate activation, cell error and input / forget gate deltas are read again by the same thread at the
            // next step of the chunk: they stay in shared memory when the group has few enough chunks (else global memory).
            float *carry_s = reinterpret_cast<float *>(gbase + G::B_CARRY);
            const bool carry = (ncl <= G::CARRY) && !(LL && NC == 64);   // (one chunk of 64: measured slower, the kernel is out of registers)

            // everything a step reads besides the recurrent error is fetched when the previous chunk-step is done
            float f_dy[CPT], f_act[CPT][4], f_c[CPT], f_cp[CPT], f_nfg[CPT], f_nce[CPT], f_ndig[CPT], f_ndfg[CPT];
            auto fetch = [&](int s2, int cl2) {
                const int Tcc = Tc_s[cl2];
                const int t = d ? s2 : Tcc - 1 - s2;
                const int next = d ? t - 1 : t + 1, prevc = d ? t + 1 : t - 1;
                const bool lastCall = d ? (t == Tcc - 1) : (t == 0);
                const int p0 = (sl + cl2 * a.nslices) * NC;
                const float *ce_nxt = a.bf.cerr + (size_t)((s2 + 1) & 1) * P * ls;
#pragma unroll
                for (int i = 0; i < CPT; ++i) {
                    const int n = slot * CPT + i, pg = p0 + n;
                    f_dy[i] = f_c[i] = f_cp[i] = f_nfg[i] = f_nce[i] = f_ndig[i] = f_ndfg[i] = 0.0f;
#pragma unroll
                    for (int g = 0; g < 4; ++g) f_act[i][g] = 0.0f;
                    if (pg < P && t < lens_s[cl2 * NC + n]) {
                        const size_t f = (size_t)t * P + pg;
                        f_dy[i] = a.dy[f * ls + u];
                        const float *ap = a.bf.acts + f * 4 * ls + u;
#pragma unroll
                        for (int g = 0; g < 4; ++g) f_act[i][g] = ap[(size_t)g * ls];
                        f_c[i] = a.bf.cells[f * ls + u];
                        if (!lastCall) f_cp[i] = a.bf.cells[((size_t)prevc * P + pg) * ls + u];
                        if (s2 > 0 && carry) {
                            const float *cr = carry_s + (size_t)(cl2 * 4) * (NC * UPC) + et * CPT + i;
                            f_nfg[i] = cr[0]; f_nce[i] = cr[NC * UPC]; f_ndig[i] = cr[2 * NC * UPC]; f_ndfg[i] = cr[3 * NC * UPC];
                        } else if (s2 > 0) {
                            const size_t fn = (size_t)next * P + pg;
                            f_nfg[i] = a.bf.acts[fn * 4 * ls + 2 * (size_t)ls + u];
                            f_nce[i] = ce_nxt[(size_t)pg * ls + u];
                            f_ndig[i] = a.bf.deltas[fn * 4 * ls + ls + u];
                            f_ndfg[i] = a.bf.deltas[fn * 4 * ls + 2 * (size_t)ls + u];
                        }
                    }
                }
            };
            int s = 0, cl = -1;
            bool more = next_item(s, cl, ncl, Tc_s, Tmax);
            if (more) fetch(s, cl);
            while (more) {
                if (give_up_s) break;
                const int Tcc = Tc_s[cl];
                const int ac = sl + cl * a.nslices, p0 = ac * NC;
                const int t = d ? s : Tcc - 1 - s;
                const bool firstCall = (s == 0), lastCall = d ? (t == Tcc - 1) : (t == 0);
                const bool feeds = (s + 1 < Tcc);   // the next step needs these deltas as tensor-core operand
                float er[CPT];
#pragma unroll
                for (int i = 0; i < CPT; ++i) er[i] = 0.0f;
                bool ok = true;
                const int ti = mc_c;
                (void)ti;
                if (et == 0) PTC_TRACE_B(1, ti, 0);
                if (s > 0) {
                    const int buf = mc_c & 1;
                    const uint32_t ph = (uint32_t)(mc_c >> 1) & 1u;
                    ++mc_c;
                    ok = mbar_wait_bounded<false>(e_full(buf), ph, &give_up_s, WAIT_CYCLES);
                    if (et == 0) PTC_TRACE_B(1, ti, 1);
                    if (ok) {
#pragma unroll
                        for (int i = 0; i < CPT; ++i) er[i] = esum[(buf * NC + slot * CPT + i) * UPC + jj];
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(e_free(buf));
                }
                int pbuf = 0;
                if (feeds) {
                    pbuf = mp_c & 1;
                    const uint32_t pph = (uint32_t)(mp_c >> 1) & 1u;
                    ++mp_c;
                    // operand buffer pbuf: the MMAs of the chunk-step before last, in every block of the cluster, have read it
                    if (ok) ok = mbar_wait_bounded<true>(b_free(pbuf), pph ^ 1u, &give_up_s, WAIT_CYCLES);
                }
                // the cell threads leave together or not at all (named barriers follow)
                if (bar_named_or(1, CT, !ok)) { give_up_s = 1; atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT); break; }
                if (et == 0) PTC_TRACE_B(1, ti, 2);
                float *ce_cur = a.bf.cerr + (size_t)(s & 1) * P * ls;
                const uint32_t bb_w = sbase + G::B_B + (uint32_t)pbuf * G::B_BUF;
                float dl_r[CPT][4], ce_r[CPT];
#pragma unroll
                for (int i = 0; i < CPT; ++i) {
                    const int n = slot * CPT + i, pg = p0 + n;
                    float dni = 0.0f, dig = 0.0f, dfg = 0.0f, dog = 0.0f, ce = 0.0f;
                    if (pg < P && t < lens_s[cl * NC + n]) {
                        const float e = f_dy[i] + er[i];
                        const float ni = f_act[i][0], ig = f_act[i][1], fg = f_act[i][2], og = f_act[i][3];
                        const float tc = fast_tanh(f_c[i]);
                        dog = d_logistic(og) * tc * e;
                        ce = og * d_tanh(tc) * e + p_og * dog;
                        if (!firstCall) ce += f_nfg[i] * f_nce[i] + p_ig * f_ndig[i] + p_fg * f_ndfg[i];
                        dni = ig * d_tanh(ni) * ce;
                        if (!lastCall) dfg = d_logistic(fg) * f_cp[i] * ce;
                        dig = d_logistic(ig) * ni * ce;
                        dni = limited_error(dni); dig = limited_error(dig); dfg = limited_error(dfg); dog = limited_error(dog);
                    }
                    if (feeds) {
                        // this cell's four deltas as fp16 hi / lo, straight into this block's operand buffer: element
                        // (sequence n, gate row g*32 + q*8 + jj) lives in chunk g*4 + q, row n of its core matrix
                        const float dl[4] = {dni, dig, dfg, dog};
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            const unsigned x = split_f16(dl[g]);
                            const uint32_t o = (uint32_t)(g * 4 + q) * (NC * 16u) + (uint32_t)(n >> 3) * 128u + (uint32_t)(n & 7) * 16u + (uint32_t)jj * 2u;
                            asm volatile("st.shared.b16 [%0], %1;" ::"r"(bb_w + o), "h"((unsigned short)(x & 0xffffu)) : "memory");
                            asm volatile("st.shared.b16 [%0], %1;" ::"r"(bb_w + G::B_HL + o), "h"((unsigned short)(x >> 16)) : "memory");
                        }
                    }
                    dl_r[i][0] = dni; dl_r[i][1] = dig; dl_r[i][2] = dfg; dl_r[i][3] = dog; ce_r[i] = ce;
                    if (carry) {
                        float *cr = carry_s + (size_t)(cl * 4) * (NC * UPC) + et * CPT + i;
                        cr[0] = f_act[i][2]; cr[NC * UPC] = ce; cr[2 * NC * UPC] = dig; cr[3 * NC * UPC] = dfg;
                    }
                }
                if (et == 0) PTC_TRACE_B(1, ti, 3);
                if (feeds && SELF_SEND) {
                    // One chunk per group: the step is a chain of latencies, and a bulk copy costs its issuer a microsecond.
                    // Each warp sends the 16-byte pieces it has just written (its sequences, all gates, hi and lo) to the three
                    // peers itself, with st.async counted on the peer's barrier, and announces its part of the local copy.
                    fence_async_smem();
                    __syncwarp();
                    const int wq = et >> 5;                           // this cell warp covers sequences 4*CPT*wq .. +4*CPT
#pragma unroll
                    for (int i2 = 0; i2 < CPT; ++i2) {
                        const int c = lane + 32 * i2, nl = c % (4 * CPT), gh = c / (4 * CPT);
                        const int n = 4 * CPT * wq + nl, g = gh & 3, hl = gh >> 2;
                        const uint32_t o = (uint32_t)hl * G::B_HL + (uint32_t)(g * 4 + q) * (NC * 16u) + (uint32_t)(n >> 3) * 128u + (uint32_t)(n & 7) * 16u;
                        uint32_t v0, v1, v2, v3;
                        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3) : "r"(bb_w + o) : "memory");
#pragma unroll
                        for (int pr = 1; pr < KS; ++pr) {
                            const uint32_t peer = (uint32_t)((q + pr) & (KS - 1));
                            st_async_v4(map_to_rank(bb_w + o, peer), v0, v1, v2, v3, map_to_rank(b_full(pbuf), peer));
                        }
                    }
                    if (lane == 0) {
                        if (et == 0) mbar_expect_tx(b_full(pbuf), (uint32_t)(KS - 1) * 8u * NC * 16u);   // the bytes the peers deliver
                        else mbar_arrive(b_full(pbuf));
                    }
                } else if (feeds) {
                    // this warp's share of the operand is in place: visible to the async proxy, then over to the sender warp
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(s_full(pbuf));
                }
                if (et == 0) PTC_TRACE_B(1, ti, 4);
                // the layer's own copies go out after the hand-over (the proxy fence above would wait for them)
#pragma unroll
                for (int i = 0; i < CPT; ++i) {
                    const int pg = p0 + slot * CPT + i;
                    if (pg < P) {
                        const size_t o = ((size_t)t * P + pg) * 4 * ls + u;
                        a.bf.deltas[o] = dl_r[i][0]; a.bf.deltas[o + ls] = dl_r[i][1];
                        a.bf.deltas[o + 2 * (size_t)ls] = dl_r[i][2]; a.bf.deltas[o + 3 * (size_t)ls] = dl_r[i][3];
                        if (!carry) ce_cur[(size_t)pg * ls + u] = ce_r[i];
                    }
                }
                more = next_item(s, cl, ncl, Tc_s, Tmax);
                if (more) fetch(s, cl);
                if (et == 0) PTC_TRACE_B(1, ti, 5);
            }
            // frames beyond a chunk's longest sequence: zero deltas (they are operands of the gradient GEMMs)
            for (int c2 = 0; c2 < ncl; ++c2) {
                const int p0 = (sl + c2 * a.nslices) * NC;
                for (int i = slot; i < (T - Tc_s[c2]) * NC; i += 4 * CW) {
                    const int t = Tc_s[c2] + i / NC, pg = p0 + i % NC;
                    if (pg < P) {
                        const size_t o = ((size_t)t * P + pg) * 4 * ls + u;
                        a.bf.deltas[o] = 0.0f; a.bf.deltas[o + ls] = 0.0f; a.bf.deltas[o + 2 * (size_t)ls] = 0.0f; a.bf.deltas[o + 3 * (size_t)ls] = 0.0f;
                    }
                }
            }
        } else if (warp == CW + 11) {
            // ------------------------------------ sender: the block's share of operand B to the three peers ------------------------------------
            // One bulk copy per (hi/lo, gate, peer): NC x 16 contiguous bytes, counted on the peer's barrier.  Issuing such a
            // copy holds its thread for a microsecond or so, which is why the cell warps do not do it themselves.
            int s = 0, cl = -1;
            while (!SELF_SEND && next_item(s, cl, ncl, Tc_s, Tmax)) {
                if (s + 1 >= Tc_s[cl]) continue;
                if (give_up_s) break;
                const int pbuf = mp_s & 1;
                const uint32_t pph = (uint32_t)(mp_s >> 1) & 1u;
                ++mp_s;
                const bool ok = mbar_wait_bounded<false>(s_full(pbuf), pph, &give_up_s, WAIT_CYCLES);
                if (!__all_sync(0xffffffffu, ok)) { give_up_s = 1; atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT); break; }
                const uint32_t bb_w = sbase + G::B_B + (uint32_t)pbuf * G::B_BUF;
                // one arrival per phase; it also announces the bytes the peers deliver into this buffer
                if (lane == 0) mbar_expect_tx(b_full(pbuf), (uint32_t)(KS - 1) * 8u * NC * 16u);
                if (lane < 8 * (KS - 1)) {
                    const int pr = (q + 1 + lane / 8) & (KS - 1), hl = (lane >> 2) & 1, g = lane & 3;
                    const uint32_t o = (uint32_t)hl * G::B_HL + (uint32_t)(g * 4 + q) * (NC * 16u);
                    bulk_s2c(map_to_rank(bb_w + o, (uint32_t)pr), bb_w + o, NC * 16u, map_to_rank(b_full(pbuf), (uint32_t)pr));
                }
                __syncwarp();
            }
        } else if (warp <= CW + 4) {
            // ------------------------------------------------ drain: partial output errors to global memory ------------------------------------------------
            const int q4 = warp & 3;
            const uint32_t lane_base = tmem + ((uint32_t)(32 * q4) << 16);
            int s = 0, cl = -1;
            while (next_item(s, cl, ncl, Tc_s, Tmax)) {
                if (s + 1 >= Tc_s[cl]) continue;
                if (give_up_s) break;
                const int buf = mp_d & 1;
                const uint32_t ph = (uint32_t)(mp_d >> 1) & 1u;
                const int ti = mp_d;
                (void)ti;
                ++mp_d;
                if (warp == CW + 1 && lane == 0) PTC_TRACE_B(3, ti, 0);
                const bool ok = mbar_wait_bounded<false>(acc_full(buf), ph, &give_up_s, WAIT_CYCLES);
                if (warp == CW + 1 && lane == 0) PTC_TRACE_B(3, ti, 1);
                if (!__all_sync(0xffffffffu, ok)) { give_up_s = 1; atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT); break; }
                tc_fence_after();
                // the MMAs of this chunk-step are complete: the peers may refill their copy of operand buffer buf
                if (warp == CW + 1 && lane < KS && lane != q) mbar_arrive_cluster_relaxed(map_to_rank(b_free(buf), (uint32_t)lane));
                const int ac = sl + cl * a.nslices;
                const size_t xoff = (((dch + ac) * 2 + (s & 1)) * RT + r) * (size_t)(NC * ELS) + KSL * q + 32 * q4 + lane;
#pragma unroll
                for (int c0 = 0; c0 < NC; c0 += 16) {
                    uint32_t mn[16], cx[16], mn1[16], cx1[16];
                    tmem_ld16(lane_base + (uint32_t)(buf * 256 + c0), mn);
                    tmem_ld16(lane_base + (uint32_t)(buf * 256 + 64 + c0), cx);
                    tmem_ld16(lane_base + (uint32_t)(buf * 256 + 128 + c0), mn1);
                    tmem_ld16(lane_base + (uint32_t)(buf * 256 + 192 + c0), cx1);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        const float v = ((__uint_as_float(mn[c]) + __uint_as_float(mn1[c])) +
                                         (__uint_as_float(cx[c]) + __uint_as_float(cx1[c])) * LO_UNSCALE) * invS;
                        // one chunk per group: self-validating words {step tag : float}, no release fence, no counters
                        if (LL) st_tagged(reinterpret_cast<u64 *>(a.xe) + xoff + (size_t)(c0 + c) * ELS, a.tag_base + (unsigned)s, __float_as_uint(v));
                        else a.xe[xoff + (size_t)(c0 + c) * ELS] = v;
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (warp == CW + 1 && lane == 0) PTC_TRACE_B(3, ti, 2);
                if (lane == 0) {
                    mbar_arrive(acc_free(buf));
                    if (!LL) {
                        // this warp's quarter of the partial errors is on its way: hand it to the publisher (same buffer parity)
                        if (!mbar_wait_bounded<false>(rel_free(buf), ph ^ 1u, &give_up_s, WAIT_CYCLES)) give_up_s = 1;
                        mbar_arrive(rel_full(buf));
                    }
                }
            }
        } else if (warp == CW + 9) {
            // ------------------------------------ publisher: the block's step counter follows its partial errors ------------------------------------
            int s = 0, cl = -1;
            while (!LL && next_item(s, cl, ncl, Tc_s, Tmax)) {
                if (s + 1 >= Tc_s[cl]) continue;
                if (give_up_s) break;
                const int pb = mp_p & 1;
                const uint32_t pph = (uint32_t)(mp_p >> 1) & 1u;
                ++mp_p;
                const bool ok = mbar_wait_bounded<false>(rel_full(pb), pph, &give_up_s, WAIT_CYCLES);
                if (!__all_sync(0xffffffffu, ok)) { give_up_s = 1; atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT); break; }
                if (lane == 0) {
                    st_release_u32(a.flags + (dch + (size_t)(sl + cl * a.nslices)) * G::GROUP + bidx, a.tag_base + (unsigned)s);
                    mbar_arrive(rel_free(pb));
                }
                __syncwarp();
            }
        } else {
            // ------------------------------------------------ gather + reduce the partial output errors ------------------------------------------------
            const int rt = tid - 32 * (CW + 5);
            float *esum = reinterpret_cast<float *>(gbase + G::B_ESUM);
            const int n = rt >> 1, hf = rt & 1;          // sequence n, units 4*hf .. 4*hf+3 of this block
            const bool active = n < NC;
            const int qu = r >> 2;                       // the slice this block's units belong to: their partials come from blocks (rs, qu)
            int s = 0, cl = -1;
            while (next_item(s, cl, ncl, Tc_s, Tmax)) {
                if (s == 0) continue;
                if (give_up_s) break;
                const int buf = mc_r & 1;
                const uint32_t ph = (uint32_t)(mc_r >> 1) & 1u;
                const int ti = mc_r;
                (void)ti;
                ++mc_r;
                const int ac = sl + cl * a.nslices;
                if (rt == 0) PTC_TRACE_B(2, ti, 0);
                bool ok = __all_sync(0xffffffffu, mbar_wait_bounded<false>(e_free(buf), ph ^ 1u, &give_up_s, WAIT_CYCLES));
                if (rt == 0) PTC_TRACE_B(2, ti, 1);
                if constexpr (LL) {
                    const unsigned tag = a.tag_base + (unsigned)(s - 1);
                    const u64 *base = reinterpret_cast<const u64 *>(a.xe) + (((dch + ac) * 2 + ((s - 1) & 1)) * RT) * (size_t)(NC * ELS) + 32 * r + q * UPC;
                    // first only one source's words per thread (little traffic while the producers are still busy) ...
                    {
                        const u64 *p = base + (size_t)((r + 1) & (RT - 1)) * NC * ELS + (size_t)(rt >> 2) * ELS + 2 * (rt & 3);
                        for (unsigned round = 0; ok; ++round) {
                            u64 w0, w1;
                            ld_tagged2(p, w0, w1);
                            if ((unsigned)(w0 >> 32) == tag && (unsigned)(w1 >> 32) == tag) break;
                            if (round >= POLL_LIMIT || give_up_s || ((round & 1023u) == 1023u && ld_relaxed_s32(a.status) != 0)) ok = false;
                        }
                    }
                    // ... then all 16 sources of each (sequence, unit pair), re-reading only what has not shown the tag yet
#pragma unroll 1
                    for (int pi = rt; pi < NC * UPC / 2 && ok; pi += 128) {
                        const int n2 = pi >> 2, jp = pi & 3;
                        const u64 *src = base + (size_t)n2 * ELS + 2 * jp;
                        u64 wa[RT], wb[RT];
                        unsigned done = 0;
                        for (unsigned round = 0; done != (1u << RT) - 1u; ++round) {
#pragma unroll
                            for (int rs = 0; rs < RT; ++rs)
                                if (!(done & (1u << rs))) ld_tagged2(src + (size_t)rs * NC * ELS, wa[rs], wb[rs]);
#pragma unroll
                            for (int rs = 0; rs < RT; ++rs)
                                if (!(done & (1u << rs)) && (unsigned)(wa[rs] >> 32) == tag && (unsigned)(wb[rs] >> 32) == tag) done |= 1u << rs;
                            if (done != (1u << RT) - 1u &&
                                (round >= POLL_LIMIT || give_up_s || ((round & 1023u) == 1023u && ld_relaxed_s32(a.status) != 0))) {
                                ok = false;
                                break;
                            }
                        }
                        float e0 = 0.0f, e1 = 0.0f;
                        if (ok) {
#pragma unroll
                            for (int rs = 0; rs < RT; ++rs) { e0 += __uint_as_float((unsigned)wa[rs]); e1 += __uint_as_float((unsigned)wb[rs]); }
                        }
                        *reinterpret_cast<float2 *>(esum + (buf * NC + n2) * UPC + 2 * jp) = make_float2(e0, e1);
                    }
                    if (!__all_sync(0xffffffffu, ok)) { give_up_s = 1; atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT); break; }
                } else {
                // the 16 blocks (rs, qu) that hold partials for this block's units
                ok = ok && poll_flags(a.flags + (dch + ac) * G::GROUP + qu, KS, a.tag_base + (unsigned)(s - 1), lane, &give_up_s, a.status);
                if (!ok) { give_up_s = 1; atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT); break; }
                if (rt == 0) PTC_TRACE_B(2, ti, 3);
                if (active) {
                    const float *src = a.xe + (((dch + ac) * 2 + ((s - 1) & 1)) * RT) * (size_t)(NC * ELS) + (size_t)n * ELS + 32 * r + q * UPC + 4 * hf;
                    float4 v[RT];
#pragma unroll
                    for (int rs = 0; rs < RT; ++rs) v[rs] = ld_l2_f4(src + (size_t)rs * NC * ELS);
                    float4 e = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                    for (int rs = 0; rs < RT; ++rs) { e.x += v[rs].x; e.y += v[rs].y; e.z += v[rs].z; e.w += v[rs].w; }
                    *reinterpret_cast<float4 *>(esum + (buf * NC + n) * UPC + 4 * hf) = e;
                }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(e_full(buf));
                if (rt == 0) PTC_TRACE_B(2, ti, 2);
            }
        }
        __syncthreads();
        if (give_up_s) break;
    }
    tc_fence_before();
    __syncthreads();
    if (give_up_s && tid == 0) atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT);
    cluster_sync_all();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

// =====================================================================================================
// weight images
// =====================================================================================================
__global__ void ptc_absmax_kernel(const float *__restrict__ wrec, int ls, int els, int D, unsigned *maxbits) {
    // recurrent block: W[g][d][j][k] at g*ls*els + d*els*els + j*els + k
    const size_t total = (size_t)4 * ls * els;
    unsigned m0 = 0u, m1 = 0u;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int d = (int)((i / ((size_t)els * els)) % D);
        const unsigned b = __float_as_uint(fabsf(wrec[i]));
        if (b < 0x7f800000u) {   // NaN / Inf weights do not set the scale
            if (d == 0) m0 = max(m0, b); else m1 = max(m1, b);
        }
    }
    for (int o = 16; o; o >>= 1) {
        m0 = max(m0, __shfl_xor_sync(0xffffffffu, m0, o));
        m1 = max(m1, __shfl_xor_sync(0xffffffffu, m1, o));
    }
    if ((threadIdx.x & 31) == 0) {
        if (m0) atomicMax(maxbits, m0);
        if (m1) atomicMax(maxbits + 1, m1);
    }
}
__global__ void ptc_scale_kernel(const unsigned *maxbits, float *scale, int D) {
    const int d = threadIdx.x;
    if (d >= D) return;
    const float mx = __uint_as_float(maxbits[d]);
    int e = 0;
    if (mx > 0.0f) e = 13 - ilogbf(mx);   // 2^13 <= mx * 2^e < 2^14
    e = max(-100, min(100, e));
    scale[2 * d] = ldexpf(1.0f, e);
    scale[2 * d + 1] = ldexpf(1.0f, -e);
}

// One thread per 16-byte chunk (8 fp16 values) of the images.  Forward image of block (d, r, q): [hi/lo][2 column
// blocks][128 rows = gate*32 + jj][64 source units of slice q], 128-byte rows with the 128-byte swizzle.  Backward
// image: [hi/lo][2 column blocks][128 rows = source unit of slice q][64 gate rows of row tile r].
template <int ELS>
__global__ void ptc_image_kernel(const float *__restrict__ wrec, const float *__restrict__ scale, uint4 *__restrict__ img_f,
                                 uint4 *__restrict__ img_b, int ls, int D) {
    constexpr int RT = ELS / 32;
    const size_t per_block = A_BYTES / 16;
    const size_t total = (size_t)D * RT * KS * per_block;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < 2 * total; i += (size_t)gridDim.x * blockDim.x) {
        const bool bwd = i >= total;
        const size_t ii = bwd ? i - total : i;
        const int blk = (int)(ii / per_block), c = (int)(ii % per_block);
        const int q = blk % KS, r = (blk / KS) % RT, d = blk / (KS * RT);
        const int hl = c / 2048, cc = c % 2048;          // 2048 chunks of 16 bytes per 32 KB half
        const int cb = cc / 1024, row = (cc / 8) % 128, pos = cc % 8;
        const int lc = pos ^ (row & 7);                  // logical chunk stored at this swizzled position
        const float S = scale[2 * d];
        unsigned short v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            int g, jj, k;
            if (!bwd) {
                g = row / 32; jj = row % 32;
                k = KSL * q + cb * 64 + lc * 8 + e;
            } else {
                const int cl = cb * 64 + lc * 8 + e;
                g = cl / 32; jj = cl % 32;
                k = KSL * q + row;
            }
            const float w = wrec[(size_t)g * ls * ELS + (size_t)d * ELS * ELS + (size_t)(32 * r + jj) * ELS + k] * S;
            const __half h = __float2half_rn(w);
            v[e] = hl ? __half_as_ushort(__float2half_rn((w - __half2float(h)) * LO_SCALE)) : __half_as_ushort(h);
        }
        uint4 o;
        o.x = v[0] | ((unsigned)v[1] << 16); o.y = v[2] | ((unsigned)v[3] << 16);
        o.z = v[4] | ((unsigned)v[5] << 16); o.w = v[6] | ((unsigned)v[7] << 16);
        (bwd ? img_b : img_f)[ii] = o;
    }
}

struct Plan { int nc, nslices, nchunks, groups; bool ll; };
// Sequences per chunk and slices per direction: as many groups of blocks as the device holds (each (direction,
// slice) is one group's work), chunks of 32 while every group gets at most one of them, else of 64.
// Tuning (index 0 forward, 1 backward): nc32 = the largest number of chunks per group for which chunks are 32 sequences
// wide (such chunks always use the latency-optimised exchange: self-validating words instead of counters and bulk
// copies); ll = the largest number of 64-wide chunks per group that still uses that exchange.
// Measured on a B200 (one layer, 200 steps, ms per sweep).  Forward, 64 sequences: one chunk of 64 1.45, two of 32 1.52;
// 128 sequences: two chunks of 64 behind counters 1.95, with words 2.69, four of 32 2.47 (the forward's operand is collected
// by its cell warps, or for several 32-wide chunks by two gather warps: neither overlaps well with a second chunk).
// Backward (warps of its own collect the partial errors), 64 sequences: one chunk of 64 1.67, two of 32 1.10; 96: 2.28 /
// 1.50; 128: two of 64 behind counters 3.05, with words 2.45, four of 32 2.00; 160: three of 64 2.76, five of 32 2.54;
// 192: three of 64 2.99, six of 32 3.11; 256: four of 64 2.70, eight of 32 4.77.
std::atomic<int> g_ll_chunks[2] = {{1}, {2}}, g_nc32_chunks[2] = {{1}, {5}};
// backward only: the largest number of 32-wide chunks per group that run behind counters (wider fractions use chunks of 64)
std::atomic<int> g_nc32_counter_chunks{6};   // 192 sequences: three chunks of 64 2.73 ms, six of 32 2.52; 256: four of 64 2.69, eight of 32 3.21

Plan make_plan(int P, int D, int group_blocks, bool backward) {
    Plan p;
    int max_groups = sm_count() / group_blocks;
    if (max_groups < 1) max_groups = 1;
    int spd = max_groups / D;   // slices per direction that run side by side
    if (spd < 1) spd = 1;
    const int llc = g_ll_chunks[backward].load(), n32 = g_nc32_chunks[backward].load();
    const int n32c = backward ? g_nc32_counter_chunks.load() : 0;
    const bool words32 = P <= 32 * spd * n32;           // chunks of 32 with the latency-optimised exchange
    p.nc = (words32 || P <= 32 * spd * n32c) ? 32 : 64;
    p.nchunks = (P + p.nc - 1) / p.nc;
    p.nslices = p.nchunks < spd ? p.nchunks : spd;
    p.groups = D * p.nslices < max_groups ? D * p.nslices : max_groups;
    p.ll = p.nc == 32 ? words32 : (p.nchunks + p.nslices - 1) / p.nslices <= llc;
    return p;
}

template <int ELS, int NC, bool LL, bool BWD>
int launch_dir(PtcArgs &a, const Plan &pl, cudaStream_t st) {
    typedef Geo<ELS, NC> G;
    void (*kern)(PtcArgs);
    size_t smem;
    int threads;
    if constexpr (BWD) { kern = lstm_bwd_ptc_kernel<ELS, NC, LL>; smem = G::bwd_smem(); threads = bwd_threads(LL); }
    else { kern = lstm_fwd_ptc_kernel<ELS, NC, LL>; smem = G::fwd_smem(); threads = fwd_threads(LL); }
    B2_TRY(set_max_dynamic_smem((const void *)kern, (int)smem));
    cudaLaunchConfig_t cfg = cudaLaunchConfig_t{};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = KS; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.gridDim = dim3(pl.groups * G::GROUP);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B2_CUDA(cudaLaunchKernelEx(&cfg, kern, a));
    count_launch();
    return B2_OK;
}
template <int ELS, int NC, bool LL>
int launch(bool backward, PtcArgs &a, const Plan &pl, cudaStream_t st) {
    return backward ? launch_dir<ELS, NC, LL, true>(a, pl, st) : launch_dir<ELS, NC, LL, false>(a, pl, st);
}

constexpr int PTC_ELS = 512;
constexpr int PTC_GROUP = (PTC_ELS / 32) * KS;

}  // namespace

#ifdef B2_PTC_TRACE
extern "C" int b2_debug_ptc_trace(long long *out, int capacity) {
    const int n = 2 * TRACE_ROLES * TRACE_ITEMS * TRACE_SLOTS;
    if (capacity < n) return -n;
    if (cudaMemcpyFromSymbol(out, g_ptc_trace, sizeof(long long) * n) != cudaSuccess) return 0;
    return n;
}
#endif

bool lstm_ptc_supported(const LstmShape &s) {
    if (s.els != PTC_ELS || s.P < 1 || sm_count() < PTC_GROUP) return false;
    for (int b = 0; b < 2; ++b) {
        const Plan pl = make_plan(s.P, s.D, PTC_GROUP, b != 0);
        if ((pl.nchunks + pl.nslices - 1) / pl.nslices > MAXC) return false;
    }
    return true;
}

void lstm_ptc_set_plan(bool backward, int ll_chunks, int nc32_chunks, int nc32_counter_chunks) {
    g_ll_chunks[backward].store(ll_chunks < 1 ? 1 : ll_chunks);
    g_nc32_chunks[backward].store(nc32_chunks < 1 ? 1 : nc32_chunks);
    if (backward) g_nc32_counter_chunks.store(nc32_counter_chunks < 0 ? 0 : nc32_counter_chunks);
}

size_t lstm_ptc_image_bytes(int els, int D) { return (size_t)2 * D * 4 * els * els * 2; }   // hi + lo, fp16

void lstm_ptc_exchange_sizes(int els, int P, int D, size_t *xh_bytes, size_t *xe_floats, size_t *flag_words) {
    // sized for either exchange and for the chunking of either sweep: operand images / floats, or 8-byte tagged words
    // ([2 parities][NC][els] per chunk forward, times 16 row tiles backward)
    *xh_bytes = *xe_floats = *flag_words = 0;
    for (int b = 0; b < 2; ++b) {
        const Plan pl = make_plan(P, D, PTC_GROUP, b != 0);
        const size_t dch = (size_t)D * pl.nchunks;
        const size_t words = (size_t)2 * pl.nc * els;
        *xh_bytes = std::max(*xh_bytes, dch * words * 8);            // >= the operand images (2 * 4 * 4 * NC * 128 bytes)
        *xe_floats = std::max(*xe_floats, dch * words * (els / 32) * 2);
        *flag_words = std::max(*flag_words, dch * PTC_GROUP);
    }
}

int lstm_ptc_prepare(const LstmShape &s, const float *w, const PtcBuffers &pb, cudaStream_t st) {
    const LstmOffsets off = lstm_offsets(s.pls, s.ls, s.els);
    B2_CUDA(cudaMemsetAsync(pb.maxbits, 0, 2 * sizeof(unsigned), st));
    ptc_absmax_kernel<<<sm_count(), 256, 0, st>>>(w + off.rec, s.ls, s.els, s.D, pb.maxbits);
    ptc_scale_kernel<<<1, 32, 0, st>>>(pb.maxbits, pb.scale, s.D);
    ptc_image_kernel<PTC_ELS><<<sm_count() * 4, 256, 0, st>>>(w + off.rec, pb.scale, pb.wimg_f, pb.wimg_b, s.ls, s.D);
    count_launch(3);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

int lstm_ptc_sweep(bool backward, const LstmShape &s, const LstmBuffers &b, const PtcBuffers &pb, const float *w, float *y,
                   const float *dy, int *status, unsigned *tag_next, cudaStream_t st) {
    if (!lstm_ptc_supported(s)) return 1;
    const Plan pl = make_plan(s.P, s.D, PTC_GROUP, backward);
    PtcArgs a;
    a.sh = s; a.bf = b; a.w = w; a.y = y; a.dy = dy;
    a.wimg = backward ? pb.wimg_b : pb.wimg_f;
    a.scale = pb.scale; a.xh = pb.xh; a.xe = pb.xe; a.flags = pb.flags; a.status = status;
    a.tag_base = *tag_next;
    a.nslices = pl.nslices; a.nchunks = pl.nchunks;
    // chunks of 32 only occur with the latency-optimised exchange (see make_plan)
    int rc;
    if (pl.nc == 32 && !pl.ll) rc = launch_dir<PTC_ELS, 32, false, true>(a, pl, st);   // backward sweep only (make_plan)
    else if (pl.nc == 32) rc = launch<PTC_ELS, 32, true>(backward, a, pl, st);
    else rc = pl.ll ? launch<PTC_ELS, 64, true>(backward, a, pl, st) : launch<PTC_ELS, 64, false>(backward, a, pl, st);
    if (rc == B2_OK) *tag_next += (unsigned)s.T + 1u;
    return rc;
}

}  // namespace b2
