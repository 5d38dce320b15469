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
// (main + cross * 2^-11) / S carries 22 mantissa bits of each operand, like the 3xTF32 split of the large GEMMs,
// at half the shared memory and half the instructions.  A main accumulator never takes more than 8 MMAs (K = 128):
// tensor-memory accumulation truncates, so longer chains are cut into segments that CUDA cores add.
//
// Decomposition (els = units per direction, here 512: 16 row tiles x 2 contraction slices = 32 blocks a group).
//   forward : block (r, q) keeps W_rec rows {gate g, unit 32r + jj} x source units [256q, 256q + 256) (128 x 256,
//             hi + lo = 128 KB).  Per step it multiplies them with h[t-1] of its slice (operand B, N = 16 or 32
//             sequences), the two blocks of a row tile exchange halves of the 128 x N partial sums through
//             distributed shared memory (st.async + transaction barrier) and each finishes 16 units: gate
//             activations, peepholes, cell state, h.  h goes to all blocks that need it through L2 as tagged
//             64-bit words {step tag : hi16 : lo16}: one round trip delivers "ready" and the operand.
//   backward: the same weight tile, stored transposed, is operand A of  e[k] = sum_c W[c][k] delta[c]  with the
//             block's own row tile as the contraction range: block (r, q) turns the gate deltas of row tile r
//             (both blocks of the pair compute 16 units' deltas and hand them to each other through distributed
//             shared memory, already as fp16 operand chunks) into partial output errors of source units
//             [256q, 256q + 256) and publishes them through L2 as tagged words {step tag : float}; the block that
//             owns a unit adds the 16 partials in a fixed order (bitwise deterministic) and runs the error functor.
// Groups of sequences ("chunks" of N) are independent; a group of blocks works on several chunks in turn, so that
// the exchange of one chunk overlaps the tensor-core work of another.  Warps are specialised (gather / MMA issue /
// tensor-memory drain / cell math) and hand buffers to each other through mbarriers.
//
// Every wait is bounded (cycle budget of about two seconds, poll-round limit for the L2 words): on expiry the
// thread records B2_ERR_STEP_TIMEOUT in the layer's status word and raises the block's give-up flag, every role
// leaves its loops, the cluster meets at its hardware barrier, tensor memory is released and the block returns.
#include <cuda_fp16.h>

#include "common.cuh"
#include "ptx.cuh"

namespace b2 {
namespace {

using namespace ptx;

constexpr int NMAX = 32;                 // sequences per chunk at most
constexpr int MAXC = 16;                 // chunks a group of blocks works on at most
constexpr int KSL = 256;                 // contraction extent a block holds (forward: source units)
constexpr long long WAIT_CYCLES = 4000000000LL;
constexpr unsigned POLL_LIMIT = 1u << 21;
constexpr float LO_SCALE = 2048.0f, LO_UNSCALE = 1.0f / 2048.0f;

constexpr int FWD_THREADS = 32 * 13;     // warp 0 MMA issue, 1-4 drain + cell math, 5-12 gather
constexpr int BWD_THREADS = 32 * 17;     // warp 0 MMA issue, 1-4 cell math, 5-8 drain, 9-16 gather + reduce

// Optional timing trace (build with -DB2_PTC_TRACE): block 0 records clock64() at the hand-over points of its
// roles for the first chunk-steps of a launch; b2_debug_ptc_trace copies the records out.
#ifdef B2_PTC_TRACE
constexpr int TRACE_ITEMS = 96, TRACE_SLOTS = 8, TRACE_ROLES = 4;
__device__ long long g_ptc_trace[TRACE_ROLES][TRACE_ITEMS][TRACE_SLOTS];
#define PTC_TRACE(role, item, slot)                                                                  \
    do {                                                                                             \
        if (blockIdx.x == 0 && (item) < TRACE_ITEMS) g_ptc_trace[role][item][slot] = clock64();      \
    } while (0)
#define PTC_TRACE_VAL(role, item, slot, v)                                                           \
    do {                                                                                             \
        if (blockIdx.x == 0 && (item) < TRACE_ITEMS) g_ptc_trace[role][item][slot] = (long long)(v); \
    } while (0)
#else
#define PTC_TRACE(role, item, slot) do { } while (0)
#define PTC_TRACE_VAL(role, item, slot, v) do { } while (0)
#endif

struct PtcArgs {
    LstmShape sh;
    LstmBuffers bf;
    const float *w;
    float *y;              // forward: block outputs
    const float *dy;       // backward: output errors
    const uint4 *wimg;     // the blocks' weight images, 128 KB each, [direction][row tile][slice]
    const float *scale;    // [direction][2]: S, 1/S
    u64 *xh;               // forward exchange  [direction][chunk][step parity][n][els]
    u64 *xe;               // backward exchange [direction][chunk][step parity][row tile][n][els]
    int *status;
    unsigned tag_base;
    int nslices;           // sequence slices per direction (chunks are dealt to the slices round robin)
    int nchunks;           // chunks of NC sequences in all
};

__device__ __forceinline__ void split_f16(float x, unsigned &hi, unsigned &lo) {
    const __half h = __float2half_rn(x);
    const __half l = __float2half_rn((x - __half2float(h)) * LO_SCALE);
    hi = (unsigned)__half_as_ushort(h);
    lo = (unsigned)__half_as_ushort(l);
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
    static constexpr int KS = ELS / KSL;           // blocks of a row tile = cluster size
    static constexpr int RT = ELS / 32;            // row tiles per direction
    static constexpr int UPC = 32 / KS;            // units a block finishes
    static constexpr int GROUP = RT * KS;          // blocks per group
    static constexpr int NSUB = 128 / UPC;         // cell threads per unit
    static constexpr int CPT = NC / NSUB;          // cells (sequences) per cell thread
    static_assert(ELS % KSL == 0 && KS >= 1 && KS <= 2 && RT <= 16, "instantiated for 256 and 512 units per direction");
    static_assert(NC == 16 || NC == 32, "chunks of 16 or 32 sequences");
    static_assert(CPT >= 1, "bad cell mapping");
    static constexpr uint32_t A_BYTES = 128 * 1024;                     // hi + lo
    static constexpr uint32_t ZBLK = 4 * NC * UPC * 4;                  // one 4-gate x NC x UPC block of partial sums
    // forward
    static constexpr uint32_t FB_HL = 4 * NMAX * 128, FB_BUF = 2 * FB_HL;   // B: [buffer][hi/lo][4 column blocks][32 rows x 128 B]
    static constexpr uint32_t F_B = A_BYTES, F_ZOWN = F_B + 2 * FB_BUF, F_ZRECV = F_ZOWN + ZBLK;
    static constexpr uint32_t F_END = F_ZRECV + 2 * (KS - 1) * ZBLK;
    // backward
    static constexpr uint32_t BB_HL = 2 * NMAX * 128, BB_BUF = 2 * BB_HL;   // B: [buffer][hi/lo][2 column blocks][32 rows x 128 B]
    static constexpr uint32_t B_B = A_BYTES, B_ESUM = B_B + 2 * BB_BUF, B_DSTAGE = B_ESUM + 2 * NC * UPC * 4;
    static constexpr uint32_t B_END = B_DSTAGE + 2 * NC * 4 * UPC * 2;
    static constexpr size_t fwd_smem() { return F_END + 1024; }
    static constexpr size_t bwd_smem() { return B_END + 1024; }
};

// copies this block's 128 KB weight image into shared memory (generic proxy) and hands it to the tensor core
__device__ __forceinline__ void load_weight_image(unsigned char *dst, const uint4 *src, int nthreads) {
    uint4 *d4 = reinterpret_cast<uint4 *>(dst);
    for (int i = threadIdx.x; i < (128 * 1024) / 16; i += nthreads) d4[i] = __ldg(src + i);
    fence_async_smem();
    __syncthreads();
}

// =====================================================================================================
// forward
// =====================================================================================================
template <int ELS, int NC>
__global__ void __launch_bounds__(FWD_THREADS, 1) lstm_fwd_ptc_kernel(PtcArgs a) {
    typedef Geo<ELS, NC> G;
    constexpr int KS = G::KS, RT = G::RT, UPC = G::UPC, CPT = G::CPT, NSUB = G::NSUB;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) u64 bars[10];
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int give_up_s;
    __shared__ int lens_s[MAXC * NMAX], Tc_s[MAXC], Tmax_s;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char *gbase = smem_raw + (sbase - smem_u32(smem_raw));
    const uint32_t bar0 = smem_u32(bars);
    auto b_full = [&](int b) { return bar0 + 8u * (uint32_t)b; };          // gather warps -> MMA
    auto b_free = [&](int b) { return bar0 + 8u * (uint32_t)(2 + b); };    // MMA -> gather warps
    auto acc_full = [&](int b) { return bar0 + 8u * (uint32_t)(4 + b); };  // MMA -> drain
    auto acc_free = [&](int b) { return bar0 + 8u * (uint32_t)(6 + b); };  // drain -> MMA
    auto zr_full = [&](int b) { return bar0 + 8u * (uint32_t)(8 + b); };   // the pair's partial sums have arrived

    const int P = a.sh.P, T = a.sh.T, ls = a.sh.ls, D = a.sh.D;
    const int grp = blockIdx.x / G::GROUP, ngroups = gridDim.x / G::GROUP;
    const int bidx = blockIdx.x % G::GROUP, r = bidx / KS;
    const int q = KS > 1 ? (int)cluster_ctarank() : 0;
    const LstmOffsets off = lstm_offsets(a.sh.pls, ls, ELS);

    if (tid == 0) {
        for (int b = 0; b < 2; ++b) {
            mbar_init(b_full(b), 8); mbar_init(b_free(b), 1); mbar_init(acc_full(b), 1); mbar_init(acc_free(b), 4);
            mbar_init(zr_full(b), 1);
        }
        give_up_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc(smem_u32(&tmem_base_s), 256);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    // a peer's shared memory and barriers may be touched only once the peer runs
    if (KS > 1) cluster_sync_all();

    int m_g = 0, m_m = 0, m_e = 0;   // running count of MMA items per role (buffer = count & 1)
    const int nwork = D * a.nslices;
    for (int wi = grp; wi < nwork; wi += ngroups) {
        const int d = wi % D, sl = wi / D;
        const int ncl = (a.nchunks - sl + a.nslices - 1) / a.nslices;
        load_weight_image(gbase, a.wimg + (size_t)((d * RT + r) * KS + q) * (G::A_BYTES / 16), FWD_THREADS);
        find_lengths<NC>(a, sl, ncl, lens_s, Tc_s, &Tmax_s, FWD_THREADS);
        const int Tmax = Tmax_s;
        const float invS = a.scale[2 * d + 1];
        const size_t xh_d = (size_t)d * a.nchunks;

        if (warp == 0) {
            // ------------------------------------------------ MMA issue ------------------------------------------------
            if (lane == 0) {
                const uint32_t idesc = idesc_f16(128, NC);
                int s = 0, cl = -1;
                while (next_item(s, cl, ncl, Tc_s, Tmax)) {
                    if (s == 0) continue;
                    if (give_up_s) break;
                    const int buf = m_m & 1;
                    const uint32_t ph = (uint32_t)(m_m >> 1) & 1u;
                    const int ti = m_m;
                    ++m_m;
                    PTC_TRACE(0, ti, 0);
                    if (!mbar_wait_bounded<false>(b_full(buf), ph, &give_up_s, WAIT_CYCLES) ||
                        !mbar_wait_bounded<false>(acc_free(buf), ph ^ 1u, &give_up_s, WAIT_CYCLES)) {
                        give_up_s = 1;
                        break;
                    }
                    PTC_TRACE(0, ti, 1);
                    fence_async_smem();
                    tc_fence_after();
                    const uint32_t acc = tmem + (uint32_t)buf * 96u;
                    const uint32_t bb = sbase + G::F_B + (uint32_t)buf * G::FB_BUF;
#pragma unroll
                    for (int ks = 0; ks < 16; ++ks) {
                        const uint32_t ao = (uint32_t)(ks >> 2) * 16384u + (uint32_t)(ks & 3) * 32u;
                        const uint32_t bo = (uint32_t)(ks >> 2) * (NMAX * 128u) + (uint32_t)(ks & 3) * 32u;
                        const u64 ahi = desc_kmajor_sw128(sbase + ao, 1024), alo = desc_kmajor_sw128(sbase + 65536u + ao, 1024);
                        const u64 bhi = desc_kmajor_sw128(bb + bo, 1024), blo = desc_kmajor_sw128(bb + G::FB_HL + bo, 1024);
                        mma_f16(acc + 64u, alo, bhi, idesc, ks ? 1u : 0u);
                        mma_f16(acc + 64u, ahi, blo, idesc, 1u);
                        mma_f16(acc + (uint32_t)(ks >> 3) * 32u, ahi, bhi, idesc, (ks & 7) ? 1u : 0u);
                    }
                    mma_commit(b_free(buf));
                    mma_commit(acc_full(buf));
                    PTC_TRACE(0, ti, 2);
                }
            }
        } else if (warp <= 4) {
            // ------------------------------------ drain tensor memory, exchange halves, cell math ------------------------------------
            const int et = tid - 32;
            const int gate = warp & 3;                       // the tensor-memory lane quarter this warp may read = the gate
            const uint32_t lane_base = tmem + ((uint32_t)(32 * gate) << 16);
            const int jj = et % UPC, sub = et / UPC;        // cell role: unit jj of this block, sequences sub*CPT .. +CPT
            const int j = 32 * r + q * UPC + jj;            // unit inside the direction
            const int u = d * ELS + j;
            float b4[4], pw[3];
#pragma unroll
            for (int g = 0; g < 4; ++g) b4[g] = a.sh.bias * __ldg(a.w + off.bias + (size_t)g * ls + u);
#pragma unroll
            for (int g = 0; g < 3; ++g) pw[g] = __ldg(a.w + off.peep + (size_t)g * ls + u);
            float *zown = reinterpret_cast<float *>(gbase + G::F_ZOWN);
            const float *zrecv = reinterpret_cast<const float *>(gbase + G::F_ZRECV);

            float pre[CPT][4], cpv[CPT];
            auto fetch = [&](int s, int cl) {
                const int t = d ? Tc_s[cl] - 1 - s : s, prev = d ? t + 1 : t - 1;
                const int p0 = (sl + cl * a.nslices) * NC;
#pragma unroll
                for (int i = 0; i < CPT; ++i) {
                    const int n = sub * CPT + i, pg = p0 + n;
                    cpv[i] = 0.0f;
#pragma unroll
                    for (int g = 0; g < 4; ++g) pre[i][g] = 0.0f;
                    if (pg < P && t < lens_s[cl * NC + n]) {
                        const float *ap = a.bf.acts + ((size_t)t * P + pg) * 4 * ls + u;
#pragma unroll
                        for (int g = 0; g < 4; ++g) pre[i][g] = ap[(size_t)g * ls];
                        if (s > 0) cpv[i] = a.bf.cells[((size_t)prev * P + pg) * ls + u];
                    }
                }
            };
            int s = 0, cl = -1;
            bool more = next_item(s, cl, ncl, Tc_s, Tmax);
            if (more) fetch(s, cl);
            while (more) {
                if (give_up_s) break;
                const int ac = sl + cl * a.nslices, p0 = ac * NC;
                const int t = d ? Tc_s[cl] - 1 - s : s;
                float z[CPT][4];
#pragma unroll
                for (int i = 0; i < CPT; ++i)
#pragma unroll
                    for (int g = 0; g < 4; ++g) z[i][g] = 0.0f;
                bool ok = true;
                const int ti = m_e;
                if (s > 0) {
                    const int buf = m_e & 1;
                    const uint32_t ph = (uint32_t)(m_e >> 1) & 1u;
                    ++m_e;
                    if (et == 0) PTC_TRACE(1, ti, 0);
                    if (KS > 1 && et == 0) mbar_expect_tx(zr_full(buf), (uint32_t)(KS - 1) * G::ZBLK);
                    ok = mbar_wait_bounded<false>(acc_full(buf), ph, &give_up_s, WAIT_CYCLES);
                    if (et == 0) PTC_TRACE(1, ti, 1);
                    if (ok) {
                        tc_fence_after();
                        float v[NC];
#pragma unroll
                        for (int c0 = 0; c0 < NC; c0 += 16) {
                            uint32_t m0[16], m1[16], cx[16];
                            tmem_ld16(lane_base + (uint32_t)(buf * 96 + c0), m0);
                            tmem_ld16(lane_base + (uint32_t)(buf * 96 + 32 + c0), m1);
                            tmem_ld16(lane_base + (uint32_t)(buf * 96 + 64 + c0), cx);
                            tmem_ld_wait();
#pragma unroll
                            for (int c = 0; c < 16; ++c)
                                v[c0 + c] = ((__uint_as_float(m0[c]) + __uint_as_float(m1[c])) + __uint_as_float(cx[c]) * LO_UNSCALE) * invS;
                        }
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(acc_free(buf));
                        // row (gate, lane): unit lane of the row tile belongs to block lane / UPC of the pair
                        const int tr = lane / UPC, tj = lane % UPC;
                        if (tr == q) {
#pragma unroll
                            for (int qd = 0; qd < NC / 4; ++qd)
                                *reinterpret_cast<float4 *>(zown + ((gate * (NC / 4) + qd) * UPC + tj) * 4) =
                                    make_float4(v[4 * qd], v[4 * qd + 1], v[4 * qd + 2], v[4 * qd + 3]);
                        } else {
                            const int slot = q < tr ? q : q - 1;   // this block's position among the target's sources
                            const uint32_t la = sbase + G::F_ZRECV + (uint32_t)(buf * (KS - 1) + slot) * G::ZBLK;
                            const uint32_t rbar = map_to_rank(zr_full(buf), (uint32_t)tr);
#pragma unroll
                            for (int qd = 0; qd < NC / 4; ++qd)
                                st_async_v4(map_to_rank(la + (uint32_t)(((gate * (NC / 4) + qd) * UPC + tj) * 16), (uint32_t)tr),
                                            __float_as_uint(v[4 * qd]), __float_as_uint(v[4 * qd + 1]), __float_as_uint(v[4 * qd + 2]),
                                            __float_as_uint(v[4 * qd + 3]), rbar);
                        }
                    }
                    bar_named(1, 128);
                    if (et == 0) PTC_TRACE(1, ti, 2);
                    if (ok && KS > 1) ok = mbar_wait_bounded<true>(zr_full(buf), ph, &give_up_s, WAIT_CYCLES);
                    if (et == 0) PTC_TRACE(1, ti, 3);
                    if (!ok) { give_up_s = 1; atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT); }
                    if (ok) {
                        // partial sums of the contraction slices in slice order (own slice from zown, the others' as received)
#pragma unroll
                        for (int rs = 0; rs < KS; ++rs) {
                            const float *src = rs == q ? zown : zrecv + (size_t)(buf * (KS - 1) + (rs < q ? rs : rs - 1)) * (G::ZBLK / 4);
#pragma unroll
                            for (int i = 0; i < CPT; ++i) {
                                const int n = sub * CPT + i;
#pragma unroll
                                for (int g = 0; g < 4; ++g) z[i][g] += src[((g * (NC / 4) + (n >> 2)) * UPC + jj) * 4 + (n & 3)];
                            }
                        }
                    }
                    // zown is rewritten by the next item's drain; the 128 threads leave together or not at all
                    ok = !bar_named_or(1, 128, !ok);
                }
                if (!ok) break;
                if (et == 0 && s > 0) PTC_TRACE(1, ti, 4);
                // cell math (ComputeBlockOutputFn of the reference), publish h, then the layer's own state
                const bool first = (s == 0), publish = (s + 1 < Tc_s[cl]);
                u64 *xo = a.xh + (((xh_d + ac) * 2 + (s & 1)) * NC) * ELS + j;
                float ni[CPT], ig[CPT], fg[CPT], og[CPT], cs[CPT], hh[CPT];
#pragma unroll
                for (int i = 0; i < CPT; ++i) {
                    const int n = sub * CPT + i, pg = p0 + n;
                    ni[i] = ig[i] = fg[i] = og[i] = cs[i] = hh[i] = 0.0f;
                    if (pg < P && t < lens_s[cl * NC + n]) {
                        float x0 = pre[i][0] + z[i][0] + b4[0], x1 = pre[i][1] + z[i][1] + b4[1];
                        float x2 = pre[i][2] + z[i][2] + b4[2], x3 = pre[i][3] + z[i][3] + b4[3];
                        const float cp = cpv[i];
                        if (!first) { x1 += cp * pw[0]; x2 += cp * pw[1]; }
                        ni[i] = act_tanh(x0); ig[i] = act_logistic(x1); fg[i] = act_logistic(x2);
                        float c = ni[i] * ig[i];
                        if (!first) c += cp * fg[i];
                        og[i] = act_logistic(x3 + c * pw[2]);
                        cs[i] = c;
                        hh[i] = act_tanh(c) * og[i];
                    }
                    if (publish) {
                        unsigned hi, lo;
                        split_f16(hh[i], hi, lo);
                        st_tagged(xo + (size_t)n * ELS, a.tag_base + (unsigned)s, (hi << 16) | lo);
                    }
                }
#pragma unroll
                for (int i = 0; i < CPT; ++i) {
                    const int n = sub * CPT + i, pg = p0 + n;
                    if (pg < P) {
                        const size_t f = (size_t)t * P + pg;
                        float *ap = a.bf.acts + f * 4 * ls + u;
                        ap[0] = ni[i]; ap[ls] = ig[i]; ap[2 * (size_t)ls] = fg[i]; ap[3 * (size_t)ls] = og[i];   // zeros on padding
                        a.bf.cells[f * ls + u] = cs[i];
                        a.y[f * ls + u] = hh[i];
                    }
                }
                if (et == 0 && s > 0) PTC_TRACE(1, ti, 5);
                more = next_item(s, cl, ncl, Tc_s, Tmax);
                if (more) fetch(s, cl);
                if (et == 0 && s > 1) PTC_TRACE(1, ti, 6);
            }
            // frames beyond a chunk's longest sequence are padding for all its sequences: outputs are zero there
            for (int c2 = 0; c2 < ncl; ++c2) {
                const int p0 = (sl + c2 * a.nslices) * NC;
                for (int i = sub; i < (T - Tc_s[c2]) * NC; i += NSUB) {
                    const int t = Tc_s[c2] + i / NC, pg = p0 + i % NC;
                    if (pg < P) a.y[((size_t)t * P + pg) * ls + u] = 0.0f;
                }
            }
        } else {
            // ------------------------------------------------ gather h[t-1] into operand B ------------------------------------------------
            const int gt = tid - 160;
            constexpr int CH = NC / 8;   // 16-byte operand chunks (8 source units of one sequence) per thread
            int s = 0, cl = -1;
            while (next_item(s, cl, ncl, Tc_s, Tmax)) {
                if (s == 0) continue;
                if (give_up_s) break;
                const int buf = m_g & 1;
                const uint32_t ph = (uint32_t)(m_g >> 1) & 1u;
                const int ti = m_g;
                ++m_g;
                if (gt == 0) PTC_TRACE(2, ti, 0);
                if (!mbar_wait_bounded<false>(b_free(buf), ph ^ 1u, &give_up_s, WAIT_CYCLES)) { give_up_s = 1; break; }
                if (gt == 0) PTC_TRACE(2, ti, 1);
                const int ac = sl + cl * a.nslices;
                const u64 *src = a.xh + (((xh_d + ac) * 2 + ((s - 1) & 1)) * NC) * ELS + KSL * q;
                const unsigned tag = a.tag_base + (unsigned)(s - 1);
                const uint32_t bb = sbase + G::F_B + (uint32_t)buf * G::FB_BUF;
                unsigned done = 0;
                bool ok = true;
                for (unsigned round = 0; done != (1u << CH) - 1u; ++round) {
                    if (gt == 0) PTC_TRACE_VAL(2, ti, 3, round + 1);
                    u64 wds[CH][8];
#pragma unroll
                    for (int c = 0; c < CH; ++c) {
                        if (done & (1u << c)) continue;
                        const int ci = gt + 256 * c, n = ci >> 5, kc = ci & 31;
                        const u64 *p = src + (size_t)n * ELS + kc * 8;
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
                        const int ci = gt + 256 * c, n = ci >> 5, kc = ci & 31;
                        uint32_t hi[4], lo[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const unsigned w0 = (unsigned)wds[c][2 * e], w1 = (unsigned)wds[c][2 * e + 1];
                            hi[e] = (w0 >> 16) | (w1 & 0xffff0000u);
                            lo[e] = (w0 & 0xffffu) | (w1 << 16);
                        }
                        const uint32_t o = (uint32_t)(kc >> 3) * (NMAX * 128u) + (uint32_t)n * 128u + (uint32_t)(((kc & 7) ^ (n & 7)) * 16);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(bb + o), "r"(hi[0]), "r"(hi[1]), "r"(hi[2]), "r"(hi[3]) : "memory");
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(bb + G::FB_HL + o), "r"(lo[0]), "r"(lo[1]), "r"(lo[2]), "r"(lo[3]) : "memory");
                        done |= 1u << c;
                    }
                    if (done != (1u << CH) - 1u &&
                        (round >= POLL_LIMIT || give_up_s || ((round & 1023u) == 1023u && ld_relaxed_s32(a.status) != 0))) {
                        ok = false;
                        break;
                    }
                }
                if (!ok) { give_up_s = 1; atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT); break; }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(b_full(buf));
                if (gt == 0) PTC_TRACE(2, ti, 2);
            }
        }
        __syncthreads();   // every role is through this work item (the weight image may be replaced)
        if (give_up_s) break;
    }
    tc_fence_before();
    __syncthreads();
    if (give_up_s && tid == 0) atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT);
    // nobody leaves while a peer may still write into its shared memory
    if (KS > 1) cluster_sync_all();
    if (warp == 0) tmem_dealloc(tmem, 256);
}

// =====================================================================================================
// backward
// =====================================================================================================
template <int ELS, int NC>
__global__ void __launch_bounds__(BWD_THREADS, 1) lstm_bwd_ptc_kernel(PtcArgs a) {
    typedef Geo<ELS, NC> G;
    constexpr int KS = G::KS, RT = G::RT, UPC = G::UPC, CPT = G::CPT, NSUB = G::NSUB;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) u64 bars[12];
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int give_up_s;
    __shared__ int lens_s[MAXC * NMAX], Tc_s[MAXC], Tmax_s;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char *gbase = smem_raw + (sbase - smem_u32(smem_raw));
    const uint32_t bar0 = smem_u32(bars);
    auto b_full = [&](int b) { return bar0 + 8u * (uint32_t)b; };          // cell warps of the pair -> MMA
    auto b_free = [&](int b) { return bar0 + 8u * (uint32_t)(2 + b); };    // MMAs of the whole pair done -> cell warps
    auto acc_full = [&](int b) { return bar0 + 8u * (uint32_t)(4 + b); };  // MMA -> drain
    auto acc_free = [&](int b) { return bar0 + 8u * (uint32_t)(6 + b); };  // drain -> MMA
    auto e_full = [&](int b) { return bar0 + 8u * (uint32_t)(8 + b); };    // reduce warps -> cell warps
    auto e_free = [&](int b) { return bar0 + 8u * (uint32_t)(10 + b); };   // cell warps -> reduce warps

    const int P = a.sh.P, T = a.sh.T, ls = a.sh.ls, D = a.sh.D;
    const int grp = blockIdx.x / G::GROUP, ngroups = gridDim.x / G::GROUP;
    const int bidx = blockIdx.x % G::GROUP, r = bidx / KS;
    const int q = KS > 1 ? (int)cluster_ctarank() : 0;
    const LstmOffsets off = lstm_offsets(a.sh.pls, ls, ELS);

    if (tid == 0) {
        for (int b = 0; b < 2; ++b) {
            mbar_init(b_full(b), 1); mbar_init(b_free(b), KS); mbar_init(acc_full(b), 1); mbar_init(acc_free(b), 4);
            mbar_init(e_full(b), 8); mbar_init(e_free(b), 4);
        }
        give_up_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc(smem_u32(&tmem_base_s), 256);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    if (KS > 1) cluster_sync_all();

    // producer side (cell -> MMA -> drain) counts the chunk-steps whose deltas somebody consumes (s + 1 < Tc);
    // consumer side (reduce -> cell) counts the chunk-steps that receive a recurrent error (s >= 1)
    int mp_m = 0, mp_c = 0, mp_d = 0, mc_r = 0, mc_c = 0;
    const int nwork = D * a.nslices;
    for (int wi = grp; wi < nwork; wi += ngroups) {
        const int d = wi % D, sl = wi / D;
        const int ncl = (a.nchunks - sl + a.nslices - 1) / a.nslices;
        load_weight_image(gbase, a.wimg + (size_t)((d * RT + r) * KS + q) * (G::A_BYTES / 16), BWD_THREADS);
        find_lengths<NC>(a, sl, ncl, lens_s, Tc_s, &Tmax_s, BWD_THREADS);
        const int Tmax = Tmax_s;
        const float invS = a.scale[2 * d + 1];
        const size_t xe_d = (size_t)d * a.nchunks;

        if (warp == 0) {
            // ------------------------------------------------ MMA issue ------------------------------------------------
            if (lane == 0) {
                const uint32_t idesc = idesc_f16(128, NC);
                int s = 0, cl = -1;
                while (next_item(s, cl, ncl, Tc_s, Tmax)) {
                    if (s + 1 >= Tc_s[cl]) continue;
                    if (give_up_s) break;
                    const int buf = mp_m & 1;
                    const uint32_t ph = (uint32_t)(mp_m >> 1) & 1u;
                    ++mp_m;
                    if (!mbar_wait_bounded<true>(b_full(buf), ph, &give_up_s, WAIT_CYCLES) ||
                        !mbar_wait_bounded<false>(acc_free(buf), ph ^ 1u, &give_up_s, WAIT_CYCLES)) {
                        give_up_s = 1;
                        break;
                    }
                    fence_async_smem();
                    tc_fence_after();
                    const uint32_t acc = tmem + (uint32_t)buf * 128u;
                    const uint32_t bb = sbase + G::B_B + (uint32_t)buf * G::BB_BUF;
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                        for (int ks = 0; ks < 8; ++ks) {
                            const uint32_t ao = (uint32_t)mt * 32768u + (uint32_t)(ks >> 2) * 16384u + (uint32_t)(ks & 3) * 32u;
                            const uint32_t bo = (uint32_t)(ks >> 2) * (NMAX * 128u) + (uint32_t)(ks & 3) * 32u;
                            const u64 ahi = desc_kmajor_sw128(sbase + ao, 1024), alo = desc_kmajor_sw128(sbase + 65536u + ao, 1024);
                            const u64 bhi = desc_kmajor_sw128(bb + bo, 1024), blo = desc_kmajor_sw128(bb + G::BB_HL + bo, 1024);
                            mma_f16(acc + (uint32_t)(mt * 64 + 32), alo, bhi, idesc, ks ? 1u : 0u);
                            mma_f16(acc + (uint32_t)(mt * 64 + 32), ahi, blo, idesc, 1u);
                            mma_f16(acc + (uint32_t)(mt * 64), ahi, bhi, idesc, ks ? 1u : 0u);
                        }
                    mma_commit(b_free(buf));
                    mma_commit(acc_full(buf));
                }
            }
        } else if (warp <= 4) {
            // ------------------------------------------------ cell math: the error functor ------------------------------------------------
            const int et = tid - 32;
            const int jj = et % UPC, sub = et / UPC;
            const int j = 32 * r + q * UPC + jj;
            const int u = d * ELS + j;
            const float p_ig = __ldg(a.w + off.peep + u), p_fg = __ldg(a.w + off.peep + (size_t)ls + u);
            const float p_og = __ldg(a.w + off.peep + 2 * (size_t)ls + u);
            const float *esum = reinterpret_cast<const float *>(gbase + G::B_ESUM);
            unsigned short *dstage = reinterpret_cast<unsigned short *>(gbase + G::B_DSTAGE);   // [hi/lo][n][gate*UPC + jj]

            // everything a step reads besides the recurrent error is fetched when the previous chunk-step is done
            float f_dy[CPT], f_act[CPT][4], f_c[CPT], f_cp[CPT], f_nfg[CPT], f_nce[CPT], f_ndig[CPT], f_ndfg[CPT];
            auto fetch = [&](int s, int cl) {
                const int Tcc = Tc_s[cl];
                const int t = d ? s : Tcc - 1 - s;
                const int next = d ? t - 1 : t + 1, prevc = d ? t + 1 : t - 1;
                const bool lastCall = d ? (t == Tcc - 1) : (t == 0);
                const int p0 = (sl + cl * a.nslices) * NC;
                const float *ce_nxt = a.bf.cerr + (size_t)((s + 1) & 1) * P * ls;
#pragma unroll
                for (int i = 0; i < CPT; ++i) {
                    const int n = sub * CPT + i, pg = p0 + n;
                    f_dy[i] = f_c[i] = f_cp[i] = f_nfg[i] = f_nce[i] = f_ndig[i] = f_ndfg[i] = 0.0f;
#pragma unroll
                    for (int g = 0; g < 4; ++g) f_act[i][g] = 0.0f;
                    if (pg < P && t < lens_s[cl * NC + n]) {
                        const size_t f = (size_t)t * P + pg;
                        f_dy[i] = a.dy[f * ls + u];
                        const float *ap = a.bf.acts + f * 4 * ls + u;
#pragma unroll
                        for (int g = 0; g < 4; ++g) f_act[i][g] = ap[(size_t)g * ls];
                        f_c[i] = a.bf.cells[f * ls + u];
                        if (!lastCall) f_cp[i] = a.bf.cells[((size_t)prevc * P + pg) * ls + u];
                        if (s > 0) {
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
                if (s > 0) {
                    const int buf = mc_c & 1;
                    const uint32_t ph = (uint32_t)(mc_c >> 1) & 1u;
                    ++mc_c;
                    ok = mbar_wait_bounded<false>(e_full(buf), ph, &give_up_s, WAIT_CYCLES);
                    if (ok) {
#pragma unroll
                        for (int i = 0; i < CPT; ++i) er[i] = esum[(buf * NC + sub * CPT + i) * UPC + jj];
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(e_free(buf));
                }
                int pbuf = 0;
                uint32_t pph = 0;
                if (feeds) {
                    pbuf = mp_c & 1;
                    pph = (uint32_t)(mp_c >> 1) & 1u;
                    ++mp_c;
                    // operand buffer pbuf: the MMAs of the chunk-step before last, in every block of the pair, have read it
                    if (ok) ok = mbar_wait_bounded<true>(b_free(pbuf), pph ^ 1u, &give_up_s, WAIT_CYCLES);
                }
                // the 128 threads leave together or not at all (named barriers follow)
                if (bar_named_or(1, 128, !ok)) { give_up_s = 1; atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT); break; }
                float *ce_cur = a.bf.cerr + (size_t)(s & 1) * P * ls;
#pragma unroll
                for (int i = 0; i < CPT; ++i) {
                    const int n = sub * CPT + i, pg = p0 + n;
                    float dni = 0.0f, dig = 0.0f, dfg = 0.0f, dog = 0.0f, ce = 0.0f;
                    const bool real = pg < P && t < lens_s[cl * NC + n];
                    if (real) {
                        const float e = f_dy[i] + er[i];
                        const float ni = f_act[i][0], ig = f_act[i][1], fg = f_act[i][2], og = f_act[i][3];
                        const float tc = act_tanh(f_c[i]);
                        dog = d_logistic(og) * tc * e;
                        ce = og * d_tanh(tc) * e + p_og * dog;
                        if (!firstCall) ce += f_nfg[i] * f_nce[i] + p_ig * f_ndig[i] + p_fg * f_ndfg[i];
                        dni = ig * d_tanh(ni) * ce;
                        if (!lastCall) dfg = d_logistic(fg) * f_cp[i] * ce;
                        dig = d_logistic(ig) * ni * ce;
                        dni = limited_error(dni); dig = limited_error(dig); dfg = limited_error(dfg); dog = limited_error(dog);
                    }
                    if (feeds) {
                        unsigned hi, lo;
                        const float dl[4] = {dni, dig, dfg, dog};
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            split_f16(dl[g], hi, lo);
                            dstage[n * (4 * UPC) + g * UPC + jj] = (unsigned short)hi;
                            dstage[(NC + n) * (4 * UPC) + g * UPC + jj] = (unsigned short)lo;
                        }
                    }
                    if (pg < P) {
                        const size_t o = ((size_t)t * P + pg) * 4 * ls + u;
                        a.bf.deltas[o] = dni; a.bf.deltas[o + ls] = dig; a.bf.deltas[o + 2 * (size_t)ls] = dfg; a.bf.deltas[o + 3 * (size_t)ls] = dog;
                        ce_cur[(size_t)pg * ls + u] = ce;
                    }
                }
                if (feeds) {
                    bar_named(1, 128);
                    // 16-byte operand chunks (8 gate rows of one sequence) into this block's operand B and the peers'
                    const uint32_t bb = sbase + G::B_B + (uint32_t)pbuf * G::BB_BUF;
                    constexpr int CPG = UPC / 8;                       // chunks per gate in this block's share
                    constexpr int NCHUNK = 2 * NC * 4 * CPG;
                    for (int ci = et; ci < NCHUNK; ci += 128) {
                        const int oc = ci % (4 * CPG), n = (ci / (4 * CPG)) % NC, hl = ci / (4 * CPG * NC);
                        const int g = oc / CPG, part = oc % CPG;
                        const uint4 v = *reinterpret_cast<const uint4 *>(dstage + (hl * NC + n) * (4 * UPC) + g * UPC + part * 8);
                        const int clc = g * 4 + (q * UPC) / 8 + part;   // chunk index along the 128 gate rows of the row tile
                        const uint32_t o = (uint32_t)hl * G::BB_HL + (uint32_t)(clc >> 3) * (NMAX * 128u) + (uint32_t)n * 128u +
                                           (uint32_t)(((clc & 7) ^ (n & 7)) * 16);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(bb + o), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
#pragma unroll
                        for (int pr = 0; pr < KS; ++pr)
                            if (pr != q) st_async_v4(map_to_rank(bb + o, (uint32_t)pr), v.x, v.y, v.z, v.w, map_to_rank(b_full(pbuf), (uint32_t)pr));
                    }
                    fence_async_smem();
                    bar_named(1, 128);
                    // one arrival per phase; it also announces the bytes the peers deliver into this buffer
                    if (et == 0) {
                        if (KS > 1) mbar_expect_tx(b_full(pbuf), (uint32_t)(KS - 1) * 2u * NC * 4u * UPC * 2u);
                        else mbar_arrive(b_full(pbuf));
                    }
                }
                more = next_item(s, cl, ncl, Tc_s, Tmax);
                if (more) fetch(s, cl);
            }
            // frames beyond a chunk's longest sequence: zero deltas (they are operands of the gradient GEMMs)
            for (int c2 = 0; c2 < ncl; ++c2) {
                const int p0 = (sl + c2 * a.nslices) * NC;
                for (int i = sub; i < (T - Tc_s[c2]) * NC; i += NSUB) {
                    const int t = Tc_s[c2] + i / NC, pg = p0 + i % NC;
                    if (pg < P) {
                        const size_t o = ((size_t)t * P + pg) * 4 * ls + u;
                        a.bf.deltas[o] = 0.0f; a.bf.deltas[o + ls] = 0.0f; a.bf.deltas[o + 2 * (size_t)ls] = 0.0f; a.bf.deltas[o + 3 * (size_t)ls] = 0.0f;
                    }
                }
            }
        } else if (warp <= 8) {
            // ------------------------------------------------ drain: partial output errors to L2 ------------------------------------------------
            const int q4 = warp & 3;
            const uint32_t lane_base = tmem + ((uint32_t)(32 * q4) << 16);
            int s = 0, cl = -1;
            while (next_item(s, cl, ncl, Tc_s, Tmax)) {
                if (s + 1 >= Tc_s[cl]) continue;
                if (give_up_s) break;
                const int buf = mp_d & 1;
                const uint32_t ph = (uint32_t)(mp_d >> 1) & 1u;
                ++mp_d;
                if (!mbar_wait_bounded<false>(acc_full(buf), ph, &give_up_s, WAIT_CYCLES)) { give_up_s = 1; break; }
                tc_fence_after();
                // the MMAs of this chunk-step are complete: the peers may refill their copy of operand buffer buf
                if (KS > 1 && warp == 5 && lane < KS && lane != q) mbar_arrive_cluster(map_to_rank(b_free(buf), (uint32_t)lane));
                const int ac = sl + cl * a.nslices;
                u64 *xo = a.xe + ((((xe_d + ac) * 2 + (s & 1)) * RT + r) * NC) * ELS + KSL * q + 32 * q4 + lane;
                const unsigned tag = a.tag_base + (unsigned)s;
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int c0 = 0; c0 < NC; c0 += 16) {
                        uint32_t mn[16], cx[16];
                        tmem_ld16(lane_base + (uint32_t)(buf * 128 + mt * 64 + c0), mn);
                        tmem_ld16(lane_base + (uint32_t)(buf * 128 + mt * 64 + 32 + c0), cx);
                        tmem_ld_wait();
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            const float v = (__uint_as_float(mn[c]) + __uint_as_float(cx[c]) * LO_UNSCALE) * invS;
                            st_tagged(xo + (size_t)(c0 + c) * ELS + mt * 128, tag, __float_as_uint(v));
                        }
                    }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_free(buf));
            }
        } else {
            // ------------------------------------------------ gather + reduce the partial output errors ------------------------------------------------
            const int pt = tid - 288;
            float *esum = reinterpret_cast<float *>(gbase + G::B_ESUM);
            constexpr int NPAIR = NC * UPC / 2;   // (sequence, unit pair) slots of this block
            static_assert(NPAIR <= 256, "one pass of the reduce warps");
            const int n = pt / (UPC / 2), jp = pt % (UPC / 2);
            const bool active = pt < NPAIR;
            int s = 0, cl = -1;
            while (next_item(s, cl, ncl, Tc_s, Tmax)) {
                if (s == 0) continue;
                if (give_up_s) break;
                const int buf = mc_r & 1;
                const uint32_t ph = (uint32_t)(mc_r >> 1) & 1u;
                ++mc_r;
                if (!mbar_wait_bounded<false>(e_free(buf), ph ^ 1u, &give_up_s, WAIT_CYCLES)) { give_up_s = 1; break; }
                const int ac = sl + cl * a.nslices;
                const unsigned tag = a.tag_base + (unsigned)(s - 1);
                bool ok = true;
                if (active) {
                    const u64 *src = a.xe + ((((xe_d + ac) * 2 + ((s - 1) & 1)) * RT) * NC + n) * ELS + 32 * r + q * UPC + 2 * jp;
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
                    *reinterpret_cast<float2 *>(esum + (buf * NC + n) * UPC + 2 * jp) = make_float2(e0, e1);
                }
                if (!ok) { give_up_s = 1; atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT); break; }
                __syncwarp();
                if (lane == 0) mbar_arrive(e_full(buf));
            }
        }
        __syncthreads();
        if (give_up_s) break;
    }
    tc_fence_before();
    __syncthreads();
    if (give_up_s && tid == 0) atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT);
    if (KS > 1) cluster_sync_all();
    if (warp == 0) tmem_dealloc(tmem, 256);
}

// =====================================================================================================
// weight images
// =====================================================================================================
__global__ void ptc_absmax_kernel(const float *__restrict__ wrec, int ls, int els, int D, unsigned *maxbits) {
    // recurrent block: W[g][d][j][k] at g*ls*els + d*els*els + j*els + k
    const size_t total = (size_t)4 * ls * els;
    unsigned m[2] = {0u, 0u};
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int d = (int)((i / ((size_t)els * els)) % D);
        const unsigned b = __float_as_uint(fabsf(wrec[i]));
        if (b < 0x7f800000u && b > m[d]) m[d] = b;   // NaN / Inf weights do not set the scale
    }
    for (int d = 0; d < D; ++d) {
        unsigned v = m[d];
        for (int o = 16; o; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
        if ((threadIdx.x & 31) == 0 && v) atomicMax(maxbits + d, v);
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

// One thread per 16-byte chunk (8 fp16 values) of the images.  Forward image of block (d, r, q): [hi/lo][4 column
// blocks][128 rows = gate*32 + jj][64 source units], 128-byte rows with the 128-byte swizzle.  Backward image:
// [hi/lo][2 m tiles][2 column blocks][128 rows = source unit][64 gate rows].
template <int ELS>
__global__ void ptc_image_kernel(const float *__restrict__ wrec, const float *__restrict__ scale, uint4 *__restrict__ img_f,
                                 uint4 *__restrict__ img_b, int ls, int D) {
    constexpr int KS = ELS / KSL, RT = ELS / 32;
    const size_t per_block = (128 * 1024) / 16;
    const size_t total = (size_t)D * RT * KS * per_block;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < 2 * total; i += (size_t)gridDim.x * blockDim.x) {
        const bool bwd = i >= total;
        const size_t ii = bwd ? i - total : i;
        const int blk = (int)(ii / per_block), c = (int)(ii % per_block);
        const int q = blk % KS, r = (blk / KS) % RT, d = blk / (KS * RT);
        const int hl = c / 4096, cc = c % 4096;          // 4096 chunks of 16 bytes per 64 KB half
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
                const int mt = cb / 2, cl = (cb % 2) * 64 + lc * 8 + e;
                g = cl / 32; jj = cl % 32;
                k = KSL * q + mt * 128 + row;
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

struct Plan { int nc, nslices, nchunks, groups; };
// Sequences per chunk and slices per direction: as many groups of blocks as the device holds (each (direction,
// slice) is one group's work), chunks of 16 while every group gets at most one of them, else of 32.
Plan make_plan(int P, int D, int group_blocks) {
    Plan p;
    int max_groups = sm_count() / group_blocks;
    if (max_groups < 1) max_groups = 1;
    int spd = max_groups / D;   // slices per direction that run side by side
    if (spd < 1) spd = 1;
    p.nc = P <= 16 * spd ? 16 : 32;
    p.nchunks = (P + p.nc - 1) / p.nc;
    p.nslices = p.nchunks < spd ? p.nchunks : spd;
    p.groups = D * p.nslices < max_groups ? D * p.nslices : max_groups;
    return p;
}

template <int ELS, int NC>
int launch(bool backward, PtcArgs &a, const Plan &pl, cudaStream_t st) {
    typedef Geo<ELS, NC> G;
    void (*kern)(PtcArgs) = backward ? lstm_bwd_ptc_kernel<ELS, NC> : lstm_fwd_ptc_kernel<ELS, NC>;
    const size_t smem = backward ? G::bwd_smem() : G::fwd_smem();
    B2_TRY(set_max_dynamic_smem((const void *)kern, (int)smem));
    cudaLaunchConfig_t cfg = cudaLaunchConfig_t{};
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (G::KS > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = G::KS; attr[na].val.clusterDim.y = 1; attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.gridDim = dim3(pl.groups * G::GROUP);
    cfg.blockDim = dim3(backward ? BWD_THREADS : FWD_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = na;
    B2_CUDA(cudaLaunchKernelEx(&cfg, kern, a));
    count_launch();
    return B2_OK;
}

}  // namespace

#ifdef B2_PTC_TRACE
extern "C" int b2_debug_ptc_trace(long long *out, int capacity) {
    const int n = TRACE_ROLES * TRACE_ITEMS * TRACE_SLOTS;
    if (capacity < n) return -n;
    if (cudaMemcpyFromSymbol(out, g_ptc_trace, sizeof(long long) * n) != cudaSuccess) return 0;
    return n;
}
#endif

bool lstm_ptc_supported(const LstmShape &s) {
    if (s.els != 512 || s.P < 1) return false;
    const Plan pl = make_plan(s.P, s.D, 32);
    const int ncl = (pl.nchunks + pl.nslices - 1) / pl.nslices;
    return ncl <= MAXC && sm_count() >= 32;
}

size_t lstm_ptc_image_bytes(int els, int D) { return (size_t)2 * D * 4 * els * els * 2; }   // hi + lo, fp16

void lstm_ptc_exchange_words(int els, int P, int D, size_t *xh_words, size_t *xe_words) {
    const Plan pl = make_plan(P, D, (els / 32) * (els / KSL));
    const size_t slots = (size_t)D * pl.nchunks * 2 * pl.nc * els;
    *xh_words = slots;
    *xe_words = slots * (els / 32);
}

int lstm_ptc_prepare(const LstmShape &s, const float *w, const PtcBuffers &pb, cudaStream_t st) {
    const LstmOffsets off = lstm_offsets(s.pls, s.ls, s.els);
    B2_CUDA(cudaMemsetAsync(pb.maxbits, 0, 2 * sizeof(unsigned), st));
    ptc_absmax_kernel<<<sm_count(), 256, 0, st>>>(w + off.rec, s.ls, s.els, s.D, pb.maxbits);
    ptc_scale_kernel<<<1, 32, 0, st>>>(pb.maxbits, pb.scale, s.D);
    ptc_image_kernel<512><<<sm_count() * 4, 256, 0, st>>>(w + off.rec, pb.scale, pb.wimg_f, pb.wimg_b, s.ls, s.D);
    count_launch(3);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

int lstm_ptc_sweep(bool backward, const LstmShape &s, const LstmBuffers &b, const PtcBuffers &pb, const float *w, float *y,
                   const float *dy, int *status, unsigned *tag_next, cudaStream_t st) {
    if (!lstm_ptc_supported(s)) return 1;
    const Plan pl = make_plan(s.P, s.D, 32);
    PtcArgs a;
    a.sh = s; a.bf = b; a.w = w; a.y = y; a.dy = dy;
    a.wimg = backward ? pb.wimg_b : pb.wimg_f;
    a.scale = pb.scale; a.xh = pb.xh; a.xe = pb.xe; a.status = status;
    a.tag_base = *tag_next;
    a.nslices = pl.nslices; a.nchunks = pl.nchunks;
    int rc = pl.nc == 16 ? launch<512, 16>(backward, a, pl, st) : launch<512, 32>(backward, a, pl, st);
    if (rc == B2_OK) *tag_next += (unsigned)s.T + 1u;
    return rc;
}

}  // namespace b2
