// Persistent LSTM recurrence kernels: ONE launch runs all timesteps of a layer's forward (or
// BPTT backward) sweep, both directions concurrently.
//
// Replaces the reference's per-timestep loop of 4 cublasSgemm + 1 Thrust functor per direction
// (layers/LstmLayer.cu:1805-1858,1878-1927 forward with ComputeBlockOutputFn :57-185;
//  :2115-2176,2195-2253 backward with ComputeBlockErrorsFn :237-405 of the reference).
//
// Decomposition.  Sequences are independent, so the work splits into items (direction, slice of
// PS sequences).  An item is processed by a GROUP of G = els/JB thread blocks; block g owns hidden
// units [g*JB, (g+1)*JB) with all four gates: a 4*JB x els slice of the recurrent weights that
// stays in REGISTERS for the whole sweep (4*JB*els = 32768 floats = 128 per thread).  Only the
// blocks of one group ever wait for each other; there is no grid-wide barrier.
//
//   forward : every block needs the whole h[t-1] (els x PS) of its group  -> all-gather
//   backward: block g turns its own gate deltas into PARTIAL sums of the output error of every
//             unit k (same weight slice, other contraction index) and sends each partial to the
//             block that owns k, which adds the G partials in a fixed order -> reduce-scatter
//
// Register tiles.  The per-step products read their vector operand (h[t-1] resp. the gate deltas)
// from shared memory as warp-wide broadcasts, which deliver only 16 bytes per 4 shared-memory
// cycles.  Each thread therefore multiplies every value it loads with FOUR weights:
//   forward : thread = (unit jj, k-range of 32): the 4 gate rows of its unit x 32 source units
//   backward: thread = (4 adjacent source units k, 32 of the block's gate rows)
// so that a step needs 32 broadcast loads per thread and sequence quad instead of 128; the partial
// sums of the k-ranges (row ranges) are combined through shared memory.
//
// Exchange.  Two transports, same data flow:
//  * thread-block cluster (groups of <= 8 blocks: 128 or 256 units per direction): values are stored
//    straight into the peers' shared memory (distributed shared memory, st.shared::cluster) and one
//    hardware cluster barrier (arrive.release / wait.acquire) per step orders them;
//  * L2 (any group size): the flag travels inside the datum: one naturally aligned 64-bit word
//    {step tag : float bits}, written with st.relaxed.gpu and polled with ld.relaxed.gpu, so one L2
//    round trip delivers both "ready" and the value; no fence, no atomics.  Polling goes in rounds
//    (all outstanding loads are issued before any is examined).  Buffers are double-buffered over
//    the step parity and over the item parity.
//
// Every software wait is bounded: after SPIN_LIMIT polling rounds (about a second) the thread
// records B2_ERR_STEP_TIMEOUT in the layer's status word and sets its give-up flag; the next block
// barrier ORs the flags (__syncthreads_or) and the block leaves its loops without waiting again.
// The L2 variant is launched cooperatively so that all blocks of a group are resident together;
// clusters are co-scheduled by the hardware.
#include <cstdio>
#include <cstdlib>

#include "common.cuh"

namespace b2 {
namespace {

constexpr int NT = 256;
constexpr unsigned SPIN_LIMIT = 1u << 21;
typedef unsigned long long u64;

__device__ __forceinline__ void st_pair(u64 *p, float v, unsigned tag) {
    u64 x = ((u64)tag << 32) | (u64)__float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(x) : "memory");
}
__device__ __forceinline__ u64 ld_pair(const u64 *p) {
    u64 x;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(x) : "l"(p) : "memory");
    return x;
}
__device__ __forceinline__ int ld_status(const int *p) {
    int x;
    asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(x) : "l"(p) : "memory");
    return x;
}
// Gather COUNT tagged values (thread-strided) into v[].  Polling goes in ROUNDS: every round re-issues
// the loads of all values that have not shown the tag yet and only then examines them, so a round
// costs one L2 round trip no matter how many values a thread waits for.  Bounded: after SPIN_LIMIT
// rounds (about a second), or when another block has reported a timeout, the thread records
// B2_ERR_STEP_TIMEOUT, sets *gave_up and returns zeros.
template <int COUNT>
__device__ __forceinline__ void gather_pairs(float (&v)[(COUNT + NT - 1) / NT], const u64 *xb, unsigned tag, int tid,
                                             int *gave_up, int *status) {
    constexpr int NW = (COUNT + NT - 1) / NT;
    u64 x[NW];
#pragma unroll
    for (int q = 0; q < NW; ++q) x[q] = ~((u64)tag << 32);   // any word whose tag differs
    if (!*gave_up) {
        for (unsigned it = 0;; ++it) {
#pragma unroll
            for (int q = 0; q < NW; ++q) {
                const int i = tid + q * NT;
                if ((COUNT % NT == 0 || i < COUNT) && (unsigned)(x[q] >> 32) != tag) x[q] = ld_pair(xb + i);
            }
            bool all = true;
#pragma unroll
            for (int q = 0; q < NW; ++q) {
                const int i = tid + q * NT;
                if (COUNT % NT == 0 || i < COUNT) all = all && ((unsigned)(x[q] >> 32) == tag);
            }
            if (all) break;
            if (it >= SPIN_LIMIT || ((it & 1023u) == 1023u && ld_status(status) != 0)) {
                *gave_up = 1;
                atomicCAS(status, 0, (int)B2_ERR_STEP_TIMEOUT);
                break;
            }
        }
    }
#pragma unroll
    for (int q = 0; q < NW; ++q) v[q] = ((unsigned)(x[q] >> 32) == tag) ? __uint_as_float((unsigned)x[q]) : 0.0f;
}

// One block waits, with the sweeps' own gather, for a tag that nothing writes: the wait must run out, record
// B2_ERR_STEP_TIMEOUT and return (see lstm_selftest_bounded_wait).
__global__ void __launch_bounds__(NT) bounded_wait_selftest_kernel(const u64 *xb, int *status, float *out) {
    float v[1];
    int gave_up = 0;
    gather_pairs<NT>(v, xb, 0x5EEDu, (int)threadIdx.x, &gave_up, status);
    const int any = __syncthreads_or(gave_up);
    if (threadIdx.x == 0) out[0] = any ? 1.0f : 0.0f;
}

// ---- thread-block cluster exchange
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t map_to_rank(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}

// shared-memory barrier with transaction count: the peers of a cluster deliver h with st.async, which both
// writes the data into this block's shared memory and counts the bytes on this barrier
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
// bounded: false when the budget (about a second) ran out or another block reported a timeout
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, const int *status) {
    for (unsigned it = 0; it < SPIN_LIMIT; ++it) {
        if (mbar_try(bar, parity)) return true;
        if ((it & 1023u) == 1023u && ld_status(status) != 0) return false;
    }
    return false;
}
__device__ __forceinline__ void st_async_v4(uint32_t raddr, float4 v, uint32_t rbar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(raddr),
                 "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w), "r"(rbar)
                 : "memory");
}
__device__ __forceinline__ void st_async_f32(uint32_t raddr, float v, uint32_t rbar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.f32 [%0], %1, [%2];" ::"r"(raddr), "f"(v), "r"(rbar)
                 : "memory");
}

struct PersistArgs {
    LstmShape sh;
    LstmBuffers bf;
    const float *w;
    float *y;          // forward: block outputs (written); backward: unused
    const float *dy;   // backward: output errors (read)
    u64 *xchg;         // exchange buffers, per slot (L2 transport)
    int *status;       // 0 ok, else an error code
    unsigned tag_base;
    int n_items;       // D * ceil((p_hi - p_lo) / PS)
    int p_lo, p_hi;    // the sequences this launch handles: items cover p_lo .. p_hi-1 in slices of PS
};

template <int ELS, int JB, int PS>
struct Geo {
    static constexpr int R = 4 * JB;                 // gate rows owned by a block
    static constexpr int G = ELS / JB;               // blocks per group
    static constexpr int CELLS = JB * PS;            // (unit, sequence) cells owned by a block
    static constexpr int CPT = (CELLS + NT - 1) / NT;
    static constexpr int PC = PS < 8 ? PS : 8;       // sequences per accumulation pass (register budget)
    // forward: thread = (unit jj, k-split ks): weights W[4 gates of jj][ks*KPT .. +KPT)
    static constexpr int KSPLIT = NT / JB;
    static constexpr int KPT = ELS / KSPLIT;
    // backward: thread = (k-quad kq, row-split rs): weights W[rs*RPT .. +RPT)[4*kq .. +4)
    static constexpr int KQ = ELS / 4;
    static constexpr int RSPLIT = NT / KQ;
    static constexpr int RPT = R / RSPLIT;
    static constexpr int NPART = NT / CELLS >= 1 ? NT / CELLS : 1;   // threads per cell when summing partials
    static_assert(NT % JB == 0 && ELS % KSPLIT == 0 && ELS % JB == 0 && 4 * KPT <= 128, "bad forward geometry");
    static_assert(ELS % 4 == 0 && NT % KQ == 0 && R % RSPLIT == 0 && 4 * RPT <= 128, "bad backward geometry");
    static_assert(CELLS <= NT ? NT % CELLS == 0 : CELLS % NT == 0, "cells must tile the block");
    // dynamic shared memory, in floats
    static constexpr int FWD_HS = ELS * PS, FWD_RED = NT * 4 * PS;
    static constexpr int BWD_PE = ELS * PS, BWD_PE2 = NT, BWD_DS = R * PS, BWD_REDB = RSPLIT * ELS * PS;
    // forward: when the block owns few cells, the k-split partial sums are first combined by all threads
    static constexpr int NPARTF = (4 * CELLS < NT) ? NT / (4 * CELLS) : 1;
    static constexpr int FWD_RED2 = NPARTF > 1 ? NT : 4;
    static_assert(KSPLIT % NPARTF == 0, "k-splits must divide over the reduce parts");
    static constexpr size_t fwd_smem(bool cl) { return sizeof(float) * ((cl ? 2 : 1) * FWD_HS + FWD_RED + FWD_RED2); }
    static constexpr size_t bwd_smem(bool cl) { return sizeof(float) * ((cl ? 2 : 1) * BWD_PE + BWD_PE2 + BWD_DS + BWD_REDB); }
};

extern __shared__ __align__(16) float smem_dyn[];

// =================================================================================================
// forward
// =================================================================================================
template <int ELS, int JB, int PS, bool CL>
__global__ void __launch_bounds__(NT, 1) lstm_fwd_persistent_kernel(PersistArgs a) {
    typedef Geo<ELS, JB, PS> Gm;
    constexpr int G = Gm::G, CELLS = Gm::CELLS, CPT = Gm::CPT, KSPLIT = Gm::KSPLIT, KPT = Gm::KPT, PC = Gm::PC;
    // h[t-1] of the group's sequences, [k][p]; with clusters the peers write it directly, double-buffered
    float *hs_all = smem_dyn;
    // k-split partial sums of the gate pre-activations, [ks][gate][p][jj]
    float *red = smem_dyn + (CL ? 2 : 1) * Gm::FWD_HS;
    float *red2 = red + Gm::FWD_RED;   // [part][gate][p][jj], only when NPARTF > 1
    constexpr int NPARTF = Gm::NPARTF;
    int gave_up = 0;   // this thread ran out of its wait budget; combined block-wide by __syncthreads_or

    const int tid = threadIdx.x;
    const int g = blockIdx.x % G, slot = blockIdx.x / G, nslots = gridDim.x / G;
    const int jj_f = tid % JB, ks = tid / JB;
    const int j0 = g * JB;
    const int P = a.sh.P, T = a.sh.T, ls = a.sh.ls, D = a.sh.D;
    const LstmOffsets off = lstm_offsets(a.sh.pls, ls, ELS);
    u64 *xslot = a.xchg + (size_t)slot * 4 * ELS * PS;
    // cluster transport: one transaction barrier per h buffer, a staging row to send 4 sequences of a unit at once
    __shared__ __align__(8) unsigned long long hbar[2];
    __shared__ float hstage[CL ? CELLS : 1];
    unsigned hphase[2] = {0u, 0u};   // phases of each buffer's barrier this block has waited for
    if constexpr (CL) {
        if (tid == 0) {
            mbar_init(smem_addr(&hbar[0]), 1);
            mbar_init(smem_addr(&hbar[1]), 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
    }
    // a peer's shared memory (and barriers) may only be touched once that peer has started running
    if constexpr (CL) { cluster_arrive(); cluster_wait(); }

    float wreg[4][KPT];
    int cur_d = -1;
    for (int item = slot; item < a.n_items; item += nslots) {
        const int d = item % D, p0 = a.p_lo + (item / D) * PS, seq = item / nslots;
        if (d != cur_d) {
            // W_rec[gate][d][j0+jj][k] from the source-major copy [d][k][gate][j] (coalesced over j)
            const float *wt = a.bf.wrecT + (size_t)d * ELS * 4 * ELS;
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
                for (int kk = 0; kk < KPT; ++kk)
                    wreg[q][kk] = __ldg(wt + ((size_t)(ks * KPT + kk) * 4 + q) * ELS + j0 + jj_f);
            cur_d = d;
        }
        const unsigned tag0 = a.tag_base + (unsigned)seq * (unsigned)(T + 1);
        u64 *xitem = xslot + (size_t)(seq & 1) * 2 * ELS * PS;

        // per-cell constants and state
        float b4[CPT][4], pw[CPT][3], cprev[CPT];
#pragma unroll
        for (int ci = 0; ci < CPT; ++ci) {
            const int c = tid + ci * NT;
            const int u = d * ELS + j0 + (c % JB);
            cprev[ci] = 0.0f;
            if (c < CELLS) {
#pragma unroll
                for (int q = 0; q < 4; ++q) b4[ci][q] = a.sh.bias * __ldg(a.w + off.bias + (size_t)q * ls + u);
#pragma unroll
                for (int q = 0; q < 3; ++q) pw[ci][q] = __ldg(a.w + off.peep + (size_t)q * ls + u);
            }
        }

        bool dead = false;
        // pre-activations and padding flags are fetched ONE STEP AHEAD: they come from HBM (the projection of a
        // long fraction does not fit L2) and a step is shorter than that latency
        float a4n[CPT][4];
        int moden[CPT];  // 0 compute, 1 padding frame, 2 sequence slot beyond the launch's range
        // Padding frames (pattern type NONE) trail a sequence, as the data set writes them: the first one is
        // found once per item by bisection, so that the step loop does not wait on a pattern-type load
        int seqlen[CPT];
#pragma unroll
        for (int ci = 0; ci < CPT; ++ci) {
            const int c = tid + ci * NT;
            seqlen[ci] = T;
            if (c < CELLS && p0 + c / JB < a.p_hi && a.sh.Tmin < T) {
                const int pg = p0 + c / JB;
                int lo = a.sh.Tmin, hi = T;   // frames below Tmin are real for every sequence
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if (a.bf.pat[(size_t)mid * P + pg] == PAT_NONE) hi = mid; else lo = mid + 1;
                }
                seqlen[ci] = lo;
            }
        }
        auto fetch = [&](int sn) {
            const int tn = d ? T - 1 - sn : sn;
#pragma unroll
            for (int ci = 0; ci < CPT; ++ci) {
                const int c = tid + ci * NT;
                moden[ci] = 2;
                if (c < CELLS) {
                    const int pg = p0 + c / JB;
                    if (pg < a.p_hi) {
                        const size_t f = (size_t)tn * P + pg;
                        const float *ap = a.bf.acts + f * 4 * ls + d * ELS + j0 + (c % JB);
#pragma unroll
                        for (int q = 0; q < 4; ++q) a4n[ci][q] = ap[(size_t)q * ls];
                        moden[ci] = tn >= seqlen[ci] ? 1 : 0;
                    }
                }
            }
        };
        if (T > 0) fetch(0);
        for (int s = 0; s < T; ++s) {
            const int t = d ? T - 1 - s : s;
            const bool first = (s == 0);
            // 1. pre-activations of this step for the block's cells (independent of the recurrence)
            float a4[CPT][4];
            int mode[CPT];
#pragma unroll
            for (int ci = 0; ci < CPT; ++ci) {
                mode[ci] = moden[ci];
#pragma unroll
                for (int q = 0; q < 4; ++q) a4[ci][q] = a4n[ci][q];
            }
            if (s + 1 < T) fetch(s + 1);
            if constexpr (CL) {
                // this step's h of all G blocks will arrive in buffer s&1 (the last step publishes nothing)
                if (tid == 0 && s + 1 < T) mbar_expect_tx(smem_addr(&hbar[s & 1]), (uint32_t)(ELS * PS * sizeof(float)));
            }
            // 2. h[t-1] of the whole group, 3. recurrent projection with register-resident weights
            if (!first) {
                const float *hs = hs_all;
                if constexpr (CL) {
                    // every block of the cluster has delivered its h[t-1] into this block's buffer
                    const int b = (s - 1) & 1;
                    if (!mbar_wait_bounded(smem_addr(&hbar[b]), hphase[b] & 1u, a.status)) {
                        gave_up = 1;
                        atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT);
                    }
                    ++hphase[b];
                    hs = hs_all + b * ELS * PS;
                    const int dead_now = __syncthreads_or(gave_up);
                    if (dead_now) { dead = true; break; }
                } else {
                    const u64 *xb = xitem + (size_t)((s - 1) & 1) * ELS * PS;
                    float hv[(ELS * PS + NT - 1) / NT];
                    gather_pairs<ELS * PS>(hv, xb, tag0 + (unsigned)s, tid, &gave_up, a.status);
#pragma unroll
                    for (int q = 0; q < (ELS * PS + NT - 1) / NT; ++q) {
                        const int i = tid + q * NT;
                        if ((ELS * PS) % NT == 0 || i < ELS * PS) hs_all[(i % ELS) * PS + (i / ELS)] = hv[q];
                    }
                    const int dead_now = __syncthreads_or(gave_up);
                    if (dead_now) { dead = true; break; }
                }
#pragma unroll 1
                for (int pc0 = 0; pc0 < PS; pc0 += PC) {
                    float acc[4][PC];
#pragma unroll
                    for (int q = 0; q < 4; ++q)
#pragma unroll
                        for (int p = 0; p < PC; ++p) acc[q][p] = 0.0f;
#pragma unroll
                    for (int kk = 0; kk < KPT; ++kk) {
                        float hvv[PC];
                        const float *hp = hs + (ks * KPT + kk) * PS + pc0;
                        if constexpr (PC % 4 == 0) {
#pragma unroll
                            for (int p4 = 0; p4 < PC / 4; ++p4) {
                                const float4 h4 = reinterpret_cast<const float4 *>(hp)[p4];
                                hvv[4 * p4] = h4.x; hvv[(4 * p4 + 1) % PC] = h4.y;
                                hvv[(4 * p4 + 2) % PC] = h4.z; hvv[(4 * p4 + 3) % PC] = h4.w;
                            }
                        } else {
#pragma unroll
                            for (int p = 0; p < PC; ++p) hvv[p] = hp[p];
                        }
#pragma unroll
                        for (int q = 0; q < 4; ++q)
#pragma unroll
                            for (int p = 0; p < PC; ++p) acc[q][p] = fmaf(wreg[q][kk], hvv[p], acc[q][p]);
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q)
#pragma unroll
                        for (int p = 0; p < PC; ++p) red[((ks * 4 + q) * PS + pc0 + p) * JB + jj_f] = acc[q][p];
                }
                __syncthreads();
                if constexpr (NPARTF > 1) {
                    // 4*CELLS gate sums, NPARTF threads each: thread = (part, output o = (gate*PS + p)*JB + jj)
                    const int o = tid % (4 * CELLS), part = tid / (4 * CELLS);
                    float sum = 0.0f;
#pragma unroll
                    for (int k2 = 0; k2 < KSPLIT / NPARTF; ++k2) sum += red[(part * (KSPLIT / NPARTF) + k2) * 4 * CELLS + o];
                    red2[part * 4 * CELLS + o] = sum;
                    __syncthreads();
                }
            }
            // 4. gate math, state update, publish h[t]
            u64 *xo = xitem + (size_t)(s & 1) * ELS * PS;
#pragma unroll
            for (int ci = 0; ci < CPT; ++ci) {
                const int c = tid + ci * NT;
                if (c >= CELLS) continue;
                const int p = c / JB, jj = c % JB;
                float h = 0.0f, ni = 0.0f, ig = 0.0f, fg = 0.0f, og = 0.0f, cs = 0.0f;
                if (mode[ci] == 1) {
                    cprev[ci] = 0.0f;
                } else if (mode[ci] == 0) {
                    float rec[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    if (!first) {
                        if constexpr (NPARTF > 1) {
#pragma unroll
                            for (int q = 0; q < 4; ++q)
#pragma unroll
                                for (int k2 = 0; k2 < NPARTF; ++k2) rec[q] += red2[k2 * 4 * CELLS + (q * PS + p) * JB + jj];
                        } else {
#pragma unroll
                            for (int q = 0; q < 4; ++q)
#pragma unroll 8
                                for (int k2 = 0; k2 < KSPLIT; ++k2) rec[q] += red[((k2 * 4 + q) * PS + p) * JB + jj];
                        }
                    }
                    ni = a4[ci][0] + rec[0] + b4[ci][0];
                    ig = a4[ci][1] + rec[1] + b4[ci][1];
                    fg = a4[ci][2] + rec[2] + b4[ci][2];
                    og = a4[ci][3] + rec[3] + b4[ci][3];
                    const float cp = cprev[ci];
                    if (!first) { ig += cp * pw[ci][0]; fg += cp * pw[ci][1]; }
                    ni = act_tanh(ni); ig = act_logistic(ig); fg = act_logistic(fg);
                    cs = ni * ig;
                    if (!first) cs += cp * fg;
                    og = act_logistic(og + cs * pw[ci][2]);
                    h = act_tanh(cs) * og;
                    cprev[ci] = cs;
                }
                if constexpr (CL) {
                    hstage[jj * PS + p] = h;
                } else {
                    st_pair(xo + (size_t)p * ELS + j0 + jj, h, tag0 + (unsigned)s + 1u);
                }
                // the peers are waiting for h: the layer's own state goes to memory after it is on its way
                if (mode[ci] != 2) {
                    const size_t f = (size_t)t * P + (p0 + p);
                    const int u = d * ELS + j0 + jj;
                    float *ap = a.bf.acts + f * 4 * ls + u;
                    ap[0] = ni; ap[ls] = ig; ap[2 * (size_t)ls] = fg; ap[3 * (size_t)ls] = og;   // zeros on padding frames
                    a.bf.cells[f * ls + u] = cs;
                    a.y[f * ls + u] = h;
                }
            }
            if constexpr (CL) {
                // thread (unit u, peer r) sends the PS sequences of unit u to block r of the cluster
                __syncthreads();
                if (s + 1 < T) {
                    for (int idx = tid; idx < JB * G; idx += NT) {
                        const int u = idx % JB, r = idx / JB;
                        const uint32_t rbar = map_to_rank(smem_addr(&hbar[s & 1]), (uint32_t)r);
                        const uint32_t la = smem_addr(hs_all + (s & 1) * ELS * PS + (j0 + u) * PS);
                        if constexpr (PS % 4 == 0) {
#pragma unroll
                            for (int p4 = 0; p4 < PS / 4; ++p4)
                                st_async_v4(map_to_rank(la + 16u * p4, (uint32_t)r),
                                            *reinterpret_cast<const float4 *>(hstage + u * PS + 4 * p4), rbar);
                        } else {
#pragma unroll
                            for (int p = 0; p < PS; ++p) st_async_f32(map_to_rank(la + 4u * p, (uint32_t)r), hstage[u * PS + p], rbar);
                        }
                    }
                }
            }
        }
        // nobody may overwrite a buffer (or leave the kernel) while a peer still reads or writes it
        if constexpr (CL) { cluster_arrive(); cluster_wait(); }
        if (dead) break;
    }
}

// =================================================================================================
// backward
// =================================================================================================
template <int ELS, int JB, int PS, bool CL>
__global__ void __launch_bounds__(NT, 1) lstm_bwd_persistent_kernel(PersistArgs a) {
    typedef Geo<ELS, JB, PS> Gm;
    constexpr int G = Gm::G, CELLS = Gm::CELLS, CPT = Gm::CPT, PC = Gm::PC;
    constexpr int KQ = Gm::KQ, RSPLIT = Gm::RSPLIT, RPT = Gm::RPT, NPART = Gm::NPART;
    constexpr int SRC_PER_PART = (G + NPART - 1) / NPART;
    // cluster transport with one thread per unit: the PS partial sums of a unit travel as 16-byte stores, the
    // receive buffers then hold [src][unit][sequence] instead of [src][sequence][unit]
    constexpr bool VEC = CL && ELS == NT && PS % 4 == 0;
    // partial sums received, [src][cell]; with clusters the peers write them directly, double-buffered
    float *pe_all = smem_dyn;
    float *pe2 = pe_all + (CL ? 2 : 1) * Gm::BWD_PE;   // first-stage sums, [part][cell]
    float *ds = pe2 + Gm::BWD_PE2;                      // this step's gate deltas, [row][p]
    float *redb = ds + Gm::BWD_DS;                      // row-split partial sums, [rs][p][k]
    int gave_up = 0;

    const int tid = threadIdx.x;
    const int g = blockIdx.x % G, slot = blockIdx.x / G, nslots = gridDim.x / G;
    const int j0 = g * JB;
    const int P = a.sh.P, T = a.sh.T, ls = a.sh.ls, D = a.sh.D;
    const LstmOffsets off = lstm_offsets(a.sh.pls, ls, ELS);
    // one exchange buffer holds, per owner block, G source blocks x CELLS tagged partial sums
    constexpr size_t XBUF = (size_t)G * G * CELLS;
    u64 *xslot = a.xchg + (size_t)slot * 4 * XBUF;
    const int kq = tid % KQ, rs = tid / KQ;
    // cluster transport: one transaction barrier per receive buffer (see the forward kernel)
    __shared__ __align__(8) unsigned long long ebar[2];
    unsigned ephase[2] = {0u, 0u};
    if constexpr (CL) {
        if (tid == 0) {
            mbar_init(smem_addr(&ebar[0]), 1);
            mbar_init(smem_addr(&ebar[1]), 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
    }
    // a peer's shared memory (and barriers) may only be touched once that peer has started running
    if constexpr (CL) { cluster_arrive(); cluster_wait(); }

    float wreg[4][RPT];
    int cur_d = -1;
    for (int item = slot; item < a.n_items; item += nslots) {
        const int d = item % D, p0 = a.p_lo + (item / D) * PS, seq = item / nslots;
        if (d != cur_d) {
            // W_rec[gate][d][j0+jj][k], row = gate*JB + jj, this thread's columns k = 4*kq .. 4*kq+3
#pragma unroll
            for (int rr = 0; rr < RPT; ++rr) {
                const int row = rs * RPT + rr;
                const float *wp = a.w + off.rec + ((size_t)(row / JB) * ls + (size_t)d * ELS + j0 + (row % JB)) * ELS + 4 * kq;
#pragma unroll
                for (int c = 0; c < 4; ++c) wreg[c][rr] = __ldg(wp + c);
            }
            cur_d = d;
        }
        const unsigned tag0 = a.tag_base + (unsigned)seq * (unsigned)(T + 1);
        u64 *xitem = xslot + (size_t)(seq & 1) * 2 * XBUF;

        float pw[CPT][3];
        float st_ce[CPT], st_dig[CPT], st_dfg[CPT], st_fg[CPT], c_keep[CPT];  // values of the step before
#pragma unroll
        for (int ci = 0; ci < CPT; ++ci) {
            const int c = tid + ci * NT;
            st_ce[ci] = st_dig[ci] = st_dfg[ci] = st_fg[ci] = c_keep[ci] = 0.0f;
            if (c < CELLS) {
                const int u = d * ELS + j0 + (c % JB);
#pragma unroll
                for (int q = 0; q < 3; ++q) pw[ci][q] = __ldg(a.w + off.peep + (size_t)q * ls + u);
            }
        }

        bool dead = false;
        // the first padding frame of each of this thread's sequences (see the forward kernel)
        int seqlen[CPT];
#pragma unroll
        for (int ci = 0; ci < CPT; ++ci) {
            const int c = tid + ci * NT;
            seqlen[ci] = T;
            if (c < CELLS && p0 + c / JB < a.p_hi && a.sh.Tmin < T) {
                const int pg = p0 + c / JB;
                int lo = a.sh.Tmin, hi = T;
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if (a.bf.pat[(size_t)mid * P + pg] == PAT_NONE) hi = mid; else lo = mid + 1;
                }
                seqlen[ci] = lo;
            }
        }
        // everything a step needs from HBM is independent of the recurrence and is fetched one step ahead
        float e_n[CPT], a4n[CPT][4], cpvn[CPT], cc_first[CPT];
        int moden[CPT];
        auto fetch = [&](int sn) {
            const int tn = d ? sn : T - 1 - sn;
            const int prevn = d ? tn + 1 : tn - 1;
#pragma unroll
            for (int ci = 0; ci < CPT; ++ci) {
                const int c = tid + ci * NT;
                moden[ci] = 2;
                cpvn[ci] = 0.0f;
                if (c < CELLS) {
                    const int pg = p0 + c / JB;
                    if (pg < a.p_hi) {
                        const size_t f = (size_t)tn * P + pg;
                        const int u = d * ELS + j0 + (c % JB);
                        moden[ci] = tn >= seqlen[ci] ? 1 : 0;
                        e_n[ci] = a.dy[f * ls + u];
                        const float *ap = a.bf.acts + f * 4 * ls + u;
#pragma unroll
                        for (int q = 0; q < 4; ++q) a4n[ci][q] = ap[(size_t)q * ls];
                        if (sn == 0) cc_first[ci] = a.bf.cells[f * ls + u];
                        if (sn != T - 1) cpvn[ci] = a.bf.cells[((size_t)prevn * P + pg) * ls + u];
                    }
                }
            }
        };
        if (T > 0) fetch(0);
        for (int s = 0; s < T; ++s) {
            const int t = d ? s : T - 1 - s;
            const bool firstCall = (s == 0), lastCall = (s == T - 1);
            // 1. this step's inputs (fetched during the step before), then the next step's fetch
            float e_in[CPT], a4[CPT][4], cc[CPT], cpv[CPT];
            int mode[CPT];
#pragma unroll
            for (int ci = 0; ci < CPT; ++ci) {
                mode[ci] = moden[ci];
                e_in[ci] = e_n[ci];
                cpv[ci] = cpvn[ci];
                cc[ci] = firstCall ? cc_first[ci] : c_keep[ci];
#pragma unroll
                for (int q = 0; q < 4; ++q) a4[ci][q] = a4n[ci][q];
            }
            if (s + 1 < T) fetch(s + 1);
            if constexpr (CL) {
                // this step's partial sums of all G blocks will arrive in buffer s&1 (the last step sends nothing)
                if (tid == 0 && !lastCall) mbar_expect_tx(smem_addr(&ebar[s & 1]), (uint32_t)(G * CELLS * sizeof(float)));
            }
            // 2. partial sums of the recurrent error from every block of the group
            const float *pe = pe_all;
            if (!firstCall) {
                if constexpr (CL) {
                    // every block of the cluster has delivered its partial sums into this block's buffer
                    const int b = (s - 1) & 1;
                    if (!mbar_wait_bounded(smem_addr(&ebar[b]), ephase[b] & 1u, a.status)) {
                        gave_up = 1;
                        atomicCAS(a.status, 0, (int)B2_ERR_STEP_TIMEOUT);
                    }
                    ++ephase[b];
                    pe = pe_all + b * G * CELLS;
                    const int dead_now = __syncthreads_or(gave_up);
                    if (dead_now) { dead = true; break; }
                } else {
                    const u64 *xb = xitem + (size_t)((s - 1) & 1) * XBUF + (size_t)g * G * CELLS;
                    float pv[(G * CELLS + NT - 1) / NT];
                    gather_pairs<G * CELLS>(pv, xb, tag0 + (unsigned)s, tid, &gave_up, a.status);
#pragma unroll
                    for (int q = 0; q < (G * CELLS + NT - 1) / NT; ++q) {
                        const int i = tid + q * NT;
                        if ((G * CELLS) % NT == 0 || i < G * CELLS) pe_all[i] = pv[q];
                    }
                    const int dead_now = __syncthreads_or(gave_up);
                    if (dead_now) { dead = true; break; }
                }
                if constexpr (CELLS <= NT) {
                    const int c = tid % CELLS, part = tid / CELLS;
                    float sum = 0.0f;
#pragma unroll 4
                    for (int q = 0; q < SRC_PER_PART; ++q) {
                        const int src = part * SRC_PER_PART + q;
                        if (src < G) sum += pe[src * CELLS + c];
                    }
                    pe2[part * CELLS + c] = sum;
                    __syncthreads();
                }
            }
            // 3. cell errors and gate deltas (ComputeBlockErrorsFn)
            float dd[CPT][4];
            // the deltas go to memory after the partial sums the peers wait for have been sent
            auto store_deltas = [&]() {
#pragma unroll
                for (int ci = 0; ci < CPT; ++ci) {
                    const int c = tid + ci * NT;
                    if (c >= CELLS || mode[ci] == 2) continue;
                    const size_t f = (size_t)t * P + (p0 + c / JB);
                    float *dl = a.bf.deltas + f * 4 * ls + d * ELS + j0 + (c % JB);
                    dl[0] = dd[ci][0]; dl[ls] = dd[ci][1]; dl[2 * (size_t)ls] = dd[ci][2]; dl[3 * (size_t)ls] = dd[ci][3];
                }
            };
#pragma unroll
            for (int ci = 0; ci < CPT; ++ci) {
                const int c = tid + ci * NT;
                if (c >= CELLS) continue;
                const int p = c / JB, jj = c % JB;
                float dni = 0.0f, dig = 0.0f, dfg = 0.0f, dog = 0.0f, ce = 0.0f;
                if (mode[ci] == 0) {
                    float e = e_in[ci];
                    if (!firstCall) {
                        if constexpr (CELLS <= NT) {
#pragma unroll
                            for (int q = 0; q < NPART; ++q) e += pe2[q * CELLS + (VEC ? jj * PS + p : c)];
                        } else {
                            for (int src = 0; src < G; ++src) e += pe[src * CELLS + (VEC ? jj * PS + p : c)];
                        }
                    }
                    const float ni = a4[ci][0], ig = a4[ci][1], fg = a4[ci][2], og = a4[ci][3];
                    const float tc = act_tanh(cc[ci]);
                    dog = d_logistic(og) * tc * e;
                    ce = og * d_tanh(tc) * e + pw[ci][2] * dog;
                    if (!firstCall) ce += st_fg[ci] * st_ce[ci] + pw[ci][0] * st_dig[ci] + pw[ci][1] * st_dfg[ci];
                    dni = ig * d_tanh(ni) * ce;
                    if (!lastCall) dfg = d_logistic(fg) * cpv[ci] * ce;
                    dig = d_logistic(ig) * ni * ce;
                    dni = limited_error(dni); dig = limited_error(dig);
                    dfg = limited_error(dfg); dog = limited_error(dog);
                    st_fg[ci] = fg;
                } else {
                    st_fg[ci] = 0.0f;
                }
                st_ce[ci] = ce; st_dig[ci] = dig; st_dfg[ci] = dfg;
                c_keep[ci] = cpv[ci];   // c[prevc] is the next step's own cell state
                dd[ci][0] = dni; dd[ci][1] = dig; dd[ci][2] = dfg; dd[ci][3] = dog;
                ds[(0 * JB + jj) * PS + p] = dni;
                ds[(1 * JB + jj) * PS + p] = dig;
                ds[(2 * JB + jj) * PS + p] = dfg;
                ds[(3 * JB + jj) * PS + p] = dog;
            }
            if (lastCall) { store_deltas(); break; }
            __syncthreads();
            // 4. this block's contribution to the output error of every unit k at the next step
            u64 *xo = xitem + (size_t)(s & 1) * XBUF;
            const unsigned tag = tag0 + (unsigned)s + 1u;
            // where partial (k, p) of this source block goes: into the owner's [src][cell] buffer
            auto send = [&](int k, int p, float v) {
                const int cell = p * JB + (k % JB);
                if constexpr (CL)
                    st_async_f32(map_to_rank(smem_addr(pe_all + ((s & 1) * G + g) * CELLS + cell), (uint32_t)(k / JB)), v,
                                 map_to_rank(smem_addr(&ebar[s & 1]), (uint32_t)(k / JB)));
                else
                    st_pair(xo + ((size_t)(k / JB) * G + g) * CELLS + cell, v, tag);
            };
#pragma unroll 1
            for (int pc0 = 0; pc0 < PS; pc0 += PC) {
                float acc[4][PC];
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int p = 0; p < PC; ++p) acc[c][p] = 0.0f;
#pragma unroll
                for (int rr = 0; rr < RPT; ++rr) {
                    float dv[PC];
                    const float *dp = ds + (rs * RPT + rr) * PS + pc0;
                    if constexpr (PC % 4 == 0) {
#pragma unroll
                        for (int p4 = 0; p4 < PC / 4; ++p4) {
                            const float4 v4 = reinterpret_cast<const float4 *>(dp)[p4];
                            dv[4 * p4] = v4.x; dv[(4 * p4 + 1) % PC] = v4.y;
                            dv[(4 * p4 + 2) % PC] = v4.z; dv[(4 * p4 + 3) % PC] = v4.w;
                        }
                    } else {
#pragma unroll
                        for (int p = 0; p < PC; ++p) dv[p] = dp[p];
                    }
#pragma unroll
                    for (int c = 0; c < 4; ++c)
#pragma unroll
                        for (int p = 0; p < PC; ++p) acc[c][p] = fmaf(wreg[c][rr], dv[p], acc[c][p]);
                }
#pragma unroll
                for (int p = 0; p < PC; ++p)
                    *reinterpret_cast<float4 *>(redb + ((size_t)(rs * PS + pc0 + p) * ELS + 4 * kq)) =
                        make_float4(acc[0][p], acc[1][p], acc[2][p], acc[3][p]);
            }
            // combine the row-splits and send with consecutive threads on consecutive units (coalesced)
            __syncthreads();
            if constexpr (VEC) {
                // thread = unit k; its PS sums go to the owner of k in 16-byte pieces
                float v[PS];
#pragma unroll
                for (int p = 0; p < PS; ++p) {
                    v[p] = 0.0f;
#pragma unroll
                    for (int q = 0; q < RSPLIT; ++q) v[p] += redb[(size_t)(q * PS + p) * ELS + tid];
                }
                const uint32_t owner = (uint32_t)(tid / JB);
                const uint32_t rbar = map_to_rank(smem_addr(&ebar[s & 1]), owner);
                const uint32_t la = smem_addr(pe_all + ((s & 1) * G + g) * CELLS + (tid % JB) * PS);
#pragma unroll
                for (int p4 = 0; p4 < PS / 4; ++p4)
                    st_async_v4(map_to_rank(la + 16u * p4, owner), make_float4(v[4 * p4], v[4 * p4 + 1], v[4 * p4 + 2], v[4 * p4 + 3]), rbar);
            } else {
#pragma unroll
                for (int q0 = 0; q0 < (ELS * PS + NT - 1) / NT; ++q0) {
                    const int i = tid + q0 * NT;
                    if ((ELS * PS) % NT != 0 && i >= ELS * PS) break;
                    const int k = i % ELS, p = i / ELS;
                    float v = 0.0f;
#pragma unroll
                    for (int q = 0; q < RSPLIT; ++q) v += redb[(size_t)(q * PS + p) * ELS + k];
                    send(k, p, v);
                }
            }
            store_deltas();
        }
        // item boundary: nobody may overwrite a buffer (or leave the kernel) while a peer still reads it
        if constexpr (CL) { cluster_arrive(); cluster_wait(); }
        if (dead) break;
    }
}

// ---- host side ----------------------------------------------------------------------------------
int num_sms() { return sm_count(); }

template <int ELS, int JB, int PS, bool CL>
int prepare_kernel(bool backward, void (**kern)(PersistArgs), size_t *smem) {
    typedef Geo<ELS, JB, PS> Gm;
    *kern = backward ? lstm_bwd_persistent_kernel<ELS, JB, PS, CL> : lstm_fwd_persistent_kernel<ELS, JB, PS, CL>;
    *smem = backward ? Gm::bwd_smem(CL) : Gm::fwd_smem(CL);
    return set_max_dynamic_smem((const void *)*kern, (int)*smem);
}

inline void cluster_config(cudaLaunchConfig_t *cfg, cudaLaunchAttribute *attr, int G, int blocks, size_t smem, cudaStream_t st) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = G;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    *cfg = cudaLaunchConfig_t{};
    cfg->gridDim = dim3(blocks);
    cfg->blockDim = dim3(NT);
    cfg->dynamicSmemBytes = smem;
    cfg->stream = st;
    cfg->attrs = attr;
    cfg->numAttrs = 1;
}

// groups of at most 8 blocks run as thread-block clusters (distributed shared memory exchange)
template <int ELS, int JB, int PS>
int launch_cluster(bool backward, PersistArgs &a, cudaStream_t st, int *items_per_slot) {
    typedef Geo<ELS, JB, PS> Gm;
    if constexpr (Gm::G > 8) {
        return 1;
    } else {
        void (*kern)(PersistArgs);
        size_t smem;
        B2_TRY((prepare_kernel<ELS, JB, PS, true>(backward, &kern, &smem)));
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attr[1];
        cluster_config(&cfg, attr, Gm::G, Gm::G, smem, st);
        int max_clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg) != cudaSuccess || max_clusters < 1) {
            cudaGetLastError();
            return 1;   // no room for a cluster of this size: the caller uses the L2 exchange
        }
        int nslots = max_clusters < a.n_items ? max_clusters : a.n_items;
        *items_per_slot = (a.n_items + nslots - 1) / nslots;
        cfg.gridDim = dim3(nslots * Gm::G);
        B2_CUDA(cudaLaunchKernelEx(&cfg, kern, a));
        count_launch();
        return B2_OK;
    }
}

template <int ELS, int JB, int PS>
int launch(bool backward, bool use_cluster, PersistArgs &a, cudaStream_t st, int *items_per_slot) {
    typedef Geo<ELS, JB, PS> Gm;
    if (use_cluster) {
        int rc = launch_cluster<ELS, JB, PS>(backward, a, st, items_per_slot);
        if (rc != 1) return rc;
    }
    void (*kern)(PersistArgs);
    size_t smem;
    B2_TRY((prepare_kernel<ELS, JB, PS, false>(backward, &kern, &smem)));
    int per_sm = 0;
    B2_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, NT, smem));
    int resident = per_sm * num_sms();
    int nslots = resident / Gm::G;
    if (nslots < 1) return 1;   // the group does not fit on the device together: caller falls back
    if (nslots > a.n_items) nslots = a.n_items;
    *items_per_slot = (a.n_items + nslots - 1) / nslots;
    void *args[] = {&a};
    B2_CUDA(cudaLaunchCooperativeKernel((const void *)kern, dim3(nslots * Gm::G), dim3(NT), args, smem, st));
    count_launch();
    return B2_OK;
}

// how many clusters of G blocks of the (forward, 4 sequences) kernel the device can hold at once
template <int ELS, int JB>
int query_cluster_slots() {
    typedef Geo<ELS, JB, 4> Gm;
    void (*kern)(PersistArgs);
    size_t smem;
    if (prepare_kernel<ELS, JB, 4, true>(false, &kern, &smem) != B2_OK) return 0;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cluster_config(&cfg, attr, Gm::G, Gm::G, smem, nullptr);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
    return n;
}

}  // namespace

// hidden units per block for the register-resident geometry of `els` units per direction
bool persistent_geometry(int els, int *JB) {
    switch (els) {
        case 1024: *JB = 8; return true;
        case 512: *JB = 16; return true;
        case 256: *JB = 32; return true;
        case 128: *JB = 64; return true;
        default: return false;
    }
}

// 0 when groups of this size do not run as clusters
int persistent_cluster_slots(int els) {
    static int s256[MAX_DEVICES], s128[MAX_DEVICES];   // per device ordinal; 0 = not asked yet, else slots + 1
    const int dev = current_device();
    if (dev < 0) return 0;
    if (els == 256) { if (!s256[dev]) s256[dev] = query_cluster_slots<256, 32>() + 1; return s256[dev] - 1; }
    if (els == 128) { if (!s128[dev]) s128[dev] = query_cluster_slots<128, 64>() + 1; return s128[dev] - 1; }
    return 0;
}

// Sequences per work item.  More sequences per item amortise the per-step exchange latency over more
// work; fewer items than group slots leave SMs idle.  Take the smallest PS that lets every item have a
// slot of its own, else the largest the register budget of the geometry allows.
int persistent_ps(int els, int P, int D, bool use_cluster) {
    int JB;
    if (!persistent_geometry(els, &JB)) return 0;
    if (P == 1) return 1;
    const int G = els / JB;
    int slots = num_sms() / G;
    if (use_cluster && persistent_cluster_slots(els) > 0) slots = persistent_cluster_slots(els);
    if (slots < 1) slots = 1;
    const int max_ps = els >= 1024 ? 8 : 16;
    for (int ps = 4; ps <= max_ps; ps *= 2)
        if (D * ((P + ps - 1) / ps) <= slots) return ps;
    return max_ps;
}

size_t lstm_persistent_xchg_words(int els, int P, int D) {
    int JB;
    if (!persistent_geometry(els, &JB)) return 0;
    int PS = persistent_ps(els, P, D, false);
    if (persistent_ps(els, P, D, true) > PS) PS = persistent_ps(els, P, D, true);
    const int G = els / JB;
    int max_slots = num_sms() / G;
    if (max_slots < 1) max_slots = 1;
    size_t fwd = (size_t)4 * els * PS, bwd = (size_t)4 * G * G * JB * PS;
    return (size_t)max_slots * (fwd > bwd ? fwd : bwd);
}

// Runs the bounded wait of the sweeps on a word whose tag never arrives.  *status_out receives what the
// kernel recorded (B2_ERR_STEP_TIMEOUT expected), *gave_up whether the block left through the timeout
// path.  Takes about as long as the wait budget (a second or two); the context stays usable.
int lstm_selftest_bounded_wait(int *status_out, int *gave_up, cudaStream_t st) {
    u64 *xb = nullptr;
    int *status = nullptr;
    float *out = nullptr;
    B2_CUDA(cudaMalloc(&xb, NT * sizeof(u64)));
    B2_CUDA(cudaMalloc(&status, sizeof(int)));
    B2_CUDA(cudaMalloc(&out, sizeof(float)));
    B2_CUDA(cudaMemsetAsync(xb, 0, NT * sizeof(u64), st));
    B2_CUDA(cudaMemsetAsync(status, 0, sizeof(int), st));
    B2_CUDA(cudaMemsetAsync(out, 0, sizeof(float), st));
    bounded_wait_selftest_kernel<<<1, NT, 0, st>>>(xb, status, out);
    count_launch();
    int hs = 0;
    float ho = 0.0f;
    cudaError_t e = cudaMemcpyAsync(&hs, status, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(&ho, out, sizeof(float), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    cudaFree(xb); cudaFree(status); cudaFree(out);
    B2_CUDA(e);
    if (status_out) *status_out = hs;
    if (gave_up) *gave_up = ho != 0.0f ? 1 : 0;
    return B2_OK;
}

namespace {
// one launch over the sequences p_lo .. p_hi-1 with PS sequences per work item
int run_part(bool backward, bool use_cluster, PersistArgs a, int els, int PS, int p_lo, int p_hi, cudaStream_t st, int *ips) {
    a.p_lo = p_lo; a.p_hi = p_hi;
    a.n_items = a.sh.D * ((p_hi - p_lo + PS - 1) / PS);
    int rc = 1;
#define CASE_PS(E, J, Q) \
    case Q: rc = launch<E, J, Q>(backward, use_cluster, a, st, ips); break;
#define CASE(E, J, MORE)                                         \
    case E:                                                      \
        switch (PS) {                                            \
            CASE_PS(E, J, 1) CASE_PS(E, J, 4) CASE_PS(E, J, 8) MORE \
            default: return 1;                                   \
        }                                                        \
        break;
    switch (els) {
        CASE(1024, 8, )
        CASE(512, 16, CASE_PS(512, 16, 16))
        CASE(256, 32, CASE_PS(256, 32, 2) CASE_PS(256, 32, 16))
        CASE(128, 64, CASE_PS(128, 64, 2) CASE_PS(128, 64, 16))
        default: return 1;
    }
#undef CASE
#undef CASE_PS
    return rc;
}

// second stream for the part of a sweep that runs beside the cluster launch; one per host thread and device,
// so that handles driven from different threads (or living on different devices) do not share the fork / join
// events
struct AuxStream { cudaStream_t stream = nullptr; cudaEvent_t fork = nullptr, join = nullptr; };
thread_local AuxStream g_aux[MAX_DEVICES];
int ensure_aux(AuxStream **out) {
    const int dev = current_device();
    if (dev < 0) { set_error("no current CUDA device"); return B2_ERR_CUDA; }
    AuxStream &a = g_aux[dev];
    if (!a.stream) {
        B2_CUDA(cudaStreamCreateWithFlags(&a.stream, cudaStreamNonBlocking));
        B2_CUDA(cudaEventCreateWithFlags(&a.fork, cudaEventDisableTiming));
        B2_CUDA(cudaEventCreateWithFlags(&a.join, cudaEventDisableTiming));
    }
    *out = &a;
    return B2_OK;
}
}  // namespace

// How a sweep is laid out (measured per-step costs on B200: exchange through L2 1.4 us + 0.27 us per
// sequence of an item; through the cluster's shared memory 0.8 us + 0.29 us per sequence, but only as many
// groups run as clusters as fit side by side):
//   L2:      every item through L2, PS as persistent_ps picks it
//   CLUSTER: every item as a cluster
//   MIXED:   as many 4-sequence items as there are cluster slots run as clusters; the remaining sequences
//            run beside them, on the SMs the clusters leave free, as 2- or 4-sequence items through L2
struct SweepPlan { int kind; int ps_main; int split; int ps_rest; };
enum { PLAN_L2 = 0, PLAN_CLUSTER = 1, PLAN_MIXED = 2 };
static SweepPlan plan_sweep(int els, int P, int D, int transport) {
    SweepPlan pl{PLAN_L2, persistent_ps(els, P, D, false), P, 0};
    int JB;
    if (!persistent_geometry(els, &JB)) return pl;
    const int G = els / JB;
    const int C = G <= 8 ? persistent_cluster_slots(els) : 0;
    if (transport == 0 || C < 1) return pl;
    if (transport == 1) {   // clusters for everything (more than one pass if they do not fit)
        pl.kind = PLAN_CLUSTER;
        pl.ps_main = persistent_ps(els, P, D, true);
        return pl;
    }
    if (P == 1) return pl;
    const int slots = num_sms() / G > 0 ? num_sms() / G : 1;
    const int items_l2 = D * ((P + pl.ps_main - 1) / pl.ps_main);
    double best = ((items_l2 + slots - 1) / slots) * (1.4 + 0.27 * pl.ps_main);
    for (int ps = 4; ps <= 16; ps *= 2)
        if (D * ((P + ps - 1) / ps) <= C) {
            const double t = 0.8 + 0.29 * ps;
            if (t < best) { best = t; pl = SweepPlan{PLAN_CLUSTER, ps, P, 0}; }
            break;
        }
    const int slices = C / D;                       // 4-sequence cluster items per direction
    const int rest = P - 4 * slices;
    if (slices >= 1 && rest > 0) {
        const int free_sms = num_sms() - slices * D * G;
        for (int pr = 2; pr <= 4; pr *= 2)
            if (D * ((rest + pr - 1) / pr) * G <= free_sms) {
                const double t = (0.8 + 0.29 * 4 > 1.4 + 0.27 * pr) ? 0.8 + 0.29 * 4 : 1.4 + 0.27 * pr;
                if (t < best) { best = t; pl = SweepPlan{PLAN_MIXED, 4, 4 * slices, pr}; }
                break;
            }
    }
    return pl;
}

// returns B2_OK, an error, or 1 when this shape has no persistent kernel (caller uses the stepwise one).
// transport: 0 exchange through L2, 1 thread-block clusters, 2 whichever layout the cost model prefers
int lstm_persistent(bool backward, int transport, const LstmShape &s, const LstmBuffers &b, const float *w, float *y,
                    const float *dy, unsigned long long *xchg, int *status, unsigned *tag_next, cudaStream_t st) {
    int JB;
    if (!persistent_geometry(s.els, &JB) || !xchg) return 1;
    PersistArgs a;
    a.sh = s; a.bf = b; a.w = w; a.y = y; a.dy = dy; a.xchg = xchg; a.status = status;
    a.tag_base = *tag_next;
    const SweepPlan pl = plan_sweep(s.els, s.P, s.D, transport);
    int ips = 1, rc;
    if (pl.kind == PLAN_MIXED) {
        AuxStream *aux = nullptr;
        B2_TRY(ensure_aux(&aux));
        B2_CUDA(cudaEventRecord(aux->fork, st));
        B2_CUDA(cudaStreamWaitEvent(aux->stream, aux->fork, 0));
        int ips_cl = 1;
        rc = run_part(backward, true, a, s.els, pl.ps_main, 0, pl.split, st, &ips_cl);
        if (rc != B2_OK) return rc;
        rc = run_part(backward, false, a, s.els, pl.ps_rest, pl.split, s.P, aux->stream, &ips);
        B2_CUDA(cudaEventRecord(aux->join, aux->stream));
        B2_CUDA(cudaStreamWaitEvent(st, aux->join, 0));
    } else {
        rc = run_part(backward, pl.kind == PLAN_CLUSTER, a, s.els, pl.ps_main, 0, s.P, st, &ips);
    }
    if (rc == B2_OK) *tag_next += (unsigned)ips * (unsigned)(s.T + 1) + 1u;
    return rc;
}

}  // namespace b2
