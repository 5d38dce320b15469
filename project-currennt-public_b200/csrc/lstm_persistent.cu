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
// Exchange through L2 with the flag inside the datum: a value travels as one naturally aligned
// 64-bit word {step tag : float bits}, written with st.relaxed.gpu and polled with
// ld.relaxed.gpu, so one L2 round trip delivers both "ready" and the value; no fence, no atomics.
// Buffers are double-buffered over the step parity and over the item parity.
//
// Every wait is bounded: after SPIN_LIMIT polls (about a second) the thread records
// B2_ERR_STEP_TIMEOUT in the layer's status word and sets its give-up flag; the next block barrier
// ORs the flags (__syncthreads_or) and the block leaves its loops without waiting again.  The host
// launches cooperatively so that all blocks of a group are resident together.
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

struct PersistArgs {
    LstmShape sh;
    LstmBuffers bf;
    const float *w;
    float *y;          // forward: block outputs (written); backward: unused
    const float *dy;   // backward: output errors (read)
    u64 *xchg;         // exchange buffers, per slot
    int *status;       // 0 ok, else an error code
    unsigned tag_base;
    int n_items;       // D * ceil(P / PS)
};

template <int ELS, int JB, int PS>
struct Geo {
    static constexpr int R = 4 * JB;                 // gate rows owned by a block
    static constexpr int G = ELS / JB;               // blocks per group
    static constexpr int CELLS = JB * PS;            // (unit, sequence) cells owned by a block
    static constexpr int CPT = (CELLS + NT - 1) / NT;
    // forward: thread = (row r, k-split ks), weights W[r][ks*KPT .. +KPT)
    static constexpr int KSPLIT = NT / R;
    static constexpr int KPT = ELS / KSPLIT;
    // backward: thread = (columns k, row-split rs), weights W[rs*RPT .. +RPT)[k]
    static constexpr int CPTK = ELS >= NT ? ELS / NT : 1;
    static constexpr int RSPLIT = ELS >= NT ? 1 : NT / ELS;
    static constexpr int RPT = R / RSPLIT;
    static constexpr int NPART = NT / CELLS >= 1 ? NT / CELLS : 1;   // threads per cell when summing partials
    static_assert(R <= NT && NT % R == 0 && ELS % KSPLIT == 0 && ELS % JB == 0, "bad geometry");
    static_assert(KPT <= 128 && CPTK * RPT <= 128, "weight slice does not fit the register budget");
    static_assert(CELLS <= NT ? NT % CELLS == 0 : CELLS % NT == 0, "cells must tile the block");
};

// =================================================================================================
// forward
// =================================================================================================
template <int ELS, int JB, int PS>
__global__ void __launch_bounds__(NT, 1) lstm_fwd_persistent_kernel(PersistArgs a) {
    typedef Geo<ELS, JB, PS> Gm;
    constexpr int R = Gm::R, G = Gm::G, CELLS = Gm::CELLS, CPT = Gm::CPT, KSPLIT = Gm::KSPLIT, KPT = Gm::KPT;
    __shared__ __align__(16) float hs[ELS * PS];             // h[t-1] of the group's sequences, [k][p]
    __shared__ __align__(16) float red[KSPLIT * R * PS];     // k-split partial sums, [ks][r][p]
    int gave_up = 0;   // this thread ran out of its wait budget; combined block-wide by __syncthreads_or

    const int tid = threadIdx.x;
    const int g = blockIdx.x % G, slot = blockIdx.x / G, nslots = gridDim.x / G;
    const int r = tid % R, ks = tid / R;
    const int gate_r = r / JB, jj_r = r % JB;
    const int j0 = g * JB;
    const int P = a.sh.P, T = a.sh.T, ls = a.sh.ls, D = a.sh.D;
    const LstmOffsets off = lstm_offsets(a.sh.pls, ls, ELS);
    u64 *xslot = a.xchg + (size_t)slot * 4 * ELS * PS;

    __syncthreads();

    float wreg[KPT];
    int cur_d = -1;
    for (int item = slot; item < a.n_items; item += nslots) {
        const int d = item % D, p0 = (item / D) * PS, seq = item / nslots;
        if (d != cur_d) {
            // W_rec[gate][d][j0+jj][k] from the source-major copy [d][k][gate][j] (coalesced over j)
            const float *wt = a.bf.wrecT + (size_t)d * ELS * 4 * ELS;
#pragma unroll
            for (int kk = 0; kk < KPT; ++kk)
                wreg[kk] = __ldg(wt + ((size_t)(ks * KPT + kk) * 4 + gate_r) * ELS + j0 + jj_r);
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
        for (int s = 0; s < T; ++s) {
            const int t = d ? T - 1 - s : s;
            const bool first = (s == 0);
            // 1. pre-activations of this step for the block's cells (independent of the recurrence)
            float a4[CPT][4];
            int mode[CPT];  // 0 compute, 1 padding frame, 2 sequence slot beyond P
#pragma unroll
            for (int ci = 0; ci < CPT; ++ci) {
                const int c = tid + ci * NT;
                mode[ci] = 2;
                if (c < CELLS) {
                    const int pg = p0 + c / JB;
                    if (pg < P) {
                        const size_t f = (size_t)t * P + pg;
                        const float *ap = a.bf.acts + f * 4 * ls + d * ELS + j0 + (c % JB);
#pragma unroll
                        for (int q = 0; q < 4; ++q) a4[ci][q] = ap[(size_t)q * ls];
                        mode[ci] = (t >= a.sh.Tmin && a.bf.pat[f] == PAT_NONE) ? 1 : 0;
                    }
                }
            }
            // 2. gather h[t-1] of the whole group, 3. recurrent projection with register-resident weights
            if (!first) {
                const u64 *xb = xitem + (size_t)((s - 1) & 1) * ELS * PS;
                float hv[(ELS * PS + NT - 1) / NT];
                gather_pairs<ELS * PS>(hv, xb, tag0 + (unsigned)s, tid, &gave_up, a.status);
#pragma unroll
                for (int q = 0; q < (ELS * PS + NT - 1) / NT; ++q) {
                    const int i = tid + q * NT;
                    if ((ELS * PS) % NT == 0 || i < ELS * PS) hs[(i % ELS) * PS + (i / ELS)] = hv[q];
                }
                const int dead_now = __syncthreads_or(gave_up);
                if (dead_now) { dead = true; break; }
                float acc[PS];
#pragma unroll
                for (int p = 0; p < PS; ++p) acc[p] = 0.0f;
                if constexpr (PS % 4 == 0) {
                    constexpr int Q = PS / 4;
                    const float4 *h4 = reinterpret_cast<const float4 *>(hs) + ks * KPT * Q;
#pragma unroll
                    for (int kk = 0; kk < KPT; ++kk) {
#pragma unroll
                        for (int q = 0; q < Q; ++q) {
                            const float4 h = h4[kk * Q + q];
                            acc[4 * q + 0] = fmaf(wreg[kk], h.x, acc[4 * q + 0]);
                            acc[(4 * q + 1) % PS] = fmaf(wreg[kk], h.y, acc[(4 * q + 1) % PS]);
                            acc[(4 * q + 2) % PS] = fmaf(wreg[kk], h.z, acc[(4 * q + 2) % PS]);
                            acc[(4 * q + 3) % PS] = fmaf(wreg[kk], h.w, acc[(4 * q + 3) % PS]);
                        }
                    }
                } else {
                    const float4 *h4 = reinterpret_cast<const float4 *>(hs + ks * KPT);
                    float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll
                    for (int kk = 0; kk < KPT; kk += 4) {
                        const float4 h = h4[kk / 4];
                        a0 = fmaf(wreg[kk], h.x, a0);
                        a1 = fmaf(wreg[kk + 1], h.y, a1);
                        a2 = fmaf(wreg[kk + 2], h.z, a2);
                        a3 = fmaf(wreg[kk + 3], h.w, a3);
                    }
                    acc[0] = (a0 + a1) + (a2 + a3);
                }
#pragma unroll
                for (int p = 0; p < PS; ++p) red[(ks * R + r) * PS + p] = acc[p];
                __syncthreads();
            }
            // 4. gate math, state update, publish h[t]
            u64 *xo = xitem + (size_t)(s & 1) * ELS * PS;
#pragma unroll
            for (int ci = 0; ci < CPT; ++ci) {
                const int c = tid + ci * NT;
                if (c >= CELLS) continue;
                const int p = c / JB, jj = c % JB;
                float h = 0.0f;
                if (mode[ci] != 2) {
                    const size_t f = (size_t)t * P + (p0 + p);
                    const int u = d * ELS + j0 + jj;
                    float *ap = a.bf.acts + f * 4 * ls + u;
                    if (mode[ci] == 1) {
                        ap[0] = 0.0f; ap[ls] = 0.0f; ap[2 * (size_t)ls] = 0.0f; ap[3 * (size_t)ls] = 0.0f;
                        a.bf.cells[f * ls + u] = 0.0f;
                        cprev[ci] = 0.0f;
                    } else {
                        float rec[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                        if (!first) {
#pragma unroll
                            for (int q = 0; q < 4; ++q)
#pragma unroll
                                for (int k2 = 0; k2 < KSPLIT; ++k2) rec[q] += red[(k2 * R + q * JB + jj) * PS + p];
                        }
                        float ni = a4[ci][0] + rec[0] + b4[ci][0];
                        float ig = a4[ci][1] + rec[1] + b4[ci][1];
                        float fg = a4[ci][2] + rec[2] + b4[ci][2];
                        float og = a4[ci][3] + rec[3] + b4[ci][3];
                        const float cp = cprev[ci];
                        if (!first) { ig += cp * pw[ci][0]; fg += cp * pw[ci][1]; }
                        ni = act_tanh(ni); ig = act_logistic(ig); fg = act_logistic(fg);
                        float cs = ni * ig;
                        if (!first) cs += cp * fg;
                        og = act_logistic(og + cs * pw[ci][2]);
                        h = act_tanh(cs) * og;
                        ap[0] = ni; ap[ls] = ig; ap[2 * (size_t)ls] = fg; ap[3 * (size_t)ls] = og;
                        a.bf.cells[f * ls + u] = cs;
                        cprev[ci] = cs;
                    }
                    a.y[f * ls + u] = h;
                }
                st_pair(xo + (size_t)p * ELS + j0 + jj, h, tag0 + (unsigned)s + 1u);
            }
        }
        if (dead) break;
    }
}

// =================================================================================================
// backward
// =================================================================================================
template <int ELS, int JB, int PS>
__global__ void __launch_bounds__(NT, 1) lstm_bwd_persistent_kernel(PersistArgs a) {
    typedef Geo<ELS, JB, PS> Gm;
    constexpr int R = Gm::R, G = Gm::G, CELLS = Gm::CELLS, CPT = Gm::CPT;
    constexpr int CPTK = Gm::CPTK, RSPLIT = Gm::RSPLIT, RPT = Gm::RPT, NPART = Gm::NPART;
    constexpr int SRC_PER_PART = (G + NPART - 1) / NPART;
    __shared__ __align__(16) float pe[G * CELLS];            // partial sums received, [src][cell]
    __shared__ __align__(16) float pe2[NPART * CELLS];       // first-stage sums, [part][cell]
    __shared__ __align__(16) float ds[R * PS];               // this step's gate deltas, [r][p]
    __shared__ __align__(16) float redb[RSPLIT > 1 ? RSPLIT * ELS * PS : 1];
    int gave_up = 0;

    const int tid = threadIdx.x;
    const int g = blockIdx.x % G, slot = blockIdx.x / G, nslots = gridDim.x / G;
    const int j0 = g * JB;
    const int P = a.sh.P, T = a.sh.T, ls = a.sh.ls, D = a.sh.D;
    const LstmOffsets off = lstm_offsets(a.sh.pls, ls, ELS);
    // one exchange buffer holds, per owner block, G source blocks x CELLS tagged partial sums
    constexpr size_t XBUF = (size_t)G * G * CELLS;
    u64 *xslot = a.xchg + (size_t)slot * 4 * XBUF;
    const int kcol = tid % ELS, rs = (ELS >= NT) ? 0 : tid / ELS;

    __syncthreads();

    float wreg[CPTK][RPT];
    int cur_d = -1;
    for (int item = slot; item < a.n_items; item += nslots) {
        const int d = item % D, p0 = (item / D) * PS, seq = item / nslots;
        if (d != cur_d) {
            // W_rec[gate][d][j0+jj][k], row r = gate*JB + jj; consecutive threads read consecutive k
#pragma unroll
            for (int c = 0; c < CPTK; ++c)
#pragma unroll
                for (int rr = 0; rr < RPT; ++rr) {
                    const int row = rs * RPT + rr, k = (ELS >= NT) ? tid + c * NT : kcol;
                    wreg[c][rr] = __ldg(a.w + off.rec + ((size_t)(row / JB) * ls + (size_t)d * ELS + j0 + (row % JB)) * ELS + k);
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
        for (int s = 0; s < T; ++s) {
            const int t = d ? s : T - 1 - s;
            const int prevc = d ? t + 1 : t - 1;
            const bool firstCall = (s == 0), lastCall = (s == T - 1);
            // 1. everything this step needs from HBM (independent of the recurrence)
            float e_in[CPT], a4[CPT][4], cc[CPT], cpv[CPT];
            int mode[CPT];
#pragma unroll
            for (int ci = 0; ci < CPT; ++ci) {
                const int c = tid + ci * NT;
                mode[ci] = 2;
                cpv[ci] = 0.0f;
                if (c < CELLS) {
                    const int pg = p0 + c / JB;
                    if (pg < P) {
                        const size_t f = (size_t)t * P + pg;
                        const int u = d * ELS + j0 + (c % JB);
                        mode[ci] = (t >= a.sh.Tmin && a.bf.pat[f] == PAT_NONE) ? 1 : 0;
                        e_in[ci] = a.dy[f * ls + u];
                        const float *ap = a.bf.acts + f * 4 * ls + u;
#pragma unroll
                        for (int q = 0; q < 4; ++q) a4[ci][q] = ap[(size_t)q * ls];
                        cc[ci] = firstCall ? a.bf.cells[f * ls + u] : c_keep[ci];
                        if (!lastCall) cpv[ci] = a.bf.cells[((size_t)prevc * P + pg) * ls + u];
                    }
                }
            }
            // 2. partial sums of the recurrent error from every block of the group
            if (!firstCall) {
                const u64 *xb = xitem + (size_t)((s - 1) & 1) * XBUF + (size_t)g * G * CELLS;
                float pv[(G * CELLS + NT - 1) / NT];
                gather_pairs<G * CELLS>(pv, xb, tag0 + (unsigned)s, tid, &gave_up, a.status);
#pragma unroll
                for (int q = 0; q < (G * CELLS + NT - 1) / NT; ++q) {
                    const int i = tid + q * NT;
                    if ((G * CELLS) % NT == 0 || i < G * CELLS) pe[i] = pv[q];
                }
                const int dead_now = __syncthreads_or(gave_up);
                if (dead_now) { dead = true; break; }
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
                            for (int q = 0; q < NPART; ++q) e += pe2[q * CELLS + c];
                        } else {
                            for (int src = 0; src < G; ++src) e += pe[src * CELLS + c];
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
                if (mode[ci] != 2) {
                    const size_t f = (size_t)t * P + (p0 + p);
                    float *dl = a.bf.deltas + f * 4 * ls + d * ELS + j0 + jj;
                    dl[0] = dni; dl[ls] = dig; dl[2 * (size_t)ls] = dfg; dl[3 * (size_t)ls] = dog;
                }
                ds[(0 * JB + jj) * PS + p] = dni;
                ds[(1 * JB + jj) * PS + p] = dig;
                ds[(2 * JB + jj) * PS + p] = dfg;
                ds[(3 * JB + jj) * PS + p] = dog;
            }
            if (lastCall) break;
            __syncthreads();
            // 4. this block's contribution to the output error of every unit k at the next step
            float acc[CPTK][PS];
#pragma unroll
            for (int c = 0; c < CPTK; ++c)
#pragma unroll
                for (int p = 0; p < PS; ++p) acc[c][p] = 0.0f;
#pragma unroll
            for (int rr = 0; rr < RPT; ++rr) {
                const int row = rs * RPT + rr;
                float dv[PS];
                if constexpr (PS % 4 == 0) {
#pragma unroll
                    for (int q = 0; q < PS / 4; ++q) {
                        const float4 v = reinterpret_cast<const float4 *>(ds)[row * (PS / 4) + q];
                        dv[4 * q] = v.x; dv[(4 * q + 1) % PS] = v.y; dv[(4 * q + 2) % PS] = v.z; dv[(4 * q + 3) % PS] = v.w;
                    }
                } else {
#pragma unroll
                    for (int p = 0; p < PS; ++p) dv[p] = ds[row * PS + p];
                }
#pragma unroll
                for (int c = 0; c < CPTK; ++c)
#pragma unroll
                    for (int p = 0; p < PS; ++p) acc[c][p] = fmaf(wreg[c][rr], dv[p], acc[c][p]);
            }
            u64 *xo = xitem + (size_t)(s & 1) * XBUF;
            const unsigned tag = tag0 + (unsigned)s + 1u;
            if constexpr (RSPLIT > 1) {
#pragma unroll
                for (int p = 0; p < PS; ++p) redb[(rs * ELS + kcol) * PS + p] = acc[0][p];
                __syncthreads();
                for (int i = tid; i < ELS * PS; i += NT) {
                    const int k = i % ELS, p = i / ELS;
                    float v = 0.0f;
#pragma unroll
                    for (int q = 0; q < RSPLIT; ++q) v += redb[(q * ELS + k) * PS + p];
                    st_pair(xo + ((size_t)(k / JB) * G + g) * CELLS + p * JB + (k % JB), v, tag);
                }
            } else {
#pragma unroll
                for (int c = 0; c < CPTK; ++c) {
                    const int k = tid + c * NT;
#pragma unroll
                    for (int p = 0; p < PS; ++p)
                        st_pair(xo + ((size_t)(k / JB) * G + g) * CELLS + p * JB + (k % JB), acc[c][p], tag);
                }
            }
        }
        if (dead) break;
    }
}

// ---- host side ----------------------------------------------------------------------------------
int g_num_sms = 0;
int num_sms() {
    if (!g_num_sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    }
    return g_num_sms;
}

template <int ELS, int JB, int PS>
int launch(bool backward, PersistArgs &a, cudaStream_t st, int *items_per_slot) {
    typedef Geo<ELS, JB, PS> Gm;
    void (*kern)(PersistArgs) = backward ? lstm_bwd_persistent_kernel<ELS, JB, PS> : lstm_fwd_persistent_kernel<ELS, JB, PS>;
    int per_sm = 0;
    B2_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, NT, 0));
    int resident = per_sm * num_sms();
    int nslots = resident / Gm::G;
    if (nslots < 1) return 1;   // the group does not fit on the device together: caller falls back
    if (nslots > a.n_items) nslots = a.n_items;
    *items_per_slot = (a.n_items + nslots - 1) / nslots;
    void *args[] = {&a};
    B2_CUDA(cudaLaunchCooperativeKernel((const void *)kern, dim3(nslots * Gm::G), dim3(NT), args, 0, st));
    count_launch();
    return B2_OK;
}

}  // namespace

// blocks per group and exchange words per slot for the geometry chosen for (els, PS)
bool persistent_geometry(int els, int *JB) {
    switch (els) {
        case 1024: *JB = 8; return true;
        case 512: *JB = 16; return true;
        case 256: *JB = 32; return true;
        case 128: *JB = 64; return true;
        default: return false;
    }
}

// Sequences per work item.  More sequences per item amortise the per-step exchange latency over more
// work; fewer items than group slots leave SMs idle.  Take the smallest PS that lets every item have a
// slot of its own, else the largest the register budget of the geometry allows.
int persistent_ps(int els, int P, int D) {
    int JB;
    if (!persistent_geometry(els, &JB)) return 0;
    if (P == 1) return 1;
    const int G = els / JB;
    int slots = num_sms() / G;
    if (slots < 1) slots = 1;
    const int max_ps = els >= 1024 ? 8 : 16;
    for (int ps = 4; ps <= max_ps; ps *= 2)
        if (D * ((P + ps - 1) / ps) <= slots) return ps;
    return max_ps;
}

size_t lstm_persistent_xchg_words(int els, int P, int D) {
    int JB;
    if (!persistent_geometry(els, &JB)) return 0;
    const int PS = persistent_ps(els, P, D), G = els / JB;
    int max_slots = num_sms() / G;
    if (max_slots < 1) max_slots = 1;
    size_t fwd = (size_t)4 * els * PS, bwd = (size_t)4 * G * G * JB * PS;
    return (size_t)max_slots * (fwd > bwd ? fwd : bwd);
}

// returns B2_OK, an error, or 1 when this shape has no persistent kernel (caller uses the stepwise one)
int lstm_persistent(bool backward, const LstmShape &s, const LstmBuffers &b, const float *w, float *y, const float *dy,
                    unsigned long long *xchg, int *status, unsigned *tag_next, cudaStream_t st) {
    int JB;
    if (!persistent_geometry(s.els, &JB) || !xchg) return 1;
    PersistArgs a;
    a.sh = s; a.bf = b; a.w = w; a.y = y; a.dy = dy; a.xchg = xchg; a.status = status;
    a.tag_base = *tag_next;
    const int PS = persistent_ps(s.els, s.P, s.D);
    a.n_items = s.D * ((s.P + PS - 1) / PS);
    int ips = 1, rc = 1;
#define CASE_PS(E, J, Q) \
    case Q: rc = launch<E, J, Q>(backward, a, st, &ips); break;
#define CASE(E, J, WITH16)                                       \
    case E:                                                      \
        switch (PS) {                                            \
            CASE_PS(E, J, 1) CASE_PS(E, J, 4) CASE_PS(E, J, 8) WITH16 \
            default: return 1;                                   \
        }                                                        \
        break;
    switch (s.els) {
        CASE(1024, 8, )
        CASE(512, 16, CASE_PS(512, 16, 16))
        CASE(256, 32, CASE_PS(256, 32, 16))
        CASE(128, 64, CASE_PS(128, 64, 16))
        default: return 1;
    }
#undef CASE
#undef CASE_PS
    if (rc == B2_OK) *tag_next += (unsigned)ips * (unsigned)(s.T + 1) + 1u;
    return rc;
}

}  // namespace b2
