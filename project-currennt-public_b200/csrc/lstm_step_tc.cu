// Tensor-core recurrence for large batches: per timestep ONE batched tcgen05 GEMM (all four gates,
// both directions) for the recurrent product and ONE fused gate kernel.
//
// Same arithmetic as the reference's time loops (layers/LstmLayer.cu:1805-1858,1878-1927 forward,
// :2115-2176,2195-2253 backward: 4 cublasSgemm + one Thrust functor per step and direction), used
// when parallel_sequences x units is large enough that the per-step product (4*els x els x P) belongs
// on the tensor cores; the persistent FFMA kernels (lstm_persistent.cu) win when it is small.
//
//   forward  step: rec[d][p][g*els+j]  = sum_k W_rec[g][d][j][k] * h_d[prev][p][k]     (3xTF32 GEMM,
//                  batches = (direction, gate), K split over blocks, partial sums to scratch)
//                  gates: pre-activation = projection + sum of the K-split partials; cell math;
//                  writes the activations, c, h and the tf32 hi/lo parts of h (the next step's
//                  GEMM operand, later also the weight-gradient GEMM's)
//   backward step: erec[d][p][k] = sum_{g,j} W_rec[g][d][j][k] * delta_g,d[next][p][j]  (one batch per
//                  direction, contraction over the four gate blocks = segmented K)
//                  gates: e = dY + partials; cell errors and clipped gate deltas; writes the deltas
//                  and their hi/lo parts
// The GEMM's tensor maps are encoded once per sweep (tc_plan_*); a step only changes coordinates.
#include "common.cuh"

namespace b2 {
namespace {

__device__ __forceinline__ void split_store(float x, float *hi, float *lo) {
    uint32_t h, l;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
    const float rem = x - __uint_as_float(h);
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(rem));
    *hi = __uint_as_float(h);
    *lo = __uint_as_float(l);
}

struct TcStepArgs {
    LstmShape sh;
    LstmBuffers bf;
    const float *w;
    float *y;           // forward: block outputs
    const float *dy;    // backward: output errors
    float *y_hi, *y_lo; // [T*P][ls]
    float *d_hi, *d_lo; // [T*P][4*ls]
    const float *part;  // K-split partial sums of this step's recurrent product
    int nsplit;         // 0 on the first step of a sweep (no recurrent term)
    int s;              // step index of the sweep
};

// one thread per cell (direction d, sequence p, unit j); ComputeBlockOutputFn of the reference
__global__ void __launch_bounds__(128) tc_fwd_gates_kernel(TcStepArgs a) {
    const int els = a.sh.els, ls = a.sh.ls, P = a.sh.P, T = a.sh.T, D = a.sh.D;
    const int j = blockIdx.x * 128 + threadIdx.x, p = blockIdx.y, d = blockIdx.z;
    if (j >= els) return;
    const int t = d ? T - 1 - a.s : a.s, prev = d ? t + 1 : t - 1;
    const bool first = (a.s == 0);
    const LstmOffsets off = lstm_offsets(a.sh.pls, ls, els);
    const int u = d * els + j;
    const size_t f = (size_t)t * P + p;
    float *ap = a.bf.acts + f * 4 * ls + u;
    float h = 0.0f;
    if (t >= a.sh.Tmin && a.bf.pat[f] == PAT_NONE) {
        ap[0] = 0.0f; ap[ls] = 0.0f; ap[2 * (size_t)ls] = 0.0f; ap[3 * (size_t)ls] = 0.0f;
        a.bf.cells[f * ls + u] = 0.0f;
    } else {
        float pre[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) pre[g] = ap[(size_t)g * ls];
        for (int z = 0; z < a.nsplit; ++z) {
            const float *rp = a.part + (((size_t)z * D + d) * P + p) * 4 * els + j;
#pragma unroll
            for (int g = 0; g < 4; ++g) pre[g] += rp[(size_t)g * els];
        }
        float ni = pre[0] + a.sh.bias * a.w[off.bias + 0 * (size_t)ls + u];
        float ig = pre[1] + a.sh.bias * a.w[off.bias + 1 * (size_t)ls + u];
        float fg = pre[2] + a.sh.bias * a.w[off.bias + 2 * (size_t)ls + u];
        float og = pre[3] + a.sh.bias * a.w[off.bias + 3 * (size_t)ls + u];
        float cp = 0.0f;
        if (!first) {
            cp = a.bf.cells[((size_t)prev * P + p) * ls + u];
            ig += cp * a.w[off.peep + 0 * (size_t)ls + u];
            fg += cp * a.w[off.peep + 1 * (size_t)ls + u];
        }
        ni = act_tanh(ni); ig = act_logistic(ig); fg = act_logistic(fg);
        float cs = ni * ig;
        if (!first) cs += cp * fg;
        og = act_logistic(og + cs * a.w[off.peep + 2 * (size_t)ls + u]);
        h = act_tanh(cs) * og;
        ap[0] = ni; ap[ls] = ig; ap[2 * (size_t)ls] = fg; ap[3 * (size_t)ls] = og;
        a.bf.cells[f * ls + u] = cs;
    }
    a.y[f * ls + u] = h;
    split_store(h, a.y_hi + f * ls + u, a.y_lo + f * ls + u);
}

// ComputeBlockErrorsFn of the reference; the cell-state errors of the previous step live in bf.cerr
__global__ void __launch_bounds__(128) tc_bwd_gates_kernel(TcStepArgs a) {
    const int els = a.sh.els, ls = a.sh.ls, P = a.sh.P, T = a.sh.T, D = a.sh.D;
    const int j = blockIdx.x * 128 + threadIdx.x, p = blockIdx.y, d = blockIdx.z;
    if (j >= els) return;
    const int t = d ? a.s : T - 1 - a.s;
    const int next = d ? t - 1 : t + 1, prevc = d ? t + 1 : t - 1;
    const bool firstCall = (a.s == 0), lastCall = (a.s == T - 1);
    const LstmOffsets off = lstm_offsets(a.sh.pls, ls, els);
    const int u = d * els + j;
    const size_t f = (size_t)t * P + p;
    float *ce_cur = a.bf.cerr + (size_t)(a.s & 1) * P * ls;
    const float *ce_nxt = a.bf.cerr + (size_t)((a.s + 1) & 1) * P * ls;
    float dni = 0.0f, dig = 0.0f, dfg = 0.0f, dog = 0.0f, ce = 0.0f;
    if (!(t >= a.sh.Tmin && a.bf.pat[f] == PAT_NONE)) {
        float e = a.dy[f * ls + u];
        for (int z = 0; z < a.nsplit; ++z) e += a.part[(((size_t)z * D + d) * P + p) * els + j];
        const float *ap = a.bf.acts + f * 4 * ls + u;
        const float ni = ap[0], ig = ap[ls], fg = ap[2 * (size_t)ls], og = ap[3 * (size_t)ls];
        const float tc = act_tanh(a.bf.cells[f * ls + u]);
        const float p_ig = a.w[off.peep + 0 * (size_t)ls + u], p_fg = a.w[off.peep + 1 * (size_t)ls + u];
        const float p_og = a.w[off.peep + 2 * (size_t)ls + u];
        dog = d_logistic(og) * tc * e;
        ce = og * d_tanh(tc) * e + p_og * dog;
        if (!firstCall) {
            const size_t fn = (size_t)next * P + p;
            const float *an = a.bf.acts + fn * 4 * ls + u;
            const float *dn = a.bf.deltas + fn * 4 * ls + u;
            ce += an[2 * (size_t)ls] * ce_nxt[(size_t)p * ls + u] + p_ig * dn[ls] + p_fg * dn[2 * (size_t)ls];
        }
        dni = ig * d_tanh(ni) * ce;
        if (!lastCall) dfg = d_logistic(fg) * a.bf.cells[((size_t)prevc * P + p) * ls + u] * ce;
        dig = d_logistic(ig) * ni * ce;
        dni = limited_error(dni); dig = limited_error(dig); dfg = limited_error(dfg); dog = limited_error(dog);
    }
    ce_cur[(size_t)p * ls + u] = ce;
    const size_t o = f * 4 * ls + u;
    a.bf.deltas[o] = dni; a.bf.deltas[o + ls] = dig; a.bf.deltas[o + 2 * (size_t)ls] = dfg; a.bf.deltas[o + 3 * (size_t)ls] = dog;
    split_store(dni, a.d_hi + o, a.d_lo + o);
    split_store(dig, a.d_hi + o + ls, a.d_lo + o + ls);
    split_store(dfg, a.d_hi + o + 2 * (size_t)ls, a.d_lo + o + 2 * (size_t)ls);
    split_store(dog, a.d_hi + o + 3 * (size_t)ls, a.d_lo + o + 3 * (size_t)ls);
}

}  // namespace

namespace {
// K-splits: enough blocks to fill the SMs (148 on a B200), each split a whole number of 32-slabs
int pick_splits(int tiles, int k) {
    int best = 1;
    for (int s = 1; s <= 8; s *= 2)
        if ((k / 32) % s == 0 && k / s >= 64 && tiles * s <= 160) best = s;
    return best;
}
int fwd_tiles(const LstmShape &s) { return 4 * s.D * ((s.els + 127) / 128) * ((s.P + 127) / 128); }
int bwd_tiles(const LstmShape &s) { return s.D * ((s.els + 127) / 128) * ((s.P + 127) / 128); }
}  // namespace

bool lstm_tc_supported(const LstmShape &s) { return s.els >= 128 && (s.els % 32) == 0 && (s.ls % 4) == 0; }

size_t lstm_tc_part_floats(int P, int els, int D) {
    LstmShape s{};
    s.P = P; s.els = els; s.D = D;
    size_t f = (size_t)pick_splits(fwd_tiles(s), els) * D * P * 4 * els;
    size_t b = (size_t)pick_splits(bwd_tiles(s), 4 * els) * D * P * els;
    return f > b ? f : b;
}

int lstm_forward_tc(const LstmShape &s, const LstmBuffers &bf, const TcRecBuffers &rb, const float *w, float *y, int *status,
                    cudaStream_t st) {
    const int els = s.els, ls = s.ls, P = s.P, T = s.T, D = s.D;
    const LstmOffsets off = lstm_offsets(s.pls, ls, els);
    // recurrent block of the weight vector as ONE [4*ls rows c][els] matrix (k contiguous), split once
    B2_TRY(split_tf32(w + off.rec, els, 4 * ls, els, rb.wrec_hi, rb.wrec_lo, els, st));
    SplitOperand A{rb.wrec_hi, rb.wrec_lo, els, true};
    SplitOperand B{rb.y_hi, rb.y_lo, ls, true};
    const int splits = pick_splits(fwd_tiles(s), els);
    TcPlan *plan = nullptr;
    if (T > 1) B2_TRY(tc_plan_create(&plan, A, els, 4L * ls, B, ls, (long)T * P, els, P, els, splits, 0, 0, 4L * els));
    TcStepArgs a;
    a.sh = s; a.bf = bf; a.w = w; a.y = y; a.dy = nullptr;
    a.y_hi = rb.y_hi; a.y_lo = rb.y_lo; a.d_hi = rb.d_hi; a.d_lo = rb.d_lo; a.part = rb.part;
    dim3 grid((els + 127) / 128, P, D);
    int rc = B2_OK;
    for (int i = 0; i < T && rc == B2_OK; ++i) {
        a.s = i;
        a.nsplit = 0;
        if (i > 0) {
            TcBatch bt[8];
            for (int d = 0; d < D; ++d) {
                const int t = d ? T - 1 - i : i, prev = d ? t + 1 : t - 1;
                for (int g = 0; g < 4; ++g) {
                    TcBatch &b = bt[d * 4 + g];
                    b.a_in = 0; b.a_out = g * ls + d * els;
                    b.b_in = d * els; b.b_out = prev * P;
                    b.c_off = ((long long)d * P) * 4 * els + (long long)g * els;
                }
            }
            rc = tc_plan_launch(plan, rb.part, bt, 4 * D, (long long)D * P * 4 * els, status, st);
            a.nsplit = splits;
        }
        if (rc == B2_OK) {
            tc_fwd_gates_kernel<<<grid, 128, 0, st>>>(a);
            count_launch();
        }
    }
    if (plan) tc_plan_destroy(plan);
    B2_TRY(rc);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

int lstm_backward_tc(const LstmShape &s, const LstmBuffers &bf, const TcRecBuffers &rb, const float *w, const float *dy,
                     int *status, cudaStream_t st) {
    const int els = s.els, ls = s.ls, P = s.P, T = s.T, D = s.D;
    // rb.wrec_hi/lo still hold this step's recurrent weights (the forward sweep split them)
    SplitOperand A{rb.wrec_hi, rb.wrec_lo, els, false};     // e[k] = sum_c W[c][k] delta[c]: k is the m index
    SplitOperand B{rb.d_hi, rb.d_lo, 4L * ls, true};
    const int splits = pick_splits(bwd_tiles(s), 4 * els);
    TcPlan *plan = nullptr;
    if (T > 1)
        B2_TRY(tc_plan_create(&plan, A, els, 4L * ls, B, 4L * ls, (long)T * P, els, P, 4 * els, splits, els, ls, els));
    TcStepArgs a;
    a.sh = s; a.bf = bf; a.w = w; a.y = nullptr; a.dy = dy;
    a.y_hi = rb.y_hi; a.y_lo = rb.y_lo; a.d_hi = rb.d_hi; a.d_lo = rb.d_lo; a.part = rb.part;
    dim3 grid((els + 127) / 128, P, D);
    int rc = B2_OK;
    for (int i = 0; i < T && rc == B2_OK; ++i) {
        a.s = i;
        a.nsplit = 0;
        if (i > 0) {
            TcBatch bt[2];
            for (int d = 0; d < D; ++d) {
                const int t = d ? i : T - 1 - i, next = d ? t - 1 : t + 1;
                bt[d].a_in = 0; bt[d].a_out = d * els;       // rows c = g*ls + d*els + j of the weight matrix
                bt[d].b_in = d * els; bt[d].b_out = next * P; // the same c inside a frame of deltas
                bt[d].c_off = (long long)d * P * els;
            }
            rc = tc_plan_launch(plan, rb.part, bt, D, (long long)D * P * els, status, st);
            a.nsplit = splits;
        }
        if (rc == B2_OK) {
            tc_bwd_gates_kernel<<<grid, 128, 0, st>>>(a);
            count_launch();
        }
    }
    if (plan) tc_plan_destroy(plan);
    B2_TRY(rc);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

}  // namespace b2
