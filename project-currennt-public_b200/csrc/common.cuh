// Shared declarations of the b2lstm library: status handling, the activation functions of the
// reference toolkit as device code, and the launch prototypes of every kernel family.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/b2lstm.h"

namespace b2 {

// ---- status -------------------------------------------------------------------------------
void set_error(const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what, const char *file, int line);
#define B2_CUDA(call)                                                              \
    do {                                                                           \
        cudaError_t e__ = (call);                                                  \
        if (e__ != cudaSuccess) return ::b2::cuda_fail(e__, #call, __FILE__, __LINE__); \
    } while (0)
#define B2_TRY(call)                  \
    do {                              \
        int rc__ = (call);            \
        if (rc__ != B2_OK) return rc__; \
    } while (0)

// every kernel launch of the library goes through this counter (b2_net_launch_count)
extern unsigned long long g_launches;
inline void count_launch(int n = 1) { g_launches += (unsigned long long)n; }

// ---- per-device facts (device.cu) ---------------------------------------------------------------
constexpr int MAX_DEVICES = 64;
int current_device();   // ordinal of the current device, -1 when there is none
int sm_count();         // multiprocessors of the current device
// cudaFuncSetAttribute(MaxDynamicSharedMemorySize), once per kernel and device (the attribute is per context)
int set_max_dynamic_smem(const void *func, int bytes);

// ---- activation functions ---------------------------------------------------------------------
// Same formulas and cut-offs as activation_functions/{Logistic,Tanh,Maxmin1}.cuh of the
// reference: logistic saturates exactly at |x| >= 88.722839, tanh(x) = 2*logistic(2x) - 1.
// expf (not __expf) keeps the result within 1-2 ulp of the host libm the reference's Cpu
// device uses.
__device__ __forceinline__ float act_logistic(float x) {
    const float lim = 88.722839f;
    if (x < lim) {
        if (x > -lim) return 1.0f / (1.0f + expf(-x));
        return 0.0f;
    }
    return 1.0f;
}
__device__ __forceinline__ float d_logistic(float y) { return y * (1.0f - y); }
__device__ __forceinline__ float act_tanh(float x) { return 2.0f * act_logistic(2.0f * x) - 1.0f; }
__device__ __forceinline__ float d_tanh(float y) { return 1.0f - y * y; }
// helpers/limitedError.cuh: clip to [-1, 1]
__device__ __forceinline__ float limited_error(float e) { return e < -1.0f ? -1.0f : (e > 1.0f ? 1.0f : e); }

enum Act { ACT_TANH = 0, ACT_LOGISTIC = 1, ACT_IDENTITY = 2 };
enum { PAT_NONE = 0 };

// ---- GEMM family (gemm_ffma.cu, gemm_tc.cu) -------------------------------------------------------
// C(m x n, column-major, ldc) = A' B' (+ C).  A'(i,k) = A[i*sam + k*sak], B'(k,j) = B[k*sbk + j*sbn].
// `ws` is split-K scratch of at least ws_floats floats (may be NULL: then no split).
int gemm_ffma(float *C, long ldc, const float *A, long sam, long sak, const float *B, long sbk, long sbn, int m,
              int n, int k, bool accumulate, float *ws, size_t ws_floats, cudaStream_t st);

// Tensor-core path (gemm_tc.cu): operands are first split into tf32 hi/lo parts, stored densely as
// [outer][ld] with the contiguous index padded to a multiple of 4 floats.
struct SplitOperand {
    const float *hi, *lo;   // the two parts; they hold halves when f16 is set
    long ld;                // elements between consecutive rows
    bool kmajor;            // true: the contraction index k is the contiguous one; false: m (resp. n) is
    bool f16 = false;       // fp16 parts with a power-of-two scale (tf32 parts otherwise)
    const unsigned *maxbits = nullptr;   // f16: device word with the bit pattern of the operand's largest finite |x|
    // shifts both parts by `elems` elements
    void advance(size_t elems) {
        if (f16) { hi = (const float *)((const unsigned short *)hi + elems); lo = (const float *)((const unsigned short *)lo + elems); }
        else { hi += elems; lo += elems; }
    }
};
// bump arena for the hi/lo copies; grows by reallocation (which waits for the device)
struct TcScratch {
    float *base = nullptr;
    size_t cap = 0, used = 0;
    int reserve(size_t floats);
    float *take(size_t floats);
    void release();
};
size_t split_floats(int outer, int inner, bool f16 = true);
int split_tf32(const float *src, long s_outer, int outer, int inner, float *hi, float *lo, long ldp, cudaStream_t st);
// bound > 0: the caller's promise that no |entry| exceeds it (saves the pass that finds the largest entry)
int split_f16(const float *src, long s_outer, int outer, int inner, void *hi, void *lo, long ldp, unsigned *maxbits,
              cudaStream_t st, float bound = 0.0f);
int split_operand(TcScratch &sc, const float *src, long s_outer, int outer, int inner, bool kmajor, SplitOperand *out,
                  cudaStream_t st, bool f16 = true, float bound = 0.0f);
bool gemm_tc_supported(const SplitOperand &A, const SplitOperand &B, int m, int n, int k);
int gemm_tc(float *C, long ldc, const SplitOperand &A, const SplitOperand &B, int m, int n, int k, bool accumulate,
            float *ws, size_t ws_floats, int *status, cudaStream_t st);
// Planned, batched launches of the tensor-core kernel: tensor maps encoded once, many launches that
// differ in coordinate offsets.  Batch b shifts operand A by (a_in, a_out) and B by (b_in, b_out) in
// (contiguous index, other index) coordinates and writes split z to C + c_off + z*c_split_stride.
struct TcBatch { int a_in, a_out, b_in, b_out; long long c_off; };
struct TcPlan;
int tc_plan_create(TcPlan **out, const SplitOperand &A, long a_inner, long a_outer, const SplitOperand &B, long b_inner,
                   long b_outer, int m, int n, int k, int splits, int kseg_len, int kseg_stride, long ldc);
int tc_plan_launch(const TcPlan *p, float *C, const TcBatch *batches, int nbatch, long long c_split_stride, int *status,
                   cudaStream_t st);
void tc_plan_destroy(TcPlan *p);
// sums the K-split partials a batched launch wrote to ws (batch b, split z at (b*splits + z)*m*n) into
// C + c_off[b] with leading dimension ldc
int tc_batched_reduce(float *C, const long long *c_off, int nbatch, long ldc, const float *ws, int m, int n, int splits,
                      cudaStream_t st);
int tc_sm_count();
bool gemm_wants_tc(long sam, long sak, long sbk, long sbn, int m, int n, int k);
// picks the tensor-core kernel when the shape qualifies (and sc/status are given), else FFMA
int gemm_auto(float *C, long ldc, const float *A, long sam, long sak, const float *B, long sbk, long sbn, int m, int n,
              int k, bool accumulate, bool force_ffma, TcScratch *sc, float *ws, size_t ws_floats, int *status,
              cudaStream_t st);

// ---- feed-forward / loss / optimizer elementwise kernels (elementwise.cu) -------------------------
// y[f*ls + u] = act(y + bias*b[u]) over n = frames*ls elements
int ff_bias_act(float *y, const float *b, float bias, int ls, size_t n, int act, cudaStream_t st);
// delta[i] = act'(y[i]) * err[i], in place on err
int ff_delta(float *err, const float *y, size_t n, int act, cudaStream_t st);
// out[u] = scale * sum_f m[f*ld + u], u < cols, f < rows; deterministic two-stage reduction
int column_sums(float *out, const float *m, long ld, int cols, long rows, float scale, float *ws, size_t ws_floats,
                cudaStream_t st);
// SSE: err_partial -> *loss_dev (double) = 0.5*sum (t-y)^2 over non-padding frames
int sse_loss(double *loss_dev, const float *y, const float *tgt, const char *pat, int ls, size_t frames, double *ws,
             cudaStream_t st);
// dy = y - t on real frames, 0 on padding
int sse_grad(float *dy, const float *y, const float *tgt, const char *pat, int ls, size_t frames, cudaStream_t st);
// steepest descent with momentum; zeroes NaN/Inf gradient entries first
int sgd_update(float *w, float *g, float *delta, size_t n, float lr, float mom, cudaStream_t st);
// the same after shaping the gradient: option 1 AdaGrad, 2 average over *frac_len_dev frames, 3 plain SGD that
// accumulates the AdaGrad statistics, 5 Adam; stats holds n floats (2n for Adam)
int sgd_update_opt(float *w, float *g, float *delta, float *stats, size_t n, float lr, float mom, int option,
                   const float *frac_len_dev, float beta1_accum, float beta2_accum, cudaStream_t st);
int fill_value(float *p, size_t n, float v, cudaStream_t st);
// acc = g (first) or acc + g
int accumulate(float *acc, const float *g, size_t n, bool first, cudaStream_t st);
int fill_zero(void *p, size_t bytes, cudaStream_t st);

// ---- LSTM recurrence (lstm_step.cu, lstm_persistent.cu) -------------------------------------------
struct LstmShape {
    int P, T, Tmin, pls, ls, els, D;  // D = directions (1 or 2)
    float bias;
};
struct LstmBuffers {
    float *acts;        // [T*P][4*ls]: pre-activations from the input projection, overwritten by the
                        //              post-activation ni, ig, fg, og; column c = g*ls + dir*els + j
    float *cells;       // [T*P][ls]:   cell states, column dir*els + j
    float *deltas;      // [T*P][4*ls]: gate deltas, same column order as acts
    float *cerr;        // [2][P][ls]:  cell-state errors of the two most recent steps (stepwise kernels)
    float *wrecT;       // [D][els][4][els]: recurrent weights, source unit major (forward sweep)
    const char *pat;    // [T*P]
};
// one launch per timestep, both directions in the same launch
int lstm_forward_stepwise(const LstmShape &s, const LstmBuffers &b, const float *w, float *y, cudaStream_t st);
int lstm_backward_stepwise(const LstmShape &s, const LstmBuffers &b, const float *w, const float *dy,
                           cudaStream_t st);
// transpose the recurrent block of the weight vector into LstmBuffers::wrecT
int lstm_prepare_wrecT(const LstmShape &s, const float *w, float *wrecT, cudaStream_t st);
// bias and peephole gradients (the vector part of the weight update), written into dw
int lstm_vector_grads(const LstmShape &s, const LstmBuffers &b, float *dw, float *ws, size_t ws_floats,
                      cudaStream_t st);

// tensor-core recurrence for large batches (lstm_step_tc.cu): one batched tcgen05 GEMM + one gate
// kernel per timestep.  The buffers hold the tf32 hi/lo parts of the recurrent weights, of the block
// outputs and of the gate deltas, and the K-split partial sums of one step.
struct TcRecBuffers {
    float *wrec_hi = nullptr, *wrec_lo = nullptr;   // [4*ls][els]
    float *y_hi = nullptr, *y_lo = nullptr;         // [T*P][ls]
    float *d_hi = nullptr, *d_lo = nullptr;         // [T*P][4*ls]
    float *part = nullptr;
};
bool lstm_tc_supported(const LstmShape &s);
size_t lstm_tc_part_floats(int P, int els, int D);
int lstm_forward_tc(const LstmShape &s, const LstmBuffers &bf, const TcRecBuffers &rb, const float *w, float *y, int *status,
                    cudaStream_t st);
int lstm_backward_tc(const LstmShape &s, const LstmBuffers &bf, const TcRecBuffers &rb, const float *w, const float *dy,
                     int *status, cudaStream_t st);

// persistent tensor-core recurrence (lstm_ptc.cu): recurrent weights resident in shared memory as fp16 hi/lo
// tcgen05 operands for the whole sweep.  Returns B2_OK, an error, or 1 when the shape is not covered.
struct PtcBuffers {
    unsigned *maxbits = nullptr;                   // [2] largest |w| of the recurrent block per direction (float bits)
    float *scale = nullptr;                        // [direction][2]: S, 1/S
    uint4 *wimg_f = nullptr, *wimg_b = nullptr;    // per-block weight images of the forward / backward sweep
    unsigned char *xh = nullptr;                   // forward exchange: fp16 operand images of h, per chunk, step parity, slice
    float *xe = nullptr;                           // backward exchange: partial output errors, per chunk, step parity, row tile
    unsigned *flags = nullptr;                     // step counters the blocks publish to each other
};
bool lstm_ptc_supported(const LstmShape &s);
size_t lstm_ptc_image_bytes(int els, int D);
void lstm_ptc_set_plan(bool backward, int ll_chunks, int nc32_chunks, int nc32_counter_chunks);
void lstm_ptc_exchange_sizes(int els, int P, int D, size_t *xh_bytes, size_t *xe_floats, size_t *flag_words);
int lstm_ptc_prepare(const LstmShape &s, const float *w, const PtcBuffers &pb, cudaStream_t st);
int lstm_ptc_sweep(bool backward, const LstmShape &s, const LstmBuffers &b, const PtcBuffers &pb, const float *w, float *y,
                   const float *dy, int *status, unsigned *tag_next, cudaStream_t st);

// persistent kernels (lstm_persistent.cu).  Return B2_OK, an error, or 1 when the shape has no
// persistent kernel (the caller then uses the stepwise kernels).
bool persistent_geometry(int els, int *JB);   // hidden units per block of the register-resident geometry
size_t lstm_persistent_xchg_words(int els, int P, int D);
int persistent_ps(int els, int P, int D, bool use_cluster);   // sequences per work item for a shape (0: no persistent kernel)
// transport: 0 = the blocks of a group exchange through L2; 1 = groups of <= 8 blocks run as thread-block
// clusters and exchange through distributed shared memory; 2 = the layout a cost model prefers (clusters for as
// many items as fit side by side, the remaining sequences through L2 on the SMs the clusters leave free)
int lstm_persistent(bool backward, int transport, const LstmShape &s, const LstmBuffers &b, const float *w, float *y,
                    const float *dy, unsigned long long *xchg, int *status, unsigned *tag_next, cudaStream_t st);
int lstm_selftest_bounded_wait(int *status_out, int *gave_up, cudaStream_t st);

// offsets inside the (b)lstm weight vector
struct LstmOffsets {
    size_t bias, rec, peep, total;
};
__host__ __device__ inline LstmOffsets lstm_offsets(int pls, int ls, int els) {
    LstmOffsets o;
    o.bias = (size_t)4 * ls * pls;
    o.rec = o.bias + (size_t)4 * ls;
    o.peep = o.rec + (size_t)4 * ls * els;
    o.total = o.peep + (size_t)3 * ls;
    return o;
}

}  // namespace b2
