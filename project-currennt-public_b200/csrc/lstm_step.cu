// Stepwise LSTM recurrence: one kernel launch per timestep, both directions in the same launch.
//
// This is the plain form of the two time loops of the reference's LstmLayer
// (layers/LstmLayer.cu:1805-1858,1878-1927 forward; :2115-2176,2195-2253 backward): what the
// reference does with four cublasSgemm calls plus one Thrust functor per step and direction
// (ComputeBlockOutputFn :57-185, ComputeBlockErrorsFn :237-405) is one fused launch here.  It
// accepts any shape and is the comparison partner of the persistent kernels.
#include "common.cuh"

namespace b2 {
namespace {

constexpr int PT = 4;     // sequences per thread
constexpr int JT = 128;   // hidden units per block
constexpr int KC = 128;   // source units staged in shared memory at a time

// Forward cell for step index s of each direction (forward direction: t = s, backward: t = T-1-s).
__global__ void __launch_bounds__(JT) lstm_fwd_step_kernel(LstmShape sh, LstmBuffers bf, const float *__restrict__ w,
                                                           float *__restrict__ y, int s) {
    const int d = blockIdx.z;
    const int els = sh.els, ls = sh.ls, P = sh.P;
    const int t = d ? sh.T - 1 - s : s;
    const int prev = d ? t + 1 : t - 1;
    const bool first = (s == 0);
    const int j = blockIdx.x * JT + threadIdx.x;
    const int p0 = blockIdx.y * PT;
    const LstmOffsets off = lstm_offsets(sh.pls, ls, els);

    __shared__ float hs[PT][KC];
    float acc[4][PT];
#pragma unroll
    for (int g = 0; g < 4; ++g)
#pragma unroll
        for (int q = 0; q < PT; ++q) acc[g][q] = 0.0f;

    if (!first) {
        const float *wt = bf.wrecT + (size_t)d * els * 4 * els;  // [k][g][j]
        for (int k0 = 0; k0 < els; k0 += KC) {
            __syncthreads();
            for (int e = threadIdx.x; e < PT * KC; e += JT) {
                int q = e / KC, kk = e % KC;
                int p = p0 + q, k = k0 + kk;
                hs[q][kk] = (p < P && k < els) ? y[((size_t)prev * P + p) * ls + d * els + k] : 0.0f;
            }
            __syncthreads();
            if (j < els) {
                int kn = min(KC, els - k0);
                for (int kk = 0; kk < kn; ++kk) {
                    const float *wr = wt + ((size_t)(k0 + kk) * 4) * els + j;
                    float w0 = __ldg(wr), w1 = __ldg(wr + els), w2 = __ldg(wr + 2 * els), w3 = __ldg(wr + 3 * els);
#pragma unroll
                    for (int q = 0; q < PT; ++q) {
                        float h = hs[q][kk];
                        acc[0][q] = fmaf(w0, h, acc[0][q]);
                        acc[1][q] = fmaf(w1, h, acc[1][q]);
                        acc[2][q] = fmaf(w2, h, acc[2][q]);
                        acc[3][q] = fmaf(w3, h, acc[3][q]);
                    }
                }
            }
        }
    }
    if (j >= els) return;

    const int u = d * els + j;
    const float b_ni = sh.bias * w[off.bias + 0 * ls + u], b_ig = sh.bias * w[off.bias + 1 * ls + u];
    const float b_fg = sh.bias * w[off.bias + 2 * ls + u], b_og = sh.bias * w[off.bias + 3 * ls + u];
    const float p_ig = w[off.peep + 0 * ls + u], p_fg = w[off.peep + 1 * ls + u], p_og = w[off.peep + 2 * ls + u];
    const bool check = t >= sh.Tmin;
#pragma unroll
    for (int q = 0; q < PT; ++q) {
        int p = p0 + q;
        if (p >= P) break;
        size_t f = (size_t)t * P + p;
        float *a = bf.acts + f * 4 * ls + u;
        if (check && bf.pat[f] == PAT_NONE) {
            // padding frame: block output and cell state are defined as zero
            y[f * ls + u] = 0.0f;
            bf.cells[f * ls + u] = 0.0f;
            a[0] = 0.0f; a[ls] = 0.0f; a[2 * ls] = 0.0f; a[3 * ls] = 0.0f;
            continue;
        }
        float ni = a[0] + acc[0][q], ig = a[ls] + acc[1][q], fg = a[2 * ls] + acc[2][q], og = a[3 * ls] + acc[3][q];
        ni += b_ni; ig += b_ig; fg += b_fg; og += b_og;
        float cprev = 0.0f;
        if (!first) {
            cprev = bf.cells[((size_t)prev * P + p) * ls + u];
            ig += cprev * p_ig;
            fg += cprev * p_fg;
        }
        ni = act_tanh(ni); ig = act_logistic(ig); fg = act_logistic(fg);
        float c = ni * ig;
        if (!first) c += cprev * fg;
        og += c * p_og;
        og = act_logistic(og);
        a[0] = ni; a[ls] = ig; a[2 * ls] = fg; a[3 * ls] = og;
        bf.cells[f * ls + u] = c;
        y[f * ls + u] = act_tanh(c) * og;
    }
}

// Backward cell for step index s (forward direction: t = T-1-s, backward direction: t = s).
__global__ void __launch_bounds__(JT) lstm_bwd_step_kernel(LstmShape sh, LstmBuffers bf, const float *__restrict__ w,
                                                           const float *__restrict__ dy, int s) {
    const int d = blockIdx.z;
    const int els = sh.els, ls = sh.ls, P = sh.P;
    const int t = d ? s : sh.T - 1 - s;
    const int next = d ? t - 1 : t + 1;    // the step processed just before this one
    const int prevc = d ? t + 1 : t - 1;   // the step whose cell state fed this one in the forward pass
    const bool firstCall = (s == 0), lastCall = (s == sh.T - 1);
    const int j = blockIdx.x * JT + threadIdx.x;
    const int p0 = blockIdx.y * PT;
    const LstmOffsets off = lstm_offsets(sh.pls, ls, els);

    __shared__ float ds[PT][KC];
    float acc[PT];
#pragma unroll
    for (int q = 0; q < PT; ++q) acc[q] = 0.0f;

    if (!firstCall) {
        // e[j] += sum over gates g and target units jj of W_rec[g][d][jj][j] * delta_g[next][jj]
        const int ktot = 4 * els;  // index kk = g*els + jj
        for (int k0 = 0; k0 < ktot; k0 += KC) {
            __syncthreads();
            for (int e = threadIdx.x; e < PT * KC; e += JT) {
                int q = e / KC, kk = k0 + e % KC;
                int p = p0 + q;
                float v = 0.0f;
                if (p < P && kk < ktot) {
                    int g = kk / els, jj = kk % els;
                    v = bf.deltas[((size_t)next * P + p) * 4 * ls + g * ls + d * els + jj];
                }
                ds[q][e % KC] = v;
            }
            __syncthreads();
            if (j < els) {
                int kn = min(KC, ktot - k0);
                for (int i = 0; i < kn; ++i) {
                    int kk = k0 + i;
                    int g = kk / els, jj = kk % els;
                    float wv = __ldg(w + off.rec + ((size_t)g * ls + d * els + jj) * els + j);
#pragma unroll
                    for (int q = 0; q < PT; ++q) acc[q] = fmaf(wv, ds[q][i], acc[q]);
                }
            }
        }
    }
    if (j >= els) return;

    const int u = d * els + j;
    const float p_ig = w[off.peep + 0 * ls + u], p_fg = w[off.peep + 1 * ls + u], p_og = w[off.peep + 2 * ls + u];
    const bool check = t >= sh.Tmin;
    float *ce_cur = bf.cerr + (size_t)(s & 1) * P * ls;
    const float *ce_nxt = bf.cerr + (size_t)((s + 1) & 1) * P * ls;
#pragma unroll
    for (int q = 0; q < PT; ++q) {
        int p = p0 + q;
        if (p >= P) break;
        size_t f = (size_t)t * P + p;
        float *dl = bf.deltas + f * 4 * ls + u;
        if (check && bf.pat[f] == PAT_NONE) {
            dl[0] = 0.0f; dl[ls] = 0.0f; dl[2 * ls] = 0.0f; dl[3 * ls] = 0.0f;
            ce_cur[(size_t)p * ls + u] = 0.0f;
            continue;
        }
        const float *a = bf.acts + f * 4 * ls + u;
        float e = dy[f * ls + u] + acc[q];
        float ni = a[0], ig = a[ls], fg = a[2 * ls], og = a[3 * ls];
        float c = bf.cells[f * ls + u];
        float tc = act_tanh(c);
        float dog = d_logistic(og) * tc * e;
        float ce = og * d_tanh(tc) * e + p_og * dog;
        if (!firstCall) {
            size_t fn = (size_t)next * P + p;
            const float *an = bf.acts + fn * 4 * ls + u;
            const float *dn = bf.deltas + fn * 4 * ls + u;
            ce += an[2 * ls] * ce_nxt[(size_t)p * ls + u] + p_ig * dn[ls] + p_fg * dn[2 * ls];
        }
        float dni = ig * d_tanh(ni) * ce;
        float dfg = 0.0f;
        if (!lastCall) dfg = d_logistic(fg) * bf.cells[((size_t)prevc * P + p) * ls + u] * ce;
        float dig = d_logistic(ig) * ni * ce;
        dl[0] = limited_error(dni); dl[ls] = limited_error(dig);
        dl[2 * ls] = limited_error(dfg); dl[3 * ls] = limited_error(dog);
        ce_cur[(size_t)p * ls + u] = ce;
    }
}

// wrecT[d][k][g][j] = W_rec[g][d][j][k]
__global__ void wrec_transpose_kernel(int ls, int els, int D, const float *__restrict__ wrec, float *__restrict__ out) {
    __shared__ float tile[32][33];
    // matrix per (g, d): rows j (slow), cols k (fast) -> out rows k, cols j
    int gd = blockIdx.z, g = gd / D, d = gd % D;
    const float *src = wrec + ((size_t)g * ls + (size_t)d * els) * els;
    int k = blockIdx.x * 32 + threadIdx.x, jb = blockIdx.y * 32;
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        int j = jb + r;
        tile[r][threadIdx.x] = (j < els && k < els) ? src[(size_t)j * els + k] : 0.0f;
    }
    __syncthreads();
    int j = jb + threadIdx.x, kb = blockIdx.x * 32;
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        int kk = kb + r;
        if (j < els && kk < els) out[(((size_t)d * els + kk) * 4 + g) * els + j] = tile[threadIdx.x][r];
    }
}

// Bias and peephole gradients: per unit u and frame chunk, partial sums of
//   delta_g[f][u] (4 gates), c[f -/+ P]*delta_ig/fg[f] and c[f]*delta_og[f]
// (layers/LstmLayer.cu:524-541,574-610 of the reference), then a fixed-order reduction.
__global__ void lstm_vgrad_partial_kernel(LstmShape sh, LstmBuffers bf, float *__restrict__ ws, int frames_per_chunk) {
    const int ls = sh.ls, els = sh.els, P = sh.P;
    const int u = blockIdx.x * blockDim.x + threadIdx.x;
    if (u >= ls) return;
    const int d = u / els;
    const long N = (long)sh.T * P;
    long f0 = (long)blockIdx.y * frames_per_chunk, f1 = min(N, f0 + frames_per_chunk);
    float s[7] = {0, 0, 0, 0, 0, 0, 0};
#pragma unroll 4
    for (long f = f0; f < f1; ++f) {
        const float *dl = bf.deltas + (size_t)f * 4 * ls + u;
        float dni = dl[0], dig = dl[ls], dfg = dl[2 * ls], dog = dl[3 * ls];
        s[0] += dni; s[1] += dig; s[2] += dfg; s[3] += dog;
        // forward direction pairs delta[t] with c[t-1] (skips t = 0); backward with c[t+1] (skips t = T-1)
        long fo = d ? f + P : f - P;
        if (fo >= 0 && fo < N) {
            float co = bf.cells[(size_t)fo * ls + u];
            s[4] += co * dig;
            s[5] += co * dfg;
        }
        s[6] += bf.cells[(size_t)f * ls + u] * dog;
    }
    float *o = ws + (size_t)blockIdx.y * 7 * ls;
#pragma unroll
    for (int i = 0; i < 7; ++i) o[(size_t)i * ls + u] = s[i];
}
// 32 entries x 8 chunk phases per block; fixed summation order
__global__ void __launch_bounds__(256) lstm_vgrad_reduce_kernel(LstmShape sh, int chunks, const float *__restrict__ ws,
                                                                float *__restrict__ dw) {
    __shared__ float part[8][33];
    const int ls = sh.ls;
    const int i = blockIdx.x * 32 + threadIdx.x;  // 0 .. 7*ls
    float s = 0.0f;
    if (i < 7 * ls)
        for (int c = threadIdx.y; c < chunks; c += 8) s += ws[(size_t)c * 7 * ls + i];
    part[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y != 0 || i >= 7 * ls) return;
    float t = 0.0f;
#pragma unroll
    for (int y = 0; y < 8; ++y) t += part[y][threadIdx.x];
    const LstmOffsets off = lstm_offsets(sh.pls, ls, sh.els);
    int which = i / ls, u = i % ls;
    if (which < 4) dw[off.bias + (size_t)which * ls + u] = sh.bias * t;
    else dw[off.peep + (size_t)(which - 4) * ls + u] = t;
}

}  // namespace

int lstm_prepare_wrecT(const LstmShape &s, const float *w, float *wrecT, cudaStream_t st) {
    const LstmOffsets off = lstm_offsets(s.pls, s.ls, s.els);
    dim3 grid((s.els + 31) / 32, (s.els + 31) / 32, 4 * s.D), block(32, 8);
    wrec_transpose_kernel<<<grid, block, 0, st>>>(s.ls, s.els, s.D, w + off.rec, wrecT);
    count_launch();
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

int lstm_forward_stepwise(const LstmShape &s, const LstmBuffers &b, const float *w, float *y, cudaStream_t st) {
    dim3 grid((s.els + JT - 1) / JT, (s.P + PT - 1) / PT, s.D);
    for (int i = 0; i < s.T; ++i) lstm_fwd_step_kernel<<<grid, JT, 0, st>>>(s, b, w, y, i);
    count_launch(s.T);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

int lstm_backward_stepwise(const LstmShape &s, const LstmBuffers &b, const float *w, const float *dy,
                           cudaStream_t st) {
    dim3 grid((s.els + JT - 1) / JT, (s.P + PT - 1) / PT, s.D);
    for (int i = 0; i < s.T; ++i) lstm_bwd_step_kernel<<<grid, JT, 0, st>>>(s, b, w, dy, i);
    count_launch(s.T);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

int lstm_vector_grads(const LstmShape &s, const LstmBuffers &b, float *dw, float *ws, size_t ws_floats,
                      cudaStream_t st) {
    long N = (long)s.T * s.P;
    // chunks of frames: enough blocks to fill the device several times over, bounded by the scratch
    int fpc = 64;
    const long max_chunks = (long)(ws_floats / ((size_t)7 * s.ls));
    if (max_chunks < 1) {
        set_error("lstm_vector_grads: scratch too small");
        return B2_ERR_BAD_SHAPE;
    }
    if ((N + fpc - 1) / fpc > max_chunks) fpc = (int)((N + max_chunks - 1) / max_chunks);
    int chunks = (int)((N + fpc - 1) / fpc);
    dim3 grid((s.ls + 127) / 128, chunks);
    lstm_vgrad_partial_kernel<<<grid, 128, 0, st>>>(s, b, ws, fpc);
    lstm_vgrad_reduce_kernel<<<(7 * s.ls + 31) / 32, dim3(32, 8), 0, st>>>(s, chunks, ws, dw);
    count_launch(2);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

}  // namespace b2
