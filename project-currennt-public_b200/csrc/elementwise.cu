// HBM-bound elementwise and reduction kernels around the LSTM stack: feed-forward bias +
// activation and delta, column sums (bias gradients), the SSE objective and its gradient, and the
// steepest-descent update.  Reference counterparts (paths inside CURRENNT_codes/currennt_lib/src/):
//   layers/FeedForwardLayer.cu:53-74 (ComputeOutputFn), :106-116 (ComputeDeltaFn),
//                              :118-138 (ComputeBiasWeightUpdateFn)
//   layers/SsePostOutputLayer.cu:94-136 (ComputeSseFn, ComputeOutputErrorFn)
//   optimizers/SteepestDescentOptimizer.cu:74-100 (UpdateWeightFn)
// Grids are sized in multiples of the 148 SMs and grid-stride over the data with 128-bit accesses
// where the alignment allows.
#include "common.cuh"

namespace b2 {
namespace {

constexpr int SMS = 148;

__device__ __forceinline__ float apply_act(int act, float a) {
    return act == ACT_TANH ? act_tanh(a) : (act == ACT_LOGISTIC ? act_logistic(a) : a);
}
__device__ __forceinline__ float apply_deriv(int act, float y) {
    return act == ACT_TANH ? d_tanh(y) : (act == ACT_LOGISTIC ? d_logistic(y) : 1.0f);
}

__global__ void ff_bias_act_kernel(float *__restrict__ y, const float *__restrict__ b, float bias, int ls, size_t n,
                                   int act) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    if ((ls & 3) == 0) {
        size_t n4 = n / 4;
        float4 *y4 = reinterpret_cast<float4 *>(y);
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
            float4 v = y4[i];
            int u = (int)((i * 4) % ls);
            v.x = apply_act(act, v.x + bias * __ldg(b + u));
            v.y = apply_act(act, v.y + bias * __ldg(b + u + 1));
            v.z = apply_act(act, v.z + bias * __ldg(b + u + 2));
            v.w = apply_act(act, v.w + bias * __ldg(b + u + 3));
            y4[i] = v;
        }
    } else {
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
            y[i] = apply_act(act, y[i] + bias * __ldg(b + (i % ls)));
    }
}

__global__ void ff_delta_kernel(float *__restrict__ err, const float *__restrict__ y, size_t n, int act) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t n4 = n / 4;
    float4 *e4 = reinterpret_cast<float4 *>(err);
    const float4 *y4 = reinterpret_cast<const float4 *>(y);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 e = e4[i], v = y4[i];
        e.x *= apply_deriv(act, v.x); e.y *= apply_deriv(act, v.y);
        e.z *= apply_deriv(act, v.z); e.w *= apply_deriv(act, v.w);
        e4[i] = e;
    }
    for (size_t i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        err[i] = apply_deriv(act, y[i]) * err[i];
}

__global__ void column_sums_partial_kernel(float *__restrict__ ws, const float *__restrict__ m, long ld, int cols,
                                           long rows, int rows_per_chunk) {
    int u = blockIdx.x * blockDim.x + threadIdx.x;
    if (u >= cols) return;
    long r0 = (long)blockIdx.y * rows_per_chunk, r1 = min(rows, r0 + rows_per_chunk);
    float s = 0.0f;
#pragma unroll 8
    for (long r = r0; r < r1; ++r) s += m[(size_t)r * ld + u];
    ws[(size_t)blockIdx.y * cols + u] = s;
}
// 32 columns x 8 chunk phases per block: phase y adds chunks y, y+8, ...; the 8 sums are added in fixed order
__global__ void __launch_bounds__(256) column_sums_reduce_kernel(float *__restrict__ out, const float *__restrict__ ws, int cols,
                                                                 int chunks, float scale) {
    __shared__ float part[8][33];
    const int u = blockIdx.x * 32 + threadIdx.x;
    float s = 0.0f;
    if (u < cols)
        for (int c = threadIdx.y; c < chunks; c += 8) s += ws[(size_t)c * cols + u];
    part[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && u < cols) {
        float t = 0.0f;
#pragma unroll
        for (int y = 0; y < 8; ++y) t += part[y][threadIdx.x];
        out[u] = scale * t;
    }
}

__global__ void sse_partial_kernel(double *__restrict__ ws, const float *__restrict__ y, const float *__restrict__ tgt,
                                   const char *__restrict__ pat, int ls, size_t n) {
    float s = 0.0f;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        if (pat[i / ls] == PAT_NONE) continue;
        float d = tgt[i] - y[i];
        s = fmaf(d, d, s);
    }
    double v = (double)s;
    __shared__ double red[32];
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.0;
        for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
        if (threadIdx.x == 0) ws[blockIdx.x] = v;
    }
}
__global__ void sse_final_kernel(double *__restrict__ loss, const double *__restrict__ ws, int blocks) {
    double v = 0.0;
    for (int i = threadIdx.x; i < blocks; i += 32) v += ws[i];
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    if (threadIdx.x == 0) *loss = 0.5 * v;
}

__global__ void sse_grad_kernel(float *__restrict__ dy, const float *__restrict__ y, const float *__restrict__ tgt,
                                const char *__restrict__ pat, int ls, size_t n) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        dy[i] = pat[i / ls] == PAT_NONE ? 0.0f : y[i] - tgt[i];
}

__global__ void sgd_update_kernel(float *__restrict__ w, float *__restrict__ g, float *__restrict__ delta, size_t n,
                                  float lr, float mom) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float gi = g[i];
        if (isnan(gi) || isinf(gi)) { gi = 0.0f; g[i] = 0.0f; }
        float dl = mom * delta[i] - lr * gi;
        delta[i] = dl;
        w[i] = w[i] + dl;
    }
}

// Gradient shaping of SteepestDescentOptimizer::_updateWeights (SteepestDescentOptimizer.cu:127-194,
// 306-395) fused with the update functor: option 1 AdaGrad, 2 average over the fraction's frames,
// 3 SGD that only accumulates the AdaGrad statistics, 5 Adam (constants of MacroDefine.hpp:39-42).
__global__ void sgd_update_opt_kernel(float *__restrict__ w, float *__restrict__ g, float *__restrict__ delta,
                                      float *__restrict__ stats, size_t n, float lr, float mom, int option,
                                      const float *__restrict__ frac_len, float beta1_accum, float beta2_accum) {
    const float fracLength = *frac_len;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float gi = g[i];
        if (isnan(gi) || isinf(gi)) { gi = 0.0f; g[i] = 0.0f; }
        const float ave = gi / fracLength;
        if (option == 2) {
            gi = ave;
        } else if (option == 1 || option == 3) {
            const float st = stats[i] + ave * ave;
            stats[i] = st;
            if (option == 1) gi = ave / sqrtf(st);
        } else if (option == 5) {
            const float m = stats[2 * i] * 0.9f + ave * (1.0f - 0.9f);
            const float v = stats[2 * i + 1] * 0.999f + ave * ave * (1.0f - 0.999f);
            stats[2 * i] = m;
            stats[2 * i + 1] = v;
            gi = (m / (1.0f - beta1_accum)) / (sqrtf(v / (1.0f - beta2_accum)) + 0.00000001f);
        }
        float dl = mom * delta[i] - lr * gi;
        delta[i] = dl;
        w[i] = w[i] + dl;
    }
}
// m_curWeightUpdates of batch learning (optimizers/Optimizer.cu:186-196): copy on the first fraction, add after
__global__ void accumulate_kernel(float *__restrict__ acc, const float *__restrict__ g, size_t n, int first) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) acc[i] = first ? g[i] : acc[i] + g[i];
}
__global__ void fill_value_kernel(float *p, size_t n, float v) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = v;
}

inline int grid_for(size_t n, int threads, int per_sm = 8) {
    size_t b = (n + threads - 1) / threads;
    size_t cap = (size_t)SMS * per_sm;
    if (b > cap) b = cap;
    if (b < 1) b = 1;
    return (int)b;
}

}  // namespace

int fill_zero(void *p, size_t bytes, cudaStream_t st) {
    if (!bytes) return B2_OK;
    B2_CUDA(cudaMemsetAsync(p, 0, bytes, st));
    return B2_OK;
}

int ff_bias_act(float *y, const float *b, float bias, int ls, size_t n, int act, cudaStream_t st) {
    if (!n) return B2_OK;
    ff_bias_act_kernel<<<grid_for(n / 4 + 1, 256), 256, 0, st>>>(y, b, bias, ls, n, act);
    count_launch();
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

int ff_delta(float *err, const float *y, size_t n, int act, cudaStream_t st) {
    if (!n || act == ACT_IDENTITY) return B2_OK;  // identity: deriv = 1, delta = err unchanged
    ff_delta_kernel<<<grid_for(n / 4 + 1, 256), 256, 0, st>>>(err, y, n, act);
    count_launch();
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

int column_sums(float *out, const float *m, long ld, int cols, long rows, float scale, float *ws, size_t ws_floats,
                cudaStream_t st) {
    // rows (frames) per partial sum: enough blocks to fill the device several times, bounded by the scratch
    int rpc = 64;
    const long max_chunks = cols > 0 ? (long)(ws_floats / (size_t)cols) : 0;
    if (max_chunks < 1) {
        set_error("column_sums: scratch too small");
        return B2_ERR_BAD_SHAPE;
    }
    if ((rows + rpc - 1) / rpc > max_chunks) rpc = (int)((rows + max_chunks - 1) / max_chunks);
    int chunks = (int)((rows + rpc - 1) / rpc);
    if (chunks < 1) chunks = 1;
    dim3 grid((cols + 127) / 128, chunks);
    column_sums_partial_kernel<<<grid, 128, 0, st>>>(ws, m, ld, cols, rows, rpc);
    column_sums_reduce_kernel<<<(cols + 31) / 32, dim3(32, 8), 0, st>>>(out, ws, cols, chunks, scale);
    count_launch(2);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

int sse_loss(double *loss_dev, const float *y, const float *tgt, const char *pat, int ls, size_t frames, double *ws,
             cudaStream_t st) {
    size_t n = frames * (size_t)ls;
    int blocks = grid_for(n, 256, 4);  // <= 592 partials; ws holds 1024 doubles
    sse_partial_kernel<<<blocks, 256, 0, st>>>(ws, y, tgt, pat, ls, n);
    sse_final_kernel<<<1, 32, 0, st>>>(loss_dev, ws, blocks);
    count_launch(2);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

int sse_grad(float *dy, const float *y, const float *tgt, const char *pat, int ls, size_t frames, cudaStream_t st) {
    size_t n = frames * (size_t)ls;
    if (!n) return B2_OK;
    sse_grad_kernel<<<grid_for(n, 256), 256, 0, st>>>(dy, y, tgt, pat, ls, n);
    count_launch();
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

int sgd_update(float *w, float *g, float *delta, size_t n, float lr, float mom, cudaStream_t st) {
    if (!n) return B2_OK;
    sgd_update_kernel<<<grid_for(n, 256), 256, 0, st>>>(w, g, delta, n, lr, mom);
    count_launch();
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

int sgd_update_opt(float *w, float *g, float *delta, float *stats, size_t n, float lr, float mom, int option,
                   const float *frac_len_dev, float beta1_accum, float beta2_accum, cudaStream_t st) {
    if (!n) return B2_OK;
    sgd_update_opt_kernel<<<grid_for(n, 256), 256, 0, st>>>(w, g, delta, stats, n, lr, mom, option, frac_len_dev, beta1_accum,
                                                         beta2_accum);
    count_launch();
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

int accumulate(float *acc, const float *g, size_t n, bool first, cudaStream_t st) {
    if (!n) return B2_OK;
    accumulate_kernel<<<grid_for(n, 256), 256, 0, st>>>(acc, g, n, first ? 1 : 0);
    count_launch();
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

int fill_value(float *p, size_t n, float v, cudaStream_t st) {
    if (!n) return B2_OK;
    fill_value_kernel<<<grid_for(n, 256), 256, 0, st>>>(p, n, v);
    count_launch();
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

}  // namespace b2
