// FFMA (CUDA-core fp32) GEMM with arbitrary operand strides.
//
// Stands where the reference calls helpers::Matrix::assignProduct/addProduct -> cublasSgemm
// (helpers/Matrix.cu:354-377, helpers/cublas.cu:52-84 of the reference) for shapes the
// tensor-core kernel does not take (ragged sizes, unaligned leading dimensions), and is the
// strict-fp32 comparison partner of that kernel.
//
// 128x128x16 tiles, 256 threads, 8x8 accumulators per thread, register prefetch of the next
// k-slab.  Optional split-K over gridDim.z into scratch followed by a fixed-order reduction, so
// the result does not depend on scheduling.
#include <atomic>

#include "common.cuh"

namespace b2 {
namespace {

constexpr int BM = 128, BN = 128, BK = 16, NT = 256;

// element (r, kk) of a tile whose rows have stride s_r and whose k index has stride s_k
// thread->element mapping follows the unit-stride dimension so that global loads coalesce
template <bool ROW_FAST>
__device__ __forceinline__ void load_tile(float (&reg)[8], const float *__restrict__ base, long s_r, long s_k,
                                          int r0, int rows, int k0, int kend, int tid) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int e = tid + i * NT;  // 0 .. 2047
        int r, kk;
        if (ROW_FAST) { r = e % 128; kk = e / 128; }
        else          { kk = e % BK; r = e / BK; }
        int gr = r0 + r, gk = k0 + kk;
        reg[i] = (gr < rows && gk < kend) ? __ldg(base + (long)gr * s_r + (long)gk * s_k) : 0.0f;
    }
}
template <bool ROW_FAST>
__device__ __forceinline__ void store_tile(const float (&reg)[8], float (*sm)[BM + 4], int tid) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int e = tid + i * NT;
        int r, kk;
        if (ROW_FAST) { r = e % 128; kk = e / 128; }
        else          { kk = e % BK; r = e / BK; }
        sm[kk][r] = reg[i];
    }
}

template <bool A_ROW_FAST, bool B_COL_FAST>
__global__ void __launch_bounds__(NT) gemm_ffma_kernel(float *__restrict__ C, long ldc, const float *__restrict__ A,
                                                       long sam, long sak, const float *__restrict__ B, long sbk,
                                                       long sbn, int M, int N, int K, int kchunk, int accumulate,
                                                       float *__restrict__ ws) {
    __shared__ __align__(16) float As[BK][BM + 4];
    __shared__ __align__(16) float Bs[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    const int kbeg = blockIdx.z * kchunk;
    const int kend = min(K, kbeg + kchunk);

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

    float ra[8], rb[8];
    load_tile<A_ROW_FAST>(ra, A, sam, sak, m0, M, kbeg, kend, tid);
    load_tile<B_COL_FAST>(rb, B, sbn, sbk, n0, N, kbeg, kend, tid);

    for (int k0 = kbeg; k0 < kend; k0 += BK) {
        store_tile<A_ROW_FAST>(ra, As, tid);
        store_tile<B_COL_FAST>(rb, Bs, tid);
        __syncthreads();
        if (k0 + BK < kend) {
            load_tile<A_ROW_FAST>(ra, A, sam, sak, m0, M, k0 + BK, kend, tid);
            load_tile<B_COL_FAST>(rb, B, sbn, sbk, n0, N, k0 + BK, kend, tid);
        }
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[8], b[8];
            *(float4 *)&a[0] = *(const float4 *)&As[kk][tx * 4];
            *(float4 *)&a[4] = *(const float4 *)&As[kk][64 + tx * 4];
            *(float4 *)&b[0] = *(const float4 *)&Bs[kk][ty * 4];
            *(float4 *)&b[4] = *(const float4 *)&Bs[kk][64 + ty * 4];
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }

    // thread owns rows m0 + {tx*4..+3, 64+tx*4..+3}, cols n0 + {ty*4..+3, 64+ty*4..+3}
    const bool split = gridDim.z > 1;
    float *dst = split ? ws + (size_t)blockIdx.z * (size_t)M * N : C;
    const long ld = split ? (long)M : ldc;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        int n = n0 + (j < 4 ? ty * 4 + j : 64 + ty * 4 + (j - 4));
        if (n >= N) continue;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            int m = m0 + (i < 4 ? tx * 4 + i : 64 + tx * 4 + (i - 4));
            if (m >= M) continue;
            float v = acc[i][j];
            float *p = dst + (long)n * ld + m;
            if (!split && accumulate) v += *p;
            *p = v;
        }
    }
}

__global__ void splitk_reduce_kernel(float *__restrict__ C, long ldc, const float *__restrict__ ws, int M, int N,
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

}  // namespace

int gemm_ffma(float *C, long ldc, const float *A, long sam, long sak, const float *B, long sbk, long sbn, int m,
              int n, int k, bool accumulate, float *ws, size_t ws_floats, cudaStream_t st) {
    if (m <= 0 || n <= 0) return B2_OK;
    if (k <= 0) {
        if (!accumulate) {
            if (ldc == m) return fill_zero(C, (size_t)m * n * sizeof(float), st);
            for (int j = 0; j < n; ++j) B2_TRY(fill_zero(C + (size_t)j * ldc, (size_t)m * sizeof(float), st));
        }
        return B2_OK;
    }
    dim3 grid((m + BM - 1) / BM, (n + BN - 1) / BN, 1);
    // split K when the output tiles alone cannot fill the GPU and K is long
    int tiles = grid.x * grid.y;
    int splits = 1;
    const int sms = sm_count();
    if (ws && tiles < sms && k >= 2048) {
        splits = (2 * sms + tiles - 1) / tiles;
        int maxs = k / 512;
        if (splits > maxs) splits = maxs;
        size_t per = (size_t)m * n;
        if (per && (size_t)splits * per > ws_floats) splits = (int)(ws_floats / per);
        if (splits < 1) splits = 1;
    }
    int kchunk = (k + splits - 1) / splits;
    kchunk = (kchunk + BK - 1) / BK * BK;
    splits = (k + kchunk - 1) / kchunk;
    grid.z = splits;
    const bool a_row = (sam == 1), b_col = (sbn == 1);
#define LAUNCH(AR, BC)                                                                                     \
    gemm_ffma_kernel<AR, BC><<<grid, NT, 0, st>>>(C, ldc, A, sam, sak, B, sbk, sbn, m, n, k, kchunk, \
                                                  accumulate ? 1 : 0, ws)
    if (a_row && b_col) LAUNCH(true, true);
    else if (a_row) LAUNCH(true, false);
    else if (b_col) LAUNCH(false, true);
    else LAUNCH(false, false);
#undef LAUNCH
    count_launch();
    B2_CUDA(cudaGetLastError());
    if (splits > 1) {
        size_t total = (size_t)m * n;
        int blocks = (int)((total + 255) / 256);
        if (blocks > sms * 8) blocks = sms * 8;
        splitk_reduce_kernel<<<blocks, 256, 0, st>>>(C, ldc, ws, m, n, splits, accumulate ? 1 : 0);
        count_launch();
        B2_CUDA(cudaGetLastError());
    }
    return B2_OK;
}

}  // namespace b2

// ---- b2_matrix_multiply_noalloc ------------------------------------------------------------------
// The split-K scratch of the FFMA GEMM normally comes from cudaMalloc.  Some hosts cannot let a
// library do that: a training program that has handed all of HBM to its own pool (a caching
// allocator, or Thrust vectors sized to fill the card), where a further cudaMalloc fails or
// fragments; or a latency-sensitive loop in which cudaMalloc's device-wide synchronisation would
// stall work on other streams.  For them this entry point keeps the scratch in a fixed array that
// is part of the library image: every GPU that loads the library holds NOALLOC_SCRATCH_FLOATS * 4
// bytes (16 MiB) until the process exits.
//
// The array name is only a host-side handle; the kernel needs its device address, which differs per
// GPU.  It is looked up with cudaGetSymbolAddress the first time the entry point runs on a device
// (with that device current) and cached.  Make that first call outside any stream capture.
// All calls on a device share the array and find the previous call's partial sums in it: nothing in
// it has to start at zero, because a launch writes every partial it later reads, but two calls whose
// kernels overlap on the GPU (different streams) race on it -- serialise them.
// With lazy module loading the driver gives the array its memory when this module is first used on a device:
// make the first call before the host program claims the rest of HBM, or that call fails with an out-of-memory
// error.  The cached address belongs to the device's primary context: after cudaDeviceReset (or the loss of
// that context) it is stale, and the library must be reloaded.
namespace {
constexpr size_t NOALLOC_SCRATCH_FLOATS = (size_t)1 << 22;
constexpr size_t NOALLOC_MAX_MN = (size_t)1 << 21;   // largest m*n accepted: leaves room for a 2-way split
constexpr int NOALLOC_MAX_DEVICES = 64;
static __device__ __align__(256) float g_noalloc_scratch[NOALLOC_SCRATCH_FLOATS];
std::atomic<float *> g_noalloc_ptr[NOALLOC_MAX_DEVICES];   // device address of the array, per device ordinal
}  // namespace

extern "C" int b2_matrix_multiply_noalloc(float *C, int ldc, const float *A, int lda, int transA, const float *B, int ldb,
                                          int transB, int m, int n, int k, int accumulate, b2_stream stream) {
    using namespace b2;
    if (!C || !A || !B) { set_error("b2_matrix_multiply_noalloc: null pointer"); return B2_ERR_BAD_ARG; }
    if (transA && transB) {
        set_error("b2_matrix_multiply_noalloc: transposing both operands is not supported");
        return B2_ERR_BAD_ARG;
    }
    if (m < 0 || n < 0 || k < 0) {
        set_error("b2_matrix_multiply_noalloc: negative dimension (m %d, n %d, k %d)", m, n, k);
        return B2_ERR_BAD_ARG;
    }
    // leading dimensions must span a column of what they address: C is m x n; A is m x k (k x m when transposed)
    // and B is k x n (n x k when transposed), all column-major
    if (ldc < m || lda < (transA ? k : m) || ldb < (transB ? n : k)) {
        set_error("b2_matrix_multiply_noalloc: leading dimension too small (ldc %d, lda %d, ldb %d for m %d, n %d, k %d)",
                  ldc, lda, ldb, m, n, k);
        return B2_ERR_BAD_ARG;
    }
    if ((size_t)m * (size_t)n > NOALLOC_MAX_MN) {
        set_error("b2_matrix_multiply_noalloc: m*n = %zu exceeds the fixed scratch limit of %zu output elements",
                  (size_t)m * (size_t)n, NOALLOC_MAX_MN);
        return B2_ERR_BAD_SHAPE;
    }
    int dev = -1;
    B2_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) {
        set_error("b2_matrix_multiply_noalloc: device ordinal %d outside 0..%d", dev, NOALLOC_MAX_DEVICES - 1);
        return B2_ERR_BAD_ARG;
    }
    float *scratch = g_noalloc_ptr[dev].load(std::memory_order_acquire);
    if (!scratch) {
        // threads that race here all look up the same address; the last store wins, with the same value
        B2_CUDA(cudaGetSymbolAddress((void **)&scratch, g_noalloc_scratch));
        g_noalloc_ptr[dev].store(scratch, std::memory_order_release);
    }
    const long sam = transA ? lda : 1, sak = transA ? 1 : lda;
    const long sbk = transB ? ldb : 1, sbn = transB ? 1 : ldb;
    return gemm_ffma(C, ldc, A, sam, sak, B, sbk, sbn, m, n, k, accumulate != 0, scratch, NOALLOC_SCRATCH_FLOATS,
                     (cudaStream_t)stream);
}
