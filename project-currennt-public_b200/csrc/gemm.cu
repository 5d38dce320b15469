// GEMM dispatch: the one place that decides between the tensor-core kernel (gemm_tc.cu) and the
// FFMA kernel (gemm_ffma.cu), and the arena that holds the hi/lo operand copies of the former.
#include "common.cuh"

namespace b2 {

int TcScratch::reserve(size_t floats) {
    if (floats <= cap) return B2_OK;
    // cudaFree waits for all outstanding work, so nothing still reads the old arena
    if (base) B2_CUDA(cudaFree(base));
    base = nullptr;
    cap = 0;
    size_t want = floats + floats / 8;
    B2_CUDA(cudaMalloc(&base, want * sizeof(float)));
    cap = want;
    return B2_OK;
}
void TcScratch::release() {
    if (base) cudaFree(base);
    base = nullptr;
    cap = used = 0;
}
float *TcScratch::take(size_t floats) {
    floats = (floats + 63) & ~(size_t)63;   // keep every piece 256-byte aligned
    if (used + floats > cap) return nullptr;
    float *p = base + used;
    used += floats;
    return p;
}

// split a strided matrix view whose contiguous index has `inner` entries and whose other index has
// `outer` entries `s_outer` floats apart; returns the dense operand description
int split_operand(TcScratch &sc, const float *src, long s_outer, int outer, int inner, bool kmajor, SplitOperand *out,
                  cudaStream_t st, bool f16, float bound) {
    if (!f16) {
        const long ldp = (inner + 3) & ~3L;
        float *hi = sc.take((size_t)outer * ldp), *lo = sc.take((size_t)outer * ldp);
        if (!hi || !lo) { set_error("split_operand: operand arena exhausted"); return B2_ERR_BAD_SHAPE; }
        B2_TRY(split_tf32(src, s_outer, outer, inner, hi, lo, ldp, st));
        *out = SplitOperand{};
        out->hi = hi; out->lo = lo; out->ld = ldp; out->kmajor = kmajor;
        return B2_OK;
    }
    // fp16 parts: rows padded to 8 halves (16 bytes, what a tensor map wants of a row pitch)
    const long ldp = (inner + 7) & ~7L;
    const size_t part = ((size_t)outer * ldp + 1) / 2;   // floats that hold one part
    float *hi = sc.take(part), *lo = sc.take(part), *mx = sc.take(1);
    if (!hi || !lo || !mx) { set_error("split_operand: operand arena exhausted"); return B2_ERR_BAD_SHAPE; }
    B2_TRY(split_f16(src, s_outer, outer, inner, hi, lo, ldp, (unsigned *)mx, st, bound));
    out->hi = hi; out->lo = lo; out->ld = ldp; out->kmajor = kmajor;
    out->f16 = true; out->maxbits = (const unsigned *)mx;
    return B2_OK;
}

size_t split_floats(int outer, int inner, bool f16) {
    if (!f16) {
        const size_t ldp = (size_t)((inner + 3) & ~3);
        return 2 * (((size_t)outer * ldp + 63) & ~(size_t)63);
    }
    const size_t ldp = (size_t)((inner + 7) & ~7);
    const size_t part = ((size_t)outer * ldp + 1) / 2;
    return 2 * ((part + 63) & ~(size_t)63) + 64;
}

bool gemm_wants_tc(long sam, long sak, long sbk, long sbn, int m, int n, int k) {
    if (m < 1 || n < 1 || k < 8) return false;
    if (!(sam == 1 || sak == 1) || !(sbk == 1 || sbn == 1)) return false;
    // tiny products are launch-latency-bound either way; keep them on the simple kernel
    return (double)m * n * k >= (double)(1 << 22);
}

int gemm_auto(float *C, long ldc, const float *A, long sam, long sak, const float *B, long sbk, long sbn, int m, int n, int k,
              bool accumulate, bool force_ffma, TcScratch *sc, float *ws, size_t ws_floats, int *status, cudaStream_t st) {
    if (force_ffma || !sc || !status || !gemm_wants_tc(sam, sak, sbk, sbn, m, n, k))
        return gemm_ffma(C, ldc, A, sam, sak, B, sbk, sbn, m, n, k, accumulate, ws, ws_floats, st);
    const bool a_k = (sak == 1), b_k = (sbk == 1);
    const int a_outer = a_k ? m : k, a_inner = a_k ? k : m;
    const int b_outer = b_k ? n : k, b_inner = b_k ? k : n;
    B2_TRY(sc->reserve(split_floats(a_outer, a_inner) + split_floats(b_outer, b_inner)));
    sc->used = 0;
    SplitOperand sa, sb;
    B2_TRY(split_operand(*sc, A, a_k ? sam : sak, a_outer, a_inner, a_k, &sa, st));
    B2_TRY(split_operand(*sc, B, b_k ? sbn : sbk, b_outer, b_inner, b_k, &sb, st));
    return gemm_tc(C, ldc, sa, sb, m, n, k, accumulate, ws, ws_floats, status, st);
}

}  // namespace b2
