// b2_lstm: one peephole (B)LSTM layer working on the caller's buffers -- the C-ABI stand-in for
// layers::LstmLayer<Gpu> of the reference (layers/LstmLayer.hpp:168-308, LstmLayer.cu:1079-2382).
//
// Data layout in HBM (frames f = t*P + p, all fp32, column-major with the frame as column):
//   acts   [4*ls x T*P]  row c = g*ls + dir*els + j; written once by the fused input projection
//                        (all four gates, both directions = ONE GEMM, M = 4*ls), then overwritten
//                        in place by the recurrence with the post-activation ni, ig, fg, og
//   cells  [ls x T*P]    cell states, row dir*els + j
//   deltas [4*ls x T*P]  gate deltas, same rows as acts; operand of the dX and dW GEMMs
//   y      [ls x T*P]    block outputs straight in the caller's outputs() vector, forward units
//                        first (no separate per-direction copy, no resort pass)
// The reference keeps 12 vectors of T*P*els per direction (LstmLayer.cu:1184-1209); this keeps
// 9*ls floats per frame against its 12*ls (+2*ls for outputs and errors on both sides).
#include <new>

#include "common.cuh"
#include "lstm_layer.hpp"

namespace b2 {

namespace {
struct Phase {
    LstmLayerImpl &l;
    Phase(LstmLayerImpl &layer, const char *name) : l(layer) { if (l.prof_begin) l.prof_begin(l.prof_ctx, name); }
    ~Phase() { if (l.prof_end) l.prof_end(l.prof_ctx); }
};
}  // namespace

int LstmLayerImpl::create(const b2_lstm_desc &d) {
    desc = d;
    D = d.bidirectional ? 2 : 1;
    if (d.size <= 0 || d.prev_size <= 0 || d.parallel_sequences <= 0 || d.max_seq_length <= 0 ||
        (d.bidirectional && (d.size & 1))) {
        set_error("b2_lstm_create: bad descriptor (size %d prev %d P %d maxT %d bidirectional %d)", d.size,
                  d.prev_size, d.parallel_sequences, d.max_seq_length, d.bidirectional);
        return B2_ERR_BAD_SHAPE;
    }
    els = d.size / D;
    size_t frames = (size_t)d.max_seq_length * d.parallel_sequences;
    size_t ls = d.size;
    B2_CUDA(cudaMalloc(&bufs.acts, frames * 4 * ls * sizeof(float)));
    B2_CUDA(cudaMalloc(&bufs.cells, frames * ls * sizeof(float)));
    B2_CUDA(cudaMalloc(&bufs.deltas, frames * 4 * ls * sizeof(float)));
    B2_CUDA(cudaMalloc(&bufs.cerr, (size_t)2 * d.parallel_sequences * ls * sizeof(float)));
    B2_CUDA(cudaMalloc(&bufs.wrecT, (size_t)D * 4 * els * els * sizeof(float)));
    size_t vg = ((frames + 255) / 256) * 7 * ls;
    ws_floats = vg > ((size_t)6 << 20) ? vg : ((size_t)6 << 20);
    B2_CUDA(cudaMalloc(&ws, ws_floats * sizeof(float)));
    if (!scratch) { own_scratch = new TcScratch; scratch = own_scratch; }
    B2_CUDA(cudaMalloc(&status_dev, sizeof(int)));
    B2_CUDA(cudaMemset(status_dev, 0, sizeof(int)));
    size_t xw = lstm_persistent_xchg_words(els, d.parallel_sequences, D);
    if (xw) {
        B2_CUDA(cudaMalloc(&xchg, xw * sizeof(unsigned long long)));
        B2_CUDA(cudaMemset(xchg, 0, xw * sizeof(unsigned long long)));   // tag 0 is never waited for
    }
    state_bytes = xw * sizeof(unsigned long long) + (frames * 9 * ls + (size_t)2 * d.parallel_sequences * ls + (size_t)D * 4 * els * els + ws_floats) *
                  sizeof(float);
    // padding frames beyond the current fraction are never read, but start from defined memory
    B2_CUDA(cudaMemset(bufs.acts, 0, frames * 4 * ls * sizeof(float)));
    B2_CUDA(cudaMemset(bufs.cells, 0, frames * ls * sizeof(float)));
    B2_CUDA(cudaMemset(bufs.deltas, 0, frames * 4 * ls * sizeof(float)));
    return B2_OK;
}

void LstmLayerImpl::destroy() {
    cudaFree(bufs.acts); cudaFree(bufs.cells); cudaFree(bufs.deltas); cudaFree(bufs.cerr); cudaFree(bufs.wrecT);
    cudaFree(ws); cudaFree(xchg); cudaFree(status_dev); cudaFree(pad_dev);
    pad_dev = nullptr;
    cudaFree(tcrec.wrec_hi); cudaFree(tcrec.wrec_lo); cudaFree(tcrec.y_hi); cudaFree(tcrec.y_lo);
    cudaFree(tcrec.d_hi); cudaFree(tcrec.d_lo); cudaFree(tcrec.part);
    tcrec = TcRecBuffers();
    cudaFree(ptc.maxbits); cudaFree(ptc.scale); cudaFree(ptc.wimg_f); cudaFree(ptc.wimg_b); cudaFree(ptc.xh); cudaFree(ptc.xe); cudaFree(ptc.flags);
    ptc = PtcBuffers();
    if (own_scratch) { own_scratch->release(); delete own_scratch; own_scratch = nullptr; scratch = nullptr; }
    bufs = LstmBuffers();
    ws = nullptr; xchg = nullptr; status_dev = nullptr;
}

LstmShape LstmLayerImpl::shape() const {
    LstmShape s;
    s.P = desc.parallel_sequences; s.T = T; s.Tmin = Tmin; s.pls = desc.prev_size; s.ls = desc.size;
    s.els = els; s.D = D; s.bias = desc.bias;
    return s;
}

namespace {
// one thread per sequence slot: a padding frame (type NONE) followed by a frame that is not one
__global__ void padding_trails_kernel(const char *pat, int T, int P, int *bad) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= P) return;
    for (int t = 0; t + 1 < T; ++t)
        if (pat[(size_t)t * P + p] == PAT_NONE && pat[(size_t)(t + 1) * P + p] != PAT_NONE) { atomicExch(bad, t + 1); return; }
}
}  // namespace

int LstmLayerImpl::load_sequences(int cur_max, int cur_min, const char *pat) {
    if (cur_max <= 0 || cur_max > desc.max_seq_length || cur_min < 0 || cur_min > cur_max || !pat) {
        set_error("b2_lstm_load_sequences: lengths %d/%d outside 1..%d", cur_max, cur_min, desc.max_seq_length);
        return B2_ERR_BAD_SHAPE;
    }
    if (check_padding) {
        // The persistent kernels find a sequence's padding once per sweep and rely on it trailing the sequence, as
        // data_sets::DataSet writes it; the reference tests every frame (layers/LstmLayer.cu:89-101).  The check costs
        // a device round trip per fraction, hence optional.
        if (!pad_dev) B2_CUDA(cudaMalloc(&pad_dev, sizeof(int)));
        B2_CUDA(cudaMemset(pad_dev, 0, sizeof(int)));
        padding_trails_kernel<<<(desc.parallel_sequences + 127) / 128, 128>>>(pat, cur_max, desc.parallel_sequences, pad_dev);
        count_launch();
        int bad = 0;
        B2_CUDA(cudaMemcpy(&bad, pad_dev, sizeof(int), cudaMemcpyDeviceToHost));
        if (bad) {
            set_error("b2_lstm_load_sequences: a real frame follows a padding frame (timestep %d): padding must trail its sequence", bad);
            return B2_ERR_BAD_ARG;
        }
    }
    T = cur_max; Tmin = cur_min; bufs.pat = pat;
    forward_done = false;
    return B2_OK;
}

int LstmLayerImpl::forward(const float *w, const float *x, float *y, cudaStream_t st) {
    if (!T) { set_error("b2_lstm_forward: no sequences loaded"); return B2_ERR_STATE; }
    if (!w || !x || !y) { set_error("b2_lstm_forward: null pointer"); return B2_ERR_BAD_ARG; }
    const LstmShape s = shape();
    const int N = s.T * s.P, ls = s.ls, pls = s.pls;
    // input projection for all gates and both directions (reference: 4*D cublasSgemm calls,
    // LstmLayer.cu:1756-1775): acts(4ls x N) = W_in^T X, W_in viewed as ONE pls x 4ls matrix
    {
        Phase ph(*this, "lstm_proj_gemm");
        B2_TRY(gemm(bufs.acts, 4 * ls, w, pls, 1, x, 1, pls, 4 * ls, N, pls, false, st));
    }
    {
        Phase ph(*this, "lstm_fwd_recurrence");
        B2_TRY(lstm_prepare_wrecT(s, w, bufs.wrecT, st));
        int rc = 1;
        ptc_used = want_ptc();
        if (ptc_used) {
            B2_TRY(ensure_ptc());
            B2_TRY(lstm_ptc_prepare(s, w, ptc, st));
            rc = lstm_ptc_sweep(false, s, bufs, ptc, w, y, nullptr, status_dev, &tag_next, st);
            fwd_path = 5;
            if (rc == 1) ptc_used = false;
        }
        tcrec_used = !ptc_used && want_tc_recurrence();
        if (ptc_used) {
        } else if (tcrec_used) {
            B2_TRY(ensure_tcrec());
            rc = lstm_forward_tc(s, bufs, tcrec, w, y, status_dev, st);
            fwd_path = 3;
        } else if (recurrence_mode >= 1) {
            rc = lstm_persistent(false, persistent_transport(), s, bufs, w, y, nullptr, xchg, status_dev, &tag_next, st);
            fwd_path = 1;
        }
        if (rc == 1) { rc = lstm_forward_stepwise(s, bufs, w, y, st); fwd_path = 0; }
        B2_TRY(rc);
    }
    forward_done = true;
    return B2_OK;
}

int LstmLayerImpl::backward(const float *w, const float *x, const float *y, const float *dy, float *dx, float *dw,
                            cudaStream_t st) {
    if (!forward_done) { set_error("b2_lstm_backward: forward pass of this fraction has not run"); return B2_ERR_STATE; }
    if (!w || !x || !y || !dy || !dw) { set_error("b2_lstm_backward: null pointer"); return B2_ERR_BAD_ARG; }
    const LstmShape s = shape();
    const int N = s.T * s.P, ls = s.ls, pls = s.pls, P = s.P;
    const LstmOffsets off = lstm_offsets(pls, ls, els);
    {
        Phase ph(*this, "lstm_bwd_recurrence");
        int rc = 1;
        if (ptc_used && recurrence_mode != 6) {
            rc = lstm_ptc_sweep(true, s, bufs, ptc, w, nullptr, dy, status_dev, &tag_next, st);
            bwd_path = 5;
        }
        if (rc != 1) {
        } else if (tcrec_used) { rc = lstm_backward_tc(s, bufs, tcrec, w, dy, status_dev, st); bwd_path = 3; }
        else if (recurrence_mode >= 1) {
            rc = lstm_persistent(true, persistent_transport(), s, bufs, w, nullptr, dy, xchg, status_dev, &tag_next, st);
            bwd_path = 1;
        }
        if (rc == 1) { rc = lstm_backward_stepwise(s, bufs, w, dy, st); bwd_path = 0; }
        B2_TRY(rc);
    }
    const int K = N - P;
    const bool tc = !force_ffma && scratch && gemm_wants_tc(1, pls, 4 * ls, 1, pls, 4 * ls, N);
    SplitOperand sD{}, sX{}, sY{}, sW{};
    if (tc) {
        // every operand of the four contractions is split into hi/lo parts ONCE and reused:
        // deltas feed dX, dW_in and dW_rec; the layouts [frame][unit] serve both as K-major and
        // as MN-major operands, only the role of the contiguous index changes
        Phase ph(*this, "lstm_split_tf32");
        const bool f16 = !tcrec_used;   // the per-timestep tensor-core recurrence leaves tf32 parts: its partners follow
        B2_TRY(scratch->reserve(split_floats(N, 4 * ls, f16) + split_floats(N, pls, f16) + split_floats(N, ls, f16) +
                                split_floats(4 * ls, pls, f16)));
        scratch->used = 0;
        if (tcrec_used) {
            // the tensor-core recurrence has already written the hi/lo parts of the deltas and of y
            sD.hi = tcrec.d_hi; sD.lo = tcrec.d_lo; sD.ld = 4 * ls; sD.kmajor = true;
            sY.hi = tcrec.y_hi; sY.lo = tcrec.y_lo; sY.ld = ls; sY.kmajor = false;
        } else {
            // the gate deltas are clipped to [-1, 1] (helpers/limitedError.cuh of the reference), |h| = |tanh(c) * og| < 1
            B2_TRY(split_operand(*scratch, bufs.deltas, 4 * ls, N, 4 * ls, true, &sD, st, true, 1.0f));
            B2_TRY(split_operand(*scratch, y, ls, N, ls, false, &sY, st, true, 1.0f));
        }
        B2_TRY(split_operand(*scratch, x, pls, N, pls, false, &sX, st, f16));
        B2_TRY(split_operand(*scratch, w, pls, 4 * ls, pls, false, &sW, st, f16));
    }
    // error to the preceding layer (reference: 4*D Sgemm, LstmLayer.cu:2298-2334): dX = W_in * deltas
    if (dx) {
        Phase ph(*this, "lstm_dx_gemm");
        if (tc) {
            SplitOperand A = sW, B = sD;
            A.kmajor = false; B.kmajor = true;
            B2_TRY(gemm_tc(dx, pls, A, B, pls, N, 4 * ls, false, ws, ws_floats, status_dev, st));
        } else {
            B2_TRY(gemm(dx, pls, w, 1, pls, bufs.deltas, 1, 4 * ls, pls, N, 4 * ls, false, st));
        }
    }
    // input weight gradients (reference: one thread per weight, serial over frames,
    // LstmLayer.cu:490-522): dW_in(pls x 4ls) = X * deltas^T, written straight into the weight layout
    {
        Phase ph(*this, "lstm_dw_in_gemm");
        if (tc) {
            SplitOperand A = sX, B = sD;
            A.kmajor = false; B.kmajor = false;
            B2_TRY(gemm_tc(dw, pls, A, B, pls, 4 * ls, N, false, ws, ws_floats, status_dev, st));
        } else {
            B2_TRY(gemm(dw, pls, x, 1, pls, bufs.deltas, 4 * ls, 1, pls, 4 * ls, N, false, st));
        }
    }
    // recurrent weight gradients (LstmLayer.cu:543-572,629-636): for gate g, direction d
    //   dW_rec[g][d](k, j) = sum_f h_d[k; f -/+ P] * delta_g,d[j; f], skipping the first (last) timestep
    {
        Phase ph(*this, "lstm_dw_rec_gemm");
        const bool tc_rec = tc && (els % 4) == 0 && gemm_wants_tc(1, ls, 4 * ls, 1, els, els, K);
        bool done = false;
        if (tc_rec && 4 * D <= 8) {
            // all 4*D products in ONE batched launch: batch = (direction, gate); K is split so that the
            // work items fill a whole number of waves; partial sums go to scratch and are added in fixed order
            const int tiles = ((els + 127) / 128) * ((els + 127) / 128) * 4 * D;
            const int sms = tc_sm_count();
            const size_t per = (size_t)els * els;
            int splits = 0;
            double best = 0.0;
            for (int sp = 1; sp <= 64 && (size_t)sp * 4 * D * per <= ws_floats && (long)sp * 256 <= K; ++sp) {
                const int waves = (tiles * sp + sms - 1) / sms;
                const double t = waves * (0.4 * ((K + sp - 1) / sp) / 64.0 + 3.0) + (double)sp * 4 * D * per * 8.0 / 5.0e6;
                if (!splits || t < best) { best = t; splits = sp; }
            }
            if (splits >= 1) {
                SplitOperand A = sY, B = sD;
                A.kmajor = false; B.kmajor = false;
                TcPlan *plan = nullptr;
                B2_TRY(tc_plan_create(&plan, A, ls, N, B, 4L * ls, N, els, els, K, splits, 0, 0, els));
                TcBatch bt[8];
                long long coff[8];
                for (int d = 0; d < D; ++d)
                    for (int g = 0; g < 4; ++g) {
                        TcBatch &b = bt[d * 4 + g];
                        b.a_in = d * els; b.a_out = d ? P : 0;                 // h of the previous step in sweep order
                        b.b_in = g * ls + d * els; b.b_out = d ? 0 : P;
                        b.c_off = (long long)(d * 4 + g) * splits * (long long)per;
                        coff[d * 4 + g] = (long long)(off.rec + ((size_t)g * ls + (size_t)d * els) * els);
                    }
                int rc = tc_plan_launch(plan, ws, bt, 4 * D, (long long)per, status_dev, st);
                tc_plan_destroy(plan);
                B2_TRY(rc);
                B2_TRY(tc_batched_reduce(dw, coff, 4 * D, els, ws, els, els, splits, st));
                done = true;
            }
        }
        for (int d = 0; d < D && !done; ++d)
            for (int g = 0; g < 4; ++g) {
                float *C = dw + off.rec + ((size_t)g * ls + (size_t)d * els) * els;
                if (tc_rec) {
                    SplitOperand A = sY, B = sD;
                    const size_t ao = (size_t)d * els + (d ? (size_t)P * sY.ld : 0);
                    const size_t bo = (size_t)g * ls + (size_t)d * els + (d ? 0 : (size_t)P * sD.ld);
                    A.advance(ao); A.kmajor = false;
                    B.advance(bo); B.kmajor = false;
                    B2_TRY(gemm_tc(C, els, A, B, els, els, K, false, ws, ws_floats, status_dev, st));
                } else {
                    const float *A = y + (size_t)d * els + (d ? (size_t)P * ls : 0);
                    const float *B = bufs.deltas + (size_t)g * ls + (size_t)d * els + (d ? 0 : (size_t)P * 4 * ls);
                    B2_TRY(gemm_ffma(C, els, A, 1, ls, B, 4 * ls, 1, els, els, K, false, ws, ws_floats, st));
                }
            }
    }
    Phase ph(*this, "lstm_vector_grads");
    B2_TRY(lstm_vector_grads(s, bufs, dw, ws, ws_floats, st));
    return B2_OK;
}

// Which recurrence runs.  Mode 3 forces the tensor-core recurrence where the shape allows it; the
// default (mode 1) picks it when the persistent kernel would need many passes of expensive steps:
// measured on B200 a persistent step costs about 1.4 us + 0.27 us per sequence of a work item, a
// tensor-core step (GEMM + gate kernel, two launches) about 10 us whatever the batch.
bool LstmLayerImpl::want_tc_recurrence() const {
    const LstmShape s = shape();
    if (force_ffma || !lstm_tc_supported(s) || (desc.size % 4) != 0) return false;
    if (recurrence_mode == 3) return true;
    if (recurrence_mode != 1 || s.P < 16) return false;
    const int ps = persistent_ps(s.els, s.P, s.D, false);
    if (ps == 0) return s.els >= 256;
    int JB = 0;
    persistent_geometry(s.els, &JB);
    int slots = sm_count() / (s.els / JB);
    if (slots < 1) slots = 1;
    const int items = s.D * ((s.P + ps - 1) / ps);
    const int passes = (items + slots - 1) / slots;
    return passes * (1.4 + 0.27 * ps) > 12.0;
}

// The persistent tensor-core kernels serve 512 units per direction.  Modes 5 and 6 force them; the default (mode 1)
// takes them from 16 parallel sequences on: measured on B200 with 32 sequences a step costs 4.5 us against 6.1 us of
// the register-resident FFMA kernels, and the gap widens with the batch (the FFMA kernels' step grows by 0.27 us per
// sequence of a work item).  Below that the FFMA kernels have the shorter step (1.65 us for one sequence).
bool LstmLayerImpl::want_ptc() const {
    const LstmShape s = shape();
    if (force_ffma || !lstm_ptc_supported(s)) return false;
    if (recurrence_mode == 5 || recurrence_mode == 6) return true;
    return recurrence_mode == 1 && s.P >= 16;
}

int LstmLayerImpl::ensure_ptc() {
    if (ptc.wimg_f) return B2_OK;
    const size_t img = lstm_ptc_image_bytes(els, D);
    size_t xh = 0, xe = 0, nf = 0;
    lstm_ptc_exchange_sizes(els, desc.parallel_sequences, D, &xh, &xe, &nf);
    B2_CUDA(cudaMalloc(&ptc.maxbits, 2 * sizeof(unsigned)));
    B2_CUDA(cudaMalloc(&ptc.scale, 4 * sizeof(float)));
    B2_CUDA(cudaMalloc(&ptc.wimg_f, img));
    B2_CUDA(cudaMalloc(&ptc.wimg_b, img));
    B2_CUDA(cudaMalloc(&ptc.xh, xh));
    B2_CUDA(cudaMalloc(&ptc.xe, xe * sizeof(float)));
    B2_CUDA(cudaMalloc(&ptc.flags, nf * sizeof(unsigned)));
    B2_CUDA(cudaMemset(ptc.xh, 0, xh));
    B2_CUDA(cudaMemset(ptc.xe, 0, xe * sizeof(float)));
    B2_CUDA(cudaMemset(ptc.flags, 0, nf * sizeof(unsigned)));   // step counters start below every tag (tags start at 1)
    state_bytes += 2 * img + xh + xe * sizeof(float) + nf * sizeof(unsigned);
    return B2_OK;
}

int LstmLayerImpl::ensure_tcrec() {
    if (tcrec.y_hi) return B2_OK;
    const size_t frames = (size_t)desc.max_seq_length * desc.parallel_sequences, ls = desc.size;
    B2_CUDA(cudaMalloc(&tcrec.wrec_hi, (size_t)4 * ls * els * sizeof(float)));
    B2_CUDA(cudaMalloc(&tcrec.wrec_lo, (size_t)4 * ls * els * sizeof(float)));
    B2_CUDA(cudaMalloc(&tcrec.y_hi, frames * ls * sizeof(float)));
    B2_CUDA(cudaMalloc(&tcrec.y_lo, frames * ls * sizeof(float)));
    B2_CUDA(cudaMalloc(&tcrec.d_hi, frames * 4 * ls * sizeof(float)));
    B2_CUDA(cudaMalloc(&tcrec.d_lo, frames * 4 * ls * sizeof(float)));
    B2_CUDA(cudaMalloc(&tcrec.part, lstm_tc_part_floats(desc.parallel_sequences, els, D) * sizeof(float)));
    state_bytes += (frames * 10 * ls + (size_t)8 * ls * els + lstm_tc_part_floats(desc.parallel_sequences, els, D)) * sizeof(float);
    return B2_OK;
}

int LstmLayerImpl::check_status(cudaStream_t st) {
    int v = 0;
    B2_CUDA(cudaMemcpyAsync(&v, status_dev, sizeof(int), cudaMemcpyDeviceToHost, st));
    B2_CUDA(cudaStreamSynchronize(st));
    if (v != 0) {
        B2_CUDA(cudaMemsetAsync(status_dev, 0, sizeof(int), st));
        set_error("a kernel of this layer gave up a bounded wait (status %d)", v);
        return v;
    }
    return B2_OK;
}

int LstmLayerImpl::gemm(float *C, long ldc, const float *A, long sam, long sak, const float *B, long sbk, long sbn,
                        int m, int n, int k, bool acc, cudaStream_t st) {
    return gemm_auto(C, ldc, A, sam, sak, B, sbk, sbn, m, n, k, acc, force_ffma, scratch, ws, ws_floats, status_dev, st);
}

}  // namespace b2

using b2::LstmLayerImpl;
struct b2_lstm {
    LstmLayerImpl impl;
};

extern "C" {

int b2_selftest_bounded_wait(int *status_out, int *gave_up) {
    return b2::lstm_selftest_bounded_wait(status_out, gave_up, nullptr);
}


size_t b2_lstm_num_weights(const b2_lstm_desc *d) {
    if (!d) return 0;
    size_t ls = d->size, pls = d->prev_size, els = d->bidirectional ? ls / 2 : ls;
    return ls * (4 * (pls + 1) + 4 * els + 3);
}

int b2_lstm_create(const b2_lstm_desc *desc, b2_lstm **out) {
    if (!desc || !out) { b2::set_error("b2_lstm_create: null argument"); return B2_ERR_BAD_ARG; }
    b2_lstm *l = new (std::nothrow) b2_lstm;
    if (!l) return B2_ERR_BAD_ARG;
    int rc = l->impl.create(*desc);
    if (rc != B2_OK) { l->impl.destroy(); delete l; return rc; }
    *out = l;
    return B2_OK;
}

void b2_lstm_destroy(b2_lstm *l) {
    if (!l) return;
    l->impl.destroy();
    delete l;
}

int b2_lstm_load_sequences(b2_lstm *l, int cur_max_len, int cur_min_len, const char *pat_types_dev) {
    if (!l) return B2_ERR_BAD_ARG;
    return l->impl.load_sequences(cur_max_len, cur_min_len, pat_types_dev);
}

int b2_lstm_forward(b2_lstm *l, const float *w, const float *x, float *y, b2_stream st) {
    if (!l) return B2_ERR_BAD_ARG;
    return l->impl.forward(w, x, y, (cudaStream_t)st);
}

int b2_lstm_backward(b2_lstm *l, const float *w, const float *x, const float *y, const float *dy, float *dx,
                     float *dw, b2_stream st) {
    if (!l) return B2_ERR_BAD_ARG;
    return l->impl.backward(w, x, y, dy, dx, dw, (cudaStream_t)st);
}

int b2_lstm_set_check_padding(b2_lstm *l, int on) {
    if (!l) return B2_ERR_BAD_ARG;
    l->impl.check_padding = on != 0;
    return B2_OK;
}

int b2_lstm_set_recurrence_mode(b2_lstm *l, int mode) {
    if (!l) return B2_ERR_BAD_ARG;
    l->impl.recurrence_mode = mode;
    return B2_OK;
}

size_t b2_lstm_state_bytes(const b2_lstm *l) { return l ? l->impl.state_bytes : 0; }

int b2_lstm_recurrence_path(const b2_lstm *l, int backward) {
    if (!l) return -1;
    return backward ? l->impl.bwd_path : l->impl.fwd_path;
}

int b2_lstm_synchronize(b2_lstm *l, b2_stream st) {
    if (!l) return B2_ERR_BAD_ARG;
    return l->impl.check_status((cudaStream_t)st);
}

}  // extern "C"
