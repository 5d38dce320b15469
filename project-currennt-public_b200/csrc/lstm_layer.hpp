// Implementation object behind the opaque b2_lstm handle; also used directly by the layer stack.
#pragma once
#include "common.cuh"

namespace b2 {

struct LstmLayerImpl {
    b2_lstm_desc desc{};
    int D = 1, els = 0;
    int T = 0, Tmin = 0;
    bool forward_done = false;
    int recurrence_mode = 1;   // 0 stepwise, 1 persistent
    bool force_ffma = false;
    bool check_padding = false;   // load_sequences verifies that padding frames trail their sequences
    int *pad_dev = nullptr;       // result word of that check
    LstmBuffers bufs{};
    float *ws = nullptr;       // scratch: split-K partials, vector-gradient partials
    size_t ws_floats = 0;
    size_t state_bytes = 0;
    // arena for the tf32 hi/lo operand copies of the tensor-core GEMMs: the layer stack lends its
    // shared one (set before create()); a stand-alone layer makes its own
    TcScratch *scratch = nullptr, *own_scratch = nullptr;
    // persistent kernels: exchange buffers, device status word, running step tag
    unsigned long long *xchg = nullptr;
    int *status_dev = nullptr;
    unsigned tag_next = 1;
    // tensor-core recurrence (large batches): hi/lo buffers, allocated on first use
    TcRecBuffers tcrec{};
    // recurrence mode 1 lets the library choose, 2 forces clusters, 4 forces L2, 5 the persistent tensor-core
    // kernels, 6 those for the forward sweep only
    int persistent_transport() const { return recurrence_mode == 2 ? 1 : (recurrence_mode == 4 ? 0 : 2); }
    bool tcrec_used = false;      // this fraction's forward sweep ran on the tensor-core recurrence
    // persistent tensor-core recurrence: weight images, exchange words (allocated on first use)
    PtcBuffers ptc{};
    bool ptc_used = false;        // this fraction's forward sweep ran on the persistent tensor-core kernels
    bool want_ptc() const;
    int ensure_ptc();
    // which recurrence the last forward / backward sweep actually ran: 0 one launch per timestep, 1 persistent
    // FFMA kernels, 3 tensor-core GEMM + gate kernel per timestep, 5 persistent tensor-core kernels
    int fwd_path = -1, bwd_path = -1;
    bool want_tc_recurrence() const;
    int ensure_tcrec();
    int check_status(cudaStream_t st);   // synchronises st; returns the kernels' status word
    // optional per-phase timing hooks (set by the layer stack when profiling is on)
    void *prof_ctx = nullptr;
    void (*prof_begin)(void *, const char *) = nullptr;
    void (*prof_end)(void *) = nullptr;

    int create(const b2_lstm_desc &d);
    void destroy();
    LstmShape shape() const;
    int load_sequences(int cur_max, int cur_min, const char *pat_dev);
    int forward(const float *w, const float *x, float *y, cudaStream_t st);
    int backward(const float *w, const float *x, const float *y, const float *dy, float *dx, float *dw,
                 cudaStream_t st);
    int gemm(float *C, long ldc, const float *A, long sam, long sak, const float *B, long sbk, long sbn, int m, int n,
             int k, bool acc, cudaStream_t st);
};

}  // namespace b2
