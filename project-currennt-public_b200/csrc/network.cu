// Layer stack, minibatch step and steepest-descent update: the host-side mirror of the reference's
// NeuralNetwork / Optimizer::_processDataSet / SteepestDescentOptimizer for the layer types of the
// LSTM training path, plus the b2_net_* and b2_matrix_* entry points of the C ABI.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <random>

#include <mutex>

#include "network.hpp"

namespace b2 {

// ---- status ---------------------------------------------------------------------------------------
static thread_local char g_err[1024] = "";
unsigned long long g_launches = 0;
float g_lstm_forget_gate_bias = 0.0f;   // the process-wide option, like the reference's Configuration singleton
float g_weights_uniform_min = -0.1f, g_weights_uniform_max = 0.1f;   // --weights_uniform_min / --weights_uniform_max (Configuration.cpp:666-670)

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}
int cuda_fail(cudaError_t e, const char *what, const char *file, int line) {
    set_error("CUDA error %d (%s) at %s:%d: %s", (int)e, cudaGetErrorString(e), file, line, what);
    return B2_ERR_CUDA;
}
const char *last_error() { return g_err; }

// ---- Layer (layers/Layer.cu:73-146,254-305) -------------------------------------------------------
Layer::Layer(NeuralNetwork &net, const json::Value &j, int P, int maxT, Layer *prev)
    : net_(net), P_(P), maxT_(maxT), prev_(prev) {
    name_ = j.has("name") ? j.at("name").str : std::string("layer");
    type_ = j.at("type").str;
    size_ = (int)j.at("size").num;
}
Layer::~Layer() {
    if (ownsBuffers_) {
        cudaFree(outputs_);
        cudaFree(outputErrors_);
    }
}
int Layer::allocate() {
    size_t n = (size_t)maxT_ * P_ * size_;
    ownsBuffers_ = true;
    B2_CUDA(cudaMalloc(&outputs_, n * sizeof(float)));
    B2_CUDA(cudaMalloc(&outputErrors_, n * sizeof(float)));
    B2_CUDA(cudaMemset(outputs_, 0, n * sizeof(float)));
    B2_CUDA(cudaMemset(outputErrors_, 0, n * sizeof(float)));
    return B2_OK;
}
int Layer::loadSequences(const Fraction &f, int) {
    curMax_ = f.T;
    curMin_ = f.Tmin;
    pat_ = f.patTypes;
    return B2_OK;
}

// ---- TrainableLayer (layers/TrainableLayer.cu:93-305) ---------------------------------------------
TrainableLayer::TrainableLayer(NeuralNetwork &net, const json::Value &j, int P, int maxT, Layer *prev)
    : Layer(net, j, P, maxT, prev) {
    bias_ = j.has("bias") ? (float)j.at("bias").num : 0.0f;
    learningRate_ = j.has("learningRate") ? (float)j.at("learningRate").num : -1.0f;
}
TrainableLayer::~TrainableLayer() {
    cudaFree(weights_);
    cudaFree(weightUpdates_);
    cudaFree(weightDeltas_);
    cudaFree(weightStats_);
    cudaFree(weightAccum_);
}
int TrainableLayer::allocateWeights(size_t n) {
    nW_ = n;
    B2_CUDA(cudaMalloc(&weights_, n * sizeof(float)));
    B2_CUDA(cudaMalloc(&weightUpdates_, n * sizeof(float)));
    B2_CUDA(cudaMalloc(&weightDeltas_, n * sizeof(float)));
    B2_CUDA(cudaMemset(weights_, 0, n * sizeof(float)));
    B2_CUDA(cudaMemset(weightUpdates_, 0, n * sizeof(float)));
    B2_CUDA(cudaMemset(weightDeltas_, 0, n * sizeof(float)));
    return B2_OK;
}

int TrainableLayer::allocateAccum() {
    if (weightAccum_) return B2_OK;
    B2_CUDA(cudaMalloc(&weightAccum_, nW_ * sizeof(float)));
    B2_CUDA(cudaMemset(weightAccum_, 0, nW_ * sizeof(float)));
    return B2_OK;
}

int TrainableLayer::allocateStats(size_t floats, float init, cudaStream_t st) {
    if (weightStats_ && statsFloats_ == floats) return fill_value(weightStats_, floats, init, st);
    if (weightStats_) { B2_CUDA(cudaStreamSynchronize(st)); cudaFree(weightStats_); weightStats_ = nullptr; }
    statsFloats_ = floats;
    if (!floats) return B2_OK;
    B2_CUDA(cudaMalloc(&weightStats_, floats * sizeof(float)));
    return fill_value(weightStats_, floats, init, st);
}

// ---- InputLayer (layers/InputLayer.cu:162-164): outputs = the fraction's inputs ------------------------
int InputLayer::loadSequences(const Fraction &f, int nnState) {
    Layer::loadSequences(f, nnState);
    // the fraction's device copy IS this layer's output vector (no second copy)
    outputs_ = const_cast<float *>(f.inputs);
    return B2_OK;
}

// ---- FeedForwardLayer (layers/FeedForwardLayer.cu:1061-1101,1634-1738) ------------------------------
FeedForwardLayer::FeedForwardLayer(NeuralNetwork &net, const json::Value &j, int P, int maxT, Layer *prev, int act)
    : TrainableLayer(net, j, P, maxT, prev), act_(act) {}

int FeedForwardLayer::computeForwardPass(int) {
    const int N = curMax_ * P_, pls = prev_->size(), ls = size_;
    {
        ProfScope ps(net_, "ff_forward_gemm");
        // outputs(ls x N) = W^T X with W the pls x ls column-major weight matrix
        B2_TRY(net_.gemm(outputs_, ls, weights_, pls, 1, prev_->outputs(), 1, pls, ls, N, pls, false));
    }
    ProfScope ps(net_, "ff_bias_act");
    return ff_bias_act(outputs_, weights_ + (size_t)ls * pls, bias_, ls, (size_t)N * ls, act_, net_.stream);
}

int FeedForwardLayer::computeBackwardPass(int) {
    const int N = curMax_ * P_, pls = prev_->size(), ls = size_;
    {
        ProfScope ps(net_, "ff_delta");
        B2_TRY(ff_delta(outputErrors_, outputs_, (size_t)N * ls, act_, net_.stream));
    }
    {
        ProfScope ps(net_, "ff_backward_gemm");
        // dX(pls x N) = W delta, overwrite (assignProduct, FeedForwardLayer.cu:1690); nobody reads the
        // errors of an input layer, so that product is skipped
        const bool wantDx = prev_->precedingLayer() != nullptr;
        const bool tc = !net_.forceFfma && gemm_wants_tc(1, pls, ls, 1, pls, ls, N) &&
                        (!wantDx || gemm_wants_tc(1, pls, 1, ls, pls, N, ls));
        if (tc) {
            // both products on the tensor cores: the deltas are split into tf32 hi/lo parts ONCE; the same
            // [frame][unit] copy serves as the K-major operand of dX and as the MN-major operand of dW
            TcScratch &sc = net_.tcScratch;
            B2_TRY(sc.reserve(split_floats(N, ls) + split_floats(N, pls) + split_floats(ls, pls)));
            sc.used = 0;
            SplitOperand sD{}, sX{}, sW{};
            B2_TRY(split_operand(sc, outputErrors_, ls, N, ls, true, &sD, net_.stream));
            if (wantDx) {
                B2_TRY(split_operand(sc, weights_, pls, ls, pls, false, &sW, net_.stream));
                B2_TRY(gemm_tc(prev_->outputErrors(), pls, sW, sD, pls, N, ls, false, net_.ws, net_.wsFloats, net_.statusDev,
                               net_.stream));
            }
            B2_TRY(split_operand(sc, prev_->outputs(), pls, N, pls, false, &sX, net_.stream));
            SplitOperand sDt = sD;
            sDt.kmajor = false;
            B2_TRY(gemm_tc(weightUpdates_, pls, sX, sDt, pls, ls, N, false, net_.ws, net_.wsFloats, net_.statusDev, net_.stream));
        } else {
            if (wantDx)
                B2_TRY(net_.gemm(prev_->outputErrors(), pls, weights_, 1, pls, outputErrors_, 1, ls, pls, N, ls, false));
            // dW(pls x ls) = X delta^T (FeedForwardLayer.cu:1719)
            B2_TRY(net_.gemm(weightUpdates_, pls, prev_->outputs(), 1, pls, outputErrors_, ls, 1, pls, ls, N, false));
        }
    }
    ProfScope ps(net_, "ff_bias_grad");
    // bias gradient = bias * sum over frames of delta (FeedForwardLayer.cu:118-138,1517-1533)
    return column_sums(weightUpdates_ + (size_t)ls * pls, outputErrors_, ls, ls, N, bias_, net_.ws, net_.wsFloats,
                       net_.stream);
}

// ---- LstmLayer ------------------------------------------------------------------------------------------
LstmLayer::LstmLayer(NeuralNetwork &net, const json::Value &j, int P, int maxT, Layer *prev, bool bidirectional)
    : TrainableLayer(net, j, P, maxT, prev), bidirectional_(bidirectional) {}
LstmLayer::~LstmLayer() { impl_.destroy(); }
static void prof_begin_cb(void *ctx, const char *name) {
    NeuralNetwork *n = (NeuralNetwork *)ctx;
    if (n->profiling) n->profBegin(name);
}
static void prof_end_cb(void *ctx) {
    NeuralNetwork *n = (NeuralNetwork *)ctx;
    if (n->profiling) n->profEnd();
}
int LstmLayer::init() {
    b2_lstm_desc d;
    d.parallel_sequences = P_; d.max_seq_length = maxT_; d.prev_size = prev_->size(); d.size = size_;
    d.bidirectional = bidirectional_ ? 1 : 0; d.bias = bias_;
    impl_.scratch = &net_.tcScratch;
    B2_TRY(impl_.create(d));
    impl_.prof_ctx = &net_;
    impl_.prof_begin = prof_begin_cb;
    impl_.prof_end = prof_end_cb;
    return allocateWeights(b2_lstm_num_weights(&d));
}
int LstmLayer::loadSequences(const Fraction &f, int nnState) {
    Layer::loadSequences(f, nnState);
    return impl_.load_sequences(f.T, f.Tmin, f.patTypes);
}
int LstmLayer::computeForwardPass(int) {
    impl_.force_ffma = net_.forceFfma;
    impl_.recurrence_mode = net_.recurrenceMode;
    return impl_.forward(weights_, prev_->outputs(), outputs_, net_.stream);
}
int LstmLayer::computeBackwardPass(int) {
    float *dx = prev_->precedingLayer() ? prev_->outputErrors() : nullptr;  // input layer: nobody reads it
    return impl_.backward(weights_, prev_->outputs(), outputs_, outputErrors_, dx, weightUpdates_, net_.stream);
}

// ---- SsePostOutputLayer (layers/SsePostOutputLayer.cu:166-267, PostOutputLayer.cu:285-311) ----------
SsePostOutputLayer::~SsePostOutputLayer() {
    cudaFree(lossDev_);
    cudaFree(lossWs_);
    if (lossPinned_) cudaFreeHost(lossPinned_);
    if (lossReady_) cudaEventDestroy(lossReady_);
}
int SsePostOutputLayer::init() {
    B2_CUDA(cudaMalloc(&lossDev_, sizeof(double)));
    B2_CUDA(cudaMalloc(&lossWs_, 1024 * sizeof(double)));
    B2_CUDA(cudaMemset(lossDev_, 0, sizeof(double)));
    B2_CUDA(cudaMallocHost(&lossPinned_, 2 * sizeof(double)));
    lossPinned_[0] = lossPinned_[1] = 0.0;
    B2_CUDA(cudaEventCreateWithFlags(&lossReady_, cudaEventDisableTiming));
    B2_CUDA(cudaEventRecord(lossReady_, net_.stream));
    return B2_OK;
}
int SsePostOutputLayer::loadSequences(const Fraction &f, int nnState) {
    Layer::loadSequences(f, nnState);
    targets_ = f.targets;  // the reference copies them into this layer's outputs(); here they stay in place
    return B2_OK;
}
int SsePostOutputLayer::calculateError(double *hostError) {
    {
        ProfScope ps(net_, "sse_loss");
        B2_TRY(sse_loss(lossDev_, prev_->outputs(), targets_, pat_, size_, (size_t)curMax_ * P_, lossWs_, net_.stream));
    }
    // the error goes to a pinned slot at once, with an event behind it: a reader then waits for the forward
    // pass only, not for whatever the stream holds after it (b2_net_read_error)
    lossSlot_ ^= 1;
    B2_CUDA(cudaMemcpyAsync(lossPinned_ + lossSlot_, lossDev_, sizeof(double), cudaMemcpyDeviceToHost, net_.stream));
    B2_CUDA(cudaEventRecord(lossReady_, net_.stream));
    if (hostError) B2_TRY(readError(hostError));
    return B2_OK;
}
int SsePostOutputLayer::readError(double *hostError) {
    B2_CUDA(cudaEventSynchronize(lossReady_));
    *hostError = lossPinned_[lossSlot_];
    return B2_OK;
}
int SsePostOutputLayer::computeBackwardPass(int) {
    ProfScope ps(net_, "sse_grad");
    return sse_grad(prev_->outputErrors(), prev_->outputs(), targets_, pat_, size_, (size_t)curMax_ * P_, net_.stream);
}

// ---- NeuralNetwork --------------------------------------------------------------------------------------
NeuralNetwork::~NeuralNetwork() {
    if (dp) dp_detach(*this);
    layers.clear();
    cudaFree(ws); cudaFree(statusDev); cudaFree(fracLenDev);
    for (int b = 0; b < 2; ++b) {
        cudaFree(inBuf[b]); cudaFree(tgBuf[b]); cudaFree(patBuf[b]);
        if (patPinned[b]) cudaFreeHost(patPinned[b]);
        if (prefetchDone[b]) cudaEventDestroy(prefetchDone[b]);
        if (bufFree[b]) cudaEventDestroy(bufFree[b]);
        if (patCopied[b]) cudaEventDestroy(patCopied[b]);
    }
    if (copyStream) cudaStreamDestroy(copyStream);
    tcScratch.release();
    for (size_t i = 0; i < eventPool.size(); ++i) cudaEventDestroy(eventPool[i]);
    for (size_t i = 0; i < prof.size(); ++i) { cudaEventDestroy(prof[i].a); cudaEventDestroy(prof[i].b); }
    for (size_t i = 0; i < gradReady.size(); ++i) cudaEventDestroy(gradReady[i]);
    if (stream) cudaStreamDestroy(stream);
    if (commStream) cudaStreamDestroy(commStream);
}

int NeuralNetwork::gemm(float *C, long ldc, const float *A, long sam, long sak, const float *B, long sbk, long sbn,
                        int m, int n, int k, bool acc) {
    return gemm_auto(C, ldc, A, sam, sak, B, sbk, sbn, m, n, k, acc, forceFfma, &tcScratch, ws, wsFloats, statusDev, stream);
}

int NeuralNetwork::create(const char *networkJson, int P_, int maxT_, unsigned seed) {
    P = P_; maxT = maxT_;
    if (P <= 0 || maxT <= 0 || !networkJson) { set_error("b2_net_create: bad arguments"); return B2_ERR_BAD_ARG; }
    launchesAtCreate = g_launches;
    json::Value doc;
    try {
        doc = json::Parser(networkJson).parse();
        const json::Value &L = doc.at("layers");
        if (L.kind != json::Value::Array || L.arr.size() < 2) throw std::runtime_error("json: 'layers' must be an array");
        // validate the topology before touching the device
        for (size_t i = 0; i < L.arr.size(); ++i) {
            const std::string ty = L.arr[i].at("type").str;
            if ((int)L.arr[i].at("size").num <= 0) throw std::runtime_error("layer size must be positive");
            if (i == 0) {
                if (ty != "input") throw std::runtime_error("the first layer must be of type 'input'");
            } else if (ty != "feedforward_tanh" && ty != "feedforward_logistic" && ty != "feedforward_identity" &&
                       ty != "lstm" && ty != "blstm" && ty != "sse") {
                throw std::runtime_error("unsupported layer type '" + ty + "'");
            } else if (ty == "sse" && i + 1 != L.arr.size()) {
                throw std::runtime_error("the sse layer must be the last layer");
            }
        }
        if (L.arr.back().at("type").str != "sse") throw std::runtime_error("the last layer must be of type 'sse'");
        int lo, hi;
        B2_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
        B2_CUDA(cudaStreamCreateWithPriority(&stream, cudaStreamNonBlocking, lo));
        B2_CUDA(cudaStreamCreateWithPriority(&commStream, cudaStreamNonBlocking, hi));
        B2_CUDA(cudaMalloc(&statusDev, sizeof(int)));
        B2_CUDA(cudaMemset(statusDev, 0, sizeof(int)));
        for (size_t i = 0; i < L.arr.size(); ++i) {
            const json::Value &j = L.arr[i];
            const std::string ty = j.at("type").str;
            Layer *prev = layers.empty() ? nullptr : layers.back().get();
            if (i == 0) {
                if (ty != "input") throw std::runtime_error("the first layer must be of type 'input'");
                layers.emplace_back(new InputLayer(*this, j, P, maxT, nullptr));
                // outputs alias the fraction's device inputs; errors are never read
            } else if (ty == "feedforward_tanh" || ty == "feedforward_logistic" || ty == "feedforward_identity") {
                int act = ty == "feedforward_tanh" ? ACT_TANH : (ty == "feedforward_logistic" ? ACT_LOGISTIC : ACT_IDENTITY);
                FeedForwardLayer *l = new FeedForwardLayer(*this, j, P, maxT, prev, act);
                layers.emplace_back(l);
                B2_TRY(l->allocate());
                B2_TRY(l->allocateWeights((size_t)l->size() * (prev->size() + 1)));
            } else if (ty == "lstm" || ty == "blstm") {
                LstmLayer *l = new LstmLayer(*this, j, P, maxT, prev, ty == "blstm");
                layers.emplace_back(l);
                B2_TRY(l->allocate());
                B2_TRY(l->init());
            } else if (ty == "sse") {
                if ((int)j.at("size").num != prev->size()) throw std::runtime_error("sse layer size must equal the preceding layer's");
                SsePostOutputLayer *l = new SsePostOutputLayer(*this, j, P, maxT, prev);
                layers.emplace_back(l);
                B2_TRY(l->init());
            } else {
                throw std::runtime_error("unsupported layer type '" + ty + "'");
            }
        }
    } catch (const std::exception &e) {
        set_error("b2_net_create: %s", e.what());
        return B2_ERR_BAD_ARG;
    }
    // fraction buffers (input layer outputs / targets / pattern types)
    size_t frames = (size_t)maxT * P;
    B2_CUDA(cudaStreamCreateWithFlags(&copyStream, cudaStreamNonBlocking));
    for (int b = 0; b < 2; ++b) {
        B2_CUDA(cudaMalloc(&inBuf[b], frames * layers.front()->size() * sizeof(float)));
        B2_CUDA(cudaMalloc(&tgBuf[b], frames * layers.back()->size() * sizeof(float)));
        B2_CUDA(cudaMalloc(&patBuf[b], frames));
        B2_CUDA(cudaMallocHost(&patPinned[b], frames));
        B2_CUDA(cudaEventCreateWithFlags(&prefetchDone[b], cudaEventDisableTiming));
        B2_CUDA(cudaEventCreateWithFlags(&bufFree[b], cudaEventDisableTiming));
        B2_CUDA(cudaEventCreateWithFlags(&patCopied[b], cudaEventDisableTiming));
    }
    wsFloats = (size_t)8 << 20;
    B2_CUDA(cudaMalloc(&ws, wsFloats * sizeof(float)));
    gradReady.resize(layers.size());
    for (size_t i = 0; i < layers.size(); ++i) B2_CUDA(cudaEventCreateWithFlags(&gradReady[i], cudaEventDisableTiming));

    // weights: from the "weights" section where present (TrainableLayer.cu:135-205), else uniform random as the reference
    // draws them (TrainableLayer.cu:219-233): ONE mt19937 seeded with the random seed serves all layers in order, and each
    // weight is boost::random::uniform_real_distribution<float>(0, max - min)(gen) + min.  That distribution, restated from
    // Boost.Random (absent here, so the stream is not pinned against Boost itself): float(draw) / (float(2^32 - 1) + 1) *
    // range, drawn again while the rounded result reaches the range.
    std::mt19937 gen(seed);
    const float wmin = g_weights_uniform_min, wrange = g_weights_uniform_max - g_weights_uniform_min;
    auto dist = [wmin, wrange](std::mt19937 &g) {
        for (;;) {
            const float numerator = static_cast<float>(g());
            const float divisor = static_cast<float>(0xffffffffu) + 1.0f;
            const float result = numerator / divisor * wrange + 0.0f;
            if (result < wrange || !(wrange > 0.0f)) return result + wmin;
        }
    };
    const json::Value *wsec = doc.find("weights");
    for (size_t i = 0; i < layers.size(); ++i) {
        TrainableLayer *t = dynamic_cast<TrainableLayer *>(layers[i].get());
        if (!t) continue;
        std::vector<float> w(t->numWeights());
        const json::Value *lw = wsec ? wsec->find(t->name()) : nullptr;
        if (lw) {
            size_t k = 0;
            const char *secs[3] = {"input", "bias", "internal"};
            for (int s = 0; s < 3; ++s) {
                const json::Value *a = lw->find(secs[s]);
                if (!a) continue;
                for (size_t q = 0; q < a->arr.size() && k < w.size(); ++q) w[k++] = (float)a->arr[q].num;
            }
            if (k != w.size()) {
                set_error("b2_net_create: layer '%s' expects %zu weights, JSON holds %zu", t->name().c_str(), w.size(), k);
                return B2_ERR_BAD_SHAPE;
            }
        } else {
            for (size_t k = 0; k < w.size(); ++k) w[k] = dist(gen);
            // --lstm_forget_gate_bias (Configuration.cpp:682-683): freshly initialised (b)lstm layers get the value added
            // to every forget-gate bias (layers/LstmLayer.cu:1147-1161); layers read from a weights section do not
            LstmLayer *l = dynamic_cast<LstmLayer *>(t);
            if (l && g_lstm_forget_gate_bias > 0.0001f) {
                const size_t ls = (size_t)l->size(), pls = (size_t)l->precedingLayer()->size();
                for (size_t k = 0; k < ls; ++k) w[4 * ls * pls + 2 * ls + k] += g_lstm_forget_gate_bias;
            }
        }
        B2_CUDA(cudaMemcpy(t->weights(), w.data(), w.size() * sizeof(float), cudaMemcpyHostToDevice));
    }
    return B2_OK;
}

// copies one fraction into buffer set b on stream st and fills fracBuf[b]
int NeuralNetwork::stageFraction(int b, int T, int nSeq, const int *lens, const float *in, const float *tg, bool onDevice,
                                 cudaStream_t st) {
    if (T <= 0 || T > maxT || nSeq <= 0 || nSeq > P || !lens || !in || !tg) {
        set_error("b2_net_load_fraction: T=%d (max %d), n_seqs=%d (P=%d)", T, maxT, nSeq, P);
        return B2_ERR_BAD_SHAPE;
    }
    int mx = 0, mn = 1 << 30;
    long real = 0;
    for (int p = 0; p < nSeq; ++p) {
        if (lens[p] <= 0 || lens[p] > T) { set_error("b2_net_load_fraction: sequence length %d outside 1..%d", lens[p], T); return B2_ERR_BAD_SHAPE; }
        mx = lens[p] > mx ? lens[p] : mx;
        mn = lens[p] < mn ? lens[p] : mn;
        real += lens[p];
    }
    // pattern types as DataSet::_makeFractionTask writes them (data_sets/DataSet.cpp:853-861)
    size_t frames = (size_t)mx * P;
    char *ph = patPinned[b];
    // the pinned staging is rewritten by the host: the previous copy out of it must have run
    B2_CUDA(cudaEventSynchronize(patCopied[b]));
    memset(ph, 0, frames);
    for (int p = 0; p < nSeq; ++p)
        for (int t = 0; t < lens[p]; ++t) ph[(size_t)t * P + p] = t == 0 ? 1 : (t == lens[p] - 1 ? 3 : 2);
    B2_CUDA(cudaMemcpyAsync(patBuf[b], ph, frames, cudaMemcpyHostToDevice, st));
    B2_CUDA(cudaEventRecord(patCopied[b], st));
    cudaMemcpyKind kind = onDevice ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
    B2_CUDA(cudaMemcpyAsync(inBuf[b], in, frames * layers.front()->size() * sizeof(float), kind, st));
    B2_CUDA(cudaMemcpyAsync(tgBuf[b], tg, frames * layers.back()->size() * sizeof(float), kind, st));
    Fraction &f = fracBuf[b];
    f.T = mx; f.Tmin = mn; f.nSeq = nSeq; f.realFrames = real;
    f.patTypes = patBuf[b]; f.inputs = inBuf[b]; f.targets = tgBuf[b];
    return B2_OK;
}

int NeuralNetwork::loadFraction(int T, int nSeq, const int *lens, const float *in, const float *tg, bool onDevice) {
    ProfScope ps(*this, "load_fraction");
    if (prefetchPending) { set_error("b2_net_load_fraction: a prefetched fraction is waiting to be used"); return B2_ERR_STATE; }
    B2_CUDA(cudaEventSynchronize(bufFree[cur]));
    B2_TRY(stageFraction(cur, T, nSeq, lens, in, tg, onDevice, stream));
    frac = fracBuf[cur];
    for (size_t i = 0; i < layers.size(); ++i) B2_TRY(layers[i]->loadSequences(frac, 0));
    return B2_OK;
}

// Start copying the NEXT fraction into the idle buffer set while the current one is being processed
// (the role of the reference's optional loader thread, data_sets/DataSet.cpp:456-489,1936-1972).
int NeuralNetwork::prefetchFraction(int T, int nSeq, const int *lens, const float *in, const float *tg) {
    if (prefetchPending) { set_error("b2_net_prefetch_fraction: the previous prefetch has not been used yet"); return B2_ERR_STATE; }
    const int b = cur ^ 1;
    // the idle set was last read by the step before the current one; the host staging by its copy
    B2_CUDA(cudaEventSynchronize(prefetchDone[b]));
    B2_CUDA(cudaStreamWaitEvent(copyStream, bufFree[b], 0));
    B2_TRY(stageFraction(b, T, nSeq, lens, in, tg, false, copyStream));
    B2_CUDA(cudaEventRecord(prefetchDone[b], copyStream));
    prefetchPending = true;
    return B2_OK;
}

int NeuralNetwork::usePrefetched() {
    if (!prefetchPending) { set_error("no prefetched fraction: call b2_net_prefetch_fraction first"); return B2_ERR_STATE; }
    const int b = cur ^ 1;
    B2_CUDA(cudaEventRecord(bufFree[cur], stream));            // everything enqueued so far has read the old set
    B2_CUDA(cudaStreamWaitEvent(stream, prefetchDone[b], 0));
    cur = b;
    prefetchPending = false;
    frac = fracBuf[cur];
    for (size_t i = 0; i < layers.size(); ++i) B2_TRY(layers[i]->loadSequences(frac, 0));
    return B2_OK;
}

int NeuralNetwork::computeForwardPass() {
    if (!frac.T) { set_error("b2_net_forward: no fraction loaded"); return B2_ERR_STATE; }
    for (size_t i = 0; i < layers.size(); ++i) B2_TRY(layers[i]->computeForwardPass(0));
    return B2_OK;
}
int NeuralNetwork::calculateError(double *hostError) {
    SsePostOutputLayer *post = dynamic_cast<SsePostOutputLayer *>(layers.back().get());
    if (!post) { set_error("the last layer is not a post-output layer"); return B2_ERR_STATE; }
    return post->calculateError(hostError);
}
int NeuralNetwork::computeBackwardPass() {
    if (!frac.T) { set_error("b2_net_backward: no fraction loaded"); return B2_ERR_STATE; }
    for (int i = (int)layers.size() - 1; i >= 1; --i) {
        B2_TRY(layers[i]->computeBackwardPass(0));
        TrainableLayer *t = dynamic_cast<TrainableLayer *>(layers[i].get());
        if (t && dp) {
            // the layer's gradient is complete: sum it over the ranks on the communication stream
            // while the layers below run their backward pass on the main stream
            B2_CUDA(cudaEventRecord(gradReady[i], stream));
            B2_CUDA(cudaStreamWaitEvent(commStream, gradReady[i], 0));
            B2_TRY(dp_allreduce_sum(*this, t->weightUpdates(), t->numWeights(), commStream));
        }
    }
    if (dp) {
        B2_CUDA(cudaEventRecord(gradReady[0], commStream));
        B2_CUDA(cudaStreamWaitEvent(stream, gradReady[0], 0));
    }
    return B2_OK;
}
// Optimizer::_processDataSet without hybrid_online_batch (optimizers/Optimizer.cu:186-196, 243-245): the
// optimizer's copy of the weight updates sums the fractions' gradients; ONE update, with frame count 1,
// follows the last fraction
int NeuralNetwork::accumulateWeightUpdates(bool first) {
    for (size_t i = 1; i < layers.size(); ++i) {
        TrainableLayer *t = dynamic_cast<TrainableLayer *>(layers[i].get());
        if (!t) continue;
        B2_TRY(t->allocateAccum());
        B2_TRY(accumulate(t->weightAccum(), t->weightUpdates(), t->numWeights(), first, stream));
    }
    return B2_OK;
}
int NeuralNetwork::updateWeightsBatch(float lr, float mom) {
    for (size_t i = 1; i < layers.size(); ++i) {
        TrainableLayer *t = dynamic_cast<TrainableLayer *>(layers[i].get());
        if (!t) continue;
        if (!t->weightAccum()) { set_error("b2_net_update_weights_batch: nothing accumulated"); return B2_ERR_STATE; }
        B2_CUDA(cudaMemcpyAsync(t->weightUpdates(), t->weightAccum(), t->numWeights() * sizeof(float), cudaMemcpyDeviceToDevice, stream));
    }
    // _updateWeights(1): the shaping options see a frame count of one; the gradients are already summed
    // over the ranks, so the count is not
    DpComm *keep = dp;
    const long frames = frac.realFrames;
    frac.realFrames = 1;
    dp = nullptr;
    const int rc = updateWeights(lr, mom);
    dp = keep;
    frac.realFrames = frames;
    return rc;
}

// a rank without a sequence in the current fraction: zero gradients into the all-reduce of every layer
int NeuralNetwork::computeBackwardPassEmpty() {
    if (!dp) { set_error("b2_net_backward_empty: no data-parallel communicator attached"); return B2_ERR_STATE; }
    for (int i = (int)layers.size() - 1; i >= 1; --i) {
        TrainableLayer *t = dynamic_cast<TrainableLayer *>(layers[i].get());
        if (!t) continue;
        B2_TRY(fill_zero(t->weightUpdates(), t->numWeights() * sizeof(float), stream));
        B2_CUDA(cudaEventRecord(gradReady[i], stream));
        B2_CUDA(cudaStreamWaitEvent(commStream, gradReady[i], 0));
        B2_TRY(dp_allreduce_sum(*this, t->weightUpdates(), t->numWeights(), commStream));
    }
    B2_CUDA(cudaEventRecord(gradReady[0], commStream));
    B2_CUDA(cudaStreamWaitEvent(stream, gradReady[0], 0));
    frac.realFrames = 0;
    return B2_OK;
}
int NeuralNetwork::trainStepEmpty(float lr, float mom) {
    B2_TRY(computeBackwardPassEmpty());
    return updateWeights(lr, mom);
}

// Optimizer constructor, option part (optimizers/Optimizer.cu:421-457): AdaGrad statistics start at
// OP_ADAGRADFACTOR, Adam's first and second moments at zero
int NeuralNetwork::setOptimizerOption(int option) {
    if (option < 0 || option > 5) {
        set_error("b2_net_set_optimizer: option %d (0 plain, 1 AdaGrad, 2 average gradient, 3 SGD + AdaGrad statistics, 4 SGD with "
                  "learning-rate decay, 5 Adam)", option);
        return B2_ERR_BAD_ARG;
    }
    optOption = option;
    adamBeta1Accum = adamBeta2Accum = 1.0f;
    if (!fracLenDev) B2_CUDA(cudaMalloc(&fracLenDev, sizeof(float)));
    for (size_t i = 0; i < layers.size(); ++i) {
        TrainableLayer *t = dynamic_cast<TrainableLayer *>(layers[i].get());
        if (!t) continue;
        if (option == 1 || option == 3) B2_TRY(t->allocateStats(t->numWeights(), 0.000001f, stream));
        else if (option == 5) B2_TRY(t->allocateStats(2 * t->numWeights(), 0.0f, stream));
        else B2_TRY(t->allocateStats(0, 0.0f, stream));
    }
    return B2_OK;
}

int NeuralNetwork::updateWeights(float lr, float mom) {
    ProfScope ps(*this, "sgd_update");
    // option 4 (OPTIMIZATION_SGD_DECAY) updates like plain SGD; its schedule lives in the training run (b2_optimizer_train)
    const bool adjust = optOption > 0 && optOption != 4;
    if (adjust) {
        // frames of the fraction (summed over the ranks of a data-parallel job): the gradient is averaged over them
        B2_TRY(fill_value(fracLenDev, 1, (float)frac.realFrames, stream));
        if (dp) B2_TRY(dp_allreduce_sum(*this, fracLenDev, 1, stream));
        if (optOption == 5) {   // SteepestDescentOptimizer.cu:339-343
            adamBeta1Accum *= 0.9f;
            adamBeta2Accum *= 0.999f;
        }
    }
    for (size_t i = 0; i < layers.size(); ++i) {
        TrainableLayer *t = dynamic_cast<TrainableLayer *>(layers[i].get());
        if (!t) continue;
        float rate = t->learningRate() >= 0.0f ? t->learningRate() : lr;  // SteepestDescentOptimizer.cu:425-426
        if (adjust)
            B2_TRY(sgd_update_opt(t->weights(), t->weightUpdates(), t->weightDeltas(), t->weightStats(), t->numWeights(), rate, mom,
                                  optOption, fracLenDev, adamBeta1Accum, adamBeta2Accum, stream));
        else
            B2_TRY(sgd_update(t->weights(), t->weightUpdates(), t->weightDeltas(), t->numWeights(), rate, mom, stream));
    }
    return B2_OK;
}
int NeuralNetwork::synchronize() {
    B2_CUDA(cudaStreamSynchronize(copyStream));
    B2_CUDA(cudaStreamSynchronize(stream));
    B2_CUDA(cudaStreamSynchronize(commStream));
    for (size_t i = 0; i < layers.size(); ++i) {
        LstmLayer *l = dynamic_cast<LstmLayer *>(layers[i].get());
        if (l) B2_TRY(l->impl().check_status(stream));
    }
    int v = 0;
    B2_CUDA(cudaMemcpy(&v, statusDev, sizeof(int), cudaMemcpyDeviceToHost));
    if (v != 0) {
        B2_CUDA(cudaMemset(statusDev, 0, sizeof(int)));
        set_error("a tensor-core GEMM gave up a bounded wait (status %d)", v);
        return v;
    }
    return B2_OK;
}

void NeuralNetwork::profBegin(const char *name) {
    ProfileEntry e;
    e.name = name;
    cudaEventCreate(&e.a);
    cudaEventCreate(&e.b);
    cudaEventRecord(e.a, stream);
    profLaunch0_ = g_launches;
    prof.push_back(e);
}
void NeuralNetwork::profEnd() {
    ProfileEntry &e = prof.back();
    cudaEventRecord(e.b, stream);
    e.launches = (int)(g_launches - profLaunch0_);
}

}  // namespace b2

// ---- C ABI ------------------------------------------------------------------------------------------------
using namespace b2;
struct b2_net {
    NeuralNetwork net;
    std::vector<std::string> profNames;
};

static TrainableLayer *trainable(b2_net *n, int i) {
    if (!n || i < 0 || i >= (int)n->net.layers.size()) return nullptr;
    return dynamic_cast<TrainableLayer *>(n->net.layers[i].get());
}

extern "C" {

b2::NeuralNetwork *b2_net_impl(b2_net *n) { return &n->net; }

const char *b2_last_error_string(void) { return b2::last_error(); }
const char *b2_version(void) { return "b2lstm 0.1 sm_100a"; }

int b2_matrix_multiply(float *C, int ldc, const float *A, int lda, int transA, const float *B, int ldb, int transB,
                       int m, int n, int k, int accumulate, int force_ffma, b2_stream stream) {
    if (!C || !A || !B) { set_error("b2_matrix_multiply: null pointer"); return B2_ERR_BAD_ARG; }
    if (transA && transB) { set_error("b2_matrix_multiply: transposing both operands is not supported"); return B2_ERR_BAD_ARG; }
    long sam = transA ? lda : 1, sak = transA ? 1 : lda;
    long sbk = transB ? ldb : 1, sbn = transB ? 1 : ldb;
    // stand-alone calls share one operand arena, split-K scratch and status word per DEVICE (the memory belongs
    // to the device that was current when it was allocated), and run one at a time on a device: the arena is
    // reused by the next call
    struct Slot { TcScratch sc; int *status = nullptr; float *ws = nullptr; std::mutex mu; };
    static Slot slots[MAX_DEVICES];
    static const size_t wsFloats = (size_t)8 << 20;
    const int dev = current_device();
    if (dev < 0) { set_error("b2_matrix_multiply: no current CUDA device"); return B2_ERR_CUDA; }
    Slot &sl = slots[dev];
    std::lock_guard<std::mutex> lk(sl.mu);
    if (!sl.status) {
        B2_CUDA(cudaMalloc(&sl.status, sizeof(int)));
        B2_CUDA(cudaMemset(sl.status, 0, sizeof(int)));
        B2_CUDA(cudaMalloc(&sl.ws, wsFloats * sizeof(float)));
    }
    TcScratch &sc = sl.sc;
    int *status = sl.status;
    float *ws = sl.ws;
    B2_TRY(gemm_auto(C, ldc, A, sam, sak, B, sbk, sbn, m, n, k, accumulate != 0, force_ffma != 0, &sc, ws, wsFloats, status,
                     (cudaStream_t)stream));
    if (!force_ffma && gemm_wants_tc(sam, sak, sbk, sbn, m, n, k)) {
        // the arena may be reused by the next call: finish, and report a timed-out wait
        int v = 0;
        B2_CUDA(cudaMemcpyAsync(&v, status, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
        B2_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
        if (v != 0) {
            B2_CUDA(cudaMemset(status, 0, sizeof(int)));
            set_error("b2_matrix_multiply: the tensor-core kernel gave up a bounded wait (status %d)", v);
            return v;
        }
    }
    return B2_OK;
}

int b2_net_create(const char *network_json, int P, int maxT, unsigned seed, b2_net **out) {
    if (!out) return B2_ERR_BAD_ARG;
    b2_net *n = new b2_net;
    int rc = n->net.create(network_json, P, maxT, seed);
    if (rc != B2_OK) { delete n; return rc; }
    *out = n;
    return B2_OK;
}
void b2_net_destroy(b2_net *n) { delete n; }
void b2_config_set_lstm_forget_gate_bias(float value) { b2::g_lstm_forget_gate_bias = value; }
void b2_config_set_weights_uniform(float min, float max) { b2::g_weights_uniform_min = min; b2::g_weights_uniform_max = max; }
void b2_config_set_ptc_plan(int backward, int ll_chunks, int nc32_chunks, int nc32_counter_chunks) {
    b2::lstm_ptc_set_plan(backward != 0, ll_chunks, nc32_chunks, nc32_counter_chunks);
}
int b2_selftest_inject_status(b2_net *n, int code) {
    if (!n) return B2_ERR_BAD_ARG;
    B2_CUDA(cudaStreamSynchronize(n->net.stream));
    B2_CUDA(cudaMemcpy(n->net.statusDev, &code, sizeof(int), cudaMemcpyHostToDevice));
    return B2_OK;
}
int b2_net_parallel_sequences(const b2_net *n) { return n ? n->net.P : 0; }
int b2_net_max_seq_length(const b2_net *n) { return n ? n->net.maxT : 0; }
int b2_net_num_layers(const b2_net *n) { return n ? (int)n->net.layers.size() : 0; }
int b2_net_layer_size(const b2_net *n, int i) {
    return (n && i >= 0 && i < (int)n->net.layers.size()) ? n->net.layers[i]->size() : 0;
}
size_t b2_net_num_weights(const b2_net *n, int i) {
    TrainableLayer *t = trainable(const_cast<b2_net *>(n), i);
    return t ? t->numWeights() : 0;
}
int b2_net_set_weights(b2_net *n, int i, const float *w) {
    TrainableLayer *t = trainable(n, i);
    if (!t || !w) { set_error("b2_net_set_weights: layer %d has no weights", i); return B2_ERR_BAD_ARG; }
    B2_CUDA(cudaMemcpyAsync(t->weights(), w, t->numWeights() * sizeof(float), cudaMemcpyHostToDevice, n->net.stream));
    B2_CUDA(cudaStreamSynchronize(n->net.stream));
    return B2_OK;
}
int b2_net_get_weights(b2_net *n, int i, float *w) {
    TrainableLayer *t = trainable(n, i);
    if (!t || !w) { set_error("b2_net_get_weights: layer %d has no weights", i); return B2_ERR_BAD_ARG; }
    B2_CUDA(cudaMemcpyAsync(w, t->weights(), t->numWeights() * sizeof(float), cudaMemcpyDeviceToHost, n->net.stream));
    B2_CUDA(cudaStreamSynchronize(n->net.stream));
    return B2_OK;
}
int b2_net_get_weight_updates(b2_net *n, int i, float *g) {
    TrainableLayer *t = trainable(n, i);
    if (!t || !g) { set_error("b2_net_get_weight_updates: layer %d has no weights", i); return B2_ERR_BAD_ARG; }
    B2_TRY(n->net.synchronize());
    B2_CUDA(cudaMemcpy(g, t->weightUpdates(), t->numWeights() * sizeof(float), cudaMemcpyDeviceToHost));
    return B2_OK;
}
float *b2_net_weights_dev(b2_net *n, int i) { TrainableLayer *t = trainable(n, i); return t ? t->weights() : nullptr; }
float *b2_net_weight_updates_dev(b2_net *n, int i) { TrainableLayer *t = trainable(n, i); return t ? t->weightUpdates() : nullptr; }
float *b2_net_outputs_dev(b2_net *n, int i) {
    if (!n || i < 0 || i >= (int)n->net.layers.size()) return nullptr;
    return i == 0 ? const_cast<float *>(n->net.frac.inputs) : n->net.layers[i]->outputs();
}
float *b2_net_output_errors_dev(b2_net *n, int i) {
    if (!n || i < 0 || i >= (int)n->net.layers.size()) return nullptr;
    return n->net.layers[i]->outputErrors();
}

int b2_net_load_fraction(b2_net *n, int T, int nSeq, const int *lens, const float *in, const float *tg) {
    if (!n) return B2_ERR_BAD_ARG;
    return n->net.loadFraction(T, nSeq, lens, in, tg, false);
}
int b2_net_load_fraction_dev(b2_net *n, int T, int nSeq, const int *lens, const float *in, const float *tg) {
    if (!n) return B2_ERR_BAD_ARG;
    return n->net.loadFraction(T, nSeq, lens, in, tg, true);
}
int b2_net_forward(b2_net *n, double *error) {
    if (!n) return B2_ERR_BAD_ARG;
    B2_TRY(n->net.computeForwardPass());
    return n->net.calculateError(error);
}
int b2_net_backward(b2_net *n) { return n ? n->net.computeBackwardPass() : B2_ERR_BAD_ARG; }
int b2_net_update_weights(b2_net *n, float lr, float mom) { return n ? n->net.updateWeights(lr, mom) : B2_ERR_BAD_ARG; }
int b2_net_accumulate_weight_updates(b2_net *n, int first) { return n ? n->net.accumulateWeightUpdates(first != 0) : B2_ERR_BAD_ARG; }
int b2_net_update_weights_batch(b2_net *n, float lr, float mom) { return n ? n->net.updateWeightsBatch(lr, mom) : B2_ERR_BAD_ARG; }
int b2_net_backward_empty(b2_net *n) { return n ? n->net.computeBackwardPassEmpty() : B2_ERR_BAD_ARG; }
int b2_net_train_step_empty(b2_net *n, float lr, float mom) { return n ? n->net.trainStepEmpty(lr, mom) : B2_ERR_BAD_ARG; }
int b2_dp_world_size(const b2_net *n) { return n ? dp_world(n->net) : 1; }
int b2_net_set_optimizer(b2_net *n, int option) { return n ? n->net.setOptimizerOption(option) : B2_ERR_BAD_ARG; }
int b2_net_get_optimizer_stats(b2_net *n, int i, float *host, size_t capacity, size_t *count) {
    TrainableLayer *t = trainable(n, i);
    if (!t) { set_error("b2_net_get_optimizer_stats: layer %d has no weights", i); return B2_ERR_BAD_ARG; }
    if (count) *count = t->statsFloats();
    if (host) {
        if (capacity < t->statsFloats()) { set_error("b2_net_get_optimizer_stats: %zu floats needed", t->statsFloats()); return B2_ERR_BAD_SHAPE; }
        B2_CUDA(cudaMemcpyAsync(host, t->weightStats(), t->statsFloats() * sizeof(float), cudaMemcpyDeviceToHost, n->net.stream));
        B2_CUDA(cudaStreamSynchronize(n->net.stream));
    }
    return B2_OK;
}

int b2_net_train_step(b2_net *n, int T, int nSeq, const int *lens, const float *in, const float *tg, float lr,
                      float mom, double *error) {
    if (!n) return B2_ERR_BAD_ARG;
    B2_TRY(n->net.loadFraction(T, nSeq, lens, in, tg, false));
    B2_TRY(n->net.computeForwardPass());
    B2_TRY(n->net.calculateError(nullptr));
    B2_TRY(n->net.computeBackwardPass());
    B2_TRY(n->net.updateWeights(lr, mom));
    if (error) {
        SsePostOutputLayer *post = dynamic_cast<SsePostOutputLayer *>(n->net.layers.back().get());
        B2_CUDA(cudaMemcpyAsync(error, post->lossDev(), sizeof(double), cudaMemcpyDeviceToHost, n->net.stream));
        B2_CUDA(cudaStreamSynchronize(n->net.stream));
    }
    return B2_OK;
}
int b2_net_prefetch_fraction(b2_net *n, int T, int nSeq, const int *lens, const float *in, const float *tg) {
    if (!n) return B2_ERR_BAD_ARG;
    return n->net.prefetchFraction(T, nSeq, lens, in, tg);
}
int b2_net_train_step_prefetched(b2_net *n, float lr, float mom, double *error) {
    if (!n) return B2_ERR_BAD_ARG;
    B2_TRY(n->net.usePrefetched());
    B2_TRY(n->net.computeForwardPass());
    B2_TRY(n->net.calculateError(nullptr));
    B2_TRY(n->net.computeBackwardPass());
    B2_TRY(n->net.updateWeights(lr, mom));
    if (error) {
        SsePostOutputLayer *post = dynamic_cast<SsePostOutputLayer *>(n->net.layers.back().get());
        B2_TRY(post->readError(error));
        B2_CUDA(cudaStreamSynchronize(n->net.stream));
    }
    return B2_OK;
}
int b2_net_read_error(b2_net *n, double *error) {
    if (!n || !error) return B2_ERR_BAD_ARG;
    SsePostOutputLayer *post = dynamic_cast<SsePostOutputLayer *>(n->net.layers.back().get());
    if (!post) { set_error("the last layer is not a post-output layer"); return B2_ERR_STATE; }
    return post->readError(error);
}
int b2_net_train_step_dev(b2_net *n, int T, int nSeq, const int *lens, const float *in, const float *tg, float lr,
                          float mom) {
    if (!n) return B2_ERR_BAD_ARG;
    B2_TRY(n->net.loadFraction(T, nSeq, lens, in, tg, true));
    B2_TRY(n->net.computeForwardPass());
    B2_TRY(n->net.calculateError(nullptr));
    B2_TRY(n->net.computeBackwardPass());
    return n->net.updateWeights(lr, mom);
}

static int copy_layer_vec(b2_net *n, int i, float *host, bool errors) {
    if (!n || !host || i < 0 || i >= (int)n->net.layers.size()) { set_error("bad layer index %d", i); return B2_ERR_BAD_ARG; }
    Layer *l = n->net.layers[i].get();
    const float *src = errors ? l->outputErrors() : (i == 0 ? n->net.frac.inputs : l->outputs());
    if (dynamic_cast<SsePostOutputLayer *>(l)) src = errors ? nullptr : n->net.frac.targets;
    if (!src) { set_error("layer %d keeps no such vector", i); return B2_ERR_BAD_ARG; }
    B2_TRY(n->net.synchronize());
    B2_CUDA(cudaMemcpy(host, src, (size_t)n->net.frac.T * n->net.P * l->size() * sizeof(float), cudaMemcpyDeviceToHost));
    return B2_OK;
}
int b2_net_get_outputs(b2_net *n, int i, float *host) { return copy_layer_vec(n, i, host, false); }
int b2_net_get_output_errors(b2_net *n, int i, float *host) { return copy_layer_vec(n, i, host, true); }
int b2_net_synchronize(b2_net *n) { return n ? n->net.synchronize() : B2_ERR_BAD_ARG; }
b2_stream b2_net_stream(b2_net *n) { return n ? (b2_stream)n->net.stream : nullptr; }
int b2_net_recurrence_path(b2_net *n, int layer, int backward) {
    if (!n || layer < 0 || layer >= (int)n->net.layers.size()) return -1;
    LstmLayer *l = dynamic_cast<LstmLayer *>(n->net.layers[layer].get());
    if (!l) return -1;
    return backward ? l->impl().bwd_path : l->impl().fwd_path;
}
int b2_net_set_recurrence_mode(b2_net *n, int mode) { if (!n) return B2_ERR_BAD_ARG; n->net.recurrenceMode = mode; return B2_OK; }
int b2_net_set_force_ffma(b2_net *n, int on) { if (!n) return B2_ERR_BAD_ARG; n->net.forceFfma = on != 0; return B2_OK; }
unsigned long long b2_net_launch_count(const b2_net *n) { return n ? g_launches - n->net.launchesAtCreate : 0; }

int b2_net_set_profiling(b2_net *n, int on) {
    if (!n) return B2_ERR_BAD_ARG;
    n->net.synchronize();
    for (size_t i = 0; i < n->net.prof.size(); ++i) { cudaEventDestroy(n->net.prof[i].a); cudaEventDestroy(n->net.prof[i].b); }
    n->net.prof.clear();
    n->net.profiling = on != 0;
    return B2_OK;
}
// Sums the recorded intervals by name (since profiling was last switched on) and clears them.
int b2_net_get_profile(b2_net *n, int cap, const char **names, float *ms, int *launches) {
    if (!n) return 0;
    n->net.synchronize();
    std::vector<std::string> order;
    std::map<std::string, std::pair<float, int> > acc;
    for (size_t i = 0; i < n->net.prof.size(); ++i) {
        ProfileEntry &e = n->net.prof[i];
        float t = 0;
        cudaEventElapsedTime(&t, e.a, e.b);
        if (!acc.count(e.name)) order.push_back(e.name);
        acc[e.name].first += t;
        acc[e.name].second += e.launches;
        cudaEventDestroy(e.a);
        cudaEventDestroy(e.b);
    }
    n->net.prof.clear();
    n->profNames = order;
    int cnt = 0;
    for (size_t i = 0; i < order.size() && cnt < cap; ++i, ++cnt) {
        names[cnt] = n->profNames[i].c_str();
        ms[cnt] = acc[order[i]].first;
        launches[cnt] = acc[order[i]].second;
    }
    return cnt;
}

}  // extern "C"
