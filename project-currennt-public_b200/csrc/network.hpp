// Host-side mirror of the reference toolkit's class structure for the training path, same names
// and call order (paths inside CURRENNT_codes/currennt_lib/src/):
//   layers::Layer            layers/Layer.hpp:42-331        -> b2::Layer
//   layers::TrainableLayer   layers/TrainableLayer.hpp      -> b2::TrainableLayer
//   layers::InputLayer / FeedForwardLayer / LstmLayer / SsePostOutputLayer
//   NeuralNetwork            NeuralNetwork.cpp:1056-1086,1367-1373,1734-1742,2864-2873,2982-2989
//   SteepestDescentOptimizer optimizers/SteepestDescentOptimizer.cu:281-472
// Every vector the reference keeps in a thrust::device_vector is a raw device allocation here.
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "common.cuh"
#include "json.hpp"
#include "lstm_layer.hpp"

namespace b2 {

class NeuralNetwork;

// what DataSetFraction hands to Layer::loadSequences (data_sets/DataSetFraction.hpp)
struct Fraction {
    int T = 0, Tmin = 0, nSeq = 0;
    long realFrames = 0;
    const char *patTypes = nullptr;   // device
    const float *inputs = nullptr;    // device, [T*P*inputSize]
    const float *targets = nullptr;   // device, [T*P*outputSize]
};

class Layer {
public:
    Layer(NeuralNetwork &net, const json::Value &j, int P, int maxT, Layer *prev);
    virtual ~Layer();
    const std::string &name() const { return name_; }
    const std::string &type() const { return type_; }
    int size() const { return size_; }
    int parallelSequences() const { return P_; }
    int maxSeqLength() const { return maxT_; }
    int curMaxSeqLength() const { return curMax_; }
    int curMinSeqLength() const { return curMin_; }
    float *outputs() { return outputs_; }
    float *outputErrors() { return outputErrors_; }
    const char *patTypes() const { return pat_; }
    Layer *precedingLayer() { return prev_; }
    virtual int loadSequences(const Fraction &f, int nnState);
    virtual int computeForwardPass(int nnState) = 0;
    virtual int computeBackwardPass(int nnState) = 0;
    int allocate();

protected:
    NeuralNetwork &net_;
    std::string name_, type_;
    int size_, P_, maxT_, curMax_ = 0, curMin_ = 0;
    const char *pat_ = nullptr;
    Layer *prev_;
    float *outputs_ = nullptr, *outputErrors_ = nullptr;
    bool ownsBuffers_ = false;
};

class TrainableLayer : public Layer {
public:
    TrainableLayer(NeuralNetwork &net, const json::Value &j, int P, int maxT, Layer *prev);
    ~TrainableLayer() override;
    size_t numWeights() const { return nW_; }
    float *weights() { return weights_; }
    float *weightUpdates() { return weightUpdates_; }
    float *weightDeltas() { return weightDeltas_; }
    float *weightStats() { return weightStats_; }
    float *weightAccum() { return weightAccum_; }
    int allocateAccum();
    size_t statsFloats() const { return statsFloats_; }
    // AdaGrad / Adam statistics (Optimizer::m_weightStats): n floats filled with `init`, or 2n zeros for Adam
    int allocateStats(size_t floats, float init, cudaStream_t st);
    float bias() const { return bias_; }
    float learningRate() const { return learningRate_; }
    int allocateWeights(size_t n);

protected:
    size_t nW_ = 0;
    float bias_, learningRate_;
    float *weights_ = nullptr, *weightUpdates_ = nullptr, *weightDeltas_ = nullptr, *weightStats_ = nullptr, *weightAccum_ = nullptr;
    size_t statsFloats_ = 0;
};

class InputLayer : public Layer {
public:
    using Layer::Layer;
    int loadSequences(const Fraction &f, int nnState) override;
    int computeForwardPass(int) override { return B2_OK; }
    int computeBackwardPass(int) override { return B2_OK; }
};

class FeedForwardLayer : public TrainableLayer {
public:
    FeedForwardLayer(NeuralNetwork &net, const json::Value &j, int P, int maxT, Layer *prev, int act);
    int computeForwardPass(int nnState) override;
    int computeBackwardPass(int nnState) override;

private:
    int act_;
};

class LstmLayer : public TrainableLayer {
public:
    LstmLayer(NeuralNetwork &net, const json::Value &j, int P, int maxT, Layer *prev, bool bidirectional);
    ~LstmLayer() override;
    int init();
    int loadSequences(const Fraction &f, int nnState) override;
    int computeForwardPass(int nnState) override;
    int computeBackwardPass(int nnState) override;
    LstmLayerImpl &impl() { return impl_; }

private:
    bool bidirectional_;
    LstmLayerImpl impl_;
};

class SsePostOutputLayer : public Layer {
public:
    using Layer::Layer;
    int loadSequences(const Fraction &f, int nnState) override;
    int computeForwardPass(int) override { return B2_OK; }
    int computeBackwardPass(int nnState) override;
    int calculateError(double *hostError);   // hostError == NULL: stay asynchronous
    int readError(double *hostError);        // waits for the last calculateError only
    double *lossDev() { return lossDev_; }
    int init();
    ~SsePostOutputLayer() override;

private:
    const float *targets_ = nullptr;
    double *lossDev_ = nullptr, *lossWs_ = nullptr;
    double *lossPinned_ = nullptr;   // two pinned slots, alternating
    int lossSlot_ = 0;
    cudaEvent_t lossReady_ = nullptr;
};

struct ProfileEntry {
    std::string name;
    cudaEvent_t a, b;
    int launches;
};

struct DpComm;  // dp_nccl.cu

class NeuralNetwork {
public:
    NeuralNetwork() {}
    ~NeuralNetwork();
    int create(const char *networkJson, int P, int maxT, unsigned seed);
    int loadFraction(int T, int nSeq, const int *lens, const float *in, const float *tg, bool onDevice);
    int computeForwardPass();
    int calculateError(double *hostError);
    int computeBackwardPass();
    int updateWeights(float lr, float mom);
    // data-parallel step of a rank that has no sequence in the current fraction: zero gradients into the sums, update
    int computeBackwardPassEmpty();
    int trainStepEmpty(float lr, float mom);
    // batch (non-stochastic) learning: gradients of the fractions of an epoch are accumulated, one update at its end
    int accumulateWeightUpdates(bool first);
    int updateWeightsBatch(float lr, float mom);
    // optimizer option of the reference (MacroDefine.hpp:32-37): 0 plain, 1 AdaGrad, 2 average gradient,
    // 3 SGD accumulating AdaGrad statistics, 5 Adam
    int setOptimizerOption(int option);
    int optOption = 0;
    float adamBeta1Accum = 1.0f, adamBeta2Accum = 1.0f;
    float *fracLenDev = nullptr;
    int synchronize();

    std::vector<std::unique_ptr<Layer> > layers;
    int P = 0, maxT = 0;
    cudaStream_t stream = nullptr, commStream = nullptr;
    Fraction frac;
    bool forceFfma = false;
    int recurrenceMode = 1;
    // shared scratch for GEMM split-K and column sums
    float *ws = nullptr;
    size_t wsFloats = 0;
    // tensor-core GEMMs: arena for the tf32 hi/lo operand copies, device status word of their waits
    TcScratch tcScratch;
    int *statusDev = nullptr;
    // device copies of the current fraction, double-buffered so that the next fraction can be copied
    // (on copyStream) while the current one is being processed
    float *inBuf[2] = {nullptr, nullptr}, *tgBuf[2] = {nullptr, nullptr};
    char *patBuf[2] = {nullptr, nullptr};
    char *patPinned[2] = {nullptr, nullptr};   // pinned host staging of the pattern types
    Fraction fracBuf[2];
    int cur = 0;
    bool prefetchPending = false;
    cudaStream_t copyStream = nullptr;
    cudaEvent_t prefetchDone[2] = {nullptr, nullptr}, bufFree[2] = {nullptr, nullptr}, patCopied[2] = {nullptr, nullptr};
    int stageFraction(int b, int T, int nSeq, const int *lens, const float *in, const float *tg, bool onDevice,
                      cudaStream_t st);
    int prefetchFraction(int T, int nSeq, const int *lens, const float *in, const float *tg);
    int usePrefetched();
    // profiling
    bool profiling = false;
    std::vector<ProfileEntry> prof;
    std::vector<cudaEvent_t> eventPool;
    void profBegin(const char *name);
    void profEnd();
    unsigned long long launchesAtCreate = 0;
    // data parallel
    DpComm *dp = nullptr;
    std::vector<cudaEvent_t> gradReady;   // one per layer
    int gemm(float *C, long ldc, const float *A, long sam, long sak, const float *B, long sbk, long sbn, int m, int n,
             int k, bool acc);

private:
    unsigned long long profLaunch0_ = 0;
};

// dp_nccl.cu
int dp_get_unique_id(void *bytes);
int dp_attach(NeuralNetwork &net, int rank, int world, const void *idBytes);
int dp_detach(NeuralNetwork &net);
int dp_allreduce_sum(NeuralNetwork &net, float *buf, size_t n, cudaStream_t st);
int dp_allreduce_double(NeuralNetwork &net, double *devValue, cudaStream_t st);
int dp_world(const NeuralNetwork &net);

struct ProfScope {
    NeuralNetwork &n;
    ProfScope(NeuralNetwork &net, const char *name) : n(net) { if (n.profiling) n.profBegin(name); }
    ~ProfScope() { if (n.profiling) n.profEnd(); }
};

}  // namespace b2
