// Test infrastructure only -- not part of the shipped library.
//
// A C-callable driver around the reference toolkit's OWN layer classes, compiled from the reference
// sources where they lie.  Two instances of the same driver:
//   ref_*      the Cpu-device classes (layers::InputLayer<Cpu>, FeedForwardLayer<Cpu,*>, LstmLayer<Cpu>,
//              SsePostOutputLayer<Cpu>): the checker of every parity test;
//   refb200_*  (only with -DREF_WITH_B200_ADAPTER, linked against libb2lstm.so) the reference's Gpu-device
//              classes with layers::LstmLayerB200<Gpu> (project-currennt-public_b200/adapter/LstmLayerB200.hpp)
//              standing where LayerFactory.cu:127-132 creates LstmLayer<Gpu>: the drop-in claim, compiled and run.  It performs the same sequence of calls
// the reference's NeuralNetwork/Optimizer make for one training fraction
// (NeuralNetwork.cpp:1367-1373 loadSequences, :1459-1460 forward, :2982-2989 calculateError,
//  :2744-2800 backward in reverse order; Optimizer.cu:85-165), because NeuralNetwork.cpp itself
// cannot be linked without libnetcdf and Boost.  All arithmetic happens inside the reference's
// functors; this file only moves buffers in and out.
//
// The steepest-descent update is the one exception: the reference's UpdateWeightFn sits in an
// anonymous namespace of SteepestDescentOptimizer.cu, which needs the whole NeuralNetwork to
// link, so ref_sgd_update() restates its three lines (SteepestDescentOptimizer.cu:74-100).
#include "Configuration.hpp"
#include "MacroDefine.hpp"
#include "activation_functions/Identity.cuh"
#include "activation_functions/Logistic.cuh"
#include "activation_functions/Tanh.cuh"
#include "helpers/JsonClasses.hpp"
#include "layers/FeedForwardLayer.hpp"
#include "layers/InputLayer.hpp"
#include "layers/LstmLayer.hpp"
#include "layers/SsePostOutputLayer.hpp"
#ifdef REF_WITH_B200_ADAPTER
#include "LstmLayerB200.hpp"
#endif
#include <thrust/copy.h>
#include "rapidjson/prettywriter.h"
#include "rapidjson/stringbuffer.h"
#include <cmath>
#include <cstdio>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

// DataSetFraction has a private constructor and names DataSet as its friend
// (data_sets/DataSetFraction.hpp:43,111).  The real DataSet needs libnetcdf, so the harness
// supplies its own class of that name whose only job is to fill a fraction from host arrays in
// the layout DataSet::_makeFractionTask produces (data_sets/DataSet.cpp:642-1022):
// time-major, parallel sequences interleaved, padded frames zero with pattern type NONE.
namespace data_sets {
class DataSet {
public:
    static DataSetFraction *make(int P, int T, int inDim, int outDim, int nSeq, const int *lens,
                                 const float *inputs, const float *targets) {
        DataSetFraction *f = new DataSetFraction;
        f->m_inputPatternSize = inDim;
        f->m_outputPatternSize = outDim;
        f->m_maxSeqLength = 0;
        f->m_minSeqLength = 1 << 30;
        f->m_inputs.assign(inputs, inputs + (size_t)T * P * inDim);
        f->m_outputs.assign(targets, targets + (size_t)T * P * outDim);
        f->m_patTypes.assign((size_t)T * P, PATTYPE_NONE);
        for (int p = 0; p < nSeq; ++p) {
            DataSetFraction::seq_info_t s;
            s.originalSeqIdx = p;
            s.length = lens[p];
            s.seqTag = "seq";
            s.exInputLength = 0;
            s.exOutputLength = 0;
            f->m_seqInfo.push_back(s);
            f->m_maxSeqLength = std::max(f->m_maxSeqLength, lens[p]);
            f->m_minSeqLength = std::min(f->m_minSeqLength, lens[p]);
            for (int t = 0; t < lens[p]; ++t) {
                char ty = PATTYPE_NORMAL;
                if (t == 0) ty = PATTYPE_FIRST;
                else if (t == lens[p] - 1) ty = PATTYPE_LAST;
                f->m_patTypes[(size_t)t * P + p] = ty;
            }
        }
        f->m_fracTotalLength = T * P;
        f->m_auxDataDim = -1;
        f->m_exInputDim = 0;
        f->m_exOutputDim = 0;
        f->m_flagDataValid = DATAFRACTION_VALID_FLAG_TRUE;
        return f;
    }
};
}  // namespace data_sets

namespace {

typedef activation_functions::Tanh ActTanh;
typedef activation_functions::Logistic ActLogistic;
typedef activation_functions::Identity ActIdentity;

Configuration *g_cfg = NULL;
char g_err[512] = "";

// which class stands for "lstm" / "blstm" on a device
template <typename TDevice, bool ADAPTER> struct LstmOf { typedef layers::LstmLayer<TDevice> type; };
#ifdef REF_WITH_B200_ADAPTER
template <typename TDevice> struct LstmOf<TDevice, true> { typedef layers::LstmLayerB200<TDevice> type; };
#endif

template <typename TDevice, bool ADAPTER>
struct RefNetT {
    typedef typename LstmOf<TDevice, ADAPTER>::type Lstm;
    int P, maxT;
    rapidjson::Document doc;
    std::vector<std::unique_ptr<layers::Layer<TDevice> > > layers;
    std::vector<std::string> types;
    std::vector<std::vector<float> > dY;  // output errors captured right before each layer's backward
    std::unique_ptr<data_sets::DataSetFraction> frac;
    std::vector<std::vector<float> > momentum;

    layers::TrainableLayer<TDevice> *trainable(int i) { return dynamic_cast<layers::TrainableLayer<TDevice> *>(layers[i].get()); }

    // network_json: {"layers":[{"size":..,"name":..,"type":..,"bias":..}, ...]} with types
    // input | feedforward_tanh | feedforward_logistic | feedforward_identity | lstm | blstm | sse.
    static RefNetT *create(const char *network_json, int P, int maxT) {
        try {
            if (!g_cfg) {
                static const char *av[] = {"ref"};
                g_cfg = new Configuration(1, av);
            }
            std::unique_ptr<RefNetT> n(new RefNetT);
            n->P = P;
            n->maxT = maxT;
            if (n->doc.template Parse<0>(network_json).HasParseError()) throw std::runtime_error("bad network json");
            rapidjson::Value &L = n->doc["layers"];
            helpers::JsonValue noWeights;
            for (rapidjson::SizeType i = 0; i < L.Size(); ++i) {
                std::string ty = L[i]["type"].GetString();
                layers::Layer<TDevice> *lay = NULL;
                if (i == 0) {
                    if (ty != "input") throw std::runtime_error("first layer must be input");
                    lay = new layers::InputLayer<TDevice>(&L[i], P, maxT, 0);
                } else {
                    layers::Layer<TDevice> &prev = *n->layers.back();
                    if (ty == "feedforward_tanh")
                        lay = new layers::FeedForwardLayer<TDevice, ActTanh>(&L[i], noWeights, prev, maxT, (int)i);
                    else if (ty == "feedforward_logistic")
                        lay = new layers::FeedForwardLayer<TDevice, ActLogistic>(&L[i], noWeights, prev, maxT, (int)i);
                    else if (ty == "feedforward_identity")
                        lay = new layers::FeedForwardLayer<TDevice, ActIdentity>(&L[i], noWeights, prev, maxT, (int)i);
                    else if (ty == "lstm")
                        lay = new Lstm(&L[i], noWeights, prev, maxT, (int)i, false);
                    else if (ty == "blstm")
                        lay = new Lstm(&L[i], noWeights, prev, maxT, (int)i, true);
                    else if (ty == "sse")
                        lay = new layers::SsePostOutputLayer<TDevice>(&L[i], prev, maxT, (int)i);
                    else
                        throw std::runtime_error("unsupported layer type " + ty);
                }
                n->layers.emplace_back(lay);
                n->types.push_back(ty);
            }
            n->dY.resize(n->layers.size());
            n->momentum.resize(n->layers.size());
            return n.release();
        } catch (const std::exception &e) {
            snprintf(g_err, sizeof g_err, "%s", e.what());
            return NULL;
        }
    }

    long num_weights(int i) {
        layers::TrainableLayer<TDevice> *t = trainable(i);
        return t ? (long)t->weights().size() : 0;
    }
    int set_weights(int i, const float *w) {
        layers::TrainableLayer<TDevice> *t = trainable(i);
        if (!t) return -1;
        thrust::copy(w, w + t->weights().size(), t->weights().begin());
        return 0;
    }
    int get_weights(int i, float *w) {
        layers::TrainableLayer<TDevice> *t = trainable(i);
        if (!t) return -1;
        thrust::copy(t->weights().begin(), t->weights().end(), w);
        return 0;
    }
    int get_weight_updates(int i, float *g) {
        layers::TrainableLayer<TDevice> *t = trainable(i);
        if (!t) return -1;
        thrust::copy(t->weightUpdates().begin(), t->weightUpdates().end(), g);
        return 0;
    }
    // inputs: T*P*inDim floats, targets: T*P*outDim floats, both [(t*P+p)*dim+d]; lens[nSeq], nSeq<=P.
    int load(int T, int nSeq, const int *lens, const float *inputs, const float *targets) {
        try {
            int inDim = layers.front()->size(), outDim = layers.back()->size();
            frac.reset(data_sets::DataSet::make(P, T, inDim, outDim, nSeq, lens, inputs, targets));
            for (size_t i = 0; i < layers.size(); ++i) layers[i]->loadSequences(*frac, NN_STATE_GAN_NOGAN_TRAIN);
            return 0;
        } catch (const std::exception &e) {
            snprintf(g_err, sizeof g_err, "%s", e.what());
            return -1;
        }
    }
    // forward through every layer, then the post-output layer's error (sum, not averaged); NaN on an exception
    double forward() {
        try {
            for (size_t i = 0; i < layers.size(); ++i) layers[i]->computeForwardPass(NN_STATE_GAN_NOGAN_TRAIN);
            layers::PostOutputLayer<TDevice> *post = dynamic_cast<layers::PostOutputLayer<TDevice> *>(layers.back().get());
            return post ? (double)post->calculateError() : 0.0;
        } catch (const std::exception &e) {
            snprintf(g_err, sizeof g_err, "%s", e.what());
            return std::nan("");
        }
    }
    int backward() {
        try {
            for (int i = (int)layers.size() - 1; i >= 0; --i) {
                typename TDevice::real_vector &e = layers[i]->outputErrors();
                dY[i].resize(e.size());
                thrust::copy(e.begin(), e.end(), dY[i].begin());
                layers[i]->computeBackwardPass(NN_STATE_GAN_NOGAN_TRAIN);
            }
            return 0;
        } catch (const std::exception &e) {
            snprintf(g_err, sizeof g_err, "%s", e.what());
            return -1;
        }
    }
    // count floats copied = T*P*size of the loaded fraction
    long get_outputs(int i, float *out) {
        size_t cnt = (size_t)layers[i]->curMaxSeqLength() * P * layers[i]->size();
        thrust::copy(layers[i]->outputs().begin(), layers[i]->outputs().begin() + cnt, out);
        return (long)cnt;
    }
    // output errors of layer i as they are AFTER the whole backward pass (for the layer below an
    // LSTM / feed-forward layer this is the dX that layer wrote)
    long get_output_errors(int i, float *out) {
        size_t cnt = (size_t)layers[i]->curMaxSeqLength() * P * layers[i]->size();
        thrust::copy(layers[i]->outputErrors().begin(), layers[i]->outputErrors().begin() + cnt, out);
        return (long)cnt;
    }
    // output errors of layer i as they were just BEFORE its own computeBackwardPass ran
    long get_output_errors_in(int i, float *out) {
        size_t cnt = (size_t)layers[i]->curMaxSeqLength() * P * layers[i]->size();
        if (dY[i].size() < cnt) return -1;
        std::copy(dY[i].begin(), dY[i].begin() + cnt, out);
        return (long)cnt;
    }
    // The document NeuralNetwork::exportLayers / exportWeights / saveNetwork write (NeuralNetwork.cpp:2993-3043,4104-4125):
    // every layer's own exportLayer and TrainableLayer::exportWeights (layers/TrainableLayer.cu:441-480) fill it, the
    // reference's rapidjson PrettyWriter turns it into text, as in saveNetwork.  Returns the length (without NUL), or
    // minus the needed capacity.
    long export_json(char *buf, long cap) {
        try {
            rapidjson::Document d;
            d.SetObject();
            rapidjson::Value layersArray(rapidjson::kArrayType);
            rapidjson::Value weightsObject(rapidjson::kObjectType);
            for (size_t i = 0; i < layers.size(); ++i) {
                layers[i]->exportLayer(&layersArray, &d.GetAllocator());
                layers::TrainableLayer<TDevice> *t = trainable((int)i);
                if (t) t->exportWeights(&weightsObject, &d.GetAllocator());
            }
            d.AddMember("layers", layersArray, d.GetAllocator());
            d.AddMember("weights", weightsObject, d.GetAllocator());
            rapidjson::StringBuffer sb;
            rapidjson::PrettyWriter<rapidjson::StringBuffer> writer(sb);
            d.Accept(writer);
            const long n = (long)sb.Size();
            if (n + 1 > cap) return -(n + 1);
            memcpy(buf, sb.GetString(), (size_t)n);
            buf[n] = 0;
            return n;
        } catch (const std::exception &e) {
            snprintf(g_err, sizeof g_err, "%s", e.what());
            return 0;
        }
    }
    // a net whose trainable layers read their weights from the document's "weights" section, as the reference does
    // when it continues from trained_network.jsn (TrainableLayer.cu:135-205)
    static RefNetT *create_with_weights(const char *network_json, int P, int maxT) {
        try {
            if (!g_cfg) {
                static const char *av[] = {"ref"};
                g_cfg = new Configuration(1, av);
            }
            std::unique_ptr<RefNetT> n(new RefNetT);
            n->P = P;
            n->maxT = maxT;
            if (n->doc.template Parse<0>(network_json).HasParseError()) throw std::runtime_error("bad network json");
            rapidjson::Value &L = n->doc["layers"];
            helpers::JsonValue weights;
            if (n->doc.HasMember("weights")) weights = helpers::JsonValue(&n->doc["weights"]);
            for (rapidjson::SizeType i = 0; i < L.Size(); ++i) {
                std::string ty = L[i]["type"].GetString();
                layers::Layer<TDevice> *lay = NULL;
                if (i == 0) lay = new layers::InputLayer<TDevice>(&L[i], P, maxT, 0);
                else {
                    layers::Layer<TDevice> &prev = *n->layers.back();
                    if (ty == "feedforward_tanh") lay = new layers::FeedForwardLayer<TDevice, ActTanh>(&L[i], weights, prev, maxT, (int)i);
                    else if (ty == "feedforward_logistic") lay = new layers::FeedForwardLayer<TDevice, ActLogistic>(&L[i], weights, prev, maxT, (int)i);
                    else if (ty == "feedforward_identity") lay = new layers::FeedForwardLayer<TDevice, ActIdentity>(&L[i], weights, prev, maxT, (int)i);
                    else if (ty == "lstm") lay = new Lstm(&L[i], weights, prev, maxT, (int)i, false);
                    else if (ty == "blstm") lay = new Lstm(&L[i], weights, prev, maxT, (int)i, true);
                    else if (ty == "sse") lay = new layers::SsePostOutputLayer<TDevice>(&L[i], prev, maxT, (int)i);
                    else throw std::runtime_error("unsupported layer type " + ty);
                }
                n->layers.emplace_back(lay);
                n->types.push_back(ty);
            }
            n->dY.resize(n->layers.size());
            n->momentum.resize(n->layers.size());
            return n.release();
        } catch (const std::exception &e) {
            snprintf(g_err, sizeof g_err, "%s", e.what());
            return NULL;
        }
    }
    // g <- 0 where NaN/Inf; delta <- momentum*delta - lr*g; w <- w + delta   (restated, see header); host vectors only
    void sgd_update(float lr, float mom) {
        for (size_t i = 0; i < layers.size(); ++i) {
            layers::TrainableLayer<TDevice> *t = trainable((int)i);
            if (!t) continue;
            size_t nw = t->weights().size();
            std::vector<float> w(nw), g(nw);
            thrust::copy(t->weights().begin(), t->weights().end(), w.begin());
            thrust::copy(t->weightUpdates().begin(), t->weightUpdates().end(), g.begin());
            if (momentum[i].size() != nw) momentum[i].assign(nw, 0.0f);
            float rate = t->learningRate() >= 0 ? t->learningRate() : lr;
            for (size_t k = 0; k < nw; ++k) {
                float gk = g[k];
                if (std::isnan(gk) || std::isinf(gk)) gk = 0;
                float d = mom * momentum[i][k] - rate * gk;
                momentum[i][k] = d;
                w[k] += d;
            }
            thrust::copy(w.begin(), w.end(), t->weights().begin());
        }
    }
};

}  // namespace

#define REF_DEFINE_API(PFX, NET)                                                                                              \
    void *PFX##create(const char *network_json, int P, int maxT) { return NET::create(network_json, P, maxT); }                \
    void PFX##destroy(void *h) { delete (NET *)h; }                                                                           \
    int PFX##num_layers(void *h) { return (int)((NET *)h)->layers.size(); }                                                   \
    int PFX##layer_size(void *h, int i) { return ((NET *)h)->layers[i]->size(); }                                             \
    long PFX##num_weights(void *h, int i) { return ((NET *)h)->num_weights(i); }                                              \
    int PFX##set_weights(void *h, int i, const float *w) { return ((NET *)h)->set_weights(i, w); }                            \
    int PFX##get_weights(void *h, int i, float *w) { return ((NET *)h)->get_weights(i, w); }                                  \
    int PFX##get_weight_updates(void *h, int i, float *g) { return ((NET *)h)->get_weight_updates(i, g); }                    \
    int PFX##load(void *h, int T, int nSeq, const int *lens, const float *inputs, const float *targets) {                     \
        return ((NET *)h)->load(T, nSeq, lens, inputs, targets);                                                              \
    }                                                                                                                         \
    double PFX##forward(void *h) { return ((NET *)h)->forward(); }                                                            \
    void PFX##backward(void *h) { ((NET *)h)->backward(); }                                                                   \
    long PFX##get_outputs(void *h, int i, float *out) { return ((NET *)h)->get_outputs(i, out); }                             \
    long PFX##get_output_errors(void *h, int i, float *out) { return ((NET *)h)->get_output_errors(i, out); }                 \
    long PFX##get_output_errors_in(void *h, int i, float *out) { return ((NET *)h)->get_output_errors_in(i, out); }           \
    void PFX##sgd_update(void *h, float lr, float mom) { ((NET *)h)->sgd_update(lr, mom); }                                   \
    long PFX##export_json(void *h, char *buf, long cap) { return ((NET *)h)->export_json(buf, cap); }                         \
    void *PFX##create_with_weights(const char *network_json, int P, int maxT) { return NET::create_with_weights(network_json, P, maxT); }

extern "C" {

const char *ref_last_error(void) { return g_err; }

typedef RefNetT<Cpu, false> RefNetCpu;
REF_DEFINE_API(ref_, RefNetCpu)

#ifdef REF_WITH_B200_ADAPTER
typedef RefNetT<Gpu, true> RefNetB200;
REF_DEFINE_API(refb200_, RefNetB200)
#endif

}  // extern "C"
