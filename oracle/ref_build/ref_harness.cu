// Test infrastructure only -- not part of the shipped library.
//
// A C-callable driver around the reference toolkit's OWN Cpu-device layer classes
// (layers::InputLayer<Cpu>, FeedForwardLayer<Cpu,*>, LstmLayer<Cpu>, SsePostOutputLayer<Cpu>),
// compiled from the reference sources where they lie.  It performs the same sequence of calls
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

struct RefNet {
    int P, maxT;
    rapidjson::Document doc;
    std::vector<std::unique_ptr<layers::Layer<Cpu> > > layers;
    std::vector<std::string> types;
    std::vector<std::vector<float> > dY;  // output errors captured right before each layer's backward
    std::unique_ptr<data_sets::DataSetFraction> frac;
    std::vector<std::vector<float> > momentum;
};

Configuration *g_cfg = NULL;
char g_err[512] = "";

layers::TrainableLayer<Cpu> *trainable(RefNet *n, int i) {
    return dynamic_cast<layers::TrainableLayer<Cpu> *>(n->layers[i].get());
}

}  // namespace

extern "C" {

const char *ref_last_error(void) { return g_err; }

// network_json: {"layers":[{"size":..,"name":..,"type":..,"bias":..}, ...]} with types
// input | feedforward_tanh | feedforward_logistic | feedforward_identity | lstm | blstm | sse.
void *ref_create(const char *network_json, int P, int maxT) {
    try {
        if (!g_cfg) {
            static const char *av[] = {"ref"};
            g_cfg = new Configuration(1, av);
        }
        std::unique_ptr<RefNet> n(new RefNet);
        n->P = P;
        n->maxT = maxT;
        if (n->doc.Parse<0>(network_json).HasParseError()) throw std::runtime_error("bad network json");
        rapidjson::Value &L = n->doc["layers"];
        helpers::JsonValue noWeights;
        for (rapidjson::SizeType i = 0; i < L.Size(); ++i) {
            std::string ty = L[i]["type"].GetString();
            layers::Layer<Cpu> *lay = NULL;
            if (i == 0) {
                if (ty != "input") throw std::runtime_error("first layer must be input");
                lay = new layers::InputLayer<Cpu>(&L[i], P, maxT, 0);
            } else {
                layers::Layer<Cpu> &prev = *n->layers.back();
                if (ty == "feedforward_tanh")
                    lay = new layers::FeedForwardLayer<Cpu, ActTanh>(&L[i], noWeights, prev, maxT, (int)i);
                else if (ty == "feedforward_logistic")
                    lay = new layers::FeedForwardLayer<Cpu, ActLogistic>(&L[i], noWeights, prev, maxT, (int)i);
                else if (ty == "feedforward_identity")
                    lay = new layers::FeedForwardLayer<Cpu, ActIdentity>(&L[i], noWeights, prev, maxT, (int)i);
                else if (ty == "lstm")
                    lay = new layers::LstmLayer<Cpu>(&L[i], noWeights, prev, maxT, (int)i, false);
                else if (ty == "blstm")
                    lay = new layers::LstmLayer<Cpu>(&L[i], noWeights, prev, maxT, (int)i, true);
                else if (ty == "sse")
                    lay = new layers::SsePostOutputLayer<Cpu>(&L[i], prev, maxT, (int)i);
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

void ref_destroy(void *h) { delete (RefNet *)h; }

int ref_num_layers(void *h) { return (int)((RefNet *)h)->layers.size(); }
int ref_layer_size(void *h, int i) { return ((RefNet *)h)->layers[i]->size(); }

long ref_num_weights(void *h, int i) {
    layers::TrainableLayer<Cpu> *t = trainable((RefNet *)h, i);
    return t ? (long)t->weights().size() : 0;
}
int ref_set_weights(void *h, int i, const float *w) {
    layers::TrainableLayer<Cpu> *t = trainable((RefNet *)h, i);
    if (!t) return -1;
    std::copy(w, w + t->weights().size(), t->weights().begin());
    return 0;
}
int ref_get_weights(void *h, int i, float *w) {
    layers::TrainableLayer<Cpu> *t = trainable((RefNet *)h, i);
    if (!t) return -1;
    std::copy(t->weights().begin(), t->weights().end(), w);
    return 0;
}
int ref_get_weight_updates(void *h, int i, float *g) {
    layers::TrainableLayer<Cpu> *t = trainable((RefNet *)h, i);
    if (!t) return -1;
    std::copy(t->weightUpdates().begin(), t->weightUpdates().end(), g);
    return 0;
}

// inputs: T*P*inDim floats, targets: T*P*outDim floats, both [(t*P+p)*dim+d]; lens[nSeq], nSeq<=P.
int ref_load(void *h, int T, int nSeq, const int *lens, const float *inputs, const float *targets) {
    RefNet *n = (RefNet *)h;
    try {
        int inDim = n->layers.front()->size(), outDim = n->layers.back()->size();
        n->frac.reset(data_sets::DataSet::make(n->P, T, inDim, outDim, nSeq, lens, inputs, targets));
        for (size_t i = 0; i < n->layers.size(); ++i) n->layers[i]->loadSequences(*n->frac, NN_STATE_GAN_NOGAN_TRAIN);
        return 0;
    } catch (const std::exception &e) {
        snprintf(g_err, sizeof g_err, "%s", e.what());
        return -1;
    }
}

// forward through every layer, then the post-output layer's error (sum, not averaged)
double ref_forward(void *h) {
    RefNet *n = (RefNet *)h;
    for (size_t i = 0; i < n->layers.size(); ++i) n->layers[i]->computeForwardPass(NN_STATE_GAN_NOGAN_TRAIN);
    layers::PostOutputLayer<Cpu> *post = dynamic_cast<layers::PostOutputLayer<Cpu> *>(n->layers.back().get());
    return post ? (double)post->calculateError() : 0.0;
}

void ref_backward(void *h) {
    RefNet *n = (RefNet *)h;
    for (int i = (int)n->layers.size() - 1; i >= 0; --i) {
        Cpu::real_vector &e = n->layers[i]->outputErrors();
        n->dY[i].assign(e.begin(), e.end());
        n->layers[i]->computeBackwardPass(NN_STATE_GAN_NOGAN_TRAIN);
    }
}

// count floats copied = T*P*size of the loaded fraction
long ref_get_outputs(void *h, int i, float *out) {
    RefNet *n = (RefNet *)h;
    size_t cnt = (size_t)n->layers[i]->curMaxSeqLength() * n->P * n->layers[i]->size();
    std::copy(n->layers[i]->outputs().begin(), n->layers[i]->outputs().begin() + cnt, out);
    return (long)cnt;
}
// output errors of layer i as they are AFTER the whole backward pass (for the layer below an
// LSTM / feed-forward layer this is the dX that layer wrote)
long ref_get_output_errors(void *h, int i, float *out) {
    RefNet *n = (RefNet *)h;
    size_t cnt = (size_t)n->layers[i]->curMaxSeqLength() * n->P * n->layers[i]->size();
    std::copy(n->layers[i]->outputErrors().begin(), n->layers[i]->outputErrors().begin() + cnt, out);
    return (long)cnt;
}
// output errors of layer i as they were just BEFORE its own computeBackwardPass ran
long ref_get_output_errors_in(void *h, int i, float *out) {
    RefNet *n = (RefNet *)h;
    size_t cnt = (size_t)n->layers[i]->curMaxSeqLength() * n->P * n->layers[i]->size();
    if (n->dY[i].size() < cnt) return -1;
    std::copy(n->dY[i].begin(), n->dY[i].begin() + cnt, out);
    return (long)cnt;
}

// g <- 0 where NaN/Inf; delta <- momentum*delta - lr*g; w <- w + delta   (restated, see header)
void ref_sgd_update(void *h, float lr, float mom) {
    RefNet *n = (RefNet *)h;
    for (size_t i = 0; i < n->layers.size(); ++i) {
        layers::TrainableLayer<Cpu> *t = trainable(n, (int)i);
        if (!t) continue;
        size_t nw = t->weights().size();
        if (n->momentum[i].size() != nw) n->momentum[i].assign(nw, 0.0f);
        float rate = t->learningRate() >= 0 ? t->learningRate() : lr;
        for (size_t k = 0; k < nw; ++k) {
            float g = t->weightUpdates()[k];
            if (std::isnan(g) || std::isinf(g)) g = 0;
            float d = mom * n->momentum[i][k] - rate * g;
            n->momentum[i][k] = d;
            t->weights()[k] += d;
        }
    }
}

}  // extern "C"
