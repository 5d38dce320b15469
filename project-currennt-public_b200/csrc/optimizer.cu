// Host side of the training run around the hot path: network export, the epoch loop with
// validation-based early stopping, and autosave / continue.
//
// Mirrors, for steepest descent with momentum and hybrid online/batch updates:
//   NeuralNetwork::exportLayers / exportWeights / saveNetwork   (NeuralNetwork.cpp:2993-3043, 4104-4125)
//   TrainableLayer::exportLayer / exportWeights                 (layers/TrainableLayer.cu:441-480)
//   Optimizer::train, _storeWeights, _restoreWeights            (optimizers/Optimizer.cu:315-352, 565-689)
//   Optimizer::exportState / importState / saveState / restoreState (Optimizer.cu:692-765, 851-933)
//   SteepestDescentOptimizer::exportState / importState         (SteepestDescentOptimizer.cu:505-522)
// The JSON documents carry the reference's member names, so a network or an autosave written here is
// read by the reference and the other way round.  Numbers are printed with 9 significant digits
// (exact for fp32); `digits` = 6 reproduces the reference's "%g".
#include <stdio.h>
#include <string.h>

#include <limits>
#include <string>
#include <vector>

#include "network.hpp"

using namespace b2;

extern "C" b2::NeuralNetwork *b2_net_impl(b2_net *n);

namespace {

void put_number(std::string &out, double v, int digits) {
    char buf[64];
    snprintf(buf, sizeof(buf), "%.*g", digits, v);
    out += buf;
}

void put_string(std::string &out, const std::string &s) {
    out += '"';
    for (char c : s) {
        switch (c) {
            case '"': out += "\\\""; break;
            case '\\': out += "\\\\"; break;
            case '\n': out += "\\n"; break;
            case '\r': out += "\\r"; break;
            case '\t': out += "\\t"; break;
            default:
                if ((unsigned char)c < 0x20) {
                    char buf[8];
                    snprintf(buf, sizeof(buf), "\\u%04X", c);
                    out += buf;
                } else {
                    out += c;
                }
        }
    }
    out += '"';
}

void put_array(std::string &out, const float *v, size_t n, int digits) {
    out += '[';
    for (size_t i = 0; i < n; ++i) {
        if (i) out += ',';
        put_number(out, v[i], digits);
    }
    out += ']';
}

// blocks of a layer's weight vector: input | bias | internal (TrainableLayer.cu:455-474)
void weight_sections(Layer *l, TrainableLayer *t, size_t *nIn, size_t *nBias) {
    const int perBlock = (l->type() == "lstm" || l->type() == "blstm") ? 4 : 1;
    *nIn = (size_t)l->size() * perBlock * l->precedingLayer()->size();
    *nBias = (size_t)l->size() * perBlock;
}

int fetch_weights(NeuralNetwork &nn, TrainableLayer *t, std::vector<float> &w) {
    w.resize(t->numWeights());
    B2_CUDA(cudaMemcpyAsync(w.data(), t->weights(), w.size() * sizeof(float), cudaMemcpyDeviceToHost, nn.stream));
    B2_CUDA(cudaStreamSynchronize(nn.stream));
    return B2_OK;
}

// "layers": [...], "weights": {...}
int export_network(NeuralNetwork &nn, std::string &out, int digits) {
    out += "\"layers\":[";
    for (size_t i = 0; i < nn.layers.size(); ++i) {
        Layer *l = nn.layers[i].get();
        if (i) out += ',';
        out += "\n{\"name\":";
        put_string(out, l->name());
        out += ",\"type\":";
        put_string(out, l->type());
        out += ",\"size\":" + std::to_string(l->size());
        if (TrainableLayer *t = dynamic_cast<TrainableLayer *>(l)) {
            out += ",\"bias\":";
            put_number(out, t->bias(), digits);
            if (t->learningRate() >= 0.0f) {
                out += ",\"learningRate\":";
                put_number(out, t->learningRate(), digits);
            }
        }
        out += '}';
    }
    out += "\n],\n\"weights\":{";
    bool first = true;
    std::vector<float> w;
    for (size_t i = 0; i < nn.layers.size(); ++i) {
        Layer *l = nn.layers[i].get();
        TrainableLayer *t = dynamic_cast<TrainableLayer *>(l);
        if (!t || !t->numWeights()) continue;
        B2_TRY(fetch_weights(nn, t, w));
        size_t nIn, nBias;
        weight_sections(l, t, &nIn, &nBias);
        if (!first) out += ',';
        first = false;
        out += '\n';
        put_string(out, l->name());
        out += ":{\"input\":";
        put_array(out, w.data(), nIn, digits);
        out += ",\"bias\":";
        put_array(out, w.data() + nIn, nBias, digits);
        out += ",\"internal\":";
        put_array(out, w.data() + nIn + nBias, w.size() - nIn - nBias, digits);
        out += '}';
    }
    out += "\n}";
    return B2_OK;
}

int write_file(const char *filename, const std::string &text) {
    FILE *f = fopen(filename, "w");
    if (!f) { set_error("Cannot open file '%s'", filename); return B2_ERR_BAD_ARG; }
    const size_t n = fwrite(text.data(), 1, text.size(), f);
    const int rc = fclose(f);
    if (n != text.size() || rc != 0) { set_error("Cannot write file '%s'", filename); return B2_ERR_BAD_ARG; }
    return B2_OK;
}

int read_file(const char *filename, std::string &text) {
    FILE *f = fopen(filename, "r");
    if (!f) { set_error("Cannot open file '%s'", filename); return B2_ERR_BAD_ARG; }
    char buf[1 << 16];
    size_t n;
    text.clear();
    while ((n = fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, n);
    fclose(f);
    return B2_OK;
}

}  // namespace

struct b2_optimizer {
    b2_net *net = nullptr;
    b2_data *trainingSet = nullptr, *validationSet = nullptr, *testSet = nullptr;
    b2_optimizer_options opt{};
    // Optimizer<TDevice> members of the same names
    bool finished = false;
    float learningRate = 0.0f;   // SteepestDescentOptimizer::m_learningRate (changeLR / adjustLR)
    int curEpoch = 0, epochsSinceLowestError = 0;
    float lowestValidationError = std::numeric_limits<float>::max();
    float curTrainingError = std::numeric_limits<float>::max();
    float curValidationError = std::numeric_limits<float>::max();
    float curTestError = std::numeric_limits<float>::max();
    float curTrainingErrorPerFrame = 0, curValidationErrorPerFrame = 0, curTestErrorPerFrame = 0;
    std::vector<std::vector<float> > bestWeights;   // [layer], empty for layers without weights

    int storeWeights() {
        NeuralNetwork &nn = *b2_net_impl(net);
        for (size_t i = 1; i < nn.layers.size(); ++i)
            if (TrainableLayer *t = dynamic_cast<TrainableLayer *>(nn.layers[i].get())) B2_TRY(fetch_weights(nn, t, bestWeights[i]));
        return B2_OK;
    }
    int restoreWeights() {
        NeuralNetwork &nn = *b2_net_impl(net);
        for (size_t i = 1; i < nn.layers.size(); ++i)
            if (TrainableLayer *t = dynamic_cast<TrainableLayer *>(nn.layers[i].get())) {
                if (bestWeights[i].size() != t->numWeights()) { set_error("best weights of layer %zu have the wrong size", i); return B2_ERR_STATE; }
                B2_CUDA(cudaMemcpyAsync(t->weights(), bestWeights[i].data(), bestWeights[i].size() * sizeof(float),
                                        cudaMemcpyHostToDevice, nn.stream));
            }
        B2_CUDA(cudaStreamSynchronize(nn.stream));
        return B2_OK;
    }
};

namespace {

int per_layer_vectors(const json::Value &doc, const char *name, NeuralNetwork &nn, std::vector<std::vector<float> > *out) {
    const json::Value *a = doc.find(name);
    if (!a || a->kind != json::Value::Array) { set_error("Array '%s' is missing or has the wrong type", name); return B2_ERR_BAD_ARG; }
    if (a->arr.size() != nn.layers.size()) { set_error("Array '%s' has a wrong size", name); return B2_ERR_BAD_SHAPE; }
    out->assign(nn.layers.size(), std::vector<float>());
    for (size_t i = 0; i < a->arr.size(); ++i) {
        const json::Value &v = a->arr[i];
        if (v.kind != json::Value::Array) { set_error("Object in '%s' is not an array", name); return B2_ERR_BAD_ARG; }
        TrainableLayer *t = dynamic_cast<TrainableLayer *>(nn.layers[i].get());
        const size_t want = (t && i > 0) ? t->numWeights() : 0;
        if (v.arr.size() != want) { set_error("Subarray in '%s' has a wrong size", name); return B2_ERR_BAD_SHAPE; }
        (*out)[i].resize(want);
        for (size_t k = 0; k < want; ++k) (*out)[i][k] = (float)v.arr[k].num;
    }
    return B2_OK;
}

void put_per_layer(std::string &out, const char *name, const std::vector<std::vector<float> > &v, int digits) {
    out += ",\n\"";
    out += name;
    out += "\":[";
    for (size_t i = 0; i < v.size(); ++i) {
        if (i) out += ",\n";
        put_array(out, v[i].data(), v[i].size(), digits);
    }
    out += ']';
}

double checked_number(const json::Value &doc, const char *name, bool *ok) {
    const json::Value *v = doc.find(name);
    if (!v || (v->kind != json::Value::Number && v->kind != json::Value::Bool)) {
        set_error("Missing value '%s'", name);
        *ok = false;
        return 0;
    }
    return v->kind == json::Value::Bool ? (v->b ? 1.0 : 0.0) : v->num;
}

}  // namespace

extern "C" {

int b2_net_export_json(b2_net *net, char *buf, size_t capacity, size_t *needed, int digits) {
    if (!net) { set_error("b2_net_export_json: null handle"); return B2_ERR_BAD_ARG; }
    if (digits <= 0) digits = 9;
    std::string out = "{\n";
    B2_TRY(export_network(*b2_net_impl(net), out, digits));
    out += "\n}\n";
    if (needed) *needed = out.size() + 1;
    if (buf) {
        if (capacity < out.size() + 1) { set_error("b2_net_export_json: buffer of %zu bytes, %zu needed", capacity, out.size() + 1); return B2_ERR_BAD_SHAPE; }
        memcpy(buf, out.c_str(), out.size() + 1);
    }
    return B2_OK;
}

int b2_net_save_network(b2_net *net, const char *filename, int digits) {
    if (!net || !filename) { set_error("b2_net_save_network: null pointer"); return B2_ERR_BAD_ARG; }
    if (digits <= 0) digits = 9;
    std::string out = "{\n";
    B2_TRY(export_network(*b2_net_impl(net), out, digits));
    out += "\n}\n";
    return write_file(filename, out);
}

// NeuralNetwork::printWeightMatrix (NeuralNetwork.cpp:3792-3880): all numbers as native floats.  Header: the number of
// layers with weights, then per layer {weights, size, preceding size, input weights per block, internal weights per
// block [, type code when with_type_codes]}; then every layer's weight vector in layer order.
int b2_net_save_weights_binary(b2_net *net, const char *filename, int with_type_codes) {
    if (!net || !filename) { set_error("b2_net_save_weights_binary: null pointer"); return B2_ERR_BAD_ARG; }
    NeuralNetwork &nn = *b2_net_impl(net);
    std::vector<float> head, body, w;
    int n = 0;
    for (size_t i = 0; i < nn.layers.size(); ++i) {
        Layer *l = nn.layers[i].get();
        TrainableLayer *t = dynamic_cast<TrainableLayer *>(l);
        if (!t) continue;
        const std::string &ty = l->type();
        const bool lstm = ty == "lstm" || ty == "blstm";
        // the TrainableLayer constructor arguments of the layer classes (FeedForwardLayer.cu: 1, 0; LstmLayer.cu: 4, (bidirectional ? 2 : 4) * size + 3)
        const int inPerBlock = lstm ? 4 : 1;
        const int internalPerBlock = lstm ? (ty == "blstm" ? 2 : 4) * l->size() + 3 : 0;
        ++n;
        head.push_back((float)t->numWeights());
        head.push_back((float)l->size());
        head.push_back((float)l->precedingLayer()->size());
        head.push_back((float)inPerBlock);
        head.push_back((float)internalPerBlock);
        if (with_type_codes) {
            const char *names[6] = {"feedforward_tanh", "feedforward_logistic", "feedforward_identity", "feedforward_relu", "lstm", "blstm"};
            int code = -1;
            for (int c = 0; c < 6; ++c)
                if (ty == names[c]) code = c;
            if (code < 0) { set_error("b2_net_save_weights_binary: no type code for layer type '%s'", ty.c_str()); return B2_ERR_BAD_ARG; }
            head.push_back((float)code);
        }
        if (t->numWeights()) {
            B2_TRY(fetch_weights(nn, t, w));
            body.insert(body.end(), w.begin(), w.end());
        }
    }
    FILE *f = fopen(filename, "wb");
    if (!f) { set_error("Cannot open file '%s'", filename); return B2_ERR_BAD_ARG; }
    const float count = (float)n;
    size_t done = fwrite(&count, sizeof(float), 1, f);
    done += fwrite(head.data(), sizeof(float), head.size(), f);
    done += fwrite(body.data(), sizeof(float), body.size(), f);
    const int rc = fclose(f);
    if (done != 1 + head.size() + body.size() || rc != 0) { set_error("Cannot write file '%s'", filename); return B2_ERR_BAD_ARG; }
    return B2_OK;
}

int b2_net_get_weight_deltas(b2_net *net, int layer, float *host) {
    NeuralNetwork &nn = *b2_net_impl(net);
    TrainableLayer *t = (net && layer >= 0 && layer < (int)nn.layers.size()) ? dynamic_cast<TrainableLayer *>(nn.layers[layer].get()) : nullptr;
    if (!t || !host) { set_error("b2_net_get_weight_deltas: layer %d has no weights", layer); return B2_ERR_BAD_ARG; }
    B2_CUDA(cudaMemcpyAsync(host, t->weightDeltas(), t->numWeights() * sizeof(float), cudaMemcpyDeviceToHost, nn.stream));
    B2_CUDA(cudaStreamSynchronize(nn.stream));
    return B2_OK;
}

int b2_net_set_weight_deltas(b2_net *net, int layer, const float *host) {
    NeuralNetwork &nn = *b2_net_impl(net);
    TrainableLayer *t = (net && layer >= 0 && layer < (int)nn.layers.size()) ? dynamic_cast<TrainableLayer *>(nn.layers[layer].get()) : nullptr;
    if (!t || !host) { set_error("b2_net_set_weight_deltas: layer %d has no weights", layer); return B2_ERR_BAD_ARG; }
    B2_CUDA(cudaMemcpyAsync(t->weightDeltas(), host, t->numWeights() * sizeof(float), cudaMemcpyHostToDevice, nn.stream));
    B2_CUDA(cudaStreamSynchronize(nn.stream));
    return B2_OK;
}

int b2_optimizer_create(b2_optimizer **out, b2_net *net, b2_data *training_set, b2_data *validation_set, b2_data *test_set,
                        const b2_optimizer_options *options) {
    if (!out || !net || !training_set || !options) { set_error("b2_optimizer_create: null pointer"); return B2_ERR_BAD_ARG; }
    b2_optimizer *o = new b2_optimizer;
    o->net = net;
    o->trainingSet = training_set;
    o->validationSet = validation_set;
    o->testSet = test_set;
    o->opt = *options;
    o->learningRate = options->learning_rate;
    if (o->opt.validate_every < 1) o->opt.validate_every = 1;
    if (o->opt.test_every < 1) o->opt.test_every = 1;
    o->bestWeights.resize(b2_net_impl(net)->layers.size());
    int rc = o->storeWeights();
    if (rc != B2_OK) { delete o; return rc; }
    *out = o;
    return B2_OK;
}

void b2_optimizer_destroy(b2_optimizer *o) { delete o; }

// Optimizer::train (Optimizer.cu:565-689), steepest descent branch
int b2_optimizer_train(b2_optimizer *o, int *finished) {
    if (!o) { set_error("b2_optimizer_train: null handle"); return B2_ERR_BAD_ARG; }
    if (!o->finished) {
        ++o->curEpoch;
        double err = 0.0;
        long long frames = 0;
        int nSeq = 0;
        long long nSteps = 0;
        if (o->opt.batch_learning) B2_TRY(b2_net_train_epoch_batch(o->net, o->trainingSet, o->learningRate, o->opt.momentum, &err, &frames));
        else B2_TRY(b2_net_train_epoch(o->net, o->trainingSet, o->learningRate, o->opt.momentum, &err, &frames));
        o->curTrainingError = (float)err;
        B2_TRY(b2_data_info(o->trainingSet, &nSeq, &nSteps, nullptr, nullptr, nullptr, nullptr));
        o->curTrainingErrorPerFrame = o->curTrainingError * ((float)nSeq / (float)nSteps);

        if (o->validationSet && o->curEpoch % o->opt.validate_every == 0) {
            B2_TRY(b2_net_train_epoch(o->net, o->validationSet, -1.0f, 0.0f, &err, &frames));
            o->curValidationError = (float)err;
            B2_TRY(b2_data_info(o->validationSet, &nSeq, &nSteps, nullptr, nullptr, nullptr, nullptr));
            o->curValidationErrorPerFrame = o->curValidationError * ((float)nSeq / (float)nSteps);
            if (o->curValidationError < o->lowestValidationError) {
                o->lowestValidationError = o->curValidationError;
                o->epochsSinceLowestError = 0;
                B2_TRY(o->storeWeights());
            } else {
                o->epochsSinceLowestError += o->opt.validate_every;
            }
        } else if (!o->validationSet) {
            o->epochsSinceLowestError = 0;
            B2_TRY(o->storeWeights());
        }
        if (o->testSet && o->curEpoch % o->opt.test_every == 0) {
            B2_TRY(b2_net_train_epoch(o->net, o->testSet, -1.0f, 0.0f, &err, &frames));
            o->curTestError = (float)err;
            B2_TRY(b2_data_info(o->testSet, &nSeq, &nSteps, nullptr, nullptr, nullptr, nullptr));
            o->curTestErrorPerFrame = o->curTestError * ((float)nSeq / (float)nSteps);
        }
        if (o->opt.max_epochs >= 0 && o->curEpoch >= o->opt.max_epochs) {
            B2_TRY(o->restoreWeights());
            o->finished = true;
        } else if (o->epochsSinceLowestError >= o->opt.max_epochs_no_best) {
            NeuralNetwork &nn = *b2_net_impl(o->net);
            if (nn.optOption == 3) {
                // OPTIMIZATION_STOCHASTIC_ADAGRAD: no best for N epochs, switch to AdaGrad on the statistics gathered so far;
                // the count starts from 1 so that the restored weights are not stored again (Optimizer.cu:654-662)
                nn.optOption = 1;
                o->epochsSinceLowestError = 1;
                o->lowestValidationError = std::numeric_limits<float>::max();
                o->learningRate = o->opt.second_learning_rate;
                B2_TRY(o->restoreWeights());
            } else if (nn.optOption == 4) {
                // OPTIMIZATION_SGD_DECAY (Optimizer.cu:663-668, SteepestDescentOptimizer::adjustLR)
                o->epochsSinceLowestError = 1;
                o->learningRate *= o->opt.lr_decay_rate;
                B2_TRY(o->restoreWeights());
            } else {
                B2_TRY(o->restoreWeights());
                o->finished = true;
            }
        }
    }
    if (finished) *finished = o->finished ? 1 : 0;
    return B2_OK;
}

int b2_optimizer_get_state(const b2_optimizer *o, b2_optimizer_state *s) {
    if (!o || !s) { set_error("b2_optimizer_get_state: null pointer"); return B2_ERR_BAD_ARG; }
    s->finished = o->finished ? 1 : 0;
    s->cur_epoch = o->curEpoch;
    s->epochs_since_lowest_error = o->epochsSinceLowestError;
    s->lowest_validation_error = o->lowestValidationError;
    s->cur_training_error = o->curTrainingError;
    s->cur_validation_error = o->curValidationError;
    s->cur_test_error = o->curTestError;
    s->cur_training_error_per_frame = o->curTrainingErrorPerFrame;
    s->cur_validation_error_per_frame = o->curValidationErrorPerFrame;
    s->cur_test_error_per_frame = o->curTestErrorPerFrame;
    s->learning_rate = o->learningRate;
    s->optimizer_option = b2_net_impl(o->net)->optOption;
    return B2_OK;
}

// Optimizer::saveState: configuration, info rows, network, optimizer state, momentum deltas
int b2_optimizer_save_state(b2_optimizer *o, const char *filename, const char *configuration, const char *info_rows, int digits) {
    if (!o || !filename) { set_error("b2_optimizer_save_state: null pointer"); return B2_ERR_BAD_ARG; }
    if (digits <= 0) digits = 9;
    NeuralNetwork &nn = *b2_net_impl(o->net);
    std::string out = "{\n\"configuration\":";
    put_string(out, configuration ? configuration : "");
    out += ",\n\"info_rows\":";
    std::string rows = info_rows ? info_rows : "";
    for (size_t p = 0; (p = rows.find('\n', p)) != std::string::npos;) rows.replace(p, 1, ";;;");
    put_string(out, rows);
    out += ",\n";
    B2_TRY(export_network(nn, out, digits));
    out += ",\n\"optimizer_finished\":";
    out += o->finished ? "true" : "false";
    out += ",\n\"optimizer_cur_epoch\":" + std::to_string(o->curEpoch);
    out += ",\n\"optimizer_epochs_since_lowest_error\":" + std::to_string(o->epochsSinceLowestError);
    const struct { const char *name; float v; } nums[] = {
        {"optimizer_lowest_validation_error", o->lowestValidationError}, {"optimizer_cur_training_error", o->curTrainingError},
        {"optimizer_cur_validation_error", o->curValidationError},       {"optimizer_cur_test_error", o->curTestError},
        {"optimizer_cur_training_class_error", 0.0f},                    {"optimizer_cur_validation_class_error", 0.0f},
        {"optimizer_cur_test_class_error", 0.0f}};
    for (const auto &n : nums) {
        out += ",\n\"";
        out += n.name;
        out += "\":";
        put_number(out, n.v, digits);
    }
    out += ",\n\"optimizer_status\":" + std::to_string(nn.optOption);   // MacroDefine.hpp OPTIMIZATION_*
    put_per_layer(out, "optimizer_best_weights", o->bestWeights, digits);
    if (nn.optOption == 1 || nn.optOption == 3 || nn.optOption == 5) {
        // AdaGrad / Adam statistics (Optimizer.cu:721-725); Adam's running beta products are not part of the
        // reference's file either and restart at 1 after a continue
        std::vector<std::vector<float> > stats(nn.layers.size());
        for (size_t i = 1; i < nn.layers.size(); ++i)
            if (TrainableLayer *t = dynamic_cast<TrainableLayer *>(nn.layers[i].get())) {
                stats[i].resize(t->statsFloats());
                if (!stats[i].empty()) B2_TRY(b2_net_get_optimizer_stats(o->net, (int)i, stats[i].data(), stats[i].size(), nullptr));
            }
        put_per_layer(out, "optimizer_status_vector", stats, digits);
    }
    if (o->opt.momentum > 0.0f) {
        std::vector<std::vector<float> > deltas(nn.layers.size());
        for (size_t i = 1; i < nn.layers.size(); ++i)
            if (TrainableLayer *t = dynamic_cast<TrainableLayer *>(nn.layers[i].get())) {
                deltas[i].resize(t->numWeights());
                B2_TRY(b2_net_get_weight_deltas(o->net, (int)i, deltas[i].data()));
            }
        put_per_layer(out, "steepest_descent_optimizer_weight_deltas", deltas, digits);
    }
    out += "\n}\n";
    return write_file(filename, out);
}

// --continue: NeuralNetwork weights from the "weights" section, then Optimizer::restoreState
int b2_optimizer_restore_state(b2_optimizer *o, const char *filename, char *info_rows, size_t info_capacity) {
    if (!o || !filename) { set_error("b2_optimizer_restore_state: null pointer"); return B2_ERR_BAD_ARG; }
    NeuralNetwork &nn = *b2_net_impl(o->net);
    std::string text;
    B2_TRY(read_file(filename, text));
    json::Value doc;
    try {
        doc = json::Parser(text.c_str()).parse();
    } catch (const std::exception &e) {
        set_error("b2_optimizer_restore_state: %s", e.what());
        return B2_ERR_BAD_ARG;
    }
    const json::Value *rows = doc.find("info_rows");
    if (!rows) { set_error("Missing value 'info_rows'"); return B2_ERR_BAD_ARG; }
    if (info_rows && info_capacity) {
        std::string r = rows->str;
        for (size_t p = 0; (p = r.find(";;;", p)) != std::string::npos;) r.replace(p, 3, "\n");
        strncpy(info_rows, r.c_str(), info_capacity - 1);
        info_rows[info_capacity - 1] = '\0';
    }
    // the network's weights
    const json::Value *wsec = doc.find("weights");
    if (!wsec) { set_error("Missing section 'weights'"); return B2_ERR_BAD_ARG; }
    for (size_t i = 1; i < nn.layers.size(); ++i) {
        TrainableLayer *t = dynamic_cast<TrainableLayer *>(nn.layers[i].get());
        if (!t) continue;
        const json::Value *lw = wsec->find(t->name());
        if (!lw) { set_error("Missing weights section for layer '%s'", t->name().c_str()); return B2_ERR_BAD_ARG; }
        std::vector<float> w(t->numWeights());
        size_t k = 0;
        const char *secs[3] = {"input", "bias", "internal"};
        for (int s = 0; s < 3; ++s) {
            const json::Value *a = lw->find(secs[s]);
            if (!a) continue;
            for (size_t q = 0; q < a->arr.size() && k < w.size(); ++q) w[k++] = (float)a->arr[q].num;
        }
        if (k != w.size()) { set_error("Invalid number of weights for layer '%s'", t->name().c_str()); return B2_ERR_BAD_SHAPE; }
        B2_TRY(b2_net_set_weights(o->net, (int)i, w.data()));
    }
    bool ok = true;
    const bool fin = checked_number(doc, "optimizer_finished", &ok) != 0.0;
    const int epoch = (int)checked_number(doc, "optimizer_cur_epoch", &ok);
    const int since = (int)checked_number(doc, "optimizer_epochs_since_lowest_error", &ok);
    const float lowest = (float)checked_number(doc, "optimizer_lowest_validation_error", &ok);
    const float tr = (float)checked_number(doc, "optimizer_cur_training_error", &ok);
    const float va = (float)checked_number(doc, "optimizer_cur_validation_error", &ok);
    const float te = (float)checked_number(doc, "optimizer_cur_test_error", &ok);
    if (!ok) return B2_ERR_BAD_ARG;
    const int option = (int)checked_number(doc, "optimizer_status", &ok);
    if (!ok) return B2_ERR_BAD_ARG;
    std::vector<std::vector<float> > best, deltas;
    B2_TRY(per_layer_vectors(doc, "optimizer_best_weights", nn, &best));
    B2_TRY(nn.setOptimizerOption(option));
    if (option == 1 || option == 3 || option == 5) {
        const json::Value *a = doc.find("optimizer_status_vector");
        if (!a || a->kind != json::Value::Array || a->arr.size() != nn.layers.size()) {
            set_error("Array 'optimizer_status_vector' is missing or has the wrong type");
            return B2_ERR_BAD_ARG;
        }
        for (size_t i = 1; i < nn.layers.size(); ++i) {
            TrainableLayer *t = dynamic_cast<TrainableLayer *>(nn.layers[i].get());
            if (!t) continue;
            const json::Value &v = a->arr[i];
            if (v.kind != json::Value::Array || v.arr.size() != t->statsFloats()) {
                set_error("Subarray in 'optimizer_status_vector' has a wrong size");
                return B2_ERR_BAD_SHAPE;
            }
            std::vector<float> h(v.arr.size());
            for (size_t k = 0; k < h.size(); ++k) h[k] = (float)v.arr[k].num;
            B2_CUDA(cudaMemcpyAsync(t->weightStats(), h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice, nn.stream));
            B2_CUDA(cudaStreamSynchronize(nn.stream));
        }
    }
    if (o->opt.momentum > 0.0f) {
        B2_TRY(per_layer_vectors(doc, "steepest_descent_optimizer_weight_deltas", nn, &deltas));
        for (size_t i = 1; i < nn.layers.size(); ++i)
            if (!deltas[i].empty()) B2_TRY(b2_net_set_weight_deltas(o->net, (int)i, deltas[i].data()));
    }
    o->finished = fin;
    o->curEpoch = epoch;
    o->epochsSinceLowestError = since;
    o->lowestValidationError = lowest;
    o->curTrainingError = tr;
    o->curValidationError = va;
    o->curTestError = te;
    o->bestWeights = best;
    return B2_OK;
}

}  // extern "C"
