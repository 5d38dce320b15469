// layers::LstmLayerB200<TDevice>: the reference-side binding of libb2lstm.
//
// A drop-in for layers::LstmLayer<Gpu> of the CURRENNT toolkit (layers/LstmLayer.hpp:168-308 of the reference): it
// derives from the toolkit's own TrainableLayer, keeps the toolkit's buffers (weights, weightUpdates, outputs,
// outputErrors, patTypes stay Thrust device vectors owned by the base classes) and forwards the three virtuals of
// the training path to the C ABI of include/b2lstm.h.  The plug-in point is LayerFactory<TDevice>::createLayer
// (LayerFactory.cu:127-132 of the reference):
//
//     else if (layerType == "lstm")  return new LstmLayerB200<TDevice>(layerChild, weightsSection, *precedingLayer, maxSeqLength, layerID, false);
//     else if (layerType == "blstm") return new LstmLayerB200<TDevice>(layerChild, weightsSection, *precedingLayer, maxSeqLength, layerID, true);
//
// Copy this file into currennt_lib/src/layers/ (it includes the toolkit's headers by their paths below src/), add
// include/ of this repository to the include path and link libb2lstm.so.  Instantiate it for Gpu only: the library
// works on device pointers.
#pragma once

#include <stdexcept>
#include <string>

#include "helpers/JsonClasses.hpp"
#include "helpers/getRawPointer.cuh"
#include "layers/TrainableLayer.hpp"

#include "b2lstm.h"

namespace layers {

template <typename TDevice>
class LstmLayerB200 : public TrainableLayer<TDevice> {
    typedef typename TDevice::real_vector real_vector;

public:
    // same constructor arguments and the same weight counts per block as the reference's LstmLayer
    // (layers/LstmLayer.cu:1079-1088): 4 input weights per block, (2 or 4) * size + 3 internal ones
    LstmLayerB200(const helpers::JsonValue &layerChild, const helpers::JsonValue &weightsSection, Layer<TDevice> &precedingLayer,
                  int maxSeqLength, int layerID, bool bidirectional)
        : TrainableLayer<TDevice>(layerChild, weightsSection, 4,
                                  (bidirectional ? 2 : 4) * helpers::safeJsonGetInt(layerChild, "size") + 3, precedingLayer,
                                  maxSeqLength, layerID),
          m_impl(NULL), m_bidirectional(bidirectional) {
        if (bidirectional && this->size() % 2 != 0) throw std::runtime_error("Cannot create a bidirectional layer with an odd layer size");
        b2_lstm_desc d;
        d.parallel_sequences = this->parallelSequences();
        d.max_seq_length = maxSeqLength;
        d.prev_size = precedingLayer.size();
        d.size = this->size();
        d.bidirectional = bidirectional ? 1 : 0;
        d.bias = this->bias();
        check(b2_lstm_create(&d, &m_impl));
        if (b2_lstm_num_weights(&d) != this->weights().size()) throw std::runtime_error("LstmLayerB200: weight count differs from the toolkit's");
    }
    virtual ~LstmLayerB200() { b2_lstm_destroy(m_impl); }

    virtual const std::string &type() const {
        static const std::string su("lstm"), sb("blstm");
        return m_bidirectional ? sb : su;
    }

    // Layer::loadSequences copies the pattern types to the device and sets the current lengths (layers/Layer.cu:254-305)
    virtual void loadSequences(const data_sets::DataSetFraction &fraction, const int nnState) {
        TrainableLayer<TDevice>::loadSequences(fraction, nnState);
        check(b2_lstm_load_sequences(m_impl, this->curMaxSeqLength(), this->curMinSeqLength(),
                                     helpers::getRawPointer(this->patTypes())));
    }
    // stream 0: the toolkit's Thrust and cuBLAS calls run on the legacy default stream, so the order is kept
    virtual void computeForwardPass(const int nnState) {
        (void)nnState;
        check(b2_lstm_forward(m_impl, helpers::getRawPointer(this->weights()), helpers::getRawPointer(this->precedingLayer().outputs()),
                              helpers::getRawPointer(this->_outputs()), 0));
    }
    virtual void computeBackwardPass(const int nnState) {
        (void)nnState;
        check(b2_lstm_backward(m_impl, helpers::getRawPointer(this->weights()), helpers::getRawPointer(this->precedingLayer().outputs()),
                               helpers::getRawPointer(this->outputs()), helpers::getRawPointer(this->outputErrors()),
                               helpers::getRawPointer(this->precedingLayer().outputErrors()),
                               helpers::getRawPointer(this->_weightUpdates()), 0));
        check(b2_lstm_synchronize(m_impl, 0));   // a given-up wait of a persistent kernel surfaces here, once per fraction
    }
    // the step-wise overloads serve auto-regressive generation only (layers/LstmLayer.cu:1951-2065): not on the training path
    virtual void computeForwardPass(const int timeStep, const int nnState) {
        (void)timeStep; (void)nnState;
        throw std::runtime_error("LstmLayerB200: step-wise forward pass is not supported");
    }
    virtual void computeBackwardPass(const int timeStep, const int nnState) {
        (void)timeStep; (void)nnState;
        throw std::runtime_error("LstmLayerB200: step-wise backward pass is not supported");
    }

private:
    static void check(int rc) {
        if (rc != B2_OK) throw std::runtime_error(b2_last_error_string());
    }
    b2_lstm *m_impl;
    bool m_bidirectional;
};

}  // namespace layers
