// C ABI of the data set (b2_data_*) and the epoch loop that feeds a net from it.
#include <string.h>

#include <string>
#include <vector>

#include "../../include/b2lstm.h"
#include "data_set.hpp"

namespace b2 {
void set_error(const char *fmt, ...);   // defined in network.cu
}
#define B2_TRY(call)                    \
    do {                                \
        int rc__ = (call);              \
        if (rc__ != B2_OK) return rc__; \
    } while (0)

struct b2_data {
    b2::DataSet ds;
    const b2::FractionView *last = nullptr;
};

// The reference takes parallel_sequences and the longest sequence of both the data set and the network from
// ONE Configuration, so they cannot disagree there; two handles can.  A fraction is laid out [T][P_data][size]:
// a net with another P would read it mis-strided (and, with a larger P, past the end of the pinned block).
static int check_data_matches_net(const char *who, b2_net *net, b2_data *data) {
    if (data->ds.inputPatternSize() != b2_net_layer_size(net, 0) ||
        data->ds.outputPatternSize() != b2_net_layer_size(net, b2_net_num_layers(net) - 1)) {
        b2::set_error("%s: the data set has %d inputs / %d targets, the network %d / %d", who,
                      data->ds.inputPatternSize(), data->ds.outputPatternSize(), b2_net_layer_size(net, 0),
                      b2_net_layer_size(net, b2_net_num_layers(net) - 1));
        return B2_ERR_BAD_SHAPE;
    }
    if (data->ds.parallelSequences() != b2_net_parallel_sequences(net) || data->ds.maxSeqLength() > b2_net_max_seq_length(net)) {
        b2::set_error("%s: the data set was opened with parallel_sequences %d and holds sequences of up to %d frames, "
                      "the network was created for parallel_sequences %d and %d frames", who, data->ds.parallelSequences(),
                      data->ds.maxSeqLength(), b2_net_parallel_sequences(net), b2_net_max_seq_length(net));
        return B2_ERR_BAD_SHAPE;
    }
    return B2_OK;
}

extern "C" {

int b2_data_open(b2_data **out, const char *const *nc_paths, int n_files, const b2_data_options *opt) {
    if (!out || !nc_paths || n_files < 1 || !opt) {
        b2::set_error("b2_data_open: null pointer or no files");
        return B2_ERR_BAD_ARG;
    }
    *out = nullptr;
    std::vector<std::string> files;
    for (int i = 0; i < n_files; ++i) {
        if (!nc_paths[i]) { b2::set_error("b2_data_open: null path"); return B2_ERR_BAD_ARG; }
        files.push_back(nc_paths[i]);
    }
    b2::DataSetOptions o;
    o.parallelSequences = opt->parallel_sequences;
    o.fraction = opt->fraction;
    o.truncSeqLength = opt->trunc_seq_length;
    o.fractionShuffling = opt->fraction_shuffling != 0;
    o.sequenceShuffling = opt->sequence_shuffling != 0;
    o.randomSeed = opt->random_seed;
    o.trainingMode = opt->training_mode != 0;
    o.loaderThreads = opt->loader_threads;
    o.shardRank = opt->shard_rank;
    o.shardCount = opt->shard_count < 1 ? 1 : opt->shard_count;
    b2_data *d = new b2_data;
    std::string err = d->ds.open(files, o);
    if (!err.empty()) {
        delete d;
        b2::set_error("%s", err.c_str());
        return B2_ERR_BAD_ARG;
    }
    *out = d;
    return B2_OK;
}

void b2_data_close(b2_data *data) { delete data; }

int b2_data_info(const b2_data *d, int *total_sequences, long long *total_timesteps, int *min_seq_length, int *max_seq_length,
                 int *input_size, int *output_size) {
    if (!d) { b2::set_error("b2_data_info: null handle"); return B2_ERR_BAD_ARG; }
    if (total_sequences) *total_sequences = d->ds.totalSequences();
    if (total_timesteps) *total_timesteps = (long long)d->ds.totalTimesteps();
    if (min_seq_length) *min_seq_length = d->ds.minSeqLength();
    if (max_seq_length) *max_seq_length = d->ds.maxSeqLength();
    if (input_size) *input_size = d->ds.inputPatternSize();
    if (output_size) *output_size = d->ds.outputPatternSize();
    return B2_OK;
}

int b2_data_output_mean_stdev(const b2_data *d, float *means, float *stdevs, int *present) {
    if (!d) { b2::set_error("b2_data_output_mean_stdev: null handle"); return B2_ERR_BAD_ARG; }
    const size_t n = (size_t)d->ds.outputPatternSize();
    if (means) memcpy(means, d->ds.outputMeans().data(), n * sizeof(float));
    if (stdevs) memcpy(stdevs, d->ds.outputStdevs().data(), n * sizeof(float));
    if (present) *present = d->ds.outputMVFlag() ? 1 : 0;
    return B2_OK;
}

int b2_data_next_fraction(b2_data *d, b2_fraction *frac) {
    if (!d || !frac) { b2::set_error("b2_data_next_fraction: null pointer"); return B2_ERR_BAD_ARG; }
    const b2::FractionView *f = d->ds.getNextFraction();
    d->last = f;
    if (!f) {
        memset(frac, 0, sizeof(*frac));
        return B2_DATA_EPOCH_END;
    }
    frac->max_seq_length = f->maxSeqLength;
    frac->min_seq_length = f->minSeqLength;
    frac->num_sequences = f->numSequences;
    frac->total_frames = f->fracTotalLength;
    frac->seq_lengths = f->seqLengths.data();
    frac->inputs = f->inputs;
    frac->targets = f->outputs;
    frac->pat_types = f->patTypes;
    return B2_OK;
}

int b2_data_fraction_seq_info(const b2_data *d, int i, char *tag, int tag_capacity, int *original_seq_idx) {
    if (!d || !d->last) { b2::set_error("b2_data_fraction_seq_info: no current fraction"); return B2_ERR_STATE; }
    if (i < 0 || i >= d->last->numSequences) { b2::set_error("b2_data_fraction_seq_info: sequence %d out of range", i); return B2_ERR_BAD_ARG; }
    if (tag && tag_capacity > 0) {
        strncpy(tag, d->last->seqTags[i].c_str(), (size_t)tag_capacity - 1);
        tag[tag_capacity - 1] = '\0';
    }
    if (original_seq_idx) *original_seq_idx = d->last->originalSeqIdx[i];
    return B2_OK;
}

void b2_data_reseed(unsigned seed) { b2::reseed_shuffle_generator(seed); }

int b2_net_train_epoch(b2_net *net, b2_data *data, float learning_rate, float momentum, double *error, long long *frames) {
    if (!net || !data) { b2::set_error("b2_net_train_epoch: null handle"); return B2_ERR_BAD_ARG; }
    B2_TRY(check_data_matches_net("b2_net_train_epoch", net, data));
    const double nSeqTotal = (double)data->ds.totalSequences();
    double errSum = 0.0;
    long long nFrames = 0;
    b2_fraction cur, nxt;
    int rc = b2_data_next_fraction(data, &cur);
    if (rc < 0) return rc;
    const bool train = learning_rate >= 0.0f;
    // a sharded data set may hand this rank an empty fraction (fewer sequences than shards at the end of
    // an epoch): the rank then only takes part in the gradient sum
    if (rc == B2_OK && train && cur.num_sequences > 0)
        B2_TRY(b2_net_prefetch_fraction(net, cur.max_seq_length, cur.num_sequences, cur.seq_lengths, cur.inputs, cur.targets));
    while (rc == B2_OK) {
        double e = 0.0;
        int rcNext;
        if (train) {
            // enqueue this fraction's step, then start the next fraction's copy while it runs
            if (cur.num_sequences > 0) B2_TRY(b2_net_train_step_prefetched(net, learning_rate, momentum, nullptr));
            else B2_TRY(b2_net_train_step_empty(net, learning_rate, momentum));
            rcNext = b2_data_next_fraction(data, &nxt);
            if (rcNext < 0) return rcNext;
            if (rcNext == B2_OK && nxt.num_sequences > 0)
                B2_TRY(b2_net_prefetch_fraction(net, nxt.max_seq_length, nxt.num_sequences, nxt.seq_lengths, nxt.inputs, nxt.targets));
            if (cur.num_sequences > 0) B2_TRY(b2_net_read_error(net, &e));
        } else {
            if (cur.num_sequences > 0) {
                B2_TRY(b2_net_load_fraction(net, cur.max_seq_length, cur.num_sequences, cur.seq_lengths, cur.inputs, cur.targets));
                B2_TRY(b2_net_forward(net, &e));
            }
            rcNext = b2_data_next_fraction(data, &nxt);
            if (rcNext < 0) return rcNext;
        }
        if (e == e) errSum += e / nSeqTotal;   // a NaN fraction is left out of the sum (Optimizer.cu:127-131)
        nFrames += cur.total_frames;
        cur = nxt;
        rc = rcNext;
    }
    // one read of every layer's status word per epoch: a sweep that gave up a bounded wait returned zeros, and
    // the caller (b2_optimizer_train) must not store weights trained on them
    B2_TRY(b2_net_synchronize(net));
    // data-parallel: the epoch's error and frame count are those of all shards
    if (b2_dp_world_size(net) > 1) {
        double fr = (double)nFrames;
        B2_TRY(b2_dp_allreduce_scalar(net, &errSum));
        B2_TRY(b2_dp_allreduce_scalar(net, &fr));
        nFrames = (long long)(fr + 0.5);
    }
    if (error) *error = errSum;
    if (frames) *frames = nFrames;
    return B2_OK;
}

// Optimizer::_processDataSet without hybrid_online_batch: forward, error, backward and accumulation per
// fraction, one update at the end
int b2_net_train_epoch_batch(b2_net *net, b2_data *data, float learning_rate, float momentum, double *error, long long *frames) {
    if (!net || !data) { b2::set_error("b2_net_train_epoch_batch: null handle"); return B2_ERR_BAD_ARG; }
    B2_TRY(check_data_matches_net("b2_net_train_epoch_batch", net, data));
    const double nSeqTotal = (double)data->ds.totalSequences();
    double errSum = 0.0;
    long long nFrames = 0;
    bool first = true;
    b2_fraction cur;
    int rc;
    while ((rc = b2_data_next_fraction(data, &cur)) == B2_OK) {
        double e = 0.0;
        if (cur.num_sequences == 0) {
            // an empty shard: this rank still takes part in the gradient sums of the fraction
            if (b2_dp_world_size(net) <= 1) continue;
            B2_TRY(b2_net_backward_empty(net));
        } else {
            B2_TRY(b2_net_load_fraction(net, cur.max_seq_length, cur.num_sequences, cur.seq_lengths, cur.inputs, cur.targets));
            B2_TRY(b2_net_forward(net, &e));
            B2_TRY(b2_net_backward(net));
        }
        B2_TRY(b2_net_accumulate_weight_updates(net, first ? 1 : 0));
        B2_TRY(b2_net_synchronize(net));        // the fraction's host buffers are recycled by the data set
        first = false;
        if (e == e) errSum += e / nSeqTotal;
        nFrames += cur.total_frames;
    }
    if (rc < 0) return rc;
    if (!first) B2_TRY(b2_net_update_weights_batch(net, learning_rate, momentum));
    if (b2_dp_world_size(net) > 1) {
        double fr = (double)nFrames;
        B2_TRY(b2_dp_allreduce_scalar(net, &errSum));
        B2_TRY(b2_dp_allreduce_scalar(net, &fr));
        nFrames = (long long)(fr + 0.5);
    }
    if (error) *error = errSum;
    if (frames) *frames = nFrames;
    return B2_OK;
}

}  // extern "C"
