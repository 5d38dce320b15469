/*
 * b2lstm -- B200 (sm_100a) implementation of the CURRENNT peephole LSTM / BLSTM training path.
 *
 * C ABI.  Plain pointers and sizes only; every function returns an int status (0 = ok, negative
 * = error, text via b2_last_error_string()).  Nothing here throws, traps or falls back to the
 * CPU: when the CUDA device or a kernel is unavailable the call fails with B2_ERR_CUDA.
 *
 * Conventions kept from the reference toolkit (paths are inside CURRENNT_codes/currennt_lib/src/):
 *   - activations are time-major with the parallel sequences interleaved: element d of frame
 *     (t, p) sits at [(t*P + p)*dim + d]                         (data_sets/DataSet.cpp:853-861)
 *   - matrices are column-major views over such vectors          (helpers/Matrix.cu:202-211)
 *   - pattern types: char per frame, 0 NONE (padding), 1 FIRST, 2 NORMAL, 3 LAST (Types.hpp:35-38)
 *   - the (b)lstm weight vector is [input | bias | recurrent | peephole]
 *                                                                (layers/LstmLayer.hpp:36-55)
 *   - a blstm's "size" is the total over both directions         (layers/LstmLayer.cu:1091-1098)
 *   - gradients are sums over frames, never averaged             (optimizers/SteepestDescentOptimizer.cu:421-438)
 *
 * Three levels, lowest first:
 *   b2_matrix_*   the GEMM wrapper                      <-> helpers::Matrix / helpers::cublas
 *   b2_lstm_*     one (b)lstm layer on caller's buffers <-> layers::LstmLayer<Gpu>
 *   b2_net_*      layer stack + minibatch step          <-> NeuralNetwork + Optimizer::_processDataSet
 *   b2_dp_*       gradient all-reduce across GPUs (no counterpart: the reference is single-GPU)
 */
#ifndef B2LSTM_H
#define B2LSTM_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* cudaStream_t without pulling the CUDA headers into the caller */
typedef void *b2_stream;

enum {
    B2_OK = 0,
    B2_ERR_BAD_SHAPE = -1,    /* sizes inconsistent with the descriptor / allocation        */
    B2_ERR_CUDA = -2,         /* a CUDA runtime call or kernel launch failed                 */
    B2_ERR_STEP_TIMEOUT = -3, /* a bounded device-side wait in a persistent kernel ran out   */
    B2_ERR_NCCL = -4,         /* NCCL missing or a collective failed                         */
    B2_ERR_BAD_ARG = -5,      /* null pointer, unknown layer type, malformed JSON ...        */
    B2_ERR_STATE = -6         /* call order violated (e.g. backward before forward)          */
};

const char *b2_last_error_string(void);
/* Library build id, e.g. "b2lstm 0.1 sm_100a". */
const char *b2_version(void);

/* ------------------------------------------------------------------------------------------
 * helpers::Matrix<Gpu>::assignProduct / addProduct          (helpers/Matrix.cu:354-377,
 * helpers/cublas.cu:52-84: cublasSgemm with alpha = 1, beta = 0 or 1).
 * C(m x n) = op(A) op(B) (+ C if accumulate), all column-major device pointers with leading
 * dimensions lda/ldb/ldc; op = transpose when the flag is non-zero.  The reference rejects
 * (transA && transB) (Matrix.cu:259-260); so does this call (B2_ERR_BAD_ARG).
 * Runs on tensor cores when the shape qualifies (operands split into scaled fp16 high and low parts,
 * three products, fp32 accumulation: the accuracy of an fp32 GEMM), otherwise as an FFMA kernel; `force_ffma` non-zero always selects the latter.
 * ------------------------------------------------------------------------------------------ */
int b2_matrix_multiply(float *C, int ldc, const float *A, int lda, int transA, const float *B, int ldb,
                       int transB, int m, int n, int k, int accumulate, int force_ffma, b2_stream stream);

/* The same product for hosts that must not have device memory allocated on their behalf (all of
 * HBM already owned by the host program's pool, or no tolerance for cudaMalloc's device-wide
 * synchronisation).  No counterpart in the reference toolkit.  Always the FFMA kernel; its split-K
 * partial sums live in a fixed 16 MiB array inside the library image (held by every GPU that loads
 * the library, until exit) instead of an allocation, so the call allocates nothing.
 * Limit: m*n <= 2^21 output elements, otherwise B2_ERR_BAD_SHAPE; negative sizes or leading
 * dimensions shorter than a column are B2_ERR_BAD_ARG.
 * The first call on a device looks up the array's device address; make it outside any stream
 * capture, and before the host program claims the rest of the GPU's memory (the driver backs the
 * array when the library's code is first used on a device).  A device reset invalidates the address
 * the library has cached.  All calls on a device share the array: calls whose kernels can overlap on the GPU
 * (different streams) race on it and must be serialised by the caller. */
int b2_matrix_multiply_noalloc(float *C, int ldc, const float *A, int lda, int transA, const float *B, int ldb,
                               int transB, int m, int n, int k, int accumulate, b2_stream stream);

/* ------------------------------------------------------------------------------------------
 * layers::LstmLayer<Gpu>                                    (layers/LstmLayer.hpp:168-308)
 * ------------------------------------------------------------------------------------------ */
typedef struct b2_lstm b2_lstm;

typedef struct {
    int parallel_sequences; /* P, Layer::parallelSequences()                                   */
    int max_seq_length;     /* frames per sequence the buffers are sized for (Layer::maxSeqLength) */
    int prev_size;          /* size of the preceding layer                                     */
    int size;               /* layer size; TOTAL over both directions for a blstm              */
    int bidirectional;      /* 0 "lstm", 1 "blstm"                   (LayerFactory.cu:127-132) */
    float bias;             /* the layer's JSON "bias" value         (TrainableLayer.cu:108-109) */
} b2_lstm_desc;

/* ls*(4*(pls+1) + 4*els + 3)                                 (layers/LstmLayer.cu:1085-1088) */
size_t b2_lstm_num_weights(const b2_lstm_desc *desc);
/* LstmLayer constructor (LstmLayer.cu:1079-1376): allocates the private state buffers on the
 * current CUDA device.  The layer keeps NO weights, outputs or errors of its own: those stay in
 * the caller's vectors and are passed to every call. */
int b2_lstm_create(const b2_lstm_desc *desc, b2_lstm **out);
void b2_lstm_destroy(b2_lstm *layer);
/* LstmLayer::loadSequences (LstmLayer.cu:1489-1533, Layer.cu:254-305): take over the current
 * fraction's shape.  pat_types_dev: device char[cur_max_len * P]; padding frames (type 0) must trail
 * their sequence, as data_sets::DataSet writes them. */
int b2_lstm_load_sequences(b2_lstm *layer, int cur_max_len, int cur_min_len, const char *pat_types_dev);
/* Non-zero makes b2_lstm_load_sequences verify that contract on the device (B2_ERR_BAD_ARG when a real frame follows a
 * padding frame) at the price of one device round trip per fraction; off by default.  The reference needs no such
 * check: it reads the pattern type of every frame (layers/LstmLayer.cu:89-101). */
int b2_lstm_set_check_padding(b2_lstm *layer, int on);
/* LstmLayer::computeForwardPass (LstmLayer.cu:1744-1949).
 * weights_dev: b2_lstm_num_weights floats; x_dev: prev_size x (T*P) = precedingLayer().outputs();
 * y_dev: size x (T*P) = outputs(), forward-direction units first, then backward-direction units.
 * Padding frames of y are written as exact zeros. */
int b2_lstm_forward(b2_lstm *layer, const float *weights_dev, const float *x_dev, float *y_dev, b2_stream stream);
/* LstmLayer::computeBackwardPass (LstmLayer.cu:2067-2382).
 * dy_dev: size x (T*P) = outputErrors() (read only); dx_dev: prev_size x (T*P) =
 * precedingLayer().outputErrors(), OVERWRITTEN (may be NULL to skip it, as for an input layer
 * nobody reads); dw_dev: weightUpdates(), OVERWRITTEN, same layout as the weights. */
int b2_lstm_backward(b2_lstm *layer, const float *weights_dev, const float *x_dev, const float *y_dev,
                     const float *dy_dev, float *dx_dev, float *dw_dev, b2_stream stream);
/* Which recurrence kernels run:
 *   0  one launch per timestep;
 *   1  persistent kernels, the library chooses the exchange between the blocks of a group (default):
 *      thread-block clusters with transaction barriers in distributed shared memory for as many work
 *      items as fit side by side, the remaining sequences through L2 on the SMs the clusters leave
 *      free; for large batches (many sequences x many units) the tensor-core recurrence of mode 3;
 *   2  persistent kernels, every group as a cluster where a group fits one (128 or 256 units per
 *      direction), through L2 otherwise;
 *   3  tensor-core recurrence (one batched tcgen05 GEMM and one gate kernel per timestep) wherever
 *      the shape allows it;
 *   4  persistent kernels, every exchange through L2;
 *   5  persistent tensor-core kernels (recurrent weights resident in shared memory as fp16 hi/lo tcgen05 operands for
 *      the whole sweep) wherever the shape allows it (512 units per direction); mode 1 picks them by itself from 16
 *      parallel sequences on;
 *   6  as 5 for the forward sweep only (the backward sweep runs on the mode-1 kernels). */
int b2_lstm_set_recurrence_mode(b2_lstm *layer, int mode);
/* Which recurrence kernels the layer's last forward (backward = 0) or backward (backward != 0) sweep really
 * ran, whatever the mode asked for: 0 one launch per timestep, 1 persistent FFMA kernels, 3 tensor-core GEMM
 * and gate kernel per timestep, 5 persistent tensor-core kernels; -1 before the first sweep.  The reference
 * has one code path (layers/LstmLayer.cu:1805-1858), so it has no such query. */
int b2_lstm_recurrence_path(const b2_lstm *layer, int backward);
/* Waits for the work enqueued on `stream` and reports what the layer's kernels recorded:
 * B2_ERR_STEP_TIMEOUT if a persistent kernel gave up a bounded wait, else B2_OK. */
int b2_lstm_synchronize(b2_lstm *layer, b2_stream stream);
/* Bytes of private device memory the layer holds. */
size_t b2_lstm_state_bytes(const b2_lstm *layer);

/* ------------------------------------------------------------------------------------------
 * NeuralNetwork + Optimizer::_processDataSet + SteepestDescentOptimizer
 * (NeuralNetwork.cpp:1056-1086,1367-1373,1734-1742,2864-2873,2982-2989;
 *  optimizers/Optimizer.cu:45-258; optimizers/SteepestDescentOptimizer.cu:74-100,421-438)
 * ------------------------------------------------------------------------------------------ */
typedef struct b2_net b2_net;

/* network_json: the reference's network file ({"layers":[{"size","name","type","bias",
 * "learningRate"?}, ...], "weights"?: {name: {"input":[..],"bias":[..],"internal":[..]}}}),
 * NeuralNetwork.cpp:1056-1086, TrainableLayer.cu:135-205.  Layer types understood: input,
 * feedforward_tanh, feedforward_logistic, feedforward_identity, lstm, blstm, sse.
 * Weights absent from the JSON are drawn U(-0.08, 0.08)... by seed `random_seed`. */
int b2_net_create(const char *network_json, int parallel_sequences, int max_seq_length, unsigned random_seed,
                  b2_net **out);
/* --lstm_forget_gate_bias (Configuration.cpp:682-683, layers/LstmLayer.cu:1147-1161): a value above 1e-4 is added to
 * every forget-gate bias of the (b)lstm layers that b2_net_create initialises at random from now on (layers whose
 * weights come from the JSON are left alone).  Process-wide, like the reference's Configuration; default 0. */
void b2_config_set_lstm_forget_gate_bias(float value);
/* --weights_uniform_min / --weights_uniform_max (Configuration.cpp:666-670; defaults -0.1, 0.1): the range of the random
 * weights of layers without a "weights" section.  b2_net_create draws them as the reference does with its default
 * weights_dist = uniform (layers/TrainableLayer.cu:219-233): one mt19937 seeded with `seed` for all layers in order, each
 * weight = boost::random::uniform_real_distribution<float>(0, max - min)(gen) + min (restated from Boost.Random).
 * Process-wide; call before b2_net_create. */
void b2_config_set_weights_uniform(float min, float max);

/* Tuning of the persistent tensor-core recurrence (no counterpart in the reference).  The sequences of a fraction are
 * processed in chunks of 32 or 64; the chunks of a group of blocks are in flight together.
 *   nc32_chunks: the largest number of chunks per group for which chunks are 32 sequences wide and use the
 *     latency-optimised exchange (self-validating words through L2 instead of step counters and bulk copies);
 *   ll_chunks: the largest number of 64-wide chunks per group that still uses that exchange;
 *   nc32_counter_chunks (backward sweep only, 0 = off): the largest number of 32-wide chunks per group that run behind
 *     step counters; wider fractions use chunks of 64 behind step counters.
 * The forward (backward = 0) and the backward sweep have settings of their own (defaults 1, 1, 0 and 2, 5, 6: the measured
 * optimum on a B200).  Every setting gives the same bits.  Call before layers or networks are created. */
void b2_config_set_ptc_plan(int backward, int ll_chunks, int nc32_chunks, int nc32_counter_chunks);
void b2_net_destroy(b2_net *net);
/* Layer::parallelSequences() / Layer::maxSeqLength() (layers/Layer.hpp:163-175) the net was created with */
int b2_net_parallel_sequences(const b2_net *net);
int b2_net_max_seq_length(const b2_net *net);
int b2_net_num_layers(const b2_net *net);
int b2_net_layer_size(const b2_net *net, int layer);
/* 0 for layers without weights */
size_t b2_net_num_weights(const b2_net *net, int layer);
/* host <-> device copies of one layer's weight vector / weightUpdates vector */
int b2_net_set_weights(b2_net *net, int layer, const float *host_w);
int b2_net_get_weights(b2_net *net, int layer, float *host_w);
int b2_net_get_weight_updates(b2_net *net, int layer, float *host_g);
/* device addresses of a layer's vectors, for callers that stay on the GPU */
float *b2_net_weights_dev(b2_net *net, int layer);
float *b2_net_weight_updates_dev(b2_net *net, int layer);
float *b2_net_outputs_dev(b2_net *net, int layer);
float *b2_net_output_errors_dev(b2_net *net, int layer);

/* NeuralNetwork::loadSequences(fraction) (NeuralNetwork.cpp:1367-1373): host buffers in the
 * fraction layout of DataSet::_makeFractionTask (DataSet.cpp:642-1022): inputs[T*P*in],
 * targets[T*P*out], padded frames zero; seq_lens[n_seqs], n_seqs <= P; T >= max(seq_lens).
 * Pattern types are derived from the lengths.  Copies host -> device (asynchronously when the
 * host buffers are pinned). */
int b2_net_load_fraction(b2_net *net, int T, int n_seqs, const int *seq_lens, const float *host_inputs,
                         const float *host_targets);
/* The same with inputs/targets already on the device (they are copied device -> device). */
int b2_net_load_fraction_dev(b2_net *net, int T, int n_seqs, const int *seq_lens, const float *dev_inputs,
                             const float *dev_targets);
/* NeuralNetwork::computeForwardPass then calculateError: *error = 0.5*sum (target-output)^2 over
 * non-padding frames (SsePostOutputLayer.cu:94-116,197-209).  Synchronises to return the scalar;
 * pass NULL to stay asynchronous. */
int b2_net_forward(b2_net *net, double *error);
/* NeuralNetwork::computeBackwardPass (layers in reverse order, NeuralNetwork.cpp:2744-2800). */
int b2_net_backward(b2_net *net);
/* SteepestDescentOptimizer::_updateWeights, plain branch: g<-0 where NaN/Inf;
 * delta<-momentum*delta-lr*g; w<-w+delta.  A layer's own "learningRate" (>= 0) overrides lr
 * (SteepestDescentOptimizer.cu:425-426).  With a data-parallel communicator attached the
 * gradients are first summed over all ranks. */
int b2_net_update_weights(b2_net *net, float learning_rate, float momentum);
/* The optimizer option of the reference (--optimizer; MacroDefine.hpp:32-37; gradient shaping in
 * SteepestDescentOptimizer::_updateWeights, SteepestDescentOptimizer.cu:127-194,306-395) applied by
 * every later update: 0 plain steepest descent (default), 1 AdaGrad, 2 gradient averaged over the
 * fraction's frames, 3 steepest descent that accumulates the AdaGrad statistics, 4 steepest descent
 * whose learning rate the training run decays (the update itself is the plain one), 5 Adam
 * (beta1 0.9, beta2 0.999, epsilon 1e-8).  What options 3 and 4 do when validation stalls: b2_optimizer_train.  Setting it (re)initialises the statistics as the
 * reference's Optimizer constructor does (Optimizer.cu:421-457).  With a data-parallel communicator
 * attached the frame count is summed over the ranks. */
int b2_net_set_optimizer(b2_net *net, int option);
/* Optimizer::m_weightStats of one layer (AdaGrad: one float per weight; Adam: m and v interleaved),
 * the "optimizer_status_vector" of an autosave.  host_out may be NULL to ask for *count only. */
int b2_net_get_optimizer_stats(b2_net *net, int layer, float *host_out, size_t capacity, size_t *count);
/* Batch (non-stochastic) learning, i.e. the reference without --hybrid_online_batch
 * (optimizers/Optimizer.cu:186-196, 243-245): after every backward pass the optimizer's copy of the
 * weight updates takes (first != 0) or adds the layer gradients; after the last fraction ONE update
 * runs on the sum, with a frame count of 1 for the shaping options. */
int b2_net_accumulate_weight_updates(b2_net *net, int first);
int b2_net_update_weights_batch(b2_net *net, float learning_rate, float momentum);
/* One iteration of the minibatch loop of Optimizer::_processDataSet (Optimizer.cu:68-231) with
 * hybrid_online_batch: load, forward, error, backward, [all-reduce], update.  *error may be NULL. */
int b2_net_train_step(b2_net *net, int T, int n_seqs, const int *seq_lens, const float *host_inputs,
                      const float *host_targets, float learning_rate, float momentum, double *error);
/* Overlap of the host -> device copy with compute (the role of the reference's optional loader
 * thread, data_sets/DataSet.cpp:456-489): b2_net_prefetch_fraction starts copying the NEXT fraction
 * (pinned host buffers, which must stay valid until the step that uses them has been enqueued) into
 * the idle half of a double buffer on a copy stream and returns at once;
 * b2_net_train_step_prefetched runs the train step on the fraction prefetched last. */
int b2_net_prefetch_fraction(b2_net *net, int T, int n_seqs, const int *seq_lens, const float *host_inputs,
                             const float *host_targets);
int b2_net_train_step_prefetched(b2_net *net, float learning_rate, float momentum, double *error);
/* Reads the error of the last forward pass back to the host; waits for the compute stream only (a
 * prefetch in flight keeps running). */
int b2_net_read_error(b2_net *net, double *error);
/* Device-resident variant of the step above (no host<->device traffic, no synchronisation). */
int b2_net_train_step_dev(b2_net *net, int T, int n_seqs, const int *seq_lens, const float *dev_inputs,
                          const float *dev_targets, float learning_rate, float momentum);
/* Copy a layer's outputs / output errors of the current fraction to the host: T*P*size floats. */
int b2_net_get_outputs(b2_net *net, int layer, float *host_out);
int b2_net_get_output_errors(b2_net *net, int layer, float *host_out);
/* Waits for everything the net has enqueued; returns B2_ERR_STEP_TIMEOUT / B2_ERR_CUDA if a
 * kernel reported a problem since the last call. */
int b2_net_synchronize(b2_net *net);
/* The stream all of the net's work is ordered on (a cudaStream_t). */
b2_stream b2_net_stream(b2_net *net);
/* The recurrence mode of every (b)lstm layer, values as for b2_lstm_set_recurrence_mode: 0 stepwise,
 * 1 persistent kernels of the library's choice (default), 2 clusters, 3 tensor-core GEMM per step,
 * 4 L2 only, 5 persistent tensor-core kernels, 6 those for the forward sweep only. */
int b2_net_set_recurrence_mode(b2_net *net, int mode);
/* b2_lstm_recurrence_path of layer `layer` of the net; -1 for layers that are no (b)lstm. */
int b2_net_recurrence_path(b2_net *net, int layer, int backward);
/* Non-zero forces the FFMA GEMM everywhere (the tensor-core GEMM is the default). */
int b2_net_set_force_ffma(b2_net *net, int on);
/* Number of kernels this library has launched on behalf of `net` since creation. */
unsigned long long b2_net_launch_count(const b2_net *net);
/* Per-kernel-class device time of the LAST train step, measured with CUDA events when
 * profiling is switched on (costs extra synchronisation).  names/ms arrays of length `cap`;
 * returns the number of entries. */
int b2_net_set_profiling(b2_net *net, int on);
int b2_net_get_profile(b2_net *net, int cap, const char **names, float *ms, int *launches);

/* Self-test of the failure path of the persistent kernels: one block waits, with the sweeps' own
 * bounded wait, for a step tag that nothing writes.  The wait runs out after its budget (a second or
 * two), the kernel records B2_ERR_STEP_TIMEOUT and returns; the context stays usable.  *status_out =
 * the recorded code, *gave_up = 1 when the block left through the timeout path.  No counterpart in
 * the reference (its kernels have no waits). */
int b2_selftest_bounded_wait(int *status_out, int *gave_up);
/* Self-test of how such a failure travels: writes `code` from the HOST into the device status word that the
 * net's kernels record a given-up wait in, exactly where a kernel would have put it (no kernel is made to fail).
 * The next b2_net_synchronize, b2_net_train_epoch or b2_optimizer_train must return `code`. */
int b2_selftest_inject_status(b2_net *net, int code);

/* ------------------------------------------------------------------------------------------
 * Data-parallel training: sequences of a fraction are dealt to the ranks, every rank holds a
 * full weight replica, weightUpdates are summed with ncclAllReduce before the update.
 * No counterpart in the reference (single GPU, single process).
 * ------------------------------------------------------------------------------------------ */
#define B2_DP_UNIQUE_ID_BYTES 128
/* rank 0 creates the id and ships the 128 bytes to the other ranks by any means */
int b2_dp_get_unique_id(void *id_bytes);
int b2_dp_attach(b2_net *net, int rank, int world_size, const void *id_bytes);
int b2_dp_detach(b2_net *net);
/* Sum a double over all ranks (loss / frame counts). Synchronises. */
int b2_dp_allreduce_scalar(b2_net *net, double *value);
/* Number of ranks of the attached communicator; 1 when none is attached. */
int b2_dp_world_size(const b2_net *net);
/* The train step of a rank that has NO sequence in the current fraction (a sharded data set near the
 * end of an epoch): zero gradients go into the all-reduce, the update runs as on the other ranks. */
int b2_net_train_step_empty(b2_net *net, float learning_rate, float momentum);
/* Its backward part alone: zero gradients into the all-reduce of every layer (batch learning). */
int b2_net_backward_empty(b2_net *net);

/* ------------------------------------------------------------------------------------------
 * Data sets: the toolkit's .nc files (netCDF classic; CURRENNT_codes/README section 5) read
 * into fractions of parallel_sequences sequences.  Host code; replaces data_sets::DataSet
 * (data_sets/DataSet.hpp:47-369) and DataSetFraction (data_sets/DataSetFraction.hpp:40-263)
 * for regression data.
 * ------------------------------------------------------------------------------------------ */
typedef struct b2_data b2_data;

typedef struct {
    int parallel_sequences;   /* --parallel_sequences */
    float fraction;           /* --train_fraction and the like: portion of each file's sequences, (0, 1] */
    int trunc_seq_length;     /* --truncate_seq: > 0 cuts sequences into segments (DataSet.cpp:1465-1500) */
    int fraction_shuffling;   /* --shuffle_fractions */
    int sequence_shuffling;   /* --shuffle_sequences */
    unsigned random_seed;     /* --random_seed: seeds the process-wide shuffle generator at its first use */
    int training_mode;        /* non-zero: segments are sorted by length (DataSet.cpp:1898-1900) */
    int loader_threads;       /* threads that convert one fraction; 0 = min(8, hardware threads) */
    /* Data-parallel sharding (no counterpart in the reference): with shard_count = S > 1 a fraction spans
     * parallel_sequences * S sequences, dealt to the shards in snake order (0 1 .. S-1, S-1 .. 1 0, ...)
     * so that frames and longest lengths balance; this handle assembles shard_rank's sequences only, padded
     * to that shard's own longest sequence.  At the end of an epoch a shard's fraction may be empty
     * (num_sequences 0).  shard_count 0 means 1. */
    int shard_rank, shard_count;
} b2_data_options;

typedef struct {
    int max_seq_length;       /* DataSetFraction::maxSeqLength: T of this fraction */
    int min_seq_length;
    int num_sequences;        /* <= parallel_sequences (the last fraction of an epoch may be short) */
    long long total_frames;   /* DataSetFraction::fracTimeLength: real frames */
    const int *seq_lengths;   /* [num_sequences] */
    const float *inputs;      /* [max_seq_length * parallel_sequences * input_size], index (t*P + p)*size + d */
    const float *targets;     /* [max_seq_length * parallel_sequences * output_size] */
    const char *pat_types;    /* [max_seq_length * parallel_sequences]: 0 none, 1 first, 2 normal, 3 last */
} b2_fraction;

/* DataSet::DataSet(ncfiles, parSeq, fraction, truncSeqLength, fracShuf, seqShuf, ...)
 * (DataSet.cpp:1303-1907).  Errors (B2_ERR_BAD_ARG) carry the reference's messages. */
int b2_data_open(b2_data **out, const char *const *nc_paths, int n_files, const b2_data_options *opt);
void b2_data_close(b2_data *data);
/* totalSequences, totalTimesteps, minSeqLength, maxSeqLength, inputPatternSize, outputPatternSize */
int b2_data_info(const b2_data *data, int *total_sequences, long long *total_timesteps, int *min_seq_length,
                 int *max_seq_length, int *input_size, int *output_size);
/* outputMeans / outputStdevs of the first file; *present = 0 (and 0 / 1 values) when the file has none */
int b2_data_output_mean_stdev(const b2_data *data, float *means, float *stdevs, int *present);
/* DataSet::getNextFraction (DataSet.cpp:1943-1995): returns B2_OK and fills *frac, or
 * B2_DATA_EPOCH_END once after the last fraction of an epoch (the reference returns a null
 * pointer there).  The buffers behind *frac are pinned when a GPU is present and stay valid for
 * the next two calls; the following fraction is assembled by a loader thread meanwhile. */
#define B2_DATA_EPOCH_END 1
int b2_data_next_fraction(b2_data *data, b2_fraction *frac);
/* seq_info_t of sequence i of the fraction returned last: utterance name, index of the segment in
 * its utterance. */
int b2_data_fraction_seq_info(const b2_data *data, int i, char *tag, int tag_capacity, int *original_seq_idx);
/* Re-seeds the process-wide generator that sequence and fraction shuffling draw from. */
void b2_data_reseed(unsigned seed);
/* One pass of Optimizer::_processDataSet over a data set with weight updates after every fraction
 * (hybrid_online_batch; optimizers/Optimizer.cu:68-231): the next fraction is copied to the device
 * while the current one trains.  *error = sum over fractions of (fraction error / totalSequences)
 * as the reference accumulates it; with learning_rate < 0 nothing is updated (validation pass:
 * forward and error only).  The data set must have been opened with the net's parallel_sequences and hold
 * no sequence longer than the net's max_seq_length (B2_ERR_BAD_SHAPE otherwise).  Before it returns the call
 * waits for the device once and reports B2_ERR_STEP_TIMEOUT if a kernel gave up a bounded wait during the
 * epoch (the weights are then not to be trusted). */
int b2_net_train_epoch(b2_net *net, b2_data *data, float learning_rate, float momentum, double *error,
                       long long *frames);
/* The same pass as batch learning (no --hybrid_online_batch): gradients of all fractions are summed,
 * the weights change once, after the last fraction. */
int b2_net_train_epoch_batch(b2_net *net, b2_data *data, float learning_rate, float momentum, double *error,
                             long long *frames);

/* ------------------------------------------------------------------------------------------
 * Network export, and the training run around the epoch loop: validation-based early
 * stopping, best-weight bookkeeping, autosave / continue.  The JSON documents use the
 * reference's member names, so files travel between the two implementations.
 * ------------------------------------------------------------------------------------------ */
/* NeuralNetwork::exportLayers + exportWeights (NeuralNetwork.cpp:2993-3043;
 * layers/TrainableLayer.cu:441-480): {"layers":[{name,type,size,bias[,learningRate]}],
 * "weights":{name:{"input":[..],"bias":[..],"internal":[..]}}} as text.  buf may be NULL to ask
 * for the size (*needed, including the terminating NUL).  digits: significant digits of every
 * number; <= 0 means 9 (exact for fp32); 6 is what the reference's writer prints ("%g"). */
int b2_net_export_json(b2_net *net, char *buf, size_t capacity, size_t *needed, int digits);
/* NeuralNetwork::saveNetwork (NeuralNetwork.cpp:4104-4125): the same document into a file
 * (trained_network.jsn). */
int b2_net_save_network(b2_net *net, const char *filename, int digits);
/* NeuralNetwork::printWeightMatrix (NeuralNetwork.cpp:3792-3880; read back by pyTools/ioTools/nnio.py
 * ReadCURRENNTWeight): the weights as one file of native floats.  Header: the number of layers with weights, then
 * per layer {number of weights, size, preceding layer's size, input weights per block, internal weights per block}
 * (and, when with_type_codes is non-zero, the reference's type code 0 feedforward_tanh, 1 _logistic, 2 _identity,
 * 3 _relu, 4 lstm, 5 blstm); then every layer's weight vector in layer order. */
int b2_net_save_weights_binary(b2_net *net, const char *filename, int with_type_codes);
/* The momentum term of SteepestDescentOptimizer (m_weightDeltas, SteepestDescentOptimizer.cu:421-438)
 * of one layer, host <-> device; part of the autosave state. */
int b2_net_get_weight_deltas(b2_net *net, int layer, float *host_out);
int b2_net_set_weight_deltas(b2_net *net, int layer, const float *host_in);

typedef struct b2_optimizer b2_optimizer;
typedef struct {
    float learning_rate;       /* --learning_rate */
    float momentum;            /* --momentum */
    int max_epochs;            /* --max_epochs; < 0: no limit */
    int max_epochs_no_best;    /* --max_epochs_no_best */
    int validate_every;        /* --validate_every */
    int test_every;            /* --test_every */
    int batch_learning;        /* non-zero: the reference WITHOUT --hybrid_online_batch (one update per epoch) */
    float second_learning_rate;/* --OptimizerSecondLR (reference default 0.01): the rate after option 3 has switched to AdaGrad */
    float lr_decay_rate;       /* --LRDecayRate (reference default 0.1): factor applied by option 4 when validation stalls */
} b2_optimizer_options;
typedef struct {
    int finished, cur_epoch, epochs_since_lowest_error;
    float lowest_validation_error;
    float cur_training_error, cur_validation_error, cur_test_error;   /* sum over fractions of error / totalSequences */
    float cur_training_error_per_frame, cur_validation_error_per_frame, cur_test_error_per_frame;
    float learning_rate;       /* the rate in use (changed by options 3 and 4 when validation stalls) */
    int optimizer_option;      /* the net's option in use (3 turns into 1 when validation stalls) */
} b2_optimizer_state;
/* optimizers::SteepestDescentOptimizer(network, trainingSet, validationSet, testSet, maxEpochs,
 * maxEpochsNoBest, validateEvery, testEvery, learningRate, momentum) (Optimizer.cu:375-421);
 * validation_set and test_set may be NULL (the reference passes empty data sets). */
int b2_optimizer_create(b2_optimizer **out, b2_net *net, b2_data *training_set, b2_data *validation_set,
                        b2_data *test_set, const b2_optimizer_options *options);
void b2_optimizer_destroy(b2_optimizer *opt);
/* Optimizer::train (Optimizer.cu:565-689): one epoch over the training set with weight updates,
 * then validation / test passes when due; stores the weights on a new lowest validation error,
 * restores the best weights and sets *finished when max_epochs or max_epochs_no_best is reached.
 * With the net's optimizer option 3 or 4 (b2_net_set_optimizer) a stall of max_epochs_no_best epochs does not end the run
 * (Optimizer.cu:653-668): option 3 switches to AdaGrad (option 1, keeping the statistics gathered so far) with
 * second_learning_rate and forgets the lowest validation error; option 4 multiplies the rate by lr_decay_rate; both
 * restore the best weights and go on with epochs_since_lowest_error = 1. */
int b2_optimizer_train(b2_optimizer *opt, int *finished);
int b2_optimizer_get_state(const b2_optimizer *opt, b2_optimizer_state *state);
/* Optimizer::saveState (Optimizer.cu:851-933, the "epochNNN.autosave" files): configuration and
 * info rows as given, network, optimizer members, best weights and momentum deltas. */
int b2_optimizer_save_state(b2_optimizer *opt, const char *filename, const char *configuration, const char *info_rows,
                            int digits);
/* --continue: weights from the file's "weights" section, then Optimizer::restoreState /
 * importState (Optimizer.cu:728-765, 915-930).  info_rows may be NULL. */
int b2_optimizer_restore_state(b2_optimizer *opt, const char *filename, char *info_rows, size_t info_capacity);

#ifdef __cplusplus
}
#endif
#endif /* B2LSTM_H */
