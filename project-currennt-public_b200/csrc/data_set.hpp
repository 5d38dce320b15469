// Host-side data set: reads the toolkit's .nc files and assembles fractions (minibatches of
// parallel_sequences sequences) in the layout the layers load.
//
// Mirrors data_sets::DataSet / DataSetFraction of the reference (data_sets/DataSet.cpp:1303-1907
// constructor: per-file sequence table, truncation into segments, sort by length in training mode;
// :491-519 sequence / fraction shuffling; :640-1020 _makeFractionTask; :1943-1995 getNextFraction
// with the loader thread) for regression data: inputs, targetPatterns, seqTags, seqLengths and the
// optional outputMeans / outputStdevs.  Differences by design: the .nc file is memory-mapped and a
// fraction is converted from big-endian straight into a pinned host buffer (no cache file, no
// intermediate copy), several threads share the conversion, and three fraction buffers rotate so
// that a fraction stays valid while the next one is assembled and the previous one is still being
// copied to the device.
#pragma once
#include <condition_variable>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "nc_file.hpp"

namespace b2 {

struct DataSetOptions {
    int parallelSequences = 1;
    float fraction = 1.0f;          // portion of each file's sequences that is used
    int truncSeqLength = 0;         // > 0: cut sequences into segments of this length
    bool fractionShuffling = false;
    bool sequenceShuffling = false;
    unsigned randomSeed = 0;
    bool trainingMode = true;       // sort the segments by length
    int loaderThreads = 0;          // 0: min(8, hardware threads)
    // data-parallel sharding: a fraction then spans parallelSequences * shardCount sequences, dealt to the
    // shards in snake order (0 1 2 .. S-1, S-1 .. 1 0, ...) so that frames and longest lengths balance;
    // this data set assembles shard shardRank's sequences only
    int shardRank = 0, shardCount = 1;
};

// what DataSetFraction exposes to Layer::loadSequences
struct FractionView {
    int maxSeqLength = 0, minSeqLength = 0;
    int numSequences = 0;
    long fracTotalLength = 0;            // real frames
    std::vector<int> seqLengths;         // [numSequences]
    std::vector<int> originalSeqIdx;     // index of each segment inside its utterance
    std::vector<std::string> seqTags;    // utterance names
    float *inputs = nullptr;             // [maxSeqLength * P * inputPatternSize], frame (t*P+p) major
    float *outputs = nullptr;            // [maxSeqLength * P * outputPatternSize]
    char *patTypes = nullptr;            // [maxSeqLength * P]
};

class DataSet {
public:
    struct sequence_t {
        int originalSeqIdx;     // index of the segment inside its utterance
        int length;
        std::string seqTag;
        int file;               // which .nc file
        long long frameBegin;   // first frame of the segment in that file's inputs / targetPatterns
        int beginInUtt;
    };

    DataSet() {}
    ~DataSet();
    DataSet(const DataSet &) = delete;
    DataSet &operator=(const DataSet &) = delete;

    // empty string on success, else the message the reference would throw
    std::string open(const std::vector<std::string> &ncfiles, const DataSetOptions &opt);
    // nullptr once per epoch, after its last fraction (as the reference's getNextFraction)
    const FractionView *getNextFraction();

    int totalSequences() const { return (int)m_sequences.size(); }
    unsigned long totalTimesteps() const { return m_totalTimesteps; }
    int minSeqLength() const { return m_minSeqLength; }
    int maxSeqLength() const { return m_maxSeqLength; }
    int inputPatternSize() const { return m_inputPatternSize; }
    int outputPatternSize() const { return m_outputPatternSize; }
    int parallelSequences() const { return m_opt.parallelSequences; }
    bool outputMVFlag() const { return m_outputMVFlag; }
    const std::vector<float> &outputMeans() const { return m_outputMeans; }
    const std::vector<float> &outputStdevs() const { return m_outputStdevs; }
    const std::vector<sequence_t> &sequences() const { return m_sequences; }
    bool pinned() const { return m_pinned; }
    const std::string &lastError() const { return m_error; }

private:
    void _shuffleSequences();
    void _shuffleFractions();
    void _makeFractionTask(int firstSeqIdx, FractionView &frac);
    void _makeFirstFractionTask(FractionView &frac);
    void _nextFracThreadFn();
    void _startTask(bool first, int firstSeqIdx);

    DataSetOptions m_opt;
    std::vector<std::unique_ptr<NcFile> > m_files;
    std::vector<const NcFile::Var *> m_inVar, m_outVar;
    std::vector<sequence_t> m_sequences;
    unsigned long m_totalTimesteps = 0;
    int m_minSeqLength = 0, m_maxSeqLength = 0;
    int m_inputPatternSize = 0, m_outputPatternSize = 0;
    bool m_outputMVFlag = false;
    std::vector<float> m_outputMeans, m_outputStdevs;
    int m_curFirstSeqIdx = -1;
    std::string m_error;

    // three rotating fraction buffers
    FractionView m_frac[3];
    void *m_block[3] = {nullptr, nullptr, nullptr};
    bool m_pinned = false;
    int m_build = 0;       // buffer the loader thread fills next

    // loader thread (thread_data_t of the reference)
    std::thread m_thread;
    std::mutex m_mutex;
    std::condition_variable m_cv;
    bool m_terminate = false, m_hasTask = false, m_finished = false;
    bool m_taskFirst = false;
    int m_taskSeqIdx = 0;
    int m_taskBuf = 0, m_readyBuf = -1;
    bool m_threadStarted = false;
};

// the process-wide generator behind sequence and fraction shuffling (see data_set.cpp)
void reseed_shuffle_generator(unsigned seed);

}  // namespace b2
