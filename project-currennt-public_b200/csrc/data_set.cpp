// Data set and fraction assembly; see data_set.hpp.  Host code only (pinned memory comes from the
// CUDA runtime when a device is present, else from the C library).
#include "data_set.hpp"

#include <cuda_runtime.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <limits>
#include <random>

namespace b2 {
namespace {

enum { PATTYPE_NONE = 0, PATTYPE_FIRST = 1, PATTYPE_NORMAL = 2, PATTYPE_LAST = 3 };   // Types.hpp:35-38

// The reference draws every shuffle from ONE process-wide boost::mt19937, seeded with the configured
// random seed at first use and shared by all data sets (DataSet.cpp:436-448).  std::mt19937 is the
// same generator.  boost::uniform_int<>(0, n-1) on a 32-bit engine divides the engine's range into
// n buckets of floor(2^32 / n) values (Boost.Random, generate_uniform_int) and rejects the tail.
std::mutex g_rng_mutex;
std::mt19937 *g_rng = nullptr;

unsigned rand_below(unsigned n, unsigned seed) {
    if (!g_rng) g_rng = new std::mt19937(seed);
    const unsigned range = n - 1;
    if (range == 0) return 0;
    const unsigned brange = 0xFFFFFFFFu;
    if (range == brange) return (unsigned)(*g_rng)();
    unsigned bucket = brange / (range + 1u);
    if (brange % (range + 1u) == range) ++bucket;
    for (;;) {
        unsigned r = (unsigned)(*g_rng)() / bucket;
        if (r <= range) return r;
    }
}

// std::random_shuffle(first, last, rng) as libstdc++ defines it: element i is swapped with element
// rng(i + 1), i = 1 .. n-1
template <typename T>
void random_shuffle_ref(std::vector<T> &v, unsigned seed) {
    std::lock_guard<std::mutex> lock(g_rng_mutex);
    for (size_t i = 1; i < v.size(); ++i) {
        size_t j = rand_below((unsigned)(i + 1), seed);
        if (i != j) std::swap(v[i], v[j]);
    }
}

void *alloc_host(size_t bytes, bool *pinned) {
    void *p = nullptr;
    if (cudaHostAlloc(&p, bytes, cudaHostAllocPortable) == cudaSuccess) {
        *pinned = true;
        return p;
    }
    cudaGetLastError();   // no device: plain memory serves the host-only uses
    *pinned = false;
    if (posix_memalign(&p, 4096, bytes) != 0) return nullptr;
    return p;
}

void free_host(void *p, bool pinned) {
    if (!p) return;
    if (pinned) cudaFreeHost(p);
    else free(p);
}

template <typename F>
void parallel_for(int n, int threads, F fn) {
    if (threads <= 1 || n <= 1) {
        for (int i = 0; i < n; ++i) fn(i);
        return;
    }
    if (threads > n) threads = n;
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t)
        pool.emplace_back([=]() {
            for (int i = t; i < n; i += threads) fn(i);
        });
    for (std::thread &th : pool) th.join();
}

}  // namespace

void reseed_shuffle_generator(unsigned seed) {
    std::lock_guard<std::mutex> lock(g_rng_mutex);
    delete g_rng;
    g_rng = new std::mt19937(seed);
}

DataSet::~DataSet() {
    if (m_threadStarted) {
        {
            std::lock_guard<std::mutex> lock(m_mutex);
            m_terminate = true;
            m_cv.notify_all();
        }
        m_thread.join();
    }
    for (int b = 0; b < 3; ++b) free_host(m_block[b], m_pinned);
}

std::string DataSet::open(const std::vector<std::string> &ncfiles, const DataSetOptions &opt) {
    m_opt = opt;
    if (opt.fraction <= 0 || opt.fraction > 1) return "Invalid fraction";
    if (opt.parallelSequences < 1) return "Invalid number of parallel sequences";
    if (opt.shardCount < 1 || opt.shardRank < 0 || opt.shardRank >= opt.shardCount) return "Invalid shard rank / count";
    if (ncfiles.empty()) return "No data files given";
    if (m_opt.loaderThreads <= 0) {
        unsigned hc = std::thread::hardware_concurrency();
        m_opt.loaderThreads = (int)std::min(8u, hc ? hc : 1u);
    }
    m_minSeqLength = std::numeric_limits<int>::max();
    m_maxSeqLength = std::numeric_limits<int>::min();
    int truncSeqLength = opt.truncSeqLength;

    bool first_file = true;
    for (size_t fi = 0; fi < ncfiles.size(); ++fi) {
        std::unique_ptr<NcFile> nc(new NcFile);
        std::string err = nc->open(ncfiles[fi]);
        if (!err.empty()) return err;
        uint64_t v = 0;
        if (!nc->dim("maxSeqTagLength", &v)) return "Cannot get dimension 'maxSeqTagLength'";
        if (nc->hasDim("numLabels")) return "Classification data (dimension 'numLabels') is not supported";
        if (!nc->dim("inputPattSize", &v)) return "Cannot get dimension 'inputPattSize'";
        const int inSize = (int)v;
        if (!nc->dim("targetPattSize", &v)) return "Cannot get dimension 'targetPattSize'";
        const int outSize = (int)v;
        if (first_file) {
            m_inputPatternSize = inSize;
            m_outputPatternSize = outSize;
        } else {
            if (m_outputPatternSize != outSize) return "Number of targets mismatch in NC files";
            if (m_inputPatternSize != inSize) return "Number of inputs mismatch in NC files";
        }
        if (!nc->dim("numSeqs", &v)) return "Cannot get dimension 'numSeqs'";
        int nSeq = (int)((float)(int)v * opt.fraction);
        nSeq = std::max(nSeq, 1);
        if ((uint64_t)nSeq > v) return "Cannot read array 'seqLengths'";

        const NcFile::Var *vLen = nc->var("seqLengths"), *vTag = nc->var("seqTags");
        const NcFile::Var *vIn = nc->var("inputs"), *vOut = nc->var("targetPatterns");
        if (!vLen) return "Cannot read array 'seqLengths'";
        if (!vTag) return "Cannot read variable 'seqTags'";
        if (!vIn || (int)vIn->rowElems != inSize) return "Cannot read array 'inputs'";
        if (!vOut || (int)vOut->rowElems != outSize) return "Cannot read array 'targetPatterns'";

        std::vector<int> lens(nSeq);
        if (!nc->readIntRows(*vLen, 0, nSeq, lens.data())) return "Cannot read array 'seqLengths'";

        // sequence table of this file: truncate into segments (DataSet.cpp:1443-1500)
        std::vector<sequence_t> sequences;
        long long frame = 0;
        for (int i = 0; i < nSeq; ++i) {
            int seqLength = lens[i];
            if (seqLength < 0) return "Cannot read array 'seqLengths'";
            m_totalTimesteps += (unsigned long)seqLength;
            std::string seqTag;
            if (!nc->readTextRow(*vTag, i, &seqTag)) return "Cannot read variable 'seqTags'";
            int k = 0, rePosInUtt = 0;
            while (seqLength > 0) {
                sequence_t seq;
                seq.originalSeqIdx = k;
                if (truncSeqLength > 0 && seqLength > 1.5 * truncSeqLength) seq.length = std::min(truncSeqLength, seqLength);
                else seq.length = seqLength;
                seq.seqTag = seqTag;
                seq.beginInUtt = rePosInUtt;
                seq.file = (int)fi;
                seq.frameBegin = frame;
                sequences.push_back(seq);
                seqLength -= seq.length;
                rePosInUtt += seq.length;
                frame += seq.length;
                ++k;
            }
        }
        if ((uint64_t)frame > vIn->rows) return "Cannot read array 'inputs'";
        if ((uint64_t)frame > vOut->rows) return "Cannot read array 'targetPatterns'";
        for (const sequence_t &s : sequences) {
            m_minSeqLength = std::min(m_minSeqLength, s.length);
            m_maxSeqLength = std::max(m_maxSeqLength, s.length);
        }
        if (first_file) {
            // output means + standard deviations, if they exist (DataSet.cpp:1846-1861)
            const NcFile::Var *vm = nc->var("outputMeans"), *vs = nc->var("outputStdevs");
            m_outputMeans.assign(m_outputPatternSize, 0.0f);
            m_outputStdevs.assign(m_outputPatternSize, 1.0f);
            m_outputMVFlag = false;
            if (vm && vs && (int)vm->rows == m_outputPatternSize && (int)vs->rows == m_outputPatternSize && vm->rowElems == 1 &&
                vs->rowElems == 1) {
                std::vector<float> mm(m_outputPatternSize), ss(m_outputPatternSize);
                if (nc->readFloatRows(*vm, 0, m_outputPatternSize, mm.data()) &&
                    nc->readFloatRows(*vs, 0, m_outputPatternSize, ss.data())) {
                    m_outputMeans = mm;
                    m_outputStdevs = ss;
                    m_outputMVFlag = true;
                }
            }
        }
        m_sequences.insert(m_sequences.end(), sequences.begin(), sequences.end());
        m_inVar.push_back(vIn);
        m_outVar.push_back(vOut);
        m_files.push_back(std::move(nc));
        first_file = false;
    }
    if (m_sequences.empty()) return "The data set contains no frames";
    // training: sort by length with the reference's comparator and algorithm (DataSet.cpp:430-434,1898-1900)
    if (opt.trainingMode)
        std::sort(m_sequences.begin(), m_sequences.end(),
                  [](const sequence_t &a, const sequence_t &b) { return a.length < b.length; });

    // fraction buffers: sized for the longest segment of the whole set
    const size_t slots = (size_t)m_maxSeqLength * m_opt.parallelSequences;
    const size_t inB = slots * m_inputPatternSize * sizeof(float), outB = slots * m_outputPatternSize * sizeof(float);
    const size_t inPad = (inB + 255) & ~(size_t)255, outPad = (outB + 255) & ~(size_t)255;
    for (int b = 0; b < 3; ++b) {
        bool pinned = false;
        m_block[b] = alloc_host(inPad + outPad + slots, &pinned);
        if (!m_block[b]) return "Out of host memory for the fraction buffers";
        m_pinned = pinned;
        m_frac[b].inputs = (float *)m_block[b];
        m_frac[b].outputs = (float *)((char *)m_block[b] + inPad);
        m_frac[b].patTypes = (char *)m_block[b] + inPad + outPad;
    }
    m_curFirstSeqIdx = -1;
    m_thread = std::thread(&DataSet::_nextFracThreadFn, this);
    m_threadStarted = true;
    return std::string();
}

void DataSet::_shuffleSequences() { random_shuffle_ref(m_sequences, m_opt.randomSeed); }

void DataSet::_shuffleFractions() {
    std::vector<std::vector<sequence_t> > fractions;
    for (size_t i = 0; i < m_sequences.size(); ++i) {
        if (i % ((size_t)m_opt.parallelSequences * m_opt.shardCount) == 0) fractions.resize(fractions.size() + 1);
        fractions.back().push_back(m_sequences[i]);
    }
    random_shuffle_ref(fractions, m_opt.randomSeed);
    m_sequences.clear();
    for (size_t i = 0; i < fractions.size(); ++i)
        for (size_t j = 0; j < fractions[i].size(); ++j) m_sequences.push_back(fractions[i][j]);
}

void DataSet::_makeFirstFractionTask(FractionView &frac) {
    if (m_opt.sequenceShuffling) _shuffleSequences();
    if (m_opt.fractionShuffling) _shuffleFractions();
    _makeFractionTask(0, frac);
}

// DataSet::_makeFractionTask (DataSet.cpp:640-1020): slot i of every timestep holds sequence
// firstSeqIdx + i; inputs/targets of padding frames are 0, their pattern type NONE.
void DataSet::_makeFractionTask(int firstSeqIdx, FractionView &frac) {
    const int P = m_opt.parallelSequences;
    frac.maxSeqLength = std::numeric_limits<int>::min();
    frac.minSeqLength = std::numeric_limits<int>::max();
    frac.seqLengths.clear();
    frac.originalSeqIdx.clear();
    frac.seqTags.clear();
    frac.fracTotalLength = 0;
    // position k of the (global) fraction belongs to shard k % S in even rounds, S-1 - k % S in odd rounds
    const int S = m_opt.shardCount;
    std::vector<int> mine;
    for (int k = 0; k < P * S; ++k) {
        const int seqIdx = firstSeqIdx + k;
        if (seqIdx >= (int)m_sequences.size()) break;
        const int pos = k % S, owner = ((k / S) % 2 == 0) ? pos : S - 1 - pos;
        if (owner == m_opt.shardRank) mine.push_back(seqIdx);
    }
    for (int seqIdx : mine) {
        frac.maxSeqLength = std::max(frac.maxSeqLength, m_sequences[seqIdx].length);
        frac.minSeqLength = std::min(frac.minSeqLength, m_sequences[seqIdx].length);
        frac.seqLengths.push_back(m_sequences[seqIdx].length);
        frac.originalSeqIdx.push_back(m_sequences[seqIdx].originalSeqIdx);
        frac.seqTags.push_back(m_sequences[seqIdx].seqTag);
        frac.fracTotalLength += m_sequences[seqIdx].length;
    }
    if (mine.empty()) {   // more shards than sequences in the last fraction: this shard sits the step out
        frac.maxSeqLength = frac.minSeqLength = 0;
        frac.numSequences = 0;
        return;
    }
    frac.numSequences = (int)frac.seqLengths.size();
    const int T = frac.maxSeqLength, nSeq = frac.numSequences;
    const int inSize = m_inputPatternSize, outSize = m_outputPatternSize;
    // one task per block of timesteps: the destination is written front to back
    const int chunk = 16;
    const int nChunks = (T + chunk - 1) / chunk;
    parallel_for(nChunks, m_opt.loaderThreads, [&](int c) {
        const int t0 = c * chunk, t1 = std::min(T, t0 + chunk);
        for (int t = t0; t < t1; ++t) {
            for (int i = 0; i < P; ++i) {
                const size_t slot = (size_t)t * P + i;
                float *din = frac.inputs + slot * inSize;
                float *dout = frac.outputs + slot * outSize;
                if (i < nSeq && t < frac.seqLengths[i]) {
                    const sequence_t &seq = m_sequences[mine[i]];
                    m_files[seq.file]->readFloatRows(*m_inVar[seq.file], (uint64_t)(seq.frameBegin + t), 1, din);
                    m_files[seq.file]->readFloatRows(*m_outVar[seq.file], (uint64_t)(seq.frameBegin + t), 1, dout);
                    const int len = frac.seqLengths[i];
                    frac.patTypes[slot] = (char)(t == 0 ? PATTYPE_FIRST : (t == len - 1 ? PATTYPE_LAST : PATTYPE_NORMAL));
                } else {
                    memset(din, 0, sizeof(float) * inSize);
                    memset(dout, 0, sizeof(float) * outSize);
                    frac.patTypes[slot] = (char)PATTYPE_NONE;
                }
            }
        }
    });
}

// the loader thread (DataSet.cpp:456-489)
void DataSet::_nextFracThreadFn() {
    for (;;) {
        std::unique_lock<std::mutex> lock(m_mutex);
        while (!m_hasTask && !m_terminate) m_cv.wait(lock);
        if (m_terminate) break;
        const bool first = m_taskFirst;
        const int idx = m_taskSeqIdx, buf = m_taskBuf;
        lock.unlock();
        if (first) _makeFirstFractionTask(m_frac[buf]);
        else _makeFractionTask(idx, m_frac[buf]);
        lock.lock();
        m_readyBuf = buf;
        m_finished = true;
        m_hasTask = false;
        m_cv.notify_all();
    }
}

void DataSet::_startTask(bool first, int firstSeqIdx) {
    // caller holds m_mutex
    m_taskFirst = first;
    m_taskSeqIdx = firstSeqIdx;
    m_taskBuf = m_build;
    m_build = (m_build + 1) % 3;
    m_finished = false;
    m_hasTask = true;
    m_cv.notify_all();
}

// DataSet::getNextFraction, loader-thread branch (DataSet.cpp:1943-1972): the next fraction is
// assembled while the caller works on the one returned; after the last fraction of an epoch the
// first fraction of the next epoch (after reshuffling) is already under way and nullptr is returned once.
const FractionView *DataSet::getNextFraction() {
    std::unique_lock<std::mutex> lock(m_mutex);
    if (m_curFirstSeqIdx == -1) {
        _startTask(true, 0);
        m_curFirstSeqIdx = 0;
    }
    while (!m_finished) m_cv.wait(lock);
    const FractionView *frac = nullptr;
    if (m_curFirstSeqIdx < (int)m_sequences.size()) {
        frac = &m_frac[m_readyBuf];
        m_curFirstSeqIdx += m_opt.parallelSequences * m_opt.shardCount;
        if (m_curFirstSeqIdx < (int)m_sequences.size()) _startTask(false, m_curFirstSeqIdx);
        else _startTask(true, 0);
    } else {
        m_curFirstSeqIdx = 0;
    }
    return frac;
}

}  // namespace b2
