// Per-device facts and one-time set-up, keyed by the device ordinal.
//
// The reference toolkit binds one process to one device at start-up (currennt/src/main.cpp:725-739 of the
// reference) and keeps its cuBLAS handle in a process-wide singleton (helpers/cublas.cu:33-43).  This library
// may be loaded by a host that drives several devices from one process, so nothing that belongs to a device
// or to a context is cached process-wide: multiprocessor counts, kernel attributes (they are per context),
// helper streams and the scratch of the stand-alone matrix product all live in slots per ordinal.
#include <mutex>
#include <set>
#include <utility>

#include "common.cuh"

namespace b2 {

namespace {
std::mutex g_mu;
int g_sms[MAX_DEVICES];
std::set<std::pair<const void *, int> > g_attr_done;
}  // namespace

int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return -1;
    return dev;
}

int sm_count() {
    const int dev = current_device();
    if (dev < 0) return 1;
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_sms[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 1;
        g_sms[dev] = n;
    }
    return g_sms[dev];
}

int set_max_dynamic_smem(const void *func, int bytes) {
    const int dev = current_device();
    if (dev < 0) { set_error("no current CUDA device (or an ordinal beyond %d)", MAX_DEVICES - 1); return B2_ERR_CUDA; }
    std::lock_guard<std::mutex> lk(g_mu);
    const std::pair<const void *, int> key(func, dev);
    if (g_attr_done.count(key)) return B2_OK;
    B2_CUDA(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    g_attr_done.insert(key);
    return B2_OK;
}

}  // namespace b2
