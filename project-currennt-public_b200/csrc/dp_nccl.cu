// Data-parallel gradient exchange: ncclAllReduce(sum, fp32) of each layer's weightUpdates over the
// GPUs of one box.  The reference is single-GPU (one cudaSetDevice, no communication library), so
// this file has no counterpart there; it slots in where Optimizer::_processDataSet collects
// layer->weightUpdates() (optimizers/Optimizer.cu:171-227 of the reference).
//
// NCCL is bound at run time (dlopen of libnccl.so.2) so that the library loads on hosts without it
// and shares the copy an embedding process (e.g. PyTorch) has already loaded.
#include <dlfcn.h>

#include "network.hpp"

namespace b2 {

namespace {
typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
enum { ncclFloat32 = 7, ncclFloat64 = 8, ncclSum = 0 };

struct NcclApi {
    void *lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};
NcclApi g_nccl;

int load_nccl() {
    if (g_nccl.lib) return B2_OK;
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    void *h = nullptr;
    for (int i = 0; i < 2 && !h; ++i) h = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
    if (!h) { set_error("NCCL not found: %s", dlerror()); return B2_ERR_NCCL; }
    g_nccl.GetUniqueId = (ncclResult_t(*)(ncclUniqueId *))dlsym(h, "ncclGetUniqueId");
    g_nccl.CommInitRank = (ncclResult_t(*)(ncclComm_t *, int, ncclUniqueId, int))dlsym(h, "ncclCommInitRank");
    g_nccl.CommDestroy = (ncclResult_t(*)(ncclComm_t))dlsym(h, "ncclCommDestroy");
    g_nccl.AllReduce = (ncclResult_t(*)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t))dlsym(h, "ncclAllReduce");
    g_nccl.GetErrorString = (const char *(*)(ncclResult_t))dlsym(h, "ncclGetErrorString");
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.CommDestroy || !g_nccl.AllReduce) {
        set_error("NCCL library lacks the expected symbols");
        return B2_ERR_NCCL;
    }
    g_nccl.lib = h;
    return B2_OK;
}
int nccl_fail(ncclResult_t r, const char *what) {
    set_error("NCCL error %d in %s: %s", r, what, g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "?");
    return B2_ERR_NCCL;
}
}  // namespace

struct DpComm {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
};

int dp_get_unique_id(void *bytes) {
    B2_TRY(load_nccl());
    ncclUniqueId id;
    ncclResult_t r = g_nccl.GetUniqueId(&id);
    if (r) return nccl_fail(r, "ncclGetUniqueId");
    memcpy(bytes, &id, sizeof id);
    return B2_OK;
}
int dp_attach(NeuralNetwork &net, int rank, int world, const void *idBytes) {
    if (net.dp) { set_error("b2_dp_attach: already attached"); return B2_ERR_STATE; }
    if (world < 1 || rank < 0 || rank >= world || !idBytes) { set_error("b2_dp_attach: bad rank/world"); return B2_ERR_BAD_ARG; }
    B2_TRY(load_nccl());
    ncclUniqueId id;
    memcpy(&id, idBytes, sizeof id);
    DpComm *c = new DpComm;
    c->rank = rank; c->world = world;
    ncclResult_t r = g_nccl.CommInitRank(&c->comm, world, id, rank);
    if (r) { delete c; return nccl_fail(r, "ncclCommInitRank"); }
    net.dp = c;
    return B2_OK;
}
int dp_detach(NeuralNetwork &net) {
    if (!net.dp) return B2_OK;
    net.synchronize();
    g_nccl.CommDestroy(net.dp->comm);
    delete net.dp;
    net.dp = nullptr;
    return B2_OK;
}
int dp_world(const NeuralNetwork &net) { return net.dp ? net.dp->world : 1; }
int dp_allreduce_sum(NeuralNetwork &net, float *buf, size_t n, cudaStream_t st) {
    if (!net.dp || net.dp->world == 1) return B2_OK;
    ncclResult_t r = g_nccl.AllReduce(buf, buf, n, ncclFloat32, ncclSum, net.dp->comm, st);
    if (r) return nccl_fail(r, "ncclAllReduce");
    return B2_OK;
}
int dp_allreduce_double(NeuralNetwork &net, double *dev, cudaStream_t st) {
    if (!net.dp || net.dp->world == 1) return B2_OK;
    ncclResult_t r = g_nccl.AllReduce(dev, dev, 1, ncclFloat64, ncclSum, net.dp->comm, st);
    if (r) return nccl_fail(r, "ncclAllReduce");
    return B2_OK;
}

}  // namespace b2

struct b2_net;
extern "C" {
b2::NeuralNetwork *b2_net_impl(b2_net *n);

int b2_dp_get_unique_id(void *id_bytes) {
    if (!id_bytes) return B2_ERR_BAD_ARG;
    return b2::dp_get_unique_id(id_bytes);
}
int b2_dp_attach(b2_net *net, int rank, int world, const void *id_bytes) {
    if (!net) return B2_ERR_BAD_ARG;
    return b2::dp_attach(*b2_net_impl(net), rank, world, id_bytes);
}
int b2_dp_detach(b2_net *net) {
    if (!net) return B2_ERR_BAD_ARG;
    return b2::dp_detach(*b2_net_impl(net));
}
int b2_dp_allreduce_scalar(b2_net *net, double *value) {
    if (!net || !value) return B2_ERR_BAD_ARG;
    b2::NeuralNetwork &n = *b2_net_impl(net);
    if (!n.dp || b2::dp_world(n) == 1) return B2_OK;
    double *dev = nullptr;
    B2_CUDA(cudaMalloc(&dev, sizeof(double)));
    B2_CUDA(cudaMemcpyAsync(dev, value, sizeof(double), cudaMemcpyHostToDevice, n.stream));
    int rc = b2::dp_allreduce_double(n, dev, n.stream);
    if (rc == B2_OK) {
        cudaMemcpyAsync(value, dev, sizeof(double), cudaMemcpyDeviceToHost, n.stream);
        cudaStreamSynchronize(n.stream);
    }
    cudaFree(dev);
    return rc;
}
}
