#include "comm.h"

#include <cuda_runtime.h>
#include <dlfcn.h>

#include <mutex>

#include "kn_b200.h"

namespace kn {

namespace {

// The part of NCCL's public C API this file uses (nccl.h): types restated, nothing else taken from it.
struct NcclUniqueId {
    char internal[kCommIdBytes];
};
typedef int (*GetUniqueIdFn)(NcclUniqueId*);
typedef int (*CommInitRankFn)(void** comm, int nranks, NcclUniqueId id, int rank);
typedef int (*CommDestroyFn)(void* comm);
typedef int (*AllReduceFn)(const void* send, void* recv, size_t count, int dtype, int op, void* comm, CUstream_st* stream);
typedef const char* (*GetErrorStringFn)(int);
constexpr int kNcclSum = 0, kNcclFloat16 = 6, kNcclFloat32 = 7;

struct Nccl {
    void* handle = nullptr;
    GetUniqueIdFn get_unique_id = nullptr;
    CommInitRankFn comm_init_rank = nullptr;
    CommDestroyFn comm_destroy = nullptr;
    AllReduceFn all_reduce = nullptr;
    GetErrorStringFn error_string = nullptr;
};
Nccl g_nccl;
std::mutex g_nccl_mu;

void check_nccl(int result, const char* what) {
    if (result == 0) return;
    const char* text = g_nccl.error_string ? g_nccl.error_string(result) : "?";
    fail(KN_ERR_CUDA, std::string(what) + " failed: NCCL error " + std::to_string(result) + " (" + text + ")");
}

}  // namespace

void nccl_load(const char* path) {
    std::lock_guard<std::mutex> lock(g_nccl_mu);
    if (g_nccl.handle) return;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);      // already in the process (e.g. loaded by torch)
    if (!h && path && *path) h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
    if (!h)
        fail(KN_ERR_UNSUPPORTED, "the NCCL library (libnccl.so.2) was not found: give its path to kn_nccl_load; a graph with "
                                 "all-reduce steps needs it when the communicator has more than one rank");
    Nccl n;
    n.handle = h;
    n.get_unique_id = (GetUniqueIdFn)dlsym(h, "ncclGetUniqueId");
    n.comm_init_rank = (CommInitRankFn)dlsym(h, "ncclCommInitRank");
    n.comm_destroy = (CommDestroyFn)dlsym(h, "ncclCommDestroy");
    n.all_reduce = (AllReduceFn)dlsym(h, "ncclAllReduce");
    n.error_string = (GetErrorStringFn)dlsym(h, "ncclGetErrorString");
    if (!n.get_unique_id || !n.comm_init_rank || !n.comm_destroy || !n.all_reduce || !n.error_string)
        fail(KN_ERR_UNSUPPORTED, "the NCCL library lacks one of ncclGetUniqueId, ncclCommInitRank, ncclCommDestroy, "
                                 "ncclAllReduce, ncclGetErrorString");
    g_nccl = n;
}

void comm_unique_id(void* id128) {
    KN_CHECK(id128 != nullptr, KN_ERR_INVALID_ARG, "null id buffer");
    nccl_load(nullptr);
    NcclUniqueId id;
    check_nccl(g_nccl.get_unique_id(&id), "ncclGetUniqueId");
    memcpy(id128, id.internal, kCommIdBytes);
}

Comm* comm_create(int device, int rank, int world, const void* id128) {
    KN_CHECK(id128 != nullptr, KN_ERR_INVALID_ARG, "null id buffer");
    KN_CHECK(world >= 1 && rank >= 0 && rank < world, KN_ERR_INVALID_ARG, "rank outside the communicator");
    nccl_load(nullptr);
    int count = 0;
    cudaError_t err = cudaGetDeviceCount(&count);
    KN_CHECK(err == cudaSuccess && device >= 0 && device < count, KN_ERR_NO_DEVICE, "CUDA device " + std::to_string(device) + " not available");
    int prev = -1;
    cudaGetDevice(&prev);
    err = cudaSetDevice(device);
    KN_CHECK(err == cudaSuccess, KN_ERR_CUDA, std::string("cudaSetDevice failed: ") + cudaGetErrorString(err));
    NcclUniqueId id;
    memcpy(id.internal, id128, kCommIdBytes);
    void* nccl = nullptr;
    const int result = g_nccl.comm_init_rank(&nccl, world, id, rank);
    if (prev >= 0) cudaSetDevice(prev);
    check_nccl(result, "ncclCommInitRank");
    Comm* c = new Comm();
    c->nccl = nccl;
    c->rank = rank;
    c->world = world;
    c->device = device;
    return c;
}

void comm_destroy(Comm* comm) {
    if (!comm) return;
    if (comm->nccl && g_nccl.comm_destroy) {
        int prev = -1;
        cudaGetDevice(&prev);
        cudaSetDevice(comm->device);
        g_nccl.comm_destroy(comm->nccl);
        if (prev >= 0) cudaSetDevice(prev);
    }
    delete comm;
}

void comm_all_reduce_sum(Comm* comm, const void* in, void* out, size_t count, DType dtype, CUstream_st* stream) {
    KN_CHECK(comm != nullptr && comm->nccl != nullptr, KN_ERR_INVALID_ARG, "null communicator");
    KN_CHECK(dtype == DType::F32 || dtype == DType::F16, KN_ERR_UNSUPPORTED, "all-reduce of this dtype");
    check_nccl(g_nccl.all_reduce(in, out, count, dtype == DType::F32 ? kNcclFloat32 : kNcclFloat16, kNcclSum, comm->nccl, stream),
               "ncclAllReduce");
}

}  // namespace kn
