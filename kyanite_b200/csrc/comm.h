// The communicator behind AllReduce steps: NCCL, bound at run time.
//
// The library does not link against NCCL (hosts that never run a tensor-parallel graph need none): the first
// call that needs it opens `libnccl.so.2` with dlopen (the copy already loaded into the process, if any; else the
// path given to kn_nccl_load; else the loader's search path) and resolves the five public entry points it uses.
// One communicator per process and device, created from an id that rank 0 makes and the host distributes.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>

#include "common.h"

struct CUstream_st;

namespace kn {

struct Comm {
    void* nccl = nullptr;   // ncclComm_t
    int rank = 0, world = 1, device = 0;
};

constexpr size_t kCommIdBytes = 128;   // sizeof(ncclUniqueId)

// Opens the NCCL library (idempotent).  `path` may be null.  Throws kn::Error (KN_ERR_UNSUPPORTED) if it cannot be found.
void nccl_load(const char* path);
void comm_unique_id(void* id128);
Comm* comm_create(int device, int rank, int world, const void* id128);
void comm_destroy(Comm* comm);
// Enqueues out = sum over ranks of in on `stream`.  Throws on an NCCL error.
void comm_all_reduce_sum(Comm* comm, const void* in, void* out, size_t count, DType dtype, CUstream_st* stream);

}  // namespace kn
