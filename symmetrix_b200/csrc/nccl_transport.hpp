// NCCL point-to-point transport for halo rows, loaded at run time.
//
// The library does not link against NCCL: a process that exchanges halos has NCCL in memory already (through its MPI /
// LAMMPS build or through torch), and dlopen("libnccl.so.2") resolves to that copy; a process that never calls the
// exchange entry points needs no NCCL at all. Only the handful of entry points below are used. The declarations follow
// NCCL's public header (nccl.h: ncclGetUniqueId, ncclCommInitRank, ncclCommDestroy, ncclGroupStart / End, ncclSend,
// ncclRecv, ncclAllReduce); the enumerator values used are ncclFloat32 = 7, ncclFloat64 = 8, ncclSum = 0.
#pragma once

#include <cuda_runtime.h>
#include <dlfcn.h>

#include <string>

#include "common.cuh"

namespace smx {

struct NcclApi {
    using Comm = void*;
    struct UniqueId { char internal[128]; };
    int (*GetUniqueId)(UniqueId*) = nullptr;
    int (*CommInitRank)(Comm*, int, UniqueId, int) = nullptr;
    int (*CommDestroy)(Comm) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    int (*Send)(const void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
    int (*Recv)(void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    static constexpr int kFloat32 = 7, kFloat64 = 8, kSum = 0;

    // Loads the library once per process; throws CudaError when NCCL cannot be found.
    static const NcclApi& get() {
        static NcclApi api = load();
        return api;
    }
    void check(int rc, const char* what) const {
        if (rc != 0) throw CudaError(std::string(what) + ": " + (GetErrorString ? GetErrorString(rc) : "NCCL error"));
    }

private:
    static NcclApi load() {
        void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) throw CudaError("NCCL is not available in this process (dlopen of libnccl.so.2 failed)");
        NcclApi a;
        auto sym = [&](const char* name) {
            void* p = dlsym(lib, name);
            if (!p) throw CudaError(std::string("NCCL symbol missing: ") + name);
            return p;
        };
        a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(sym("ncclGetUniqueId"));
        a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(sym("ncclCommInitRank"));
        a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(sym("ncclCommDestroy"));
        a.GroupStart = reinterpret_cast<decltype(a.GroupStart)>(sym("ncclGroupStart"));
        a.GroupEnd = reinterpret_cast<decltype(a.GroupEnd)>(sym("ncclGroupEnd"));
        a.Send = reinterpret_cast<decltype(a.Send)>(sym("ncclSend"));
        a.Recv = reinterpret_cast<decltype(a.Recv)>(sym("ncclRecv"));
        a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(sym("ncclAllReduce"));
        a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(sym("ncclGetErrorString"));
        return a;
    }
};

}  // namespace smx
