// NCCL, found at run time: the collectives of the tensor-parallel and expert-parallel entry points go through
// libnccl.so.2, opened with dlopen on the first b2_comm_* call, the way the host program opens this library and the way
// the reference opens the CUDA driver (src/cuda.rs:31-96). Nothing is linked at build time and a machine without NCCL
// still loads the library (the b2_comm_* calls then decline). Only the handful of entry points used here are declared,
// with the argument types of NCCL's public header.
#pragma once
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <mutex>

namespace b2 {

struct NcclId {
    char internal[128];  // NCCL_UNIQUE_ID_BYTES
};
typedef void* NcclComm;
enum { NCCL_UINT8 = 1, NCCL_INT32 = 2, NCCL_FLOAT32 = 7 };

struct NcclApi {
    int (*GetUniqueId)(NcclId*) = nullptr;
    int (*CommInitRank)(NcclComm*, int, NcclId, int) = nullptr;
    int (*CommDestroy)(NcclComm) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t) = nullptr;
    int (*Send)(const void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*Recv)(void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    bool ok = false;
};

// The table, loaded once per process; ok == false when libnccl.so.2 (or one of the symbols) is missing.
inline const NcclApi& nccl_api() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return;
        bool all = true;
        auto sym = [&](const char* name) {
            void* p = dlsym(h, name);
            if (!p) all = false;
            return p;
        };
        api.GetUniqueId = (int (*)(NcclId*))sym("ncclGetUniqueId");
        api.CommInitRank = (int (*)(NcclComm*, int, NcclId, int))sym("ncclCommInitRank");
        api.CommDestroy = (int (*)(NcclComm))sym("ncclCommDestroy");
        api.AllGather = (int (*)(const void*, void*, size_t, int, NcclComm, cudaStream_t))sym("ncclAllGather");
        api.Send = (int (*)(const void*, size_t, int, int, NcclComm, cudaStream_t))sym("ncclSend");
        api.Recv = (int (*)(void*, size_t, int, int, NcclComm, cudaStream_t))sym("ncclRecv");
        api.GroupStart = (int (*)())sym("ncclGroupStart");
        api.GroupEnd = (int (*)())sym("ncclGroupEnd");
        api.GetErrorString = (const char* (*)(int))sym("ncclGetErrorString");
        api.ok = all;
    });
    return api;
}

}  // namespace b2
