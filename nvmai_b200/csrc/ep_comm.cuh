// NCCL, resolved at run time: the library links nothing but the CUDA runtime, and a
// process that never shards experts never loads NCCL.  Only the handful of entry
// points the expert-parallel step uses are bound, by the names and signatures of
// NCCL's public header (nccl.h, 2.x); the few types and constants needed are
// restated here so that building does not need that header.
#pragma once

#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstddef>
#include <cstdlib>

namespace nvmai {

struct NcclUniqueId { char internal[128]; };       // ncclUniqueId, NCCL_UNIQUE_ID_BYTES = 128
typedef struct ncclComm *NcclComm;                 // ncclComm_t
constexpr int kNcclSuccess = 0;                    // ncclSuccess
constexpr int kNcclInProgress = 7;                 // ncclInProgress (a non-blocking communicator still at work)
constexpr int kNcclFloat16 = 6, kNcclFloat32 = 7;  // ncclDataType_t

struct NcclApi {
    void *lib = nullptr;
    int (*GetUniqueId)(NcclUniqueId *) = nullptr;
    int (*CommInitRank)(NcclComm *, int, NcclUniqueId, int) = nullptr;
    int (*CommDestroy)(NcclComm) = nullptr;
    int (*CommAbort)(NcclComm) = nullptr;
    int (*CommGetAsyncError)(NcclComm, int *) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, NcclComm, cudaStream_t) = nullptr;
    int (*Send)(const void *, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*Recv)(void *, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    bool ok = false;
};

// A process that already holds NCCL (a torch process, say) gets that copy back:
// dlopen by soname returns the loaded object.
inline const NcclApi &nccl_api() {
    static NcclApi api = [] {
        NcclApi a;
        // NVMAI_CUDA_NCCL_LIB names the library to load (a specific build, or a test double); default: the soname
        const char *named = std::getenv("NVMAI_CUDA_NCCL_LIB");
        if (named && *named) a.lib = dlopen(named, RTLD_NOW | RTLD_LOCAL);
        else {
            a.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
            if (!a.lib) a.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        }
        if (!a.lib) return a;
        auto sym = [&](const char *name) { return dlsym(a.lib, name); };
        a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(sym("ncclGetUniqueId"));
        a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(sym("ncclCommInitRank"));
        a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(sym("ncclCommDestroy"));
        a.CommAbort = reinterpret_cast<decltype(a.CommAbort)>(sym("ncclCommAbort"));
        a.CommGetAsyncError = reinterpret_cast<decltype(a.CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
        a.AllGather = reinterpret_cast<decltype(a.AllGather)>(sym("ncclAllGather"));
        a.Send = reinterpret_cast<decltype(a.Send)>(sym("ncclSend"));
        a.Recv = reinterpret_cast<decltype(a.Recv)>(sym("ncclRecv"));
        a.GroupStart = reinterpret_cast<decltype(a.GroupStart)>(sym("ncclGroupStart"));
        a.GroupEnd = reinterpret_cast<decltype(a.GroupEnd)>(sym("ncclGroupEnd"));
        a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.CommAbort && a.CommGetAsyncError && a.AllGather && a.Send &&
               a.Recv && a.GroupStart && a.GroupEnd;
        return a;
    }();
    return api;
}

}  // namespace nvmai
