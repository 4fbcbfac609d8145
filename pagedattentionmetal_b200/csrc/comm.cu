// All-gather of per-head attention outputs over the GPUs that share a cache sharded by KV
// head (no counterpart in the reference, which is single-device: PagedAttentionEngine.swift:249,
// PagedAttentionCABI.swift:104).  GPU r of N owns query heads [r * H/N, (r+1) * H/N); no
// collective runs on the attention path, this is only for a caller that needs the whole
// [rows][H][dim] tensor on every GPU.
//
// ncclAllGather over NVLink into [N][rows][H/N][dim], then one kernel that interleaves the
// slices into [rows][H][dim].  NCCL is looked up at run time (dlopen), so a single-GPU user
// of the library needs no NCCL; inside a process that has already loaded NCCL (PyTorch)
// that same copy is used.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <cstdint>
#include <mutex>
#include <string>

#include "kernels.h"

namespace pam {
namespace {

struct NcclApi {
    decltype(&ncclGetUniqueId) getUniqueId = nullptr;
    decltype(&ncclCommInitRank) commInitRank = nullptr;
    decltype(&ncclCommDestroy) commDestroy = nullptr;
    decltype(&ncclAllGather) allGather = nullptr;
    decltype(&ncclGetErrorString) getErrorString = nullptr;
    bool ok = false;
};

const NcclApi& nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return;
        api.getUniqueId = reinterpret_cast<decltype(api.getUniqueId)>(dlsym(h, "ncclGetUniqueId"));
        api.commInitRank = reinterpret_cast<decltype(api.commInitRank)>(dlsym(h, "ncclCommInitRank"));
        api.commDestroy = reinterpret_cast<decltype(api.commDestroy)>(dlsym(h, "ncclCommDestroy"));
        api.allGather = reinterpret_cast<decltype(api.allGather)>(dlsym(h, "ncclAllGather"));
        api.getErrorString = reinterpret_cast<decltype(api.getErrorString)>(dlsym(h, "ncclGetErrorString"));
        api.ok = api.getUniqueId && api.commInitRank && api.commDestroy && api.allGather && api.getErrorString;
    });
    return api;
}

// staging [n][rows][slice] -> full [rows][n][slice], 16-byte vectors.
__global__ void interleaveSlicesKernel(const uint4* __restrict__ staging, uint4* __restrict__ full, int n, int rows,
                                       int sliceVecs) {
    const int64_t total = static_cast<int64_t>(n) * rows * sliceVecs;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int v = static_cast<int>(i % sliceVecs);
        const int64_t t = i / sliceVecs;
        const int r = static_cast<int>(t % n);           // output order: row, rank, vector
        const int64_t row = t / n;
        full[i] = staging[(static_cast<int64_t>(r) * rows + row) * sliceVecs + v];
    }
}

}  // namespace

struct HeadComm {
    ncclComm_t comm = nullptr;
    int rank = 0, size = 1, device = 0;
};

bool commAvailable() { return nccl().ok; }

int commUniqueId(void* out128) {
    if (!nccl().ok || !out128) return -1;
    static_assert(sizeof(ncclUniqueId) == 128, "the id travels as 128 bytes");
    ncclUniqueId id;
    if (nccl().getUniqueId(&id) != ncclSuccess) return -1;
    memcpy(out128, &id, sizeof(id));
    return 0;
}

HeadComm* commCreate(const void* id128, int rank, int size, int device, std::string* error) {
    if (!nccl().ok) { if (error) *error = "NCCL could not be loaded (libnccl.so.2)"; return nullptr; }
    if (!id128 || size < 1 || rank < 0 || rank >= size) { if (error) *error = "bad rank or communicator size"; return nullptr; }
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    HeadComm* c = new HeadComm();
    c->rank = rank; c->size = size; c->device = device;
    ncclResult_t r = nccl().commInitRank(&c->comm, size, id, rank);
    if (r != ncclSuccess) {
        if (error) *error = std::string("ncclCommInitRank: ") + nccl().getErrorString(r);
        delete c;
        return nullptr;
    }
    return c;
}

void commDestroy(HeadComm* c) {
    if (!c) return;
    if (c->comm) nccl().commDestroy(c->comm);
    delete c;
}

int commRank(const HeadComm* c) { return c ? c->rank : -1; }
int commSize(const HeadComm* c) { return c ? c->size : -1; }

cudaError_t launchAllGatherHeads(HeadComm* c, const void* local, void* staging, void* full, int rows, size_t sliceBytes,
                                 cudaStream_t stream, int* launches, std::string* error) {
    if (!c || rows <= 0 || sliceBytes == 0) return cudaErrorInvalidValue;
    if (sliceBytes % 16 != 0 || (reinterpret_cast<uintptr_t>(full) & 15) || (reinterpret_cast<uintptr_t>(staging) & 15))
        return cudaErrorMisalignedAddress;
    const size_t count = static_cast<size_t>(rows) * sliceBytes;
    // one rank: the slice is the whole tensor
    if (c->size == 1) return cudaMemcpyAsync(full, local, count, cudaMemcpyDeviceToDevice, stream);
    ncclResult_t r = nccl().allGather(local, staging, count, ncclInt8, c->comm, stream);
    if (r != ncclSuccess) {
        if (error) *error = std::string("ncclAllGather: ") + nccl().getErrorString(r);
        return cudaErrorUnknown;
    }
    const int sliceVecs = static_cast<int>(sliceBytes / 16);
    const int64_t total = static_cast<int64_t>(c->size) * rows * sliceVecs;
    int blocks = static_cast<int>((total + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    interleaveSlicesKernel<<<blocks, 256, 0, stream>>>(static_cast<const uint4*>(staging), static_cast<uint4*>(full), c->size, rows,
                                                       sliceVecs);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

}  // namespace pam
