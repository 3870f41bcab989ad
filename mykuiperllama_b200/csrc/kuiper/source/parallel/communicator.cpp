// NCCL binding through dlopen; see parallel/communicator.h.
#include "parallel/communicator.h"

#include <dlfcn.h>

#include <cstring>
#include <mutex>

namespace parallel {
namespace {

// the handful of NCCL entry points the engine uses, with their public C signatures
struct IdByValue {
    char b[kUniqueIdBytes];  // ncclUniqueId is an opaque 128-byte struct passed by value
};

struct NcclApi {
    int (*GetUniqueId)(void* id) = nullptr;
    int (*CommInitRank)(void** comm, int nranks, IdByValue id, int rank) = nullptr;
    int (*AllReduce)(const void* send, void* recv, size_t count, int dtype, int op, void* comm, cudaStream_t s) = nullptr;
    int (*CommDestroy)(void* comm) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    bool ok = false;
};

constexpr int kNcclFloat32 = 7;  // ncclFloat32 in nccl.h
constexpr int kNcclSum = 0;      // ncclSum

NcclApi& api() {
    static NcclApi a;
    static std::once_flag once;
    std::call_once(once, [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return;
        a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
        a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
        a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(dlsym(h, "ncclAllReduce"));
        a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
        a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
        a.ok = a.GetUniqueId && a.CommInitRank && a.AllReduce && a.CommDestroy && a.GetErrorString;
    });
    return a;
}

base::Status nccl_status(int rc, const char* what) {
    if (rc == 0) return base::error::success();
    return base::error::internal_error(std::string(what) + ": " + api().GetErrorString(rc));
}

}  // namespace

Communicator::~Communicator() {
    if (comm_ && api().ok) api().CommDestroy(comm_);
}

base::Status Communicator::make_unique_id(void* out) {
    if (!api().ok) return base::error::internal_error("NCCL library (libnccl.so.2) could not be loaded");
    return nccl_status(api().GetUniqueId(out), "ncclGetUniqueId");
}

base::Status Communicator::init(const void* unique_id, int32_t rank, int32_t world_size) {
    if (!api().ok) return base::error::internal_error("NCCL library (libnccl.so.2) could not be loaded");
    if (!unique_id || world_size < 1 || rank < 0 || rank >= world_size)
        return base::error::invalid_argument("bad tensor-parallel rank / world size");
    if (comm_) return base::error::key_has_exits("communicator already initialised");
    IdByValue id;
    std::memcpy(id.b, unique_id, sizeof(id.b));
    base::Status st = nccl_status(api().CommInitRank(&comm_, world_size, id, rank), "ncclCommInitRank");
    if (!st) {
        comm_ = nullptr;
        return st;
    }
    rank_ = rank;
    world_size_ = world_size;
    return st;
}

base::Status Communicator::all_reduce_sum(float* data, size_t count, cudaStream_t stream) const {
    if (!comm_) return base::error::internal_error("communicator is not initialised");
    return nccl_status(api().AllReduce(data, data, count, kNcclFloat32, kNcclSum, comm_, stream), "ncclAllReduce");
}

}  // namespace parallel
