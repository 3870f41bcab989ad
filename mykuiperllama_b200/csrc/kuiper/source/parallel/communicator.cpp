// NCCL binding through dlopen; see parallel/communicator.h.
#include "parallel/communicator.h"

#include <dlfcn.h>

#include <cstring>
#include <mutex>
#include <vector>

#include "base/log.h"
#include "kuiper_b200.h"

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
    int (*AllGather)(const void* send, void* recv, size_t sendcount, int dtype, void* comm, cudaStream_t s) = nullptr;
    int (*CommDestroy)(void* comm) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    bool ok = false;
};

constexpr int kNcclFloat32 = 7;  // ncclFloat32 in nccl.h
constexpr int kNcclSum = 0;      // ncclSum
constexpr int kNcclMin = 3;      // ncclMin
constexpr int kNcclInt8 = 0;     // ncclInt8 / ncclChar

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
        a.AllGather = reinterpret_cast<decltype(a.AllGather)>(dlsym(h, "ncclAllGather"));
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
    for (int r = 0; r < world_size_ && r < 8; r++)
        if (rank_buffers_[r] && r != rank_) cudaIpcCloseMemHandle(rank_buffers_[r]);
    if (exchange_) cudaFree(exchange_);
    if (state_) cudaFree(state_);
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

base::Status Communicator::enable_one_shot(size_t max_count) {
    if (!comm_) return base::error::internal_error("communicator is not initialised");
    if (one_shot_) return base::error::success();
    if (world_size_ > 8 || !api().AllGather) return base::error::success();  // stays on NCCL
    max_count = (max_count + 31) / 32 * 32;
    if (max_count > 65536) return base::error::success();  // rows this long stay on NCCL
    const size_t bytes = kuiper_allreduce_buffer_bytes(world_size_, int64_t(max_count));
    // every step below is attempted on every rank; `good` is agreed at the end so that all ranks take the same path
    float good = 1.f;
    cudaIpcMemHandle_t mine;
    std::memset(&mine, 0, sizeof(mine));
    char* d_handles = nullptr;
    if (bytes == 0 || cudaMalloc(&exchange_, bytes) != cudaSuccess || cudaMemset(exchange_, 0, bytes) != cudaSuccess ||
        cudaMalloc(reinterpret_cast<void**>(&state_), kuiper_allreduce_state_bytes()) != cudaSuccess ||
        cudaMemset(state_, 0, kuiper_allreduce_state_bytes()) != cudaSuccess || cudaIpcGetMemHandle(&mine, exchange_) != cudaSuccess)
        good = 0.f;
    const size_t hb = sizeof(cudaIpcMemHandle_t);
    std::vector<cudaIpcMemHandle_t> all(static_cast<size_t>(world_size_));
    if (cudaMalloc(reinterpret_cast<void**>(&d_handles), hb * size_t(world_size_ + 1)) != cudaSuccess) {
        (void)cudaGetLastError();
        return base::error::internal_error("cannot allocate the handle exchange buffer");
    }
    cudaMemcpy(d_handles + hb * size_t(world_size_), &mine, hb, cudaMemcpyHostToDevice);
    base::Status st = nccl_status(api().AllGather(d_handles + hb * size_t(world_size_), d_handles, hb, kNcclInt8, comm_, nullptr),
                                  "ncclAllGather");
    if (st) {
        cudaDeviceSynchronize();
        cudaMemcpy(all.data(), d_handles, hb * size_t(world_size_), cudaMemcpyDeviceToHost);
        for (int r = 0; r < world_size_ && good > 0.f; r++) {
            if (r == rank_) {
                rank_buffers_[r] = exchange_;
            } else if (cudaIpcOpenMemHandle(&rank_buffers_[r], all[size_t(r)], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                rank_buffers_[r] = nullptr;
                good = 0.f;
            }
        }
        (void)cudaGetLastError();
        // agree: one rank without peer mappings keeps everybody on NCCL
        float* d_good = reinterpret_cast<float*>(d_handles);
        cudaMemcpy(d_good, &good, sizeof(float), cudaMemcpyHostToDevice);
        st = nccl_status(api().AllReduce(d_good, d_good, 1, kNcclFloat32, kNcclMin, comm_, nullptr), "ncclAllReduce");
        if (st) {
            cudaDeviceSynchronize();
            cudaMemcpy(&good, d_good, sizeof(float), cudaMemcpyDeviceToHost);
        }
    }
    cudaFree(d_handles);
    if (!st) return st;
    one_shot_ = good > 0.f;
    one_shot_max_count_ = max_count;
    if (!one_shot_) LOG(WARNING) << "one-shot all-reduce unavailable (no peer mapping on some rank): using NCCL";
    return base::error::success();
}

base::Status Communicator::one_shot_status(bool clear) const {
    if (!one_shot_) return base::error::success();
    // the error word is sticky on the device; once reported it is cleared so that the next call starts clean
    if (kuiper_allreduce_status(state_, clear ? 1 : 0) != 0) return base::error::internal_error(kuiper_last_error());
    return base::error::success();
}

base::Status Communicator::all_reduce_sum(float* data, size_t count, cudaStream_t stream) const {
    if (!comm_) return base::error::internal_error("communicator is not initialised");
    return nccl_status(api().AllReduce(data, data, count, kNcclFloat32, kNcclSum, comm_, stream), "ncclAllReduce");
}

base::Status Communicator::exchange_sum(float* partial, const float* residual, float* out, size_t count,
                                        cudaStream_t stream) const {
    if (!fits_one_shot(count)) return base::error::invalid_argument("row does not fit the low-latency exchange");
    if (kuiper_allreduce_sum_f32(partial, residual, out, 1, int64_t(count), rank_, world_size_, rank_buffers_,
                                 int64_t(one_shot_max_count_), state_, reinterpret_cast<kuiper_stream_t>(stream)) != 0)
        return base::error::internal_error(kuiper_last_error());
    return base::error::success();
}

base::Status Communicator::exchange_argmax(const float* logits_local, int32_t* next, int32_t rows, int32_t v_local,
                                           cudaStream_t stream) const {
    if (!one_shot_ || rows > 16) return base::error::function_not_implement("argmax exchange needs the peer-memory path and <= 16 rows");
    if (kuiper_argmax_allgather(logits_local, next, rows, v_local, rank_, world_size_, rank_buffers_,
                                int64_t(one_shot_max_count_), state_, reinterpret_cast<kuiper_stream_t>(stream)) != 0)
        return base::error::internal_error(kuiper_last_error());
    return base::error::success();
}

base::Status Communicator::all_gather(const float* in, float* out, size_t count, cudaStream_t stream) const {
    if (!comm_ || !api().AllGather) return base::error::internal_error("communicator is not initialised");
    return nccl_status(api().AllGather(in, out, count, kNcclFloat32, comm_, stream), "ncclAllGather");
}

}  // namespace parallel
