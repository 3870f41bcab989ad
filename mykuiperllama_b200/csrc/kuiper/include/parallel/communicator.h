// Tensor-parallel communicator: one NCCL communicator per process (one process per GPU),
// used for the single all-reduce that follows each row-split projection (O and down).
// The reference has no multi-GPU code at all; this is new to the engine.
//
// NCCL is loaded at run time (dlopen of libnccl.so.2) so that a single-GPU process has no
// link-time dependency on it.  The unique id is created on rank 0 and handed to the other
// ranks by the caller (torch.distributed, a file, ...).
#ifndef KUIPER_INCLUDE_PARALLEL_COMMUNICATOR_H
#define KUIPER_INCLUDE_PARALLEL_COMMUNICATOR_H

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>

#include "base/base.h"

namespace parallel {

constexpr size_t kUniqueIdBytes = 128;

class Communicator : public base::NoCopyable {
public:
    Communicator() = default;
    ~Communicator();

    // fills `out` (kUniqueIdBytes) with a fresh NCCL unique id
    static base::Status make_unique_id(void* out);

    base::Status init(const void* unique_id, int32_t rank, int32_t world_size);
    // Optional: exchange buffers for the one-shot all-reduce of small rows (<= max_count floats) over peer memory.
    // Each rank allocates its buffer, the CUDA IPC handles travel through an NCCL all-gather, and every rank maps
    // its peers' buffers.  If any rank cannot, all ranks keep using NCCL (the outcome is agreed with an all-reduce).
    base::Status enable_one_shot(size_t max_count);
    bool one_shot_enabled() const { return one_shot_; }
    // in-place sum over all ranks of `count` fp32 values through ncclAllReduce, enqueued on `stream`
    base::Status all_reduce_sum(float* data, size_t count, cudaStream_t stream) const;
    // does a row of `count` floats fit the low-latency exchange over peer memory?
    bool fits_one_shot(size_t count) const { return one_shot_ && count <= one_shot_max_count_; }
    // out = residual + sum over ranks of partial through the low-latency exchange (identical bits on every rank);
    // `partial` is zeroed afterwards (ready for the next accumulating projection).  Needs fits_one_shot(count).
    base::Status exchange_sum(float* partial, const float* residual, float* out, size_t count, cudaStream_t stream) const;
    // greedy ids over a vocabulary split across the ranks: logits_local [rows, v_local]; the same ids on every rank.
    // Through the low-latency exchange when it is enabled (rows <= 16), else an NCCL all-gather of the per-rank pairs
    // is not available and the caller gathers the logits instead (returns function_not_implement).
    base::Status exchange_argmax(const float* logits_local, int32_t* next, int32_t rows, int32_t v_local,
                                 cudaStream_t stream) const;
    // concatenation over ranks of `count` floats each: out [world][count]
    base::Status all_gather(const float* in, float* out, size_t count, cudaStream_t stream) const;
    // synchronous health check of the one-shot path: error if a bounded wait on a peer ever ran out (the result of
    // that exchange, and of everything computed from it, is void); clear = true resets the error word once reported
    base::Status one_shot_status(bool clear = false) const;

    int32_t rank() const { return rank_; }
    int32_t world_size() const { return world_size_; }
    bool ready() const { return comm_ != nullptr; }

private:
    void* comm_ = nullptr;  // ncclComm_t
    int32_t rank_ = 0;
    int32_t world_size_ = 1;
    // one-shot exchange
    bool one_shot_ = false;
    size_t one_shot_max_count_ = 0;
    void* exchange_ = nullptr;          // this rank's exchange buffer (cudaMalloc)
    uint32_t* state_ = nullptr;         // sequence number + error word
    void* rank_buffers_[8] = {};        // every rank's exchange buffer as mapped here
};

}  // namespace parallel

#endif  // KUIPER_INCLUDE_PARALLEL_COMMUNICATOR_H
