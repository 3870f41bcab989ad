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
    // in-place sum over all ranks of `count` fp32 values, enqueued on `stream`
    base::Status all_reduce_sum(float* data, size_t count, cudaStream_t stream) const;

    int32_t rank() const { return rank_; }
    int32_t world_size() const { return world_size_; }
    bool ready() const { return comm_ != nullptr; }

private:
    void* comm_ = nullptr;  // ncclComm_t
    int32_t rank_ = 0;
    int32_t world_size_ = 1;
};

}  // namespace parallel

#endif  // KUIPER_INCLUDE_PARALLEL_COMMUNICATOR_H
