// Per-model CUDA execution context.  The reference's kernel::CudaConfig
// (kuiper/include/base/cuda_config.h:17-30) is an RAII holder of one stream; this one
// additionally carries the tensor-parallel communicator handle the row-split layers
// reduce over (null on a single GPU).
#ifndef KUIPER_INCLUDE_BASE_CUDA_CONFIG_H
#define KUIPER_INCLUDE_BASE_CUDA_CONFIG_H

#include <cuda_runtime_api.h>

#include "base/base.h"

namespace kernel {

class CudaConfig : public base::NoCopyable {
public:
    explicit CudaConfig() : stream_(nullptr) {}
    explicit CudaConfig(cudaStream_t stream) : stream_(stream) {}
    ~CudaConfig();  // destroys the stream it holds
    void create();  // makes a new stream; the holder must be empty
    cudaStream_t stream() const;
    void set_stream(cudaStream_t stream);

    // opaque tensor-parallel communicator (parallel::Communicator*), not owned
    void* communicator() const { return communicator_; }
    void set_communicator(void* comm) { communicator_ = comm; }

private:
    cudaStream_t stream_ = nullptr;
    void* communicator_ = nullptr;
};

}  // namespace kernel

#endif  // KUIPER_INCLUDE_BASE_CUDA_CONFIG_H
