// Stream holder (interface: kuiper/include/base/cuda_config.h:17-30 of the reference).
#include "base/cuda_config.h"

namespace kernel {

CudaConfig::~CudaConfig() {
    if (!stream_) return;
    cudaError_t err = cudaStreamDestroy(stream_);
    if (err != cudaSuccess) LOG(ERROR) << "Failed to destroy CUDA stream: " << cudaGetErrorString(err);
}

void CudaConfig::create() {
    CHECK(stream_ == nullptr) << "CudaConfig already holds a stream";
    cudaError_t err = cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking);
    CHECK_EQ(int(err), int(cudaSuccess)) << "Failed to create CUDA stream: " << cudaGetErrorString(err);
}

cudaStream_t CudaConfig::stream() const { return stream_; }
void CudaConfig::set_stream(cudaStream_t stream) { stream_ = stream; }

}  // namespace kernel
