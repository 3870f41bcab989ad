// Model base class: owns the execution context, the named step buffers and the
// forward / predict entry points.  The reference globs a kuiper/source/model directory
// that does not exist (CMakeLists.txt:79); what it does define are the buffer names
// (model::ModelBufferType, kuiper/include/base/base.h:12-31), the KeyValueHasExist status
// (base.h:82) for a keyed buffer table, and the operator classes a model strings together.
#ifndef KUIPER_INCLUDE_MODEL_MODEL_H
#define KUIPER_INCLUDE_MODEL_MODEL_H

#include <map>
#include <memory>
#include <vector>

#include "base/cuda_config.h"
#include "model/config.h"
#include "parallel/communicator.h"
#include "tensor/tensor.h"

namespace model {

class Model {
public:
    explicit Model(base::ModelType model_type, const ModelConfig& config);
    virtual ~Model() = default;

    // allocate buffers and build the layers on `device_type` (DeviceCUDA only)
    virtual base::Status init(base::DeviceType device_type) = 0;

    // One pass over M token rows given on the host: row m is token tokens[m] at position
    // pos[m] of KV-cache sequence slot[m].  Enqueues the pass and leaves the logits in
    // ForwardOutput and the greedy ids in NextTokens; does not synchronise.
    virtual base::Status forward(const int32_t* tokens, const int32_t* pos, const int32_t* slot, int32_t M) = 0;
    // forward + greedy sampling; `next` receives M ids on the host (synchronises)
    virtual base::Status predict(const int32_t* tokens, const int32_t* pos, const int32_t* slot, int32_t M,
                                 int32_t* next) = 0;

    base::Status insert_buffer(ModelBufferType buffer_idx, const tensor::Tensor& tensor);
    tensor::Tensor& get_buffer(ModelBufferType buffer_idx);
    const tensor::Tensor& get_buffer(ModelBufferType buffer_idx) const;

    base::ModelType model_type() const { return model_type_; }
    const ModelConfig& config() const { return config_; }
    std::shared_ptr<kernel::CudaConfig> cuda_config() const { return cuda_config_; }
    cudaStream_t stream() const { return cuda_config_ ? cuda_config_->stream() : nullptr; }

    // tensor parallelism: all ranks call this with the id made on rank 0
    base::Status init_tensor_parallel(const void* unique_id);

protected:
    base::ModelType model_type_;
    ModelConfig config_;
    base::DeviceType device_type_ = base::DeviceType::DeviceUnknown;
    std::shared_ptr<kernel::CudaConfig> cuda_config_;
    std::unique_ptr<parallel::Communicator> communicator_;

public:
    const parallel::Communicator* communicator() const { return communicator_.get(); }

protected:
    std::map<ModelBufferType, tensor::Tensor> buffers_;
};

}  // namespace model

#endif  // KUIPER_INCLUDE_MODEL_MODEL_H
