// Model base: buffer table and tensor-parallel set-up.
#include "model/model.h"

#include <cstdlib>

namespace model {

Model::Model(base::ModelType model_type, const ModelConfig& config) : model_type_(model_type), config_(config) {}

base::Status Model::insert_buffer(ModelBufferType buffer_idx, const tensor::Tensor& tensor) {
    if (buffers_.count(buffer_idx) > 0)
        return base::error::key_has_exits(std::to_string(int(buffer_idx)) + " has exits in the buffers");
    if (tensor.is_empty()) return base::error::invalid_argument("The tensor is empty for inserting buffer.");
    buffers_.emplace(buffer_idx, tensor);
    return base::error::success();
}

tensor::Tensor& Model::get_buffer(ModelBufferType buffer_idx) {
    auto it = buffers_.find(buffer_idx);
    CHECK(it != buffers_.end()) << "no buffer with key " << int(buffer_idx);
    return it->second;
}

const tensor::Tensor& Model::get_buffer(ModelBufferType buffer_idx) const {
    auto it = buffers_.find(buffer_idx);
    CHECK(it != buffers_.end()) << "no buffer with key " << int(buffer_idx);
    return it->second;
}

base::Status Model::init_tensor_parallel(const void* unique_id) {
    if (config_.tp_size <= 1) return base::error::success();
    if (!cuda_config_) return base::error::internal_error("init() must run before init_tensor_parallel()");
    communicator_ = std::make_unique<parallel::Communicator>();
    base::Status st = communicator_->init(unique_id, config_.tp_rank, config_.tp_size);
    if (!st) {
        communicator_.reset();
        return st;
    }
    cuda_config_->set_communicator(communicator_.get());
    // decode rows (up to 8 of them) are summed by the one-shot exchange over peer memory (it falls back to NCCL
    // by agreement of all ranks when peer mapping is unavailable); KUIPER_TP_ONESHOT=0 keeps everything on ncclAllReduce
    const char* env = std::getenv("KUIPER_TP_ONESHOT");
    if (!(env && env[0] == '0')) {
        const int32_t rows = config_.max_batch < 8 ? config_.max_batch : 8;
        st = communicator_->enable_one_shot(size_t(rows) * size_t(config_.dim));
    }
    return st;
}

}  // namespace model
