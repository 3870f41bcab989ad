// EmbeddingLayer: bf16 table gather into fp32 rows.
#include "op/embedding.h"

#include "kernel/kernel_interface.h"

namespace op {

EmbeddingLayer::EmbeddingLayer(base::DeviceType device_type, int32_t dim, int32_t vocab_size)
    : LayerParam(device_type, LayerType::LayerEmbedding, false, "Embedding"), dim_(dim), vocab_size_(vocab_size) {
    reset_input_size(1);
    reset_output_size(1);
    reset_weights_size(1);
}

base::DataType EmbeddingLayer::weight_data_type(int32_t) const { return base::DataType::DataTypeBf16; }

base::Status EmbeddingLayer::check() const {
    base::Status status = check_tensor(get_input(0), device_type_, base::DataType::DataTypeInt32);
    if (!status) {
        LOG(ERROR) << "The token tensor error in the embedding layer.";
        return status;
    }
    status = check_tensor_with_dim(get_weight(0), device_type_, base::DataType::DataTypeBf16, vocab_size_, dim_);
    if (!status) return status;
    status = check_tensor(get_output(0), device_type_, data_type_);
    if (status && (get_output(0).size() % size_t(dim_) != 0 || get_output(0).size() / size_t(dim_) > get_input(0).size()))
        status = base::error::invalid_argument("The output tensor has a wrong shape.");
    return status;
}

base::Status EmbeddingLayer::forward() {
    base::Status status = check();
    if (!status) return status;
    kernel::get_emb_kernel(device_type_)(get_input(0), get_weight(0), get_output(0), vocab_size_, stream());
    return base::error::success();
}

}  // namespace op
