// MultiHeadAttention: GQA flash-decoding over the KV cache.
#include "op/mha.h"

#include "kernel/kernel_interface.h"

namespace op {

MultiHeadAttention::MultiHeadAttention(base::DeviceType device_type, int32_t head_num, int32_t kv_head_num,
                                       int32_t head_size)
    : Layer(device_type, LayerType::LayerMHA, "MultiHead"),
      head_num_(head_num), kv_head_num_(kv_head_num), head_size_(head_size) {
    reset_input_size(3);
    reset_output_size(1);
}

void MultiHeadAttention::set_cache(const tensor::Tensor& key_cache, const tensor::Tensor& value_cache) {
    key_cache_ = key_cache;
    value_cache_ = value_cache;
}

void MultiHeadAttention::set_workspace(const tensor::Tensor& workspace) { workspace_ = workspace; }

base::Status MultiHeadAttention::check() const {
    const int32_t row = head_num_ * head_size_;
    base::Status status = check_tensor(get_input(0), device_type_, data_type_);
    if (status && get_input(0).size() % size_t(row) != 0)
        status = base::error::invalid_argument("The query tensor has a wrong width.");
    if (!status) {
        LOG(ERROR) << "The query tensor error in the mha layer.";
        return status;
    }
    const size_t M = get_input(0).size() / size_t(row);
    for (int i = 1; i <= 2; i++) {
        status = check_tensor(get_input(i), device_type_, base::DataType::DataTypeInt32);
        if (status && get_input(i).size() < M) status = base::error::invalid_argument("seq_len / slot tensor is too short.");
        if (!status) return status;
    }
    status = check_tensor(get_output(0), device_type_, data_type_);
    if (status && get_output(0).size() != get_input(0).size())
        status = base::error::invalid_argument("The output tensor has a wrong element count.");
    if (!status) return status;
    for (const tensor::Tensor* c : {&key_cache_, &value_cache_}) {
        status = check_tensor(*c, device_type_, base::DataType::DataTypeBf16);
        if (status && (c->dims_size() != 4 || c->get_dim(1) != kv_head_num_ || c->get_dim(3) != head_size_))
            status = base::error::invalid_argument("The KV cache has a wrong shape.");
        if (!status) return status;
    }
    return base::error::success();
}

base::Status MultiHeadAttention::forward() {
    base::Status status = check();
    if (!status) return status;
    kernel::get_mha_kernel(device_type_)(get_input(0), key_cache_, value_cache_, get_input(1), get_input(2),
                                         get_output(0), head_num_, kv_head_num_, head_size_, fresh_rows_, workspace_,
                                         stream());
    return base::error::success();
}

base::Status MultiHeadAttention::forward_prefill(const tensor::Tensor& query, int32_t pos0, int32_t slot,
                                                 const tensor::Tensor& output) {
    base::Status status = check_tensor(query, device_type_, data_type_);
    const int32_t row = head_num_ * head_size_;
    if (status && (query.size() % size_t(row) != 0 || output.size() != query.size()))
        status = base::error::invalid_argument("The query / output tensors of the prefill attention have a wrong size.");
    if (!status) return status;
    status = check_tensor(output, device_type_, data_type_);
    if (!status) return status;
    const int32_t M = int32_t(query.size() / size_t(row));
    if (key_cache_.is_empty() || value_cache_.is_empty() || key_cache_.dims_size() != 4)
        return base::error::invalid_argument("The KV cache is not set.");
    if (slot < 0 || slot >= key_cache_.get_dim(0) || pos0 < 0 || pos0 + M > key_cache_.get_dim(2))
        return base::error::invalid_argument("The prompt chunk does not fit the KV cache.");
    kernel::get_mha_prefill_kernel(device_type_)(query, key_cache_, value_cache_, output, head_num_, kv_head_num_, head_size_,
                                                 pos0, slot, stream());
    return base::error::success();
}

}  // namespace op
