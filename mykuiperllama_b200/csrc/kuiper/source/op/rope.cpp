// RoPELayer: per-head q/k RMSNorm + rotary + KV-cache append.
#include "op/rope.h"

#include "kernel/kernel_interface.h"

namespace op {

RoPELayer::RoPELayer(base::DeviceType device_type, int32_t head_num, int32_t kv_head_num, int32_t head_size, float eps)
    : LayerParam(device_type, LayerType::LayerRope, false, "RoPE"),
      head_num_(head_num), kv_head_num_(kv_head_num), head_size_(head_size), eps_(eps) {
    reset_input_size(5);
    reset_output_size(1);
    reset_weights_size(2);
}

base::DataType RoPELayer::weight_data_type(int32_t) const { return base::DataType::DataTypeBf16; }

void RoPELayer::set_cache(const tensor::Tensor& key_cache, const tensor::Tensor& value_cache) {
    key_cache_ = key_cache;
    value_cache_ = value_cache;
}

base::Status RoPELayer::check() const {
    const int32_t row = (head_num_ + 2 * kv_head_num_) * head_size_;
    base::Status status = check_tensor(get_input(0), device_type_, data_type_);
    if (status && get_input(0).size() % size_t(row) != 0)
        status = base::error::invalid_argument("The qkv tensor has a wrong width.");
    if (!status) {
        LOG(ERROR) << "The qkv tensor error in the rope layer.";
        return status;
    }
    const size_t M = get_input(0).size() / size_t(row);
    for (int i = 1; i <= 2; i++) {
        status = check_tensor(get_input(i), device_type_, base::DataType::DataTypeInt32);
        if (status && get_input(i).size() < M) status = base::error::invalid_argument("pos / slot tensor is too short.");
        if (!status) return status;
    }
    for (int i = 3; i <= 4; i++) {
        status = check_tensor(get_input(i), device_type_, data_type_);
        if (!status) return status;
    }
    status = check_tensor(get_output(0), device_type_, data_type_);
    if (status && get_output(0).size() != M * size_t(head_num_) * size_t(head_size_))
        status = base::error::invalid_argument("The query output has a wrong element count.");
    if (!status) return status;
    for (int i = 0; i < 2; i++) {
        status = check_tensor_with_dim(get_weight(i), device_type_, base::DataType::DataTypeBf16, head_size_);
        if (!status) return status;
    }
    for (const tensor::Tensor* c : {&key_cache_, &value_cache_}) {
        status = check_tensor(*c, device_type_, base::DataType::DataTypeBf16);
        if (status && (c->dims_size() != 4 || c->get_dim(1) != kv_head_num_ || c->get_dim(3) != head_size_))
            status = base::error::invalid_argument("The KV cache has a wrong shape.");
        if (!status) return status;
    }
    return base::error::success();
}

base::Status RoPELayer::forward() {
    base::Status status = check();
    if (!status) return status;
    tensor::Tensor extra;
    if (!clear_extra_.is_empty() && clear_extra_row_ > 0) {
        const int32_t row = (head_num_ + 2 * kv_head_num_) * head_size_;
        const int32_t M = int32_t(get_input(0).size() / size_t(row));
        if (size_t(M) * size_t(clear_extra_row_) > clear_extra_.size())
            return base::error::invalid_argument("the extra buffer is smaller than the pass");
        extra = tensor::Tensor(base::DataType::DataTypeFp32, std::vector<int32_t>{M, clear_extra_row_}, false, nullptr,
                               const_cast<float*>(clear_extra_.ptr<float>()));
        extra.set_device_type(device_type_);
    }
    kernel::get_rope_kernel(device_type_)(get_input(0), get_weight(0), get_weight(1), get_input(3), get_input(4),
                                          get_input(1), get_input(2), get_output(0), key_cache_, value_cache_, head_num_,
                                          kv_head_num_, head_size_, eps_, clear_input_,
                                          extra.is_empty() ? nullptr : &extra, stream());
    return base::error::success();
}

base::Status RoPELayer::forward_with_attention(const tensor::Tensor& qkv, const tensor::Tensor& pos,
                                               const tensor::Tensor& slot, const tensor::Tensor& cos_cache,
                                               const tensor::Tensor& sin_cache, const tensor::Tensor& seq_len,
                                               const tensor::Tensor& attention_out, int32_t fresh_rows) {
    set_input(0, qkv);
    set_input(1, pos);
    set_input(2, slot);
    set_input(3, cos_cache);
    set_input(4, sin_cache);
    set_output(0, attention_out);  // same shape as the q output of the plain layer
    base::Status status = check();
    if (!status) return status;
    const int32_t row = (head_num_ + 2 * kv_head_num_) * head_size_;
    const int32_t M = int32_t(qkv.size() / size_t(row));
    status = check_tensor(seq_len, device_type_, base::DataType::DataTypeInt32);
    if (status && seq_len.size() < size_t(M)) status = base::error::invalid_argument("seq_len tensor is too short.");
    if (!status) return status;
    tensor::Tensor extra;
    if (!clear_extra_.is_empty() && clear_extra_row_ > 0) {
        if (size_t(M) * size_t(clear_extra_row_) > clear_extra_.size())
            return base::error::invalid_argument("the extra buffer is smaller than the pass");
        extra = tensor::Tensor(base::DataType::DataTypeFp32, std::vector<int32_t>{M, clear_extra_row_}, false, nullptr,
                               const_cast<float*>(clear_extra_.ptr<float>()));
        extra.set_device_type(device_type_);
    }
    kernel::get_rope_mha_kernel(device_type_)(qkv, get_weight(0), get_weight(1), cos_cache, sin_cache, pos, seq_len, slot,
                                              attention_out, key_cache_, value_cache_, head_num_, kv_head_num_, head_size_,
                                              eps_, fresh_rows, clear_input_, extra.is_empty() ? nullptr : &extra,
                                              attention_workspace_, stream());
    return base::error::success();
}

}  // namespace op
