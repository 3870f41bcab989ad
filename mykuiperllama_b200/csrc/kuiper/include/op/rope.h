// Per-head q/k RMSNorm, half-split rotary embedding and KV-cache append in one layer.
// Placeholder in the reference: kuiper/include/op/rope.h:1-10, tag LayerRope (op/layer.h:15).
//
// inputs : 0 qkv [M, (Nq+2Nkv)*D] Fp32, 1 pos [M] Int32, 2 slot [M] Int32,
//          3 cos [max_seq, D/2] Fp32, 4 sin [max_seq, D/2] Fp32
// output : 0 q [M, Nq*D] Fp32
// weights: 0 q_norm Bf16 [D], 1 k_norm Bf16 [D]
// caches : set_cache(k, v): Bf16 [n_slots, Nkv, max_seq, D] for this layer
#ifndef KUIPER_INCLUDE_OP_ROPE_H
#define KUIPER_INCLUDE_OP_ROPE_H

#include "op/layer.h"

namespace op {
class RoPELayer : public LayerParam {
public:
    explicit RoPELayer(base::DeviceType device_type, int32_t head_num, int32_t kv_head_num, int32_t head_size,
                       float eps = 1e-6f);
    base::Status check() const override;
    using Layer::forward;  // keep the N-ary overloads visible next to the override
    base::Status forward() override;
    void set_cache(const tensor::Tensor& key_cache, const tensor::Tensor& value_cache);
    // zero the qkv input after reading it (it then serves as the addend of an accumulating matmul)
    void set_clear_input(bool clear) { clear_input_ = clear; }
    // another Fp32 buffer the kernel zeroes on the side (an empty tensor switches it off); the model passes the
    // gate|up projection output, which is idle while this layer runs
    // row_elems: floats per token row; the kernel clears as many rows as the pass has
    void set_clear_extra(const tensor::Tensor& buffer, int32_t row_elems) {
        clear_extra_ = buffer;
        clear_extra_row_ = row_elems;
    }

    // Decode batches only (one token row per sequence slot, seq_len == pos + 1): rotary, KV append and
    // flash-decoding in one kernel.  Inputs as for forward() plus seq_len; attention_out [M, Nq*D] replaces the q
    // output; workspace as for op::MultiHeadAttention; fresh_rows as documented there.
    void set_attention_workspace(const tensor::Tensor& workspace) { attention_workspace_ = workspace; }
    base::Status forward_with_attention(const tensor::Tensor& qkv, const tensor::Tensor& pos, const tensor::Tensor& slot,
                                        const tensor::Tensor& cos_cache, const tensor::Tensor& sin_cache,
                                        const tensor::Tensor& seq_len, const tensor::Tensor& attention_out,
                                        int32_t fresh_rows);

protected:
    base::DataType weight_data_type(int32_t idx) const override;

private:
    int32_t head_num_ = 0, kv_head_num_ = 0, head_size_ = 0;
    float eps_ = 1e-6f;
    bool clear_input_ = false;
    tensor::Tensor key_cache_, value_cache_, clear_extra_, attention_workspace_;
    int32_t clear_extra_row_ = 0;
};
}  // namespace op

#endif  // KUIPER_INCLUDE_OP_ROPE_H
