// Grouped-query attention over the KV cache (flash-decoding: split KV + log-sum-exp
// combine).  Placeholder in the reference: kuiper/include/op/mha.h:1-11, tag LayerMHA
// (op/layer.h:16).
//
// inputs : 0 q [M, Nq*D] Fp32, 1 seq_len [M] Int32 (row m attends to positions
//          [0, seq_len[m])), 2 slot [M] Int32
// output : 0 [M, Nq*D] Fp32
// caches : set_cache(k, v): Bf16 [n_slots, Nkv, max_seq, D]; set_workspace(): scratch of
//          kernel::mha_workspace_bytes(...) bytes, zero-initialised once
#ifndef KUIPER_INCLUDE_OP_MHA_H
#define KUIPER_INCLUDE_OP_MHA_H

#include "base/cuda_config.h"
#include "op/layer.h"

namespace op {
class MultiHeadAttention : public Layer {
public:
    explicit MultiHeadAttention(base::DeviceType device_type, int32_t head_num, int32_t kv_head_num,
                                int32_t head_size);
    base::Status check() const override;
    using Layer::forward;  // keep the N-ary overloads visible next to the override
    base::Status forward() override;
    void set_cache(const tensor::Tensor& key_cache, const tensor::Tensor& value_cache);
    void set_workspace(const tensor::Tensor& workspace);
    // Promise about the kernel launched just before this layer on the stream: it appended at most the newest
    // `rows` cache rows of a sequence, everything below seq_len - rows (and seq_len / slot) was final before it
    // started.  The attention kernel then fetches those rows while that kernel is still finishing.  -1 = no promise.
    void set_fresh_rows(int32_t rows) { fresh_rows_ = rows; }
    // Prompt chunk: the rows of `query` are consecutive tokens of sequence `slot` starting at position pos0 (their K / V
    // rows are in the cache already); causal attention with every K / V tile loaded once per block of query rows.
    base::Status forward_prefill(const tensor::Tensor& query, int32_t pos0, int32_t slot, const tensor::Tensor& output);

private:
    int32_t head_num_ = 0, kv_head_num_ = 0, head_size_ = 0;
    int32_t fresh_rows_ = -1;
    tensor::Tensor key_cache_, value_cache_, workspace_;
};
}  // namespace op

#endif  // KUIPER_INCLUDE_OP_MHA_H
