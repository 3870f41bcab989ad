// Token embedding gather.  Placeholder in the reference: kuiper/include/op/embedding.h:1-10,
// tag LayerEmbedding (op/layer.h:12).
// input 0: tokens [M] Int32; weight 0: table Bf16 [vocab, dim]; output 0: [M, dim] Fp32.
#ifndef KUIPER_INCLUDE_OP_EMBEDDING_H
#define KUIPER_INCLUDE_OP_EMBEDDING_H

#include "op/layer.h"

namespace op {
class EmbeddingLayer : public LayerParam {
public:
    explicit EmbeddingLayer(base::DeviceType device_type, int32_t dim, int32_t vocab_size);
    base::Status check() const override;
    using Layer::forward;  // keep the N-ary overloads visible next to the override
    base::Status forward() override;

protected:
    base::DataType weight_data_type(int32_t idx) const override;

private:
    int32_t dim_ = 0, vocab_size_ = 0;
};
}  // namespace op

#endif  // KUIPER_INCLUDE_OP_EMBEDDING_H
