// SwiGLU activation out = silu(gate) * up.  Placeholder in the reference:
// kuiper/include/op/swiglu.h:1-10, tag LayerSwiGLU (op/layer.h:19).
// input 0: the fused gate|up projection [M, 2*hidden_dim] Fp32; output 0: [M, hidden_dim].
#ifndef KUIPER_INCLUDE_OP_SWIGLU_H
#define KUIPER_INCLUDE_OP_SWIGLU_H

#include "op/layer.h"

namespace op {
class SwiGLULayer : public Layer {
public:
    explicit SwiGLULayer(base::DeviceType device_type, int32_t hidden_dim);
    base::Status check() const override;
    void set_clear_input(bool clear) { clear_input_ = clear; }  // zero gate|up after reading it
    using Layer::forward;  // keep the N-ary overloads visible next to the override
    base::Status forward() override;

private:
    int32_t hidden_dim_ = 0;
    bool clear_input_ = false;
};
}  // namespace op

#endif  // KUIPER_INCLUDE_OP_SWIGLU_H
