// Residual add layer: out = in1 + in2.  Same class as the reference's VecAddLayer
// (kuiper/include/op/add.h:7-14, kuiper/source/op/add.cpp:5-49).
#ifndef KUIPER_INCLUDE_OP_ADD_H
#define KUIPER_INCLUDE_OP_ADD_H

#include "op/layer.h"

namespace op {
class VecAddLayer : public Layer {
public:
    explicit VecAddLayer(base::DeviceType device_type);
    base::Status check() const override;
    using Layer::forward;  // keep the N-ary overloads visible next to the override
    base::Status forward() override;
};
}  // namespace op

#endif  // KUIPER_INCLUDE_OP_ADD_H
