// RMSNorm y = (x * rstd) * w over the last dimension.  Placeholder in the reference:
// kuiper/include/op/rmsnorm.h:1-10, tag LayerRMSNorm (op/layer.h:13).
// weight slot 0 = Bf16 [dim]; input / output [M, dim] Fp32.
#ifndef KUIPER_INCLUDE_OP_RMSNORM_H
#define KUIPER_INCLUDE_OP_RMSNORM_H

#include "op/layer.h"

namespace op {
class RmsNormLayer : public LayerParam {
public:
    explicit RmsNormLayer(base::DeviceType device_type, int32_t dim, float eps = 1e-6f);
    base::Status check() const override;
    using Layer::forward;  // keep the N-ary overloads visible next to the override
    base::Status forward() override;

protected:
    base::DataType weight_data_type(int32_t idx) const override;

private:
    int32_t dim_ = 0;
    float eps_ = 1e-6f;
};
}  // namespace op

#endif  // KUIPER_INCLUDE_OP_RMSNORM_H
