// RmsNormLayer.
#include "op/rmsnorm.h"

#include "kernel/kernel_interface.h"

namespace op {

RmsNormLayer::RmsNormLayer(base::DeviceType device_type, int32_t dim, float eps)
    : LayerParam(device_type, LayerType::LayerRMSNorm, false, "RMSNorm"), dim_(dim), eps_(eps) {
    reset_input_size(1);
    reset_output_size(1);
    reset_weights_size(1);
}

base::DataType RmsNormLayer::weight_data_type(int32_t) const { return base::DataType::DataTypeBf16; }

base::Status RmsNormLayer::check() const {
    base::Status status = check_tensor(get_input(0), device_type_, data_type_);
    if (status && get_input(0).size() % size_t(dim_) != 0)
        status = base::error::invalid_argument("The input width is not the norm dimension.");
    if (!status) {
        LOG(ERROR) << "The input tensor error in the rmsnorm layer.";
        return status;
    }
    status = check_tensor(get_output(0), device_type_, data_type_);
    if (status && get_output(0).size() != get_input(0).size())
        status = base::error::invalid_argument("The output tensor has a wrong element count.");
    if (!status) {
        LOG(ERROR) << "The output tensor error in the rmsnorm layer.";
        return status;
    }
    return check_tensor_with_dim(get_weight(0), device_type_, base::DataType::DataTypeBf16, dim_);
}

base::Status RmsNormLayer::forward() {
    base::Status status = check();
    if (!status) return status;
    kernel::get_rmsnorm_kernel(device_type_)(get_input(0), get_weight(0), get_output(0), eps_, stream());
    return base::error::success();
}

}  // namespace op
