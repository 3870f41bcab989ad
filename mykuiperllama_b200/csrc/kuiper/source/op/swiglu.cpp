// SwiGLULayer: out = silu(gate) * up on the fused gate|up projection.
#include "op/swiglu.h"

#include "kernel/kernel_interface.h"

namespace op {

SwiGLULayer::SwiGLULayer(base::DeviceType device_type, int32_t hidden_dim)
    : Layer(device_type, LayerType::LayerSwiGLU, "SwiGLU"), hidden_dim_(hidden_dim) {
    reset_input_size(1);
    reset_output_size(1);
}

base::Status SwiGLULayer::check() const {
    base::Status status = check_tensor(get_input(0), device_type_, data_type_);
    if (status && get_input(0).size() % size_t(2 * hidden_dim_) != 0)
        status = base::error::invalid_argument("The gate|up tensor has a wrong width.");
    if (!status) {
        LOG(ERROR) << "The input tensor error in the swiglu layer.";
        return status;
    }
    status = check_tensor(get_output(0), device_type_, data_type_);
    if (status && (get_output(0).size() * 2 != get_input(0).size() ||
                   get_output(0).get_dim(get_output(0).dims_size() - 1) != hidden_dim_))
        status = base::error::invalid_argument("The output tensor has a wrong shape.");
    if (!status) LOG(ERROR) << "The output tensor error in the swiglu layer.";
    return status;
}

base::Status SwiGLULayer::forward() {
    base::Status status = check();
    if (!status) return status;
    kernel::get_swiglu_kernel(device_type_)(get_input(0), get_output(0), clear_input_, stream());
    return base::error::success();
}

}  // namespace op
