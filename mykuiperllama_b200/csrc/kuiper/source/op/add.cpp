// VecAddLayer: out = in1 + in2 (reference: kuiper/source/op/add.cpp:5-49).
#include "op/add.h"

#include "kernel/kernel_interface.h"

namespace op {

VecAddLayer::VecAddLayer(base::DeviceType device_type) : Layer(device_type, LayerType::LayerAdd, "Add") {
    reset_input_size(2);
    reset_output_size(1);
}

base::Status VecAddLayer::check() const {
    const tensor::Tensor& out = get_output(0);
    const tensor::Tensor* operands[3] = {&get_input(0), &get_input(1), &out};
    const char* names[3] = {"input tensor 1", "input tensor 2", "output tensor"};
    for (int i = 0; i < 3; i++) {
        base::Status status = check_tensor(*operands[i], device_type_, data_type_);
        if (status && operands[i]->size() != get_input(0).size())
            status = base::error::invalid_argument("The tensor has a wrong element count.");
        if (!status) {
            LOG(ERROR) << "The " << names[i] << " error in the add layer.";
            return status;
        }
    }
    return base::error::success();
}

base::Status VecAddLayer::forward() {
    base::Status status = check();
    if (!status) return status;
    if (device_type_ == base::DeviceType::DeviceCUDA) CHECK_NE(cuda_config_, nullptr);
    kernel::get_add_kernel(device_type_)(get_input(0), get_input(1), get_output(0), stream());
    return base::error::success();
}

}  // namespace op
