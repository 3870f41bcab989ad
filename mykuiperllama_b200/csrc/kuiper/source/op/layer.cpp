// BaseLayer / Layer / LayerParam (interface: kuiper/include/op/layer.h:22-156 of the
// reference; slot bookkeeping and the N-ary forward() overloads behave as
// kuiper/source/op/layer.cpp:94-231 there).
#include "op/layer.h"

#include <cstdarg>
#include <functional>
#include <numeric>

namespace op {

// ---------------------------------------------------------------- BaseLayer
BaseLayer::BaseLayer(base::DeviceType device_type, LayerType layer_type, base::DataType data_type,
                     std::string layer_name)
    : layer_name_(std::move(layer_name)), layer_type_(layer_type), data_type_(data_type), device_type_(device_type) {}

base::Status BaseLayer::set_weight(int32_t, const tensor::Tensor&) { return base::error::function_not_implement(); }

base::Status BaseLayer::set_weight(int32_t, const std::vector<int32_t>&, const void*, base::DeviceType) {
    return base::error::function_not_implement();
}

const std::string& BaseLayer::layer_name() const { return layer_name_; }
LayerType BaseLayer::layer_type() const { return layer_type_; }
base::DataType BaseLayer::data_type() const { return data_type_; }
base::DeviceType BaseLayer::device_type() const { return device_type_; }
void BaseLayer::set_layer_name(const std::string& layer_name) { layer_name_ = layer_name; }
void BaseLayer::set_device_type(base::DeviceType device_type) { device_type_ = device_type; }

// ---------------------------------------------------------------- Layer
Layer::Layer(base::DeviceType device_type, LayerType layer_type, std::string layer_name)
    : BaseLayer(device_type, layer_type, base::DataType::DataTypeFp32, std::move(layer_name)) {}

base::Status Layer::init() { return base::error::success(); }

base::Status Layer::check() const {
    return base::error::function_not_implement("The check function is not implement yet");
}

base::Status Layer::check_tensor(const tensor::Tensor& tensor, base::DeviceType device_type,
                                 base::DataType data_type) const {
    if (tensor.is_empty()) return base::error::invalid_argument("The tensor parameter is empty.");
    if (tensor.device_type() != device_type) return base::error::invalid_argument("The tensor has a wrong device type.");
    if (tensor.data_type() != data_type) return base::error::invalid_argument("The tensor has a wrong data type.");
    return base::error::success();
}

base::Status Layer::check_tensor_with_dim(const tensor::Tensor& tensor, base::DeviceType device_type,
                                          base::DataType data_type, ...) const {
    base::Status status = check_tensor(tensor, device_type, data_type);
    if (!status) return status;
    std::va_list args;
    va_start(args, data_type);
    for (int32_t i = 0; i < tensor.dims_size(); i++) {
        const int32_t expected = va_arg(args, int32_t);
        if (expected != tensor.get_dim(i)) {
            va_end(args);
            return base::error::invalid_argument("The tensor has a wrong dim in dim" + std::to_string(i));
        }
    }
    va_end(args);
    return base::error::success();
}

base::Status Layer::forward() { return base::error::function_not_implement(); }

base::Status Layer::forward(const tensor::Tensor& input1, const tensor::Tensor& output1) {
    set_input(0, input1);
    set_output(0, output1);
    return forward();
}

base::Status Layer::forward(const tensor::Tensor& input1, const tensor::Tensor& input2, const tensor::Tensor& output1) {
    set_input(0, input1);
    set_input(1, input2);
    set_output(0, output1);
    return forward();
}

base::Status Layer::forward(const tensor::Tensor& input1, const tensor::Tensor& input2, const tensor::Tensor& input3,
                            const tensor::Tensor& output1) {
    set_input(0, input1);
    set_input(1, input2);
    set_input(2, input3);
    set_output(0, output1);
    return forward();
}

base::Status Layer::forward(const tensor::Tensor& input1, const tensor::Tensor& input2, const tensor::Tensor& input3,
                            const tensor::Tensor& input4, const tensor::Tensor& output1) {
    set_input(0, input1);
    set_input(1, input2);
    set_input(2, input3);
    set_input(3, input4);
    set_output(0, output1);
    return forward();
}

base::Status Layer::forward(const tensor::Tensor& input1, const tensor::Tensor& input2, const tensor::Tensor& input3,
                            const tensor::Tensor& input4, const tensor::Tensor& input5, const tensor::Tensor& output1) {
    set_input(0, input1);
    set_input(1, input2);
    set_input(2, input3);
    set_input(3, input4);
    set_input(4, input5);
    set_output(0, output1);
    return forward();
}

void Layer::set_input(int32_t idx, const tensor::Tensor& input) {
    CHECK_GE(idx, 0);
    CHECK_LT(size_t(idx), inputs_.size());
    // index-like inputs (token ids, positions) are Int32; everything else is the layer's Fp32
    CHECK(input.data_type() == data_type_ || input.data_type() == base::DataType::DataTypeInt32);
    if (!input.is_empty()) CHECK(input.device_type() == device_type_);
    inputs_[size_t(idx)] = input;
}

void Layer::set_output(int32_t idx, const tensor::Tensor& output) {
    CHECK_GE(idx, 0);
    CHECK_LT(size_t(idx), outputs_.size());
    CHECK(output.data_type() == data_type_);
    if (!output.is_empty()) CHECK(output.device_type() == device_type_);
    outputs_[size_t(idx)] = output;
}

size_t Layer::input_size() const { return inputs_.size(); }
size_t Layer::output_size() const { return outputs_.size(); }

tensor::Tensor& Layer::get_input(int32_t idx) {
    CHECK_GE(idx, 0);
    CHECK_LT(size_t(idx), inputs_.size());
    return inputs_[size_t(idx)];
}

tensor::Tensor& Layer::get_output(int32_t idx) {
    CHECK_GE(idx, 0);
    CHECK_LT(size_t(idx), outputs_.size());
    return outputs_[size_t(idx)];
}

const tensor::Tensor& Layer::get_input(int32_t idx) const {
    CHECK_GE(idx, 0);
    CHECK_LT(size_t(idx), inputs_.size());
    return inputs_[size_t(idx)];
}

const tensor::Tensor& Layer::get_output(int32_t idx) const {
    CHECK_GE(idx, 0);
    CHECK_LT(size_t(idx), outputs_.size());
    return outputs_[size_t(idx)];
}

void Layer::reset_input_size(size_t size) { inputs_.resize(size); }
void Layer::reset_output_size(size_t size) { outputs_.resize(size); }

void Layer::set_cuda_config(std::shared_ptr<kernel::CudaConfig> cuda_config) {
    if (cuda_config) cuda_config_ = std::move(cuda_config);
}

std::shared_ptr<kernel::CudaConfig> Layer::cuda_config() const { return cuda_config_; }

void* Layer::stream() const { return cuda_config_ ? cuda_config_->stream() : nullptr; }

void Layer::to_cuda() {
    cudaStream_t s = cuda_config_ ? cuda_config_->stream() : nullptr;
    for (auto& t : inputs_)
        if (!t.is_empty()) t.to_cuda(s);
    for (auto& t : outputs_)
        if (!t.is_empty()) t.to_cuda(s);
}

// ---------------------------------------------------------------- LayerParam
LayerParam::LayerParam(base::DeviceType device_type, LayerType layer_type, bool is_quant_layer, std::string layer_name)
    : Layer(device_type, layer_type, std::move(layer_name)), is_quant_layer_(is_quant_layer) {}

size_t LayerParam::weights_size() const { return weights_.size(); }
void LayerParam::reset_weights_size(size_t size) { weights_.resize(size); }

tensor::Tensor& LayerParam::get_weight(int32_t idx) {
    CHECK_GE(idx, 0);
    CHECK_LT(size_t(idx), weights_.size());
    return weights_[size_t(idx)];
}

const tensor::Tensor& LayerParam::get_weight(int32_t idx) const {
    CHECK_GE(idx, 0);
    CHECK_LT(size_t(idx), weights_.size());
    return weights_[size_t(idx)];
}

base::DataType LayerParam::weight_data_type(int32_t) const { return base::DataType::DataTypeFp32; }

base::Status LayerParam::set_weight(int32_t idx, const tensor::Tensor& weight) {
    CHECK_GE(idx, 0);
    CHECK_LT(size_t(idx), weights_.size());
    if (weight.data_type() != weight_data_type(idx))
        return base::error::invalid_argument("The weight has a wrong data type for slot " + std::to_string(idx));
    if (!weight.is_empty()) CHECK(weight.device_type() == device_type_);
    weights_[size_t(idx)] = weight;
    return base::error::success();
}

base::Status LayerParam::set_weight(int32_t idx, const std::vector<int32_t>& dims, const void* weight_ptr,
                                    base::DeviceType device_type) {
    CHECK_GE(idx, 0);
    CHECK_LT(size_t(idx), weights_.size());
    CHECK_NE(weight_ptr, nullptr);
    // borrowed memory, quantised layers included
    tensor::Tensor weight(weight_data_type(idx), dims, false, nullptr, const_cast<void*>(weight_ptr));
    if (device_type != base::DeviceType::DeviceUnknown) weight.set_device_type(device_type);
    weights_[size_t(idx)] = weight;
    return base::error::success();
}

void LayerParam::set_scales(const tensor::Tensor& scales) {
    CHECK(!scales.is_empty());
    CHECK(scales.data_type() == base::DataType::DataTypeFp16 || scales.data_type() == data_type_);
    CHECK(scales.device_type() == device_type_);
    scales_ = scales;
}

void LayerParam::set_group_size(int32_t group_size) { group_size_ = group_size; }

int32_t LayerParam::get_scale_num() const {
    CHECK(!scales_.is_empty());
    return int32_t(scales_.size());
}

void LayerParam::to_cuda() {
    Layer::to_cuda();
    cudaStream_t s = cuda_config_ ? cuda_config_->stream() : nullptr;
    for (auto& w : weights_)
        if (!w.is_empty()) w.to_cuda(s);
    if (!scales_.is_empty()) scales_.to_cuda(s);
}

}  // namespace op
