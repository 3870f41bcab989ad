// Operator base classes.  Public interface of the reference's kuiper/include/op/layer.h
// (LayerType :8-20, BaseLayer :22-67, Layer :70-120, LayerParam :122-156).
//
// Differences a user of the reference should know:
//  - activations (layer inputs / outputs) stay Fp32 as in the reference (layer.cpp:41-42),
//    but LayerParam accepts Int32 (packed INT4), Fp16 (scales) and Bf16 weights; the
//    reference CHECKs Fp32 on every weight (layer.cpp:248) and its raw-pointer
//    set_weight() is a no-op for quantised layers (layer.cpp:268-273);
//  - check_tensor_with_dim takes the expected dims as int32_t varargs (layer.cpp:80-88);
//    callers here cast explicitly (the reference's VecAddLayer passes a size_t,
//    add.cpp:15-16).
#ifndef KUIPER_INCLUDE_OP_LAYER_H
#define KUIPER_INCLUDE_OP_LAYER_H

#include <string>
#include <vector>

#include "base/cuda_config.h"
#include "tensor/tensor.h"

namespace op {

enum class LayerType : uint8_t {
    LayerUnknown = 0,
    LayerLinear = 1,
    LayerEncode = 2,
    LayerEmbedding = 3,
    LayerRMSNorm = 4,
    LayerMatmul = 5,
    LayerRope = 6,
    LayerMHA = 7,
    LayerSoftmax = 8,
    LayerAdd = 9,
    LayerSwiGLU = 10,
};

class BaseLayer {
public:
    explicit BaseLayer(base::DeviceType device_type, LayerType layer_type, base::DataType data_type,
                       std::string layer_name = "");
    virtual ~BaseLayer() = default;

    virtual base::Status init() = 0;
    virtual base::Status check() const = 0;

    virtual base::Status forward() = 0;
    virtual base::Status forward(const tensor::Tensor& input1, const tensor::Tensor& output1) = 0;
    virtual base::Status forward(const tensor::Tensor& input1, const tensor::Tensor& input2,
                                 const tensor::Tensor& output1) = 0;
    virtual base::Status forward(const tensor::Tensor& input1, const tensor::Tensor& input2,
                                 const tensor::Tensor& input3, const tensor::Tensor& output1) = 0;
    virtual base::Status forward(const tensor::Tensor& input1, const tensor::Tensor& input2,
                                 const tensor::Tensor& input3, const tensor::Tensor& input4,
                                 const tensor::Tensor& output1) = 0;
    virtual base::Status forward(const tensor::Tensor& input1, const tensor::Tensor& input2,
                                 const tensor::Tensor& input3, const tensor::Tensor& input4,
                                 const tensor::Tensor& input5, const tensor::Tensor& output1) = 0;

    virtual void set_input(int32_t idx, const tensor::Tensor& input) = 0;
    virtual void set_output(int32_t idx, const tensor::Tensor& output) = 0;
    virtual size_t input_size() const = 0;
    virtual size_t output_size() const = 0;
    virtual tensor::Tensor& get_input(int32_t idx) = 0;
    virtual tensor::Tensor& get_output(int32_t idx) = 0;
    virtual const tensor::Tensor& get_input(int32_t idx) const = 0;
    virtual const tensor::Tensor& get_output(int32_t idx) const = 0;

    virtual base::Status set_weight(int32_t idx, const tensor::Tensor& weight);
    virtual base::Status set_weight(int32_t idx, const std::vector<int32_t>& dims, const void* weight_ptr,
                                    base::DeviceType device_type = base::DeviceType::DeviceUnknown);

    const std::string& layer_name() const;
    LayerType layer_type() const;
    base::DataType data_type() const;
    base::DeviceType device_type() const;
    void set_layer_name(const std::string& layer_name);
    void set_device_type(base::DeviceType device_type);

protected:
    std::string layer_name_;
    LayerType layer_type_ = LayerType::LayerUnknown;
    base::DataType data_type_ = base::DataType::DataTypeUnknown;
    base::DeviceType device_type_ = base::DeviceType::DeviceUnknown;
};

// operator without parameters
class Layer : public BaseLayer {
public:
    explicit Layer(base::DeviceType device_type, LayerType layer_type, std::string layer_name = "");

    base::Status init() override;
    base::Status check() const override;

    base::Status check_tensor(const tensor::Tensor& tensor, base::DeviceType device_type,
                              base::DataType data_type) const;
    // trailing arguments: one int32_t per dimension of `tensor`
    base::Status check_tensor_with_dim(const tensor::Tensor& tensor, base::DeviceType device_type,
                                       base::DataType data_type, ...) const;

    base::Status forward() override;
    base::Status forward(const tensor::Tensor& input1, const tensor::Tensor& output1) override;
    base::Status forward(const tensor::Tensor& input1, const tensor::Tensor& input2,
                         const tensor::Tensor& output1) override;
    base::Status forward(const tensor::Tensor& input1, const tensor::Tensor& input2, const tensor::Tensor& input3,
                         const tensor::Tensor& output1) override;
    base::Status forward(const tensor::Tensor& input1, const tensor::Tensor& input2, const tensor::Tensor& input3,
                         const tensor::Tensor& input4, const tensor::Tensor& output1) override;
    base::Status forward(const tensor::Tensor& input1, const tensor::Tensor& input2, const tensor::Tensor& input3,
                         const tensor::Tensor& input4, const tensor::Tensor& input5,
                         const tensor::Tensor& output1) override;

    void set_input(int32_t idx, const tensor::Tensor& input) override;
    void set_output(int32_t idx, const tensor::Tensor& output) override;
    size_t input_size() const override;
    size_t output_size() const override;
    tensor::Tensor& get_input(int32_t idx) override;
    tensor::Tensor& get_output(int32_t idx) override;
    const tensor::Tensor& get_input(int32_t idx) const override;
    const tensor::Tensor& get_output(int32_t idx) const override;

    void reset_input_size(size_t size);
    void reset_output_size(size_t size);

    void set_cuda_config(std::shared_ptr<kernel::CudaConfig> cuda_config);
    std::shared_ptr<kernel::CudaConfig> cuda_config() const;

    virtual void to_cuda();

protected:
    // the stream kernels are enqueued on (nullptr = default stream)
    void* stream() const;

    std::vector<tensor::Tensor> inputs_;
    std::vector<tensor::Tensor> outputs_;
    std::shared_ptr<kernel::CudaConfig> cuda_config_;
};

// operator with parameters (weights, and for quantised layers scales + group size)
class LayerParam : public Layer {
public:
    explicit LayerParam(base::DeviceType device_type, LayerType layer_type, bool is_quant_layer = false,
                        std::string layer_name = "");

    size_t weights_size() const;
    void reset_weights_size(size_t size);
    tensor::Tensor& get_weight(int32_t idx);
    const tensor::Tensor& get_weight(int32_t idx) const;

    base::Status set_weight(int32_t idx, const tensor::Tensor& weight) override;
    // wraps a raw pointer without taking ownership; the element type is the layer's
    // weight type for that slot (see weight_data_type)
    base::Status set_weight(int32_t idx, const std::vector<int32_t>& dims, const void* weight_ptr,
                            base::DeviceType device_type = base::DeviceType::DeviceUnknown) override;

    void set_scales(const tensor::Tensor& scales);
    void set_group_size(int32_t group_size);
    int32_t get_scale_num() const;
    int32_t group_size() const { return group_size_; }
    bool is_quant_layer() const { return is_quant_layer_; }
    const tensor::Tensor& scales() const { return scales_; }

    void to_cuda() override;

protected:
    // element type a raw-pointer weight in slot idx is interpreted as
    virtual base::DataType weight_data_type(int32_t idx) const;

    int32_t group_size_ = 0;
    bool is_quant_layer_ = false;
    tensor::Tensor scales_;
    std::vector<tensor::Tensor> weights_;
};

}  // namespace op

#endif  // KUIPER_INCLUDE_OP_LAYER_H
