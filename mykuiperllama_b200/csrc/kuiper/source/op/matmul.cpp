#include <cstdlib>
// MatmulLayer: y = x . W for INT4-AWQ (dequant-fused GEMV) and bf16 weights.
#include "op/matmul.h"

#include "kernel/kernel_interface.h"

namespace op {

MatmulLayer::MatmulLayer(base::DeviceType device_type, int32_t dim0, int32_t dim1, bool is_quant_layer)
    : LayerParam(device_type, LayerType::LayerMatmul, is_quant_layer, "Matmul"), dim0_(dim0), dim1_(dim1) {
    reset_input_size(1);
    reset_output_size(1);
    reset_weights_size(is_quant_layer ? 2 : 1);
    if (is_quant_layer) group_size_ = 128;
    if (const char* env = std::getenv("KUIPER_GEMM_MIN_ROWS")) gemm_min_rows_ = std::atoi(env);  // measurement aid
}

base::DataType MatmulLayer::weight_data_type(int32_t) const {
    return is_quant_layer_ ? base::DataType::DataTypeInt32 : base::DataType::DataTypeBf16;
}

void MatmulLayer::set_residual(bool has_residual) {
    has_residual_ = has_residual;
    reset_input_size(has_residual ? 2 : 1);
}

void MatmulLayer::set_workspace(const tensor::Tensor& workspace) { workspace_ = workspace; }

base::Status MatmulLayer::check() const {
    const tensor::Tensor& x = get_input(0);
    base::Status status = check_tensor(x, device_type_, data_type_);
    if (!status) {
        LOG(ERROR) << "The input tensor error in the matmul layer.";
        return status;
    }
    const size_t in_row = size_t(dim1_) * (input_swiglu_ ? 2 : 1);
    if (x.size() % in_row != 0) return base::error::invalid_argument("The input width is not the layer's dim1.");
    const size_t M = x.size() / in_row;
    status = check_tensor(get_output(0), device_type_, data_type_);
    if (status && get_output(0).size() != M * size_t(dim0_))
        status = base::error::invalid_argument("The output tensor has a wrong element count.");
    if (!status) {
        LOG(ERROR) << "The output tensor error in the matmul layer.";
        return status;
    }
    if (has_residual_) {
        status = check_tensor(get_input(1), device_type_, data_type_);
        if (status && get_input(1).size() != M * size_t(dim0_))
            status = base::error::invalid_argument("The residual tensor has a wrong element count.");
        if (!status) return status;
    }
    if (is_quant_layer_) {
        if (group_size_ <= 0 || dim1_ % group_size_ != 0)
            return base::error::invalid_argument("The group size does not divide the input width.");
        status = check_tensor_with_dim(get_weight(0), device_type_, base::DataType::DataTypeInt32, dim1_, dim0_ / 8);
        if (!status) return status;
        status = check_tensor_with_dim(get_weight(1), device_type_, base::DataType::DataTypeInt32, dim1_ / group_size_,
                                       dim0_ / 8);
        if (!status) return status;
        status = check_tensor_with_dim(scales_, device_type_, base::DataType::DataTypeFp16, dim1_ / group_size_, dim0_);
        if (!status) return status;
    } else {
        status = check_tensor_with_dim(get_weight(0), device_type_, base::DataType::DataTypeBf16, dim0_, dim1_);
        if (!status) return status;
    }
    return base::error::success();
}

base::Status MatmulLayer::forward() {
    base::Status status = check();
    if (!status) return status;
    if (device_type_ == base::DeviceType::DeviceCUDA) CHECK_NE(cuda_config_, nullptr);
    const int32_t M = int32_t(get_input(0).size() / (size_t(dim1_) * (input_swiglu_ ? 2 : 1)));
    if (input_swiglu_ && !(is_quant_layer_ && accumulate_ && input_norm_.is_empty()))
        return base::error::invalid_argument("the fused SwiGLU input needs a quantised layer in accumulate mode without a norm");
    if (is_quant_layer_ && act_mode_ != 0 && gemm_min_rows_ > 0 && M >= gemm_min_rows_) {
        // enough rows for the tensor cores: x and the dequantised weight go through tcgen05 as fp16
        if (accumulate_ && has_residual_) return base::error::invalid_argument("accumulate mode takes no residual input");
        const tensor::Tensor* x = &get_input(0);
        tensor::Tensor normed;
        if (accumulate_ && (!input_norm_.is_empty() || input_swiglu_)) {
            // the normalised / activated rows are written as fp16 straight into the GEMM's activation buffer (the
            // rounding is that of the separate conversion pass, which is then not needed)
            if (gemm_workspace_.is_empty() || gemm_workspace_.byte_size() < size_t(M) * size_t(dim1_) * sizeof(uint16_t))
                return base::error::invalid_argument("the tensor-core path needs its fp16 activation workspace");
            normed = tensor::Tensor(base::DataType::DataTypeFp16, std::vector<int32_t>{M, dim1_}, false, nullptr,
                                    const_cast<void*>(gemm_workspace_.ptr<void>()));
            normed.set_device_type(device_type_);
            if (input_swiglu_)
                kernel::get_swiglu_kernel(device_type_)(get_input(0), normed, false, stream());
            else
                kernel::get_rmsnorm_kernel(device_type_)(get_input(0), input_norm_, normed, input_norm_eps_, stream());
            x = &normed;
        }
        kernel::get_matmul_kernel_quant_gemm(device_type_)(*x, get_weight(0), get_weight(1), scales_, get_output(0),
                                                           has_residual_ ? &get_input(1) : nullptr, accumulate_,
                                                           group_size_, gemm_workspace_, stream());
    } else if (is_quant_layer_ && accumulate_) {
        if (has_residual_) return base::error::invalid_argument("accumulate mode takes no residual input");
        kernel::get_matmul_kernel_quant_accum(device_type_)(get_input(0), get_weight(0), get_weight(1), scales_, get_output(0),
                                                            group_size_, input_norm_.is_empty() ? nullptr : &input_norm_,
                                                            input_norm_eps_, input_swiglu_, act_mode_ == 2 ? 2 : 1, &tickets_, stream());
    } else if (is_quant_layer_) {
        kernel::get_matmul_kernel_quant(device_type_)(get_input(0), get_weight(0), get_weight(1), scales_, get_output(0),
                                                      has_residual_ ? &get_input(1) : nullptr, group_size_, act_mode_,
                                                      workspace_, stream());
    } else {
        if (has_residual_) return base::error::function_not_implement("residual on a bf16 matmul");
        kernel::get_matmul_kernel(device_type_)(get_input(0), get_weight(0), get_output(0), stream());
    }
    return base::error::success();
}

}  // namespace op
