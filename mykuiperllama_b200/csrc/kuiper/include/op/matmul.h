// Linear projection y = x . W.  The reference reserves this header as an empty
// namespace (kuiper/include/op/matmul.h:1-11) and the LayerMatmul tag (op/layer.h:14).
//
// Quantised (is_quant_layer): INT4-AWQ.  weight slot 0 = qweight Int32 [K, N/8],
// slot 1 = qzeros Int32 [K/group, N/8], set_scales() = Fp16 [K/group, N],
// set_group_size(128); input [M, K], output [M, N].
// Plain: weight slot 0 = Bf16 [N, K] (one row per output, the lm_head layout).
//
// Optional residual: with set_residual(true) the layer takes a second input [M, N] and
// writes output = input2 + x . W in the same kernel (the output may be that tensor).
#ifndef KUIPER_INCLUDE_OP_MATMUL_H
#define KUIPER_INCLUDE_OP_MATMUL_H

#include "base/cuda_config.h"
#include "op/layer.h"

namespace op {
class MatmulLayer : public LayerParam {
public:
    // dim0 = output width N, dim1 = input width K
    explicit MatmulLayer(base::DeviceType device_type, int32_t dim0, int32_t dim1, bool is_quant_layer = false);

    base::Status check() const override;
    using Layer::forward;  // keep the N-ary overloads visible next to the override
    base::Status forward() override;

    void set_residual(bool has_residual);
    // accumulate mode (quantised layers): output += x . W, the output tensor already holds the addend
    // (residual stream or zeros); no workspace, unordered fp32 summation
    void set_accumulate(bool accumulate) { accumulate_ = accumulate; }
    // accumulate mode only: the input is an un-normalised row and the layer applies RMSNorm(input; weight, eps)
    // inside the matmul kernel (weight bf16 [dim1]); saves the separate norm launch
    void set_input_norm(const tensor::Tensor& weight, float eps) {
        input_norm_ = weight;
        input_norm_eps_ = eps;
    }
    // accumulate mode only: the input is a gate|up row [M, 2*dim1] and the layer applies SwiGLU inside the matmul
    // kernel (operand = silu(gate) * up); saves the separate activation launch.  The input is only read.
    void set_input_swiglu(bool on) { input_swiglu_ = on; }
    // where RMSNorm(input) / SwiGLU(input) is written when the row count takes the tensor-core path, which has
    // no fused prologue ([max rows, dim1] fp32)
    void set_norm_scratch(const tensor::Tensor& scratch) { norm_scratch_ = scratch; }
    // quantised layers, fp16-operand mode: inputs of at least this many rows go to the tcgen05 GEMM instead of
    // the GEMV (0 = never).  With its K split (few output tiles -> several CTAs per tile) the GEMM is ahead of passes of
    // 4 rows through the GEMV from 16 rows on (4096 x 24576, 16 rows: 48 us against 4 x 12.8 us; 32 rows: 48.5 against 102).
    void set_gemm_min_rows(int32_t rows) { gemm_min_rows_ = rows; }
    // scratch of the split-K kernel: kernel::matmul_quant_workspace_bytes(M, K, N) bytes, zero-initialised once
    void set_workspace(const tensor::Tensor& workspace);
    // scratch of the tensor-core path: kernel::matmul_quant_gemm_workspace_bytes(max rows, dim1) bytes, no
    // initialisation needed
    void set_gemm_workspace(const tensor::Tensor& workspace) { gemm_workspace_ = workspace; }
    // accumulate mode: kernel::matmul_quant_ticket_bytes() zeroed bytes owned by this layer (its balance counters);
    // without them the kernel deals its work out statically
    void set_tickets(const tensor::Tensor& tickets) { tickets_ = tickets; }
    // how the INT4 kernel rounds x: 1 = fp16 operand (default), 0 = fp32 operand, 2 = block-scaled 16-bit integers for
    // single-row passes (the fastest decode kernel) and fp16 for passes of several rows
    void set_act_mode(int32_t act_mode) { act_mode_ = act_mode; }

    int32_t out_features() const { return dim0_; }
    int32_t in_features() const { return dim1_; }

protected:
    base::DataType weight_data_type(int32_t idx) const override;

private:
    int32_t dim0_ = 0;
    int32_t dim1_ = 0;
    bool has_residual_ = false;
    bool accumulate_ = false;
    bool input_swiglu_ = false;
    tensor::Tensor input_norm_;
    float input_norm_eps_ = 1e-6f;
    int32_t act_mode_ = 1;
    tensor::Tensor workspace_;
    tensor::Tensor gemm_workspace_;
    tensor::Tensor norm_scratch_;
    tensor::Tensor tickets_;
    int32_t gemm_min_rows_ = 16;  // from 16 rows on the split-K tcgen05 GEMM beats passes of 4 rows through the GEMV
};
}  // namespace op

#endif  // KUIPER_INCLUDE_OP_MATMUL_H
