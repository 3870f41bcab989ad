// Kernel registry: one function-pointer type and one getter per operator, selected by
// device.  Pattern of the reference's kuiper/source/op/kernel/kernel_interface.h:10-11
// and kernel_interface.cpp:6-14 (AddKernel / get_add_kernel), extended to every op of
// the decode path.  This is the drop-in boundary: each CUDA entry wraps one function of
// the C ABI (include/kuiper_b200.h).  There is no CPU implementation behind these
// getters: asking for DeviceCPU is a fatal error, as an unknown device is in the
// reference (kernel_interface.cpp:12).
//
// All kernels: inputs and outputs are passed as const Tensor& and outputs are written
// in place (add_kernel.cu:39); `stream` is a cudaStream_t passed as void*, nullptr =
// default stream (add_kernel.cu:31-48); launches are asynchronous and nothing allocates.
#ifndef KERNEL_INTERFACE_H
#define KERNEL_INTERFACE_H

#include "tensor/tensor.h"

namespace kernel {

using AddKernel = void (*)(const tensor::Tensor& input1, const tensor::Tensor& input2, const tensor::Tensor& output,
                           void* stream);

// output[M,N] = input[M,K] . weight[N,K]^T, weight Bf16
using MatmulKernel = void (*)(const tensor::Tensor& input, const tensor::Tensor& weight, const tensor::Tensor& output,
                              void* stream);

// output[M,N] = input[M,K] . dequant(qweight, qzeros, scales) (+ residual if not null)
using MatmulKernelQuant = void (*)(const tensor::Tensor& input, const tensor::Tensor& qweight,
                                   const tensor::Tensor& qzeros, const tensor::Tensor& scales,
                                   const tensor::Tensor& output, const tensor::Tensor* residual, int32_t group_size,
                                   int32_t act_mode, const tensor::Tensor& workspace, void* stream);

// output[M,N] += input[M,K] . dequant(...): the output already holds the addend (residual stream or zeros).
// With input_norm_weight (bf16 [K]) the operand is RMSNorm(input) formed inside the kernel.
// With input_swiglu the input is a gate|up row [M, 2K] and the operand is silu(gate) * up (no norm then).
// act_mode: 1 fp16 operand, 2 block-scaled 16-bit integer operand for single-row calls (fp16 otherwise).
// tickets (may be null): matmul_quant_ticket_bytes() zeroed bytes owned by the calling layer; with them the kernel
// hands the tail of the weight stream to whichever CTA is free, so that all CTAs finish together.
using MatmulKernelQuantAccum = void (*)(const tensor::Tensor& input, const tensor::Tensor& qweight,
                                        const tensor::Tensor& qzeros, const tensor::Tensor& scales,
                                        const tensor::Tensor& output, int32_t group_size,
                                        const tensor::Tensor* input_norm_weight, float eps, bool input_swiglu,
                                        int32_t act_mode, const tensor::Tensor* tickets, void* stream);

// Tensor-core path for M >= 16 rows: output = input . dequant(...) (+ residual), or output += ... when accumulate.
using MatmulKernelQuantGemm = void (*)(const tensor::Tensor& input, const tensor::Tensor& qweight,
                                       const tensor::Tensor& qzeros, const tensor::Tensor& scales,
                                       const tensor::Tensor& output, const tensor::Tensor* residual, bool accumulate,
                                       int32_t group_size, const tensor::Tensor& workspace, void* stream);

using RMSNormKernel = void (*)(const tensor::Tensor& input, const tensor::Tensor& weight, const tensor::Tensor& output,
                               float eps, void* stream);

using RoPEKernel = void (*)(const tensor::Tensor& qkv, const tensor::Tensor& q_norm, const tensor::Tensor& k_norm,
                            const tensor::Tensor& cos_cache, const tensor::Tensor& sin_cache, const tensor::Tensor& pos,
                            const tensor::Tensor& slot, const tensor::Tensor& q_out, const tensor::Tensor& key_cache,
                            const tensor::Tensor& value_cache, int32_t head_num, int32_t kv_head_num, int32_t head_size,
                            float eps, bool clear_input, const tensor::Tensor* clear_extra, void* stream);

// rotary + KV append + attention in one kernel (decode batches: one row per sequence slot, seq_len == pos + 1)
using RoPEMHAKernel = void (*)(const tensor::Tensor& qkv, const tensor::Tensor& q_norm, const tensor::Tensor& k_norm,
                               const tensor::Tensor& cos_cache, const tensor::Tensor& sin_cache, const tensor::Tensor& pos,
                               const tensor::Tensor& seq_len, const tensor::Tensor& slot, const tensor::Tensor& output,
                               const tensor::Tensor& key_cache, const tensor::Tensor& value_cache, int32_t head_num,
                               int32_t kv_head_num, int32_t head_size, float eps, int32_t fresh_rows, bool clear_input,
                               const tensor::Tensor* clear_extra, const tensor::Tensor& workspace, void* stream);

using MHAKernel = void (*)(const tensor::Tensor& query, const tensor::Tensor& key_cache, const tensor::Tensor& value_cache,
                           const tensor::Tensor& seq_len, const tensor::Tensor& slot, const tensor::Tensor& output,
                           int32_t head_num, int32_t kv_head_num, int32_t head_size, int32_t fresh_rows,
                           const tensor::Tensor& workspace, void* stream);

// causal attention of a prompt chunk: the M rows are consecutive tokens of one sequence starting at position pos0
using MHAPrefillKernel = void (*)(const tensor::Tensor& query, const tensor::Tensor& key_cache, const tensor::Tensor& value_cache,
                                  const tensor::Tensor& output, int32_t head_num, int32_t kv_head_num, int32_t head_size,
                                  int32_t pos0, int32_t slot, void* stream);

using SwigluKernel = void (*)(const tensor::Tensor& gate_up, const tensor::Tensor& output, bool clear_input, void* stream);

using EmbeddingKernel = void (*)(const tensor::Tensor& tokens, const tensor::Tensor& table, const tensor::Tensor& output,
                                 int32_t vocab_size, void* stream);

using ArgmaxKernel = void (*)(const tensor::Tensor& logits, const tensor::Tensor& next, void* stream);

AddKernel get_add_kernel(base::DeviceType device_type);
MatmulKernel get_matmul_kernel(base::DeviceType device_type);
MatmulKernelQuant get_matmul_kernel_quant(base::DeviceType device_type);
MatmulKernelQuantAccum get_matmul_kernel_quant_accum(base::DeviceType device_type);
MatmulKernelQuantGemm get_matmul_kernel_quant_gemm(base::DeviceType device_type);
RMSNormKernel get_rmsnorm_kernel(base::DeviceType device_type);
RoPEKernel get_rope_kernel(base::DeviceType device_type);
MHAKernel get_mha_kernel(base::DeviceType device_type);
MHAPrefillKernel get_mha_prefill_kernel(base::DeviceType device_type);
RoPEMHAKernel get_rope_mha_kernel(base::DeviceType device_type);
SwigluKernel get_swiglu_kernel(base::DeviceType device_type);
EmbeddingKernel get_emb_kernel(base::DeviceType device_type);
ArgmaxKernel get_argmax_kernel(base::DeviceType device_type);

// scratch sizes of the two kernels that need a workspace
size_t matmul_quant_workspace_bytes(int32_t M, int32_t K, int32_t N);
size_t matmul_quant_ticket_bytes();  // balance counters of one accumulate-mode layer
size_t matmul_quant_gemm_workspace_bytes(int32_t M, int32_t K);  // fp16 activation copy of the tensor-core path
size_t mha_workspace_bytes(int32_t M, int32_t head_num, int32_t head_size, int32_t max_seq);

}  // namespace kernel

#endif  // KERNEL_INTERFACE_H
