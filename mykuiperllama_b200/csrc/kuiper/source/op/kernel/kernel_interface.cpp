// Kernel registry: wraps each C-ABI entry point (include/kuiper_b200.h) in the
// Tensor-level signature the layers call, and hands it out per device like the
// reference's get_add_kernel (kuiper/source/op/kernel/kernel_interface.cpp:6-14).
// Preconditions are CHECKed the way add_kernel_cu does (add_kernel.cu:16-26), and a
// non-zero C-ABI status is fatal, mirroring its CHECK on cudaGetLastError (:50-51).
#include "kernel_interface.h"

#include "kuiper_b200.h"

namespace kernel {
namespace {

using tensor::Tensor;

#define KERNEL_OK(call)                                                              \
    do {                                                                             \
        int rc__ = (call);                                                           \
        CHECK_EQ(rc__, 0) << #call << " failed: " << kuiper_last_error();           \
    } while (0)

inline kuiper_stream_t as_stream(void* s) { return reinterpret_cast<kuiper_stream_t>(s); }

void require_cuda(const Tensor& t, const char* what) {
    CHECK(!t.is_empty()) << what << " is empty";
    CHECK(t.device_type() == base::DeviceType::DeviceCUDA) << what << " is not on the CUDA device";
}

template <typename T>
T* out_ptr(const Tensor& t) {
    return const_cast<T*>(t.ptr<T>());
}

void add_kernel_cu(const Tensor& input1, const Tensor& input2, const Tensor& output, void* stream) {
    require_cuda(input1, "add input1");
    require_cuda(input2, "add input2");
    require_cuda(output, "add output");
    CHECK_EQ(input1.size(), output.size());
    CHECK_EQ(input2.size(), output.size());
    KERNEL_OK(kuiper_add_f32(input1.ptr<float>(), input2.ptr<float>(), out_ptr<float>(output), int64_t(output.size()),
                             as_stream(stream)));
}

void matmul_kernel_cu(const Tensor& input, const Tensor& weight, const Tensor& output, void* stream) {
    require_cuda(input, "matmul input");
    require_cuda(weight, "matmul weight");
    require_cuda(output, "matmul output");
    CHECK_EQ(weight.dims_size(), 2);
    const int32_t N = weight.get_dim(0), K = weight.get_dim(1);
    CHECK_EQ(input.size() % size_t(K), size_t(0));
    const int32_t M = int32_t(input.size() / size_t(K));
    CHECK_EQ(output.size(), size_t(M) * size_t(N));
    KERNEL_OK(kuiper_bf16_gemv_f32(input.ptr<float>(), weight.ptr<uint16_t>(), out_ptr<float>(output), M, K, N,
                                   as_stream(stream)));
}

void matmul_kernel_quant_cu(const Tensor& input, const Tensor& qweight, const Tensor& qzeros, const Tensor& scales,
                            const Tensor& output, const Tensor* residual, int32_t group_size, int32_t act_mode,
                            const Tensor& workspace, void* stream) {
    require_cuda(input, "matmul input");
    require_cuda(qweight, "matmul qweight");
    require_cuda(qzeros, "matmul qzeros");
    require_cuda(scales, "matmul scales");
    require_cuda(output, "matmul output");
    CHECK_EQ(qweight.dims_size(), 2);
    const int32_t K = qweight.get_dim(0), N = qweight.get_dim(1) * 8;
    CHECK_EQ(input.size() % size_t(K), size_t(0));
    const int32_t M = int32_t(input.size() / size_t(K));
    CHECK_EQ(output.size(), size_t(M) * size_t(N));
    if (residual) {
        require_cuda(*residual, "matmul residual");
        CHECK_EQ(residual->size(), output.size());
    }
    KERNEL_OK(kuiper_awq_gemv_f32(input.ptr<float>(), qweight.ptr<int32_t>(), qzeros.ptr<int32_t>(),
                                  scales.ptr<uint16_t>(), out_ptr<float>(output),
                                  residual ? residual->ptr<float>() : nullptr, M, K, N, group_size, act_mode,
                                  out_ptr<void>(workspace), workspace.byte_size(), as_stream(stream)));
}

void matmul_kernel_quant_accum_cu(const Tensor& input, const Tensor& qweight, const Tensor& qzeros, const Tensor& scales,
                                  const Tensor& output, int32_t group_size, const Tensor* input_norm_weight, float eps,
                                  bool input_swiglu, int32_t act_mode, const Tensor* tickets, void* stream) {
    require_cuda(input, "matmul input");
    require_cuda(qweight, "matmul qweight");
    require_cuda(qzeros, "matmul qzeros");
    require_cuda(scales, "matmul scales");
    require_cuda(output, "matmul output");
    CHECK_EQ(qweight.dims_size(), 2);
    const int32_t K = qweight.get_dim(0), N = qweight.get_dim(1) * 8;
    const size_t in_row = size_t(K) * (input_swiglu ? 2 : 1);
    CHECK_EQ(input.size() % in_row, size_t(0));
    const int32_t M = int32_t(input.size() / in_row);
    CHECK_EQ(output.size(), size_t(M) * size_t(N));
    CHECK(!(input_swiglu && input_norm_weight != nullptr));
    if (input_norm_weight) {
        require_cuda(*input_norm_weight, "matmul input norm weight");
        CHECK_EQ(input_norm_weight->size(), size_t(K));
    }
    void* tk = nullptr;
    if (tickets && !tickets->is_empty()) {
        require_cuda(*tickets, "matmul balance counters");
        CHECK_GE(tickets->byte_size(), kuiper_awq_gemv_ticket_bytes());
        tk = out_ptr<void>(*tickets);
    }
    KERNEL_OK(kuiper_awq_gemv_accum_balanced_f32(input.ptr<float>(), input_norm_weight ? input_norm_weight->ptr<uint16_t>() : nullptr,
                                                 eps, input_swiglu ? 1 : 0, qweight.ptr<int32_t>(), qzeros.ptr<int32_t>(),
                                                 scales.ptr<uint16_t>(), out_ptr<float>(output), M, K, N, group_size, act_mode, tk,
                                                 as_stream(stream)));
}

void matmul_kernel_quant_gemm_cu(const Tensor& input, const Tensor& qweight, const Tensor& qzeros, const Tensor& scales,
                                 const Tensor& output, const Tensor* residual, bool accumulate, int32_t group_size,
                                 const Tensor& workspace, void* stream) {
    require_cuda(input, "matmul input");
    require_cuda(qweight, "matmul qweight");
    require_cuda(qzeros, "matmul qzeros");
    require_cuda(scales, "matmul scales");
    require_cuda(output, "matmul output");
    if (residual) require_cuda(*residual, "matmul residual");
    CHECK_EQ(qweight.dims_size(), 2);
    const int32_t K = qweight.get_dim(0), N = qweight.get_dim(1) * 8;
    CHECK_EQ(input.size() % size_t(K), size_t(0));
    const int32_t M = int32_t(input.size() / size_t(K));
    CHECK_EQ(output.size(), size_t(M) * size_t(N));
    if (input.data_type() == base::DataType::DataTypeFp16) {  // normalised / activated rows that already are fp16
        KERNEL_OK(kuiper_awq_gemm_f16in_f32(input.ptr<uint16_t>(), qweight.ptr<int32_t>(), qzeros.ptr<int32_t>(),
                                            scales.ptr<uint16_t>(), out_ptr<float>(output),
                                            residual ? residual->ptr<float>() : nullptr, accumulate ? 1 : 0, M, K, N, group_size,
                                            as_stream(stream)));
        return;
    }
    KERNEL_OK(kuiper_awq_gemm_f32(input.ptr<float>(), qweight.ptr<int32_t>(), qzeros.ptr<int32_t>(), scales.ptr<uint16_t>(),
                                  out_ptr<float>(output), residual ? residual->ptr<float>() : nullptr, accumulate ? 1 : 0, M,
                                  K, N, group_size, workspace.is_empty() ? nullptr : out_ptr<void>(workspace),
                                  workspace.is_empty() ? 0 : workspace.byte_size(), as_stream(stream)));
}

void rmsnorm_kernel_cu(const Tensor& input, const Tensor& weight, const Tensor& output, float eps, void* stream) {
    require_cuda(input, "rmsnorm input");
    require_cuda(weight, "rmsnorm weight");
    require_cuda(output, "rmsnorm output");
    const int32_t H = int32_t(weight.size());
    CHECK_EQ(input.size() % size_t(H), size_t(0));
    CHECK_EQ(input.size(), output.size());
    if (output.data_type() == base::DataType::DataTypeFp16) {
        KERNEL_OK(kuiper_rmsnorm_f16(input.ptr<float>(), weight.ptr<uint16_t>(), out_ptr<uint16_t>(output),
                                     int32_t(input.size() / size_t(H)), H, eps, as_stream(stream)));
        return;
    }
    KERNEL_OK(kuiper_rmsnorm_f32(input.ptr<float>(), weight.ptr<uint16_t>(), out_ptr<float>(output),
                                 int32_t(input.size() / size_t(H)), H, eps, as_stream(stream)));
}

void rope_kernel_cu(const Tensor& qkv, const Tensor& q_norm, const Tensor& k_norm, const Tensor& cos_cache,
                    const Tensor& sin_cache, const Tensor& pos, const Tensor& slot, const Tensor& q_out,
                    const Tensor& key_cache, const Tensor& value_cache, int32_t head_num, int32_t kv_head_num,
                    int32_t head_size, float eps, bool clear_input, const Tensor* clear_extra, void* stream) {
    require_cuda(qkv, "rope qkv");
    if (clear_extra) require_cuda(*clear_extra, "rope extra buffer");
    require_cuda(q_out, "rope q_out");
    require_cuda(key_cache, "rope key cache");
    require_cuda(value_cache, "rope value cache");
    CHECK_EQ(key_cache.dims_size(), 4);  // [n_slots, kv_heads, max_seq, head_size]
    const int32_t row = (head_num + 2 * kv_head_num) * head_size;
    CHECK_EQ(qkv.size() % size_t(row), size_t(0));
    const int32_t M = int32_t(qkv.size() / size_t(row));
    CHECK_GE(pos.size(), size_t(M));
    CHECK_GE(slot.size(), size_t(M));
    KERNEL_OK(kuiper_qknorm_rope_kvwrite(out_ptr<float>(qkv), q_norm.ptr<uint16_t>(), k_norm.ptr<uint16_t>(),
                                         cos_cache.ptr<float>(), sin_cache.ptr<float>(), pos.ptr<int32_t>(),
                                         slot.ptr<int32_t>(), M, head_num, kv_head_num, head_size, eps,
                                         key_cache.get_dim(2), key_cache.get_dim(0), out_ptr<float>(q_out),
                                         out_ptr<uint16_t>(key_cache), out_ptr<uint16_t>(value_cache), clear_input ? 1 : 0,
                                         clear_extra ? out_ptr<float>(*clear_extra) : nullptr,
                                         clear_extra ? int64_t(clear_extra->size()) : 0, as_stream(stream)));
}

void mha_kernel_cu(const Tensor& query, const Tensor& key_cache, const Tensor& value_cache, const Tensor& seq_len,
                   const Tensor& slot, const Tensor& output, int32_t head_num, int32_t kv_head_num, int32_t head_size,
                   int32_t fresh_rows, const Tensor& workspace, void* stream) {
    require_cuda(query, "mha query");
    require_cuda(output, "mha output");
    require_cuda(key_cache, "mha key cache");
    require_cuda(value_cache, "mha value cache");
    CHECK_EQ(key_cache.dims_size(), 4);
    const int32_t row = head_num * head_size;
    CHECK_EQ(query.size() % size_t(row), size_t(0));
    const int32_t M = int32_t(query.size() / size_t(row));
    CHECK_EQ(output.size(), query.size());
    KERNEL_OK(kuiper_flash_decode(query.ptr<float>(), key_cache.ptr<uint16_t>(), value_cache.ptr<uint16_t>(),
                                  seq_len.ptr<int32_t>(), slot.ptr<int32_t>(), out_ptr<float>(output), M, head_num,
                                  kv_head_num, head_size, key_cache.get_dim(2), key_cache.get_dim(0), fresh_rows,
                                  out_ptr<void>(workspace), workspace.byte_size(), as_stream(stream)));
}

void mha_prefill_kernel_cu(const Tensor& query, const Tensor& key_cache, const Tensor& value_cache, const Tensor& output,
                           int32_t head_num, int32_t kv_head_num, int32_t head_size, int32_t pos0, int32_t slot, void* stream) {
    require_cuda(query, "mha query");
    require_cuda(output, "mha output");
    require_cuda(key_cache, "mha key cache");
    require_cuda(value_cache, "mha value cache");
    CHECK_EQ(key_cache.dims_size(), 4);
    const int32_t row = head_num * head_size;
    CHECK_EQ(query.size() % size_t(row), size_t(0));
    const int32_t M = int32_t(query.size() / size_t(row));
    CHECK_EQ(output.size(), query.size());
    KERNEL_OK(kuiper_flash_prefill(query.ptr<float>(), key_cache.ptr<uint16_t>(), value_cache.ptr<uint16_t>(),
                                   out_ptr<float>(output), M, head_num, kv_head_num, head_size, key_cache.get_dim(2),
                                   key_cache.get_dim(0), pos0, slot, as_stream(stream)));
}

void rope_mha_kernel_cu(const Tensor& qkv, const Tensor& q_norm, const Tensor& k_norm, const Tensor& cos_cache,
                        const Tensor& sin_cache, const Tensor& pos, const Tensor& seq_len, const Tensor& slot,
                        const Tensor& output, const Tensor& key_cache, const Tensor& value_cache, int32_t head_num,
                        int32_t kv_head_num, int32_t head_size, float eps, int32_t fresh_rows, bool clear_input,
                        const Tensor* clear_extra, const Tensor& workspace, void* stream) {
    require_cuda(qkv, "rope+mha qkv");
    require_cuda(output, "rope+mha output");
    require_cuda(key_cache, "rope+mha key cache");
    require_cuda(value_cache, "rope+mha value cache");
    if (clear_extra) require_cuda(*clear_extra, "rope+mha extra buffer");
    CHECK_EQ(key_cache.dims_size(), 4);  // [n_slots, kv_heads, max_seq, head_size]
    const int32_t row = (head_num + 2 * kv_head_num) * head_size;
    CHECK_EQ(qkv.size() % size_t(row), size_t(0));
    const int32_t M = int32_t(qkv.size() / size_t(row));
    CHECK_EQ(output.size(), size_t(M) * size_t(head_num) * size_t(head_size));
    CHECK_GE(pos.size(), size_t(M));
    CHECK_GE(seq_len.size(), size_t(M));
    CHECK_GE(slot.size(), size_t(M));
    KERNEL_OK(kuiper_rope_flash_decode(out_ptr<float>(qkv), q_norm.ptr<uint16_t>(), k_norm.ptr<uint16_t>(),
                                       cos_cache.ptr<float>(), sin_cache.ptr<float>(), pos.ptr<int32_t>(),
                                       seq_len.ptr<int32_t>(), slot.ptr<int32_t>(), out_ptr<float>(output),
                                       out_ptr<uint16_t>(key_cache), out_ptr<uint16_t>(value_cache), M, head_num, kv_head_num,
                                       head_size, eps, key_cache.get_dim(2), key_cache.get_dim(0), fresh_rows,
                                       clear_input ? 1 : 0, clear_extra ? out_ptr<float>(*clear_extra) : nullptr,
                                       clear_extra ? int64_t(clear_extra->size()) : 0, out_ptr<void>(workspace),
                                       workspace.byte_size(), as_stream(stream)));
}

void swiglu_kernel_cu(const Tensor& gate_up, const Tensor& output, bool clear_input, void* stream) {
    require_cuda(gate_up, "swiglu input");
    require_cuda(output, "swiglu output");
    CHECK_EQ(gate_up.size(), output.size() * 2);
    const int32_t I = output.get_dim(output.dims_size() - 1);
    if (output.data_type() == base::DataType::DataTypeFp16) {
        KERNEL_OK(kuiper_swiglu_f16(out_ptr<float>(gate_up), out_ptr<uint16_t>(output), int32_t(output.size() / size_t(I)), I,
                                    clear_input ? 1 : 0, as_stream(stream)));
        return;
    }
    KERNEL_OK(kuiper_swiglu_f32(out_ptr<float>(gate_up), out_ptr<float>(output), int32_t(output.size() / size_t(I)), I,
                                clear_input ? 1 : 0, as_stream(stream)));
}

void emb_kernel_cu(const Tensor& tokens, const Tensor& table, const Tensor& output, int32_t vocab_size, void* stream) {
    require_cuda(tokens, "embedding tokens");
    require_cuda(table, "embedding table");
    require_cuda(output, "embedding output");
    const int32_t H = table.get_dim(1);
    CHECK_EQ(output.size() % size_t(H), size_t(0));
    const int32_t M = int32_t(output.size() / size_t(H));
    CHECK_GE(tokens.size(), size_t(M));
    KERNEL_OK(kuiper_embedding_bf16(tokens.ptr<int32_t>(), table.ptr<uint16_t>(), out_ptr<float>(output), M, H,
                                    vocab_size, as_stream(stream)));
}

void argmax_kernel_cu(const Tensor& logits, const Tensor& next, void* stream) {
    require_cuda(logits, "argmax logits");
    require_cuda(next, "argmax output");
    const int32_t V = logits.get_dim(logits.dims_size() - 1);
    const int32_t M = int32_t(logits.size() / size_t(V));
    CHECK_GE(next.size(), size_t(M));
    KERNEL_OK(kuiper_argmax_f32(logits.ptr<float>(), out_ptr<int32_t>(next), M, V, as_stream(stream)));
}

template <typename Fn>
Fn pick(base::DeviceType device_type, Fn cuda_fn, const char* name) {
    if (device_type == base::DeviceType::DeviceCUDA) return cuda_fn;
    LOG(FATAL) << "No " << name << " kernel for device type " << int(device_type)
               << ": this engine has CUDA kernels only.";
    return nullptr;
}

}  // namespace

AddKernel get_add_kernel(base::DeviceType d) { return pick<AddKernel>(d, add_kernel_cu, "add"); }
MatmulKernel get_matmul_kernel(base::DeviceType d) { return pick<MatmulKernel>(d, matmul_kernel_cu, "matmul"); }
MatmulKernelQuant get_matmul_kernel_quant(base::DeviceType d) {
    return pick<MatmulKernelQuant>(d, matmul_kernel_quant_cu, "quantised matmul");
}
MatmulKernelQuantAccum get_matmul_kernel_quant_accum(base::DeviceType d) {
    return pick<MatmulKernelQuantAccum>(d, matmul_kernel_quant_accum_cu, "accumulating quantised matmul");
}
MatmulKernelQuantGemm get_matmul_kernel_quant_gemm(base::DeviceType d) {
    return pick<MatmulKernelQuantGemm>(d, matmul_kernel_quant_gemm_cu, "tensor-core quantised matmul");
}
RMSNormKernel get_rmsnorm_kernel(base::DeviceType d) { return pick<RMSNormKernel>(d, rmsnorm_kernel_cu, "rmsnorm"); }
RoPEKernel get_rope_kernel(base::DeviceType d) { return pick<RoPEKernel>(d, rope_kernel_cu, "rope"); }
MHAKernel get_mha_kernel(base::DeviceType d) { return pick<MHAKernel>(d, mha_kernel_cu, "mha"); }
MHAPrefillKernel get_mha_prefill_kernel(base::DeviceType d) { return pick<MHAPrefillKernel>(d, mha_prefill_kernel_cu, "prefill mha"); }
RoPEMHAKernel get_rope_mha_kernel(base::DeviceType d) { return pick<RoPEMHAKernel>(d, rope_mha_kernel_cu, "rope+mha"); }
SwigluKernel get_swiglu_kernel(base::DeviceType d) { return pick<SwigluKernel>(d, swiglu_kernel_cu, "swiglu"); }
EmbeddingKernel get_emb_kernel(base::DeviceType d) { return pick<EmbeddingKernel>(d, emb_kernel_cu, "embedding"); }
ArgmaxKernel get_argmax_kernel(base::DeviceType d) { return pick<ArgmaxKernel>(d, argmax_kernel_cu, "argmax"); }

size_t matmul_quant_workspace_bytes(int32_t M, int32_t K, int32_t N) { return kuiper_awq_gemv_workspace_bytes(M, K, N); }
size_t matmul_quant_ticket_bytes() { return kuiper_awq_gemv_ticket_bytes(); }
size_t matmul_quant_gemm_workspace_bytes(int32_t M, int32_t K) { return kuiper_awq_gemm_workspace_bytes(M, K); }
size_t mha_workspace_bytes(int32_t M, int32_t head_num, int32_t head_size, int32_t max_seq) {
    return kuiper_flash_decode_workspace_bytes(M, head_num, head_size, max_seq);
}

}  // namespace kernel
