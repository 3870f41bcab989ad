// Qwen3-shaped INT4-AWQ decoder on one GPU or one tensor-parallel rank.
#include "model/qwen3.h"

#include <climits>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>

#include "kuiper_b200.h"
#include "model/checkpoint.h"
#include "op/kernel/kernel_interface.h"

namespace model {
namespace {

using base::DataType;
using tensor::Tensor;

#define CUDA_OK(call)                                                                        \
    do {                                                                                     \
        cudaError_t err__ = (call);                                                          \
        if (err__ != cudaSuccess)                                                            \
            return base::error::internal_error(std::string(#call) + ": " + cudaGetErrorString(err__)); \
    } while (0)

#define RETURN_IF_ERROR(expr)       \
    do {                            \
        base::Status st__ = (expr); \
        if (!st__) return st__;     \
    } while (0)

size_t round256(size_t v) { return (v + 255) / 256 * 256; }

// borrowed view of `elems` elements starting `offset` elements into a device buffer
Tensor view(const Tensor& buf, DataType dtype, std::vector<int32_t> dims, size_t offset_elems = 0) {
    char* p = const_cast<char*>(buf.ptr<char>()) + offset_elems * base::data_type_size(dtype);
    Tensor t(dtype, std::move(dims), false, nullptr, p);
    t.set_device_type(base::DeviceType::DeviceCUDA);
    return t;
}

struct QuantShape {
    int32_t K, N;
    size_t qw_bytes(int g) const { (void)g; return size_t(K) * size_t(N) / 2; }
    size_t qz_bytes(int g) const { return size_t(K / g) * size_t(N) / 2; }
    size_t s_bytes(int g) const { return size_t(K / g) * size_t(N) * 2; }
    size_t total(int g) const { return round256(qw_bytes(g)) + round256(qz_bytes(g)) + round256(s_bytes(g)); }
};

// strided copy of `rows` rows of `row_bytes` bytes, host or device source
base::Status copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t row_bytes, size_t rows,
                     bool src_on_device) {
    CUDA_OK(cudaMemcpy2D(dst, dst_pitch, src, src_pitch, row_bytes, rows,
                         src_on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice));
    return base::error::success();
}

}  // namespace

Qwen3Model::Qwen3Model(const ModelConfig& config) : Model(base::ModelType::ModelTypeQwen3, config) {}

Qwen3Model::~Qwen3Model() {
    if (cuda_config_ && cuda_config_->stream()) cudaStreamSynchronize(cuda_config_->stream());
    for (auto& kv : graphs_) cudaGraphExecDestroy(kv.second);
    for (auto& kv : graphs_unrolled_) cudaGraphExecDestroy(kv.second);
    if (host_stage_) cudaFreeHost(host_stage_);
}

base::Status Qwen3Model::init(base::DeviceType device_type) {
    if (device_type != base::DeviceType::DeviceCUDA)
        return base::error::invalid_argument("the engine runs on DeviceCUDA only");
    const ModelConfig& c = config_;
    if (c.layer_num <= 0 || c.dim <= 0 || c.head_num <= 0 || c.kv_head_num <= 0 || c.hidden_dim <= 0 ||
        c.vocab_size <= 0 || c.max_seq_len <= 0 || c.max_batch <= 0 || c.max_rows <= 0)
        return base::error::invalid_argument("model config has an empty dimension");
    if (c.head_size != 128 || c.group_size != 128)
        return base::error::invalid_argument("head_size and group_size must be 128");
    if (c.tp_size < 1 || c.tp_rank < 0 || c.tp_rank >= c.tp_size)
        return base::error::invalid_argument("bad tensor-parallel rank");
    if (c.head_num % c.kv_head_num || c.head_num % c.tp_size || c.kv_head_num % c.tp_size ||
        c.hidden_dim % (c.tp_size * c.group_size) || c.dim % c.group_size || c.max_rows < c.max_batch)
        return base::error::invalid_argument("model dimensions do not divide (heads / tp / group / rows)");

    int n_devices = 0;
    if (cudaGetDeviceCount(&n_devices) != cudaSuccess || n_devices == 0)
        return base::error::internal_error("no CUDA device is visible: the engine has no CPU path");

    device_type_ = device_type;
    cuda_config_ = std::make_shared<kernel::CudaConfig>();
    cuda_config_->create();

    const int32_t D = c.head_size, H = c.dim, R = c.max_rows;
    const int32_t Hq = local_heads(), Hkv = local_kv_heads(), I = local_hidden();
    const int32_t QKV = (Hq + 2 * Hkv) * D;
    const int g = c.group_size;
    const QuantShape sh_qkv{H, QKV}, sh_o{Hq * D, H}, sh_gu{H, 2 * I}, sh_down{I, H};

    // ---- capacity of the arena: weights + caches + step buffers + scratch
    const size_t cache_elems = size_t(c.max_batch) * Hkv * c.max_seq_len * D;
    size_t ws_mm = 0;
    size_t ws_gemm = 0;  // fp16 activation rows of the tensor-core path
    for (const QuantShape& s : {sh_qkv, sh_o, sh_gu, sh_down}) {
        ws_mm = std::max(ws_mm, kernel::matmul_quant_workspace_bytes(2, s.K, s.N));
        ws_gemm = std::max(ws_gemm, kernel::matmul_quant_gemm_workspace_bytes(R, s.K));
    }
    const size_t ws_mha = kernel::mha_workspace_bytes(R, Hq, D, c.max_seq_len);
    // tensor dimensions are 32-bit (tensor::Tensor, as in the reference): a workspace has to stay below 2 GiB
    if (ws_mm > size_t(INT32_MAX) || ws_mha > size_t(INT32_MAX) || ws_gemm > size_t(INT32_MAX))
        return base::error::invalid_argument("max_rows is too large: a kernel workspace would exceed 2 GiB");
    size_t total = 0;
    total += size_t(c.layer_num) * (sh_qkv.total(g) + sh_o.total(g) + sh_gu.total(g) + sh_down.total(g) +
                                    2 * round256(size_t(H) * 2) + 2 * round256(size_t(D) * 2) +
                                    2 * round256(cache_elems * 2));
    total += 2 * round256(size_t(c.vocab_size) * H * 2) + round256(size_t(H) * 2);
    total += 5 * round256(size_t(R) * 4);                                   // tokens, pos, seq_len, slot, next
    total += 4 * round256(size_t(R) * H * 4);                               // h, h_alt, two norm outputs
    total += round256(size_t(R) * QKV * 4) + 2 * round256(size_t(R) * Hq * D * 4);
    total += round256(size_t(R) * 2 * I * 4) + round256(size_t(R) * I * 4);
    total += round256(size_t(R) * c.vocab_size * 4) * (c.tp_size > 1 ? 3 : 1);  // + logits shard and gather under tensor parallelism
    total += 2 * round256(size_t(c.max_seq_len) * (D / 2) * 4);
    total += round256(ws_mm) + round256(ws_mha) + round256(ws_gemm) + (1u << 20);
    total += size_t(c.layer_num) * 4 * 256;  // balance counters of the four projections of a layer
    auto arena = std::make_shared<base::CUDAArenaAllocator>(total);
    weight_alloc_ = arena;

    auto dev = [&](DataType dt, std::vector<int32_t> dims) { return Tensor(dt, std::move(dims), true, weight_alloc_); };

    // ---- step buffers, named as in model::ModelBufferType
    RETURN_IF_ERROR(insert_buffer(ModelBufferType::InputTokens, dev(DataType::DataTypeInt32, {R})));
    RETURN_IF_ERROR(insert_buffer(ModelBufferType::InputPos, dev(DataType::DataTypeInt32, {R})));
    RETURN_IF_ERROR(insert_buffer(ModelBufferType::SeqLen, dev(DataType::DataTypeInt32, {R})));
    RETURN_IF_ERROR(insert_buffer(ModelBufferType::SeqSlot, dev(DataType::DataTypeInt32, {R})));
    RETURN_IF_ERROR(insert_buffer(ModelBufferType::NextTokens, dev(DataType::DataTypeInt32, {R})));
    RETURN_IF_ERROR(insert_buffer(ModelBufferType::InputEmbeddings, dev(DataType::DataTypeFp32, {R, H})));
    RETURN_IF_ERROR(insert_buffer(ModelBufferType::AttnOutput, dev(DataType::DataTypeFp32, {R, H})));
    RETURN_IF_ERROR(insert_buffer(ModelBufferType::OutputRMSNorm, dev(DataType::DataTypeFp32, {R, H})));
    RETURN_IF_ERROR(insert_buffer(ModelBufferType::FFNRMSNorm, dev(DataType::DataTypeFp32, {R, H})));
    RETURN_IF_ERROR(insert_buffer(ModelBufferType::QKVOutput, dev(DataType::DataTypeFp32, {R, QKV})));
    RETURN_IF_ERROR(insert_buffer(ModelBufferType::Query, dev(DataType::DataTypeFp32, {R, Hq * D})));
    RETURN_IF_ERROR(insert_buffer(ModelBufferType::OutputMHA, dev(DataType::DataTypeFp32, {R, Hq * D})));
    RETURN_IF_ERROR(insert_buffer(ModelBufferType::W1Output, dev(DataType::DataTypeFp32, {R, 2 * I})));
    RETURN_IF_ERROR(insert_buffer(ModelBufferType::W2Output, dev(DataType::DataTypeFp32, {R, I})));
    RETURN_IF_ERROR(insert_buffer(ModelBufferType::ForwardOutput, dev(DataType::DataTypeFp32, {R, c.vocab_size})));
    // tensor parallelism: the lm_head is split over the vocabulary (rank r holds rows [r V/tp, (r+1) V/tp)); the local
    // logits and, for passes that want the whole row, the gathered slices of all ranks
    vocab_local_ = (c.tp_size > 1 && c.vocab_size % c.tp_size == 0) ? c.vocab_size / c.tp_size : c.vocab_size;
    if (vocab_local_ != c.vocab_size) {
        RETURN_IF_ERROR(insert_buffer(ModelBufferType::LogitsShard, dev(DataType::DataTypeFp32, {R, vocab_local_})));
        RETURN_IF_ERROR(insert_buffer(ModelBufferType::LogitsGather, dev(DataType::DataTypeFp32, {c.tp_size, R, vocab_local_})));
    }
    RETURN_IF_ERROR(insert_buffer(ModelBufferType::CosCache, dev(DataType::DataTypeFp32, {c.max_seq_len, D / 2})));
    RETURN_IF_ERROR(insert_buffer(ModelBufferType::SinCache, dev(DataType::DataTypeFp32, {c.max_seq_len, D / 2})));
    RETURN_IF_ERROR(insert_buffer(ModelBufferType::MatmulWorkspace, dev(DataType::DataTypeInt8, {int32_t(ws_mm)})));
    RETURN_IF_ERROR(insert_buffer(ModelBufferType::MHAWorkspace, dev(DataType::DataTypeInt8, {int32_t(ws_mha)})));
    RETURN_IF_ERROR(insert_buffer(ModelBufferType::GemmWorkspace, dev(DataType::DataTypeInt8, {int32_t(ws_gemm)})));
    CUDA_OK(cudaMemset(get_buffer(ModelBufferType::MatmulWorkspace).ptr<void>(), 0, ws_mm));
    CUDA_OK(cudaMemset(get_buffer(ModelBufferType::MHAWorkspace).ptr<void>(), 0, ws_mha));
    // the partial-row buffer of the row-split projections starts (and is always left) zeroed
    CUDA_OK(cudaMemset(get_buffer(ModelBufferType::AttnOutput).ptr<void>(), 0, get_buffer(ModelBufferType::AttnOutput).byte_size()));
    // accumulating projections need their output buffers zero before the first pass
    CUDA_OK(cudaMemset(get_buffer(ModelBufferType::QKVOutput).ptr<void>(), 0, get_buffer(ModelBufferType::QKVOutput).byte_size()));
    CUDA_OK(cudaMemset(get_buffer(ModelBufferType::W1Output).ptr<void>(), 0, get_buffer(ModelBufferType::W1Output).byte_size()));
    for (ModelBufferType b : {ModelBufferType::InputTokens, ModelBufferType::InputPos, ModelBufferType::SeqLen,
                              ModelBufferType::SeqSlot, ModelBufferType::NextTokens})
        CUDA_OK(cudaMemset(get_buffer(b).ptr<void>(), 0, size_t(R) * 4));

    // ---- rotary tables: angle = pos * theta^(-2i/D) in double, rounded once to fp32
    {
        const int32_t half = D / 2;
        std::vector<float> cos_h(size_t(c.max_seq_len) * half), sin_h(cos_h.size());
        for (int32_t p = 0; p < c.max_seq_len; p++)
            for (int32_t i = 0; i < half; i++) {
                const double a = double(p) * std::pow(c.rope_theta, -2.0 * double(i) / double(D));
                cos_h[size_t(p) * half + i] = float(std::cos(a));
                sin_h[size_t(p) * half + i] = float(std::sin(a));
            }
        CUDA_OK(cudaMemcpy(get_buffer(ModelBufferType::CosCache).ptr<void>(), cos_h.data(), cos_h.size() * 4,
                           cudaMemcpyHostToDevice));
        CUDA_OK(cudaMemcpy(get_buffer(ModelBufferType::SinCache).ptr<void>(), sin_h.data(), sin_h.size() * 4,
                           cudaMemcpyHostToDevice));
    }

    // ---- layers
    auto make_quant = [&](const QuantShape& s, bool residual) {
        auto l = std::make_unique<op::MatmulLayer>(device_type_, s.N, s.K, true);
        l->set_cuda_config(cuda_config_);
        l->set_group_size(g);
        l->set_act_mode(c.act_mode);
        l->set_residual(residual);
        l->set_workspace(get_buffer(ModelBufferType::MatmulWorkspace));
        l->set_gemm_workspace(get_buffer(ModelBufferType::GemmWorkspace));
        {
            // balance counters of this layer object alone: launches that overlap under programmatic dependent
            // launch are always different layer objects
            Tensor tk = dev(DataType::DataTypeInt32, {int32_t(kernel::matmul_quant_ticket_bytes() / 4)});
            cudaMemset(tk.ptr<void>(), 0, tk.byte_size());
            l->set_tickets(tk);
        }
        STATUS_CHECK(l->set_weight(0, dev(DataType::DataTypeInt32, {s.K, s.N / 8})));
        STATUS_CHECK(l->set_weight(1, dev(DataType::DataTypeInt32, {s.K / g, s.N / 8})));
        l->set_scales(dev(DataType::DataTypeFp16, {s.K / g, s.N}));
        return l;
    };
    auto make_norm = [&](int32_t dim) {
        auto l = std::make_unique<op::RmsNormLayer>(device_type_, dim, c.eps);
        l->set_cuda_config(cuda_config_);
        STATUS_CHECK(l->set_weight(0, dev(DataType::DataTypeBf16, {dim})));
        return l;
    };
    // Every projection accumulates into its output (the residual stream for O and down; a buffer that its consumer
    // left zeroed for QKV and gate|up), which needs no ordered combine.  Under tensor parallelism the row-split
    // projections (O, down) accumulate into a zeroed partial-row buffer instead; the exchange that follows adds the
    // residual stream and the partial rows of all ranks and leaves the buffer zeroed again.
    accumulate_cols_ = c.act_mode != 0 && QKV % 32 == 0 && H % 32 == 0 && (2 * I) % 32 == 0;
    accumulate_ = accumulate_cols_;
    layers_.resize(size_t(c.layer_num));
    layer_loaded_.assign(size_t(c.layer_num), false);
    for (Qwen3Layer& L : layers_) {
        L.input_norm = make_norm(H);
        L.post_norm = make_norm(H);
        L.qkv = make_quant(sh_qkv, false);
        L.o = make_quant(sh_o, c.tp_size == 1 && !accumulate_);
        L.gate_up = make_quant(sh_gu, false);
        L.down = make_quant(sh_down, c.tp_size == 1 && !accumulate_);
        for (op::MatmulLayer* m : {L.qkv.get(), L.gate_up.get()}) m->set_accumulate(accumulate_cols_);
        for (op::MatmulLayer* m : {L.o.get(), L.down.get()}) m->set_accumulate(accumulate_);
        if (accumulate_cols_) {
            // the two pre-norms run inside the projections that consume them
            L.qkv->set_input_norm(L.input_norm->get_weight(0), c.eps);
            L.gate_up->set_input_norm(L.post_norm->get_weight(0), c.eps);
            // passes of 16 rows or more take the tensor-core path, which wants the normed rows materialised
            L.qkv->set_norm_scratch(get_buffer(ModelBufferType::OutputRMSNorm));
            L.gate_up->set_norm_scratch(get_buffer(ModelBufferType::FFNRMSNorm));
        }
        if (accumulate_) {
            // SwiGLU runs inside the down projection, which only reads the gate|up buffer
            L.down->set_input_swiglu(true);
            L.down->set_norm_scratch(get_buffer(ModelBufferType::W2Output));
        }
        L.key_cache = dev(DataType::DataTypeBf16, {c.max_batch, Hkv, c.max_seq_len, D});
        L.value_cache = dev(DataType::DataTypeBf16, {c.max_batch, Hkv, c.max_seq_len, D});
        CUDA_OK(cudaMemset(L.key_cache.ptr<void>(), 0, L.key_cache.byte_size()));
        CUDA_OK(cudaMemset(L.value_cache.ptr<void>(), 0, L.value_cache.byte_size()));
        L.rope = std::make_unique<op::RoPELayer>(device_type_, Hq, Hkv, D, c.eps);
        L.rope->set_cuda_config(cuda_config_);
        STATUS_CHECK(L.rope->set_weight(0, dev(DataType::DataTypeBf16, {D})));
        STATUS_CHECK(L.rope->set_weight(1, dev(DataType::DataTypeBf16, {D})));
        L.rope->set_cache(L.key_cache, L.value_cache);
        L.rope->set_clear_input(accumulate_cols_);
        // ... so this layer's rotary kernel zeroes that buffer for the next gate|up projection to accumulate into
        if (accumulate_) L.rope->set_clear_extra(get_buffer(ModelBufferType::W1Output), 2 * I);
        L.mha = std::make_unique<op::MultiHeadAttention>(device_type_, Hq, Hkv, D);
        L.mha->set_cuda_config(cuda_config_);
        L.mha->set_cache(L.key_cache, L.value_cache);
        L.mha->set_workspace(get_buffer(ModelBufferType::MHAWorkspace));
        L.rope->set_attention_workspace(get_buffer(ModelBufferType::MHAWorkspace));
        L.swiglu = std::make_unique<op::SwiGLULayer>(device_type_, I);
        L.swiglu->set_cuda_config(cuda_config_);
        L.swiglu->set_clear_input(accumulate_cols_);  // used when SwiGLU is not fused into the down projection
    }
    embedding_ = std::make_unique<op::EmbeddingLayer>(device_type_, H, c.vocab_size);
    embedding_->set_cuda_config(cuda_config_);
    STATUS_CHECK(embedding_->set_weight(0, dev(DataType::DataTypeBf16, {c.vocab_size, H})));
    final_norm_ = make_norm(H);
    lm_head_ = std::make_unique<op::MatmulLayer>(device_type_, vocab_local_, H, false);
    lm_head_->set_cuda_config(cuda_config_);
    STATUS_CHECK(lm_head_->set_weight(0, dev(DataType::DataTypeBf16, {vocab_local_, H})));
    sampler_ = std::make_unique<sampler::ArgmaxSampler>(device_type_);

    CUDA_OK(cudaMallocHost(reinterpret_cast<void**>(&host_stage_), size_t(R) * 4 * sizeof(int32_t)));
    CUDA_OK(cudaDeviceSynchronize());
    return base::error::success();
}

// ------------------------------------------------------------------ weights
base::Status Qwen3Model::load_layer(int32_t layer, const RawLayerWeights& w, bool on_device) {
    if (layer < 0 || layer >= config_.layer_num) return base::error::invalid_argument("layer index out of range");
    for (const void* p : {w.input_norm, w.post_norm, w.q_norm, w.k_norm, w.qkv_qw, w.qkv_qz, w.qkv_s, w.o_qw, w.o_qz,
                          w.o_s, w.gu_qw, w.gu_qz, w.gu_s, w.down_qw, w.down_qz, w.down_s})
        if (!p) return base::error::invalid_argument("null weight pointer");
    const ModelConfig& c = config_;
    const int32_t D = c.head_size, H = c.dim, g = c.group_size, tp = c.tp_size, r = c.tp_rank;
    const int32_t Hq = local_heads(), Hkv = local_kv_heads(), I = local_hidden();
    Qwen3Layer& L = layers_[size_t(layer)];
    const cudaMemcpyKind kind = on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;

    CUDA_OK(cudaMemcpy(L.input_norm->get_weight(0).ptr<void>(), w.input_norm, size_t(H) * 2, kind));
    CUDA_OK(cudaMemcpy(L.post_norm->get_weight(0).ptr<void>(), w.post_norm, size_t(H) * 2, kind));
    CUDA_OK(cudaMemcpy(L.rope->get_weight(0).ptr<void>(), w.q_norm, size_t(D) * 2, kind));
    CUDA_OK(cudaMemcpy(L.rope->get_weight(1).ptr<void>(), w.k_norm, size_t(D) * 2, kind));

    // Column split: copy `cols` logical columns starting at src_col of a full-width N_full
    // tensor triple into dst columns starting at dst_col.  Packed words hold 8 columns.
    auto copy_cols = [&](op::MatmulLayer& m, const void* qw, const void* qz, const void* s, int32_t K, int32_t N_full,
                         int32_t src_col, int32_t dst_col, int32_t cols) -> base::Status {
        const int32_t N_loc = m.out_features();
        char* dqw = m.get_weight(0).ptr<char>();
        char* dqz = m.get_weight(1).ptr<char>();
        char* ds = const_cast<char*>(m.scales().ptr<char>());
        RETURN_IF_ERROR(copy_2d(dqw + size_t(dst_col) / 2, size_t(N_loc) / 2, static_cast<const char*>(qw) + size_t(src_col) / 2,
                                size_t(N_full) / 2, size_t(cols) / 2, size_t(K), on_device));
        RETURN_IF_ERROR(copy_2d(dqz + size_t(dst_col) / 2, size_t(N_loc) / 2, static_cast<const char*>(qz) + size_t(src_col) / 2,
                                size_t(N_full) / 2, size_t(cols) / 2, size_t(K / g), on_device));
        RETURN_IF_ERROR(copy_2d(ds + size_t(dst_col) * 2, size_t(N_loc) * 2, static_cast<const char*>(s) + size_t(src_col) * 2,
                                size_t(N_full) * 2, size_t(cols) * 2, size_t(K / g), on_device));
        return base::error::success();
    };
    // Row split: rows [row0, row0 + K_loc) of a [K_full, N] triple (row0 a multiple of the group)
    auto copy_rows = [&](op::MatmulLayer& m, const void* qw, const void* qz, const void* s, int32_t N, int32_t row0,
                         int32_t K_loc) -> base::Status {
        CUDA_OK(cudaMemcpy(m.get_weight(0).ptr<void>(), static_cast<const char*>(qw) + size_t(row0) * N / 2,
                           size_t(K_loc) * N / 2, kind));
        CUDA_OK(cudaMemcpy(m.get_weight(1).ptr<void>(), static_cast<const char*>(qz) + size_t(row0 / g) * N / 2,
                           size_t(K_loc / g) * N / 2, kind));
        CUDA_OK(cudaMemcpy(const_cast<void*>(m.scales().ptr<void>()), static_cast<const char*>(s) + size_t(row0 / g) * N * 2,
                           size_t(K_loc / g) * N * 2, kind));
        return base::error::success();
    };

    const int32_t QKV_full = (c.head_num + 2 * c.kv_head_num) * D;
    // q heads | k heads | v heads of this rank
    RETURN_IF_ERROR(copy_cols(*L.qkv, w.qkv_qw, w.qkv_qz, w.qkv_s, H, QKV_full, r * Hq * D, 0, Hq * D));
    RETURN_IF_ERROR(copy_cols(*L.qkv, w.qkv_qw, w.qkv_qz, w.qkv_s, H, QKV_full, c.head_num * D + r * Hkv * D, Hq * D, Hkv * D));
    RETURN_IF_ERROR(copy_cols(*L.qkv, w.qkv_qw, w.qkv_qz, w.qkv_s, H, QKV_full,
                              (c.head_num + c.kv_head_num) * D + r * Hkv * D, (Hq + Hkv) * D, Hkv * D));
    // gate | up of this rank
    RETURN_IF_ERROR(copy_cols(*L.gate_up, w.gu_qw, w.gu_qz, w.gu_s, H, 2 * c.hidden_dim, r * I, 0, I));
    RETURN_IF_ERROR(copy_cols(*L.gate_up, w.gu_qw, w.gu_qz, w.gu_s, H, 2 * c.hidden_dim, c.hidden_dim + r * I, I, I));
    RETURN_IF_ERROR(copy_rows(*L.o, w.o_qw, w.o_qz, w.o_s, H, r * Hq * D, Hq * D));
    RETURN_IF_ERROR(copy_rows(*L.down, w.down_qw, w.down_qz, w.down_s, H, r * I, I));
    (void)tp;
    // device-to-device copies may return before they are done, and the engine's stream does not wait for the
    // default stream they ran on
    if (on_device) CUDA_OK(cudaDeviceSynchronize());
    layer_loaded_[size_t(layer)] = true;
    return base::error::success();
}

base::Status Qwen3Model::load_globals(const void* embed, const void* final_norm, const void* lm_head, bool on_device) {
    if (!embed || !final_norm || !lm_head) return base::error::invalid_argument("null weight pointer");
    const cudaMemcpyKind kind = on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
    const size_t table = size_t(config_.vocab_size) * config_.dim * 2;
    CUDA_OK(cudaMemcpy(embedding_->get_weight(0).ptr<void>(), embed, table, kind));
    CUDA_OK(cudaMemcpy(final_norm_->get_weight(0).ptr<void>(), final_norm, size_t(config_.dim) * 2, kind));
    // this rank's slice of the vocabulary (all of it on one GPU)
    const size_t shard = size_t(vocab_local_) * config_.dim * 2;
    const size_t shard_off = vocab_local_ != config_.vocab_size ? size_t(config_.tp_rank) * shard : 0;
    CUDA_OK(cudaMemcpy(lm_head_->get_weight(0).ptr<void>(), static_cast<const char*>(lm_head) + shard_off, shard, kind));
    if (on_device) CUDA_OK(cudaDeviceSynchronize());
    globals_loaded_ = true;
    return base::error::success();
}

// ------------------------------------------------------------------ checkpoint file
namespace {

// bf16 bits of a checkpoint tensor stored as BF16, F16 or F32 (round to nearest even)
base::Status to_bf16(const CheckpointTensor& t, int64_t expect, const std::string& name, std::vector<uint16_t>* out) {
    if (t.element_count() != expect)
        return base::error::model_parse_error(name + " has " + std::to_string(t.element_count()) + " elements, expected " + std::to_string(expect));
    out->resize(size_t(expect));
    auto f32_to_bf16 = [](float f) {
        uint32_t u;
        std::memcpy(&u, &f, 4);
        if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x40);
        u += 0x7fffu + ((u >> 16) & 1u);
        return uint16_t(u >> 16);
    };
    if (t.dtype == "BF16") {
        std::memcpy(out->data(), t.data, size_t(expect) * 2);
    } else if (t.dtype == "F32") {
        const float* p = reinterpret_cast<const float*>(t.data);
        for (int64_t i = 0; i < expect; i++) (*out)[size_t(i)] = f32_to_bf16(p[i]);
    } else if (t.dtype == "F16") {
        const uint16_t* p = reinterpret_cast<const uint16_t*>(t.data);
        for (int64_t i = 0; i < expect; i++) {
            const uint32_t h = p[i], sign = (h & 0x8000u) << 16, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu;
            uint32_t u;
            if (exp == 0) {
                if (man == 0) {
                    u = sign;
                } else {  // subnormal half: normalise
                    int e = -1;
                    uint32_t m = man;
                    do { e++; m <<= 1; } while ((m & 0x400u) == 0);
                    u = sign | uint32_t(127 - 15 - e) << 23 | (m & 0x3ffu) << 13;
                }
            } else if (exp == 31) {
                u = sign | 0x7f800000u | man << 13;
            } else {
                u = sign | (exp + 127 - 15) << 23 | man << 13;
            }
            float f;
            std::memcpy(&f, &u, 4);
            (*out)[size_t(i)] = f32_to_bf16(f);
        }
    } else {
        return base::error::model_parse_error(name + " has dtype " + t.dtype + " (BF16, F16 or F32 expected)");
    }
    return base::error::success();
}

// one INT4-AWQ projection of the file, entered through the layer hook the reference reserves for it:
// LayerParam::set_weight(idx, dims, ptr, device) with borrowed host pointers (quantised branch), set_scales()
struct StagedProjection {
    std::unique_ptr<op::MatmulLayer> layer;  // host-side layer object that only holds the borrowed tensors
    int32_t K = 0, N = 0;
};

base::Status stage_projection(const SafetensorsFile& f, const std::string& prefix, int32_t K, int32_t N, int32_t g,
                              StagedProjection* out) {
    const CheckpointTensor* qw = f.find(prefix + ".qweight");
    const CheckpointTensor* qz = f.find(prefix + ".qzeros");
    const CheckpointTensor* sc = f.find(prefix + ".scales");
    if (!qw || !qz || !sc) return base::error::model_parse_error(prefix + ": qweight / qzeros / scales missing");
    auto shape_is = [](const CheckpointTensor& t, int64_t a, int64_t b) { return t.shape.size() == 2 && t.shape[0] == a && t.shape[1] == b; };
    if (qw->dtype != "I32" || !shape_is(*qw, K, N / 8)) return base::error::model_parse_error(prefix + ".qweight is not I32 [" + std::to_string(K) + ", " + std::to_string(N / 8) + "]");
    if (qz->dtype != "I32" || !shape_is(*qz, K / g, N / 8)) return base::error::model_parse_error(prefix + ".qzeros is not I32 [in/group, out/8]");
    if (sc->dtype != "F16" || !shape_is(*sc, K / g, N)) return base::error::model_parse_error(prefix + ".scales is not F16 [in/group, out]");
    out->layer = std::make_unique<op::MatmulLayer>(base::DeviceType::DeviceCPU, N, K, true);
    out->layer->set_group_size(g);
    RETURN_IF_ERROR(out->layer->set_weight(0, {K, N / 8}, qw->data, base::DeviceType::DeviceCPU));
    RETURN_IF_ERROR(out->layer->set_weight(1, {K / g, N / 8}, qz->data, base::DeviceType::DeviceCPU));
    tensor::Tensor scales(DataType::DataTypeFp16, std::vector<int32_t>{K / g, N}, false, nullptr, const_cast<unsigned char*>(sc->data));
    scales.set_device_type(base::DeviceType::DeviceCPU);
    out->layer->set_scales(scales);
    out->K = K;
    out->N = N;
    return base::error::success();
}

// N-concatenation of staged projections that share K: packed words and zeros by word columns, scales by columns
void fuse_columns(const std::vector<const StagedProjection*>& parts, int32_t g, std::vector<int32_t>* qw, std::vector<int32_t>* qz,
                  std::vector<uint16_t>* sc) {
    const int32_t K = parts[0]->K;
    int32_t N = 0;
    for (const StagedProjection* p : parts) N += p->N;
    qw->resize(size_t(K) * (N / 8));
    qz->resize(size_t(K / g) * (N / 8));
    sc->resize(size_t(K / g) * N);
    int32_t col = 0;
    for (const StagedProjection* p : parts) {
        const int32_t* w = p->layer->get_weight(0).ptr<int32_t>();
        const int32_t* z = p->layer->get_weight(1).ptr<int32_t>();
        const uint16_t* s = p->layer->scales().ptr<uint16_t>();
        for (int32_t k = 0; k < K; k++)
            std::memcpy(qw->data() + size_t(k) * (N / 8) + col / 8, w + size_t(k) * (p->N / 8), size_t(p->N / 8) * 4);
        for (int32_t r = 0; r < K / g; r++) {
            std::memcpy(qz->data() + size_t(r) * (N / 8) + col / 8, z + size_t(r) * (p->N / 8), size_t(p->N / 8) * 4);
            std::memcpy(sc->data() + size_t(r) * N + col, s + size_t(r) * p->N, size_t(p->N) * 2);
        }
        col += p->N;
    }
}

}  // namespace

base::Status Qwen3Model::load_checkpoint(const std::string& path) {
    if (layers_.empty()) return base::error::internal_error("init() must run before load_checkpoint()");
    std::unique_ptr<SafetensorsFile> file;
    RETURN_IF_ERROR(SafetensorsFile::open(path, &file));
    const ModelConfig& c = config_;
    const int32_t D = c.head_size, H = c.dim, g = c.group_size, I = c.hidden_dim;
    auto named = [&](const std::string& name, const CheckpointTensor** t) -> base::Status {
        *t = file->find(name);
        if (!*t) return base::error::model_parse_error("tensor " + name + " is missing from " + path);
        return base::error::success();
    };
    std::vector<uint16_t> in_norm, post_norm, q_norm, k_norm, sc_qkv, sc_gu;
    std::vector<int32_t> qw_qkv, qz_qkv, qw_gu, qz_gu;
    for (int32_t l = 0; l < c.layer_num; l++) {
        const std::string base_name = "model.layers." + std::to_string(l);
        const CheckpointTensor* t = nullptr;
        RETURN_IF_ERROR(named(base_name + ".input_layernorm.weight", &t));
        RETURN_IF_ERROR(to_bf16(*t, H, base_name + ".input_layernorm.weight", &in_norm));
        RETURN_IF_ERROR(named(base_name + ".post_attention_layernorm.weight", &t));
        RETURN_IF_ERROR(to_bf16(*t, H, base_name + ".post_attention_layernorm.weight", &post_norm));
        RETURN_IF_ERROR(named(base_name + ".self_attn.q_norm.weight", &t));
        RETURN_IF_ERROR(to_bf16(*t, D, base_name + ".self_attn.q_norm.weight", &q_norm));
        RETURN_IF_ERROR(named(base_name + ".self_attn.k_norm.weight", &t));
        RETURN_IF_ERROR(to_bf16(*t, D, base_name + ".self_attn.k_norm.weight", &k_norm));
        StagedProjection q, k, v, o, gate, up, down;
        RETURN_IF_ERROR(stage_projection(*file, base_name + ".self_attn.q_proj", H, c.head_num * D, g, &q));
        RETURN_IF_ERROR(stage_projection(*file, base_name + ".self_attn.k_proj", H, c.kv_head_num * D, g, &k));
        RETURN_IF_ERROR(stage_projection(*file, base_name + ".self_attn.v_proj", H, c.kv_head_num * D, g, &v));
        RETURN_IF_ERROR(stage_projection(*file, base_name + ".self_attn.o_proj", c.head_num * D, H, g, &o));
        RETURN_IF_ERROR(stage_projection(*file, base_name + ".mlp.gate_proj", H, I, g, &gate));
        RETURN_IF_ERROR(stage_projection(*file, base_name + ".mlp.up_proj", H, I, g, &up));
        RETURN_IF_ERROR(stage_projection(*file, base_name + ".mlp.down_proj", I, H, g, &down));
        fuse_columns({&q, &k, &v}, g, &qw_qkv, &qz_qkv, &sc_qkv);   // q heads | k heads | v heads
        fuse_columns({&gate, &up}, g, &qw_gu, &qz_gu, &sc_gu);        // gate | up
        RawLayerWeights w;
        w.input_norm = in_norm.data(); w.post_norm = post_norm.data(); w.q_norm = q_norm.data(); w.k_norm = k_norm.data();
        w.qkv_qw = qw_qkv.data(); w.qkv_qz = qz_qkv.data(); w.qkv_s = sc_qkv.data();
        w.o_qw = o.layer->get_weight(0).ptr<void>(); w.o_qz = o.layer->get_weight(1).ptr<void>(); w.o_s = o.layer->scales().ptr<void>();
        w.gu_qw = qw_gu.data(); w.gu_qz = qz_gu.data(); w.gu_s = sc_gu.data();
        w.down_qw = down.layer->get_weight(0).ptr<void>(); w.down_qz = down.layer->get_weight(1).ptr<void>();
        w.down_s = down.layer->scales().ptr<void>();
        RETURN_IF_ERROR(load_layer(l, w, false));
    }
    const CheckpointTensor *embed = nullptr, *norm = nullptr;
    RETURN_IF_ERROR(named("model.embed_tokens.weight", &embed));
    RETURN_IF_ERROR(named("model.norm.weight", &norm));
    const CheckpointTensor* head = file->find("lm_head.weight");  // absent: tied to the embedding
    std::vector<uint16_t> embed_b, norm_b, head_b;
    RETURN_IF_ERROR(to_bf16(*embed, int64_t(c.vocab_size) * H, "model.embed_tokens.weight", &embed_b));
    RETURN_IF_ERROR(to_bf16(*norm, H, "model.norm.weight", &norm_b));
    if (head) RETURN_IF_ERROR(to_bf16(*head, int64_t(c.vocab_size) * H, "lm_head.weight", &head_b));
    return load_globals(embed_b.data(), norm_b.data(), head ? head_b.data() : embed_b.data(), false);
}

base::Status Qwen3Model::check_loaded() const {
    if (!globals_loaded_) return base::error::model_parse_error("embedding / lm_head weights are not loaded");
    for (size_t i = 0; i < layer_loaded_.size(); i++)
        if (!layer_loaded_[i]) return base::error::model_parse_error("layer " + std::to_string(i) + " is not loaded");
    if (config_.tp_size > 1 && !communicator_)
        return base::error::internal_error("tensor-parallel communicator is not initialised");
    return base::error::success();
}

// ------------------------------------------------------------------ one pass
base::Status Qwen3Model::upload_rows(const int32_t* tokens, const int32_t* pos, const int32_t* slot, int32_t M) {
    const int32_t R = config_.max_rows;
    if (M <= 0 || M > R) return base::error::invalid_argument("row count exceeds max_rows");
    for (int32_t m = 0; m < M; m++) {
        if (tokens[m] < 0 || tokens[m] >= config_.vocab_size) return base::error::invalid_argument("token id out of range");
        if (pos[m] < 0 || pos[m] >= config_.max_seq_len) return base::error::invalid_argument("position exceeds max_seq_len");
        if (slot[m] < 0 || slot[m] >= config_.max_batch) return base::error::invalid_argument("sequence slot out of range");
    }
    {
        std::vector<int32_t> lo(size_t(config_.max_batch), INT32_MAX), hi(size_t(config_.max_batch), -1);
        for (int32_t m = 0; m < M; m++) {
            lo[size_t(slot[m])] = std::min(lo[size_t(slot[m])], pos[m]);
            hi[size_t(slot[m])] = std::max(hi[size_t(slot[m])], pos[m]);
        }
        // a prompt chunk: one sequence, consecutive positions
        chunk_pos0_ = pos[0];
        chunk_slot_ = slot[0];
        rows_are_chunk_ = M >= kPrefillAttentionMinRows;
        for (int32_t m = 1; m < M && rows_are_chunk_; m++)
            if (slot[m] != slot[0] || pos[m] != pos[0] + m) rows_are_chunk_ = false;
        rows_compact_ = true;
        for (int32_t b = 0; b < config_.max_batch; b++)
            if (hi[size_t(b)] >= 0 && hi[size_t(b)] - lo[size_t(b)] >= M) rows_compact_ = false;
        std::vector<char> seen(size_t(config_.max_batch), 0);
        slots_distinct_ = true;
        for (int32_t m = 0; m < M; m++) {
            if (seen[size_t(slot[m])]) slots_distinct_ = false;
            seen[size_t(slot[m])] = 1;
        }
    }
    cudaStream_t s = stream();
    CUDA_OK(cudaStreamSynchronize(s));  // the pinned stage may still feed an earlier copy
    int32_t* st = host_stage_;
    for (int32_t m = 0; m < M; m++) {
        st[m] = tokens[m];
        st[R + m] = pos[m];
        st[2 * R + m] = pos[m] + 1;
        st[3 * R + m] = slot[m];
    }
    const size_t n = size_t(M) * 4;
    CUDA_OK(cudaMemcpyAsync(get_buffer(ModelBufferType::InputTokens).ptr<void>(), st, n, cudaMemcpyHostToDevice, s));
    CUDA_OK(cudaMemcpyAsync(get_buffer(ModelBufferType::InputPos).ptr<void>(), st + R, n, cudaMemcpyHostToDevice, s));
    CUDA_OK(cudaMemcpyAsync(get_buffer(ModelBufferType::SeqLen).ptr<void>(), st + 2 * R, n, cudaMemcpyHostToDevice, s));
    CUDA_OK(cudaMemcpyAsync(get_buffer(ModelBufferType::SeqSlot).ptr<void>(), st + 3 * R, n, cudaMemcpyHostToDevice, s));
    return base::error::success();
}

base::Status Qwen3Model::run_pass(int32_t M, bool inputs_settled) {
    const ModelConfig& c = config_;
    const int32_t D = c.head_size, H = c.dim;
    const int32_t Hq = local_heads(), Hkv = local_kv_heads(), I = local_hidden();
    const int32_t QKV = (Hq + 2 * Hkv) * D;
    const DataType F = DataType::DataTypeFp32, I32 = DataType::DataTypeInt32;

    const Tensor tokens = view(get_buffer(ModelBufferType::InputTokens), I32, {M});
    const Tensor pos = view(get_buffer(ModelBufferType::InputPos), I32, {M});
    const Tensor seq_len = view(get_buffer(ModelBufferType::SeqLen), I32, {M});
    const Tensor slot = view(get_buffer(ModelBufferType::SeqSlot), I32, {M});
    Tensor h = view(get_buffer(ModelBufferType::InputEmbeddings), F, {M, H});
    Tensor h_alt = view(get_buffer(ModelBufferType::AttnOutput), F, {M, H});
    const Tensor xn = view(get_buffer(ModelBufferType::OutputRMSNorm), F, {M, H});
    const Tensor xn2 = view(get_buffer(ModelBufferType::FFNRMSNorm), F, {M, H});
    const Tensor qkv = view(get_buffer(ModelBufferType::QKVOutput), F, {M, QKV});
    const Tensor q = view(get_buffer(ModelBufferType::Query), F, {M, Hq * D});
    const Tensor att = view(get_buffer(ModelBufferType::OutputMHA), F, {M, Hq * D});
    const Tensor gu = view(get_buffer(ModelBufferType::W1Output), F, {M, 2 * I});
    const Tensor act = view(get_buffer(ModelBufferType::W2Output), F, {M, I});
    const Tensor logits = view(get_buffer(ModelBufferType::ForwardOutput), F, {M, c.vocab_size});
    const Tensor next = view(get_buffer(ModelBufferType::NextTokens), I32, {M});
    const Tensor& cos_t = get_buffer(ModelBufferType::CosCache);
    const Tensor& sin_t = get_buffer(ModelBufferType::SinCache);
    const bool tp = c.tp_size > 1;

    // row-split projection: h += x.W summed over ranks
    auto project_and_reduce = [&](op::MatmulLayer& layer, const Tensor& x) -> base::Status {
        if (!tp) return accumulate_ ? layer.forward(x, h) : layer.forward(x, h, h);
        // this rank's partial row goes into the zeroed buffer (accumulated, or written by the ordered kernel)
        RETURN_IF_ERROR(layer.forward(x, h_alt));
        float* partial = const_cast<float*>(h_alt.ptr<float>());
        float* hp = const_cast<float*>(h.ptr<float>());
        const size_t count = size_t(M) * H;
        if (communicator_->fits_one_shot(count))
            return communicator_->exchange_sum(partial, hp, hp, count, stream());  // h = h + sum_r partial_r; clears partial
        RETURN_IF_ERROR(communicator_->all_reduce_sum(partial, count, stream()));
        kernel::get_add_kernel(device_type_)(h, h_alt, h, stream());
        CUDA_OK(cudaMemsetAsync(partial, 0, count * sizeof(float), stream()));
        return base::error::success();
    };

    RETURN_IF_ERROR(embedding_->forward(tokens, h));
    for (Qwen3Layer& L : layers_) {
        if (accumulate_cols_) {
            RETURN_IF_ERROR(L.qkv->forward(h, qkv));  // RMSNorm fused into the projection
        } else {
            RETURN_IF_ERROR(L.input_norm->forward(h, xn));
            RETURN_IF_ERROR(L.qkv->forward(xn, qkv));
        }
        if (accumulate_cols_ && inputs_settled && slots_distinct_) {
            // decode batch: rotary, KV append and attention in one kernel; every cache row but the one appended
            // here is older than this pass
            RETURN_IF_ERROR(L.rope->forward_with_attention(qkv, pos, slot, cos_t, sin_t, seq_len, att, 1));
        } else {
            RETURN_IF_ERROR(L.rope->forward(qkv, pos, slot, cos_t, sin_t, q));
            // the rotary kernel just before appended one cache row per token row of this pass; when the rows of a
            // sequence lie within M consecutive positions, every cache row below seq_len - M is older than this pass.
            // The promise also covers seq_len / slot, so it is only made when those were settled before the pass
            // (kernels under programmatic dependent launch may start ahead of earlier copies of the same pass).
            if (rows_are_chunk_ && !inputs_settled) {
                // prompt chunk of one sequence: tiled causal attention, K / V tiles shared by a block of query rows
                RETURN_IF_ERROR(L.mha->forward_prefill(q, chunk_pos0_, chunk_slot_, att));
            } else {
                L.mha->set_fresh_rows(rows_compact_ && inputs_settled ? M : -1);
                RETURN_IF_ERROR(L.mha->forward(q, seq_len, slot, att));
            }
        }
        RETURN_IF_ERROR(project_and_reduce(*L.o, att));
        if (accumulate_cols_) {
            RETURN_IF_ERROR(L.gate_up->forward(h, gu));
        } else {
            RETURN_IF_ERROR(L.post_norm->forward(h, xn2));
            RETURN_IF_ERROR(L.gate_up->forward(xn2, gu));
        }
        if (accumulate_) {
            RETURN_IF_ERROR(project_and_reduce(*L.down, gu));  // SwiGLU fused into the projection
        } else {
            RETURN_IF_ERROR(L.swiglu->forward(gu, act));
            RETURN_IF_ERROR(project_and_reduce(*L.down, act));
        }
    }
    if (logit_rows_ > 0) {
        // logits only for the last logit_rows_ rows of the pass
        const int32_t r0 = M - logit_rows_;
        const Tensor h_tail = view(h, F, {logit_rows_, H}, size_t(r0) * H);
        const Tensor xn_tail = view(xn, F, {logit_rows_, H}, size_t(r0) * H);
        const Tensor lg_tail = view(logits, F, {logit_rows_, c.vocab_size}, size_t(r0) * c.vocab_size);
        const Tensor nx_tail = view(next, I32, {logit_rows_}, size_t(r0));
        RETURN_IF_ERROR(final_norm_->forward(h_tail, xn_tail));
        if (vocab_local_ == c.vocab_size) {
            RETURN_IF_ERROR(lm_head_->forward(xn_tail, lg_tail));
            sampler_->sample(lg_tail, nx_tail, stream());
        } else {
            // vocabulary-split lm_head: every rank scores its slice
            const Tensor shard = view(get_buffer(ModelBufferType::LogitsShard), F, {logit_rows_, vocab_local_});
            RETURN_IF_ERROR(lm_head_->forward(xn_tail, shard));
            base::Status ex = base::error::function_not_implement("");
            if (inputs_settled)  // decode graph: only the per-rank (maximum, index) pairs travel
                ex = communicator_->exchange_argmax(shard.ptr<float>(), const_cast<int32_t*>(nx_tail.ptr<int32_t>()), logit_rows_,
                                                    vocab_local_, stream());
            if (!ex) {
                if (ex.get_err_code() != base::StatusCode::FunctionUnImplement) return ex;
                // eager passes (and ranks without the peer-memory path): gather the slices into whole rows, so that
                // read_logits() sees them, and pick on the whole row
                float* gathered = const_cast<float*>(get_buffer(ModelBufferType::LogitsGather).ptr<float>());
                const size_t slice = size_t(logit_rows_) * vocab_local_;
                RETURN_IF_ERROR(communicator_->all_gather(shard.ptr<float>(), gathered, slice, stream()));
                for (int32_t r = 0; r < c.tp_size; r++)
                    CUDA_OK(cudaMemcpy2DAsync(const_cast<float*>(lg_tail.ptr<float>()) + size_t(r) * vocab_local_,
                                              size_t(c.vocab_size) * 4, gathered + size_t(r) * slice, size_t(vocab_local_) * 4,
                                              size_t(vocab_local_) * 4, size_t(logit_rows_), cudaMemcpyDeviceToDevice, stream()));
                sampler_->sample(lg_tail, nx_tail, stream());
            }
        }
    }
    return base::error::success();
}

// Called after a stream synchronisation: a tensor-parallel exchange whose bounded wait ran out leaves this rank
// with a partial sum, so everything read back after it is void and the caller must hear about it.
base::Status Qwen3Model::check_exchange() const {
    if (config_.tp_size > 1 && communicator_) return communicator_->one_shot_status(true);
    return base::error::success();
}

// The pipelined GEMV, the tcgen05 GEMM and the fused attention kernel bound every wait and record a word on the device when one runs out
// (their results are void then).  Reading the words costs two small synchronous copies, so this runs where the caller
// already pays for a synchronisation that is not on the per-token path: after a prefill, in decode_read and synchronize.
base::Status Qwen3Model::check_kernels() const {
    if (kuiper_awq_gemv_status() != 0 || kuiper_awq_gemm_status() != 0 || kuiper_flash_decode_status() != 0)
        return base::error::internal_error(kuiper_last_error());
    return base::error::success();
}

base::Status Qwen3Model::synchronize() {
    CUDA_OK(cudaStreamSynchronize(stream()));
    RETURN_IF_ERROR(check_exchange());
    return check_kernels();
}

base::Status Qwen3Model::forward(const int32_t* tokens, const int32_t* pos, const int32_t* slot, int32_t M) {
    RETURN_IF_ERROR(check_loaded());
    if (!tokens || !pos || !slot) return base::error::invalid_argument("null input pointer");
    RETURN_IF_ERROR(upload_rows(tokens, pos, slot, M));
    logit_rows_ = M;
    return run_pass(M);
}

base::Status Qwen3Model::predict(const int32_t* tokens, const int32_t* pos, const int32_t* slot, int32_t M,
                                 int32_t* next) {
    if (!next) return base::error::invalid_argument("null output pointer");
    RETURN_IF_ERROR(forward(tokens, pos, slot, M));
    int32_t* st = host_stage_;
    CUDA_OK(cudaMemcpyAsync(st, get_buffer(ModelBufferType::NextTokens).ptr<void>(), size_t(M) * 4,
                            cudaMemcpyDeviceToHost, stream()));
    CUDA_OK(cudaStreamSynchronize(stream()));
    RETURN_IF_ERROR(check_exchange());
    std::memcpy(next, st, size_t(M) * 4);
    return base::error::success();
}

base::Status Qwen3Model::prefill(const int32_t* tokens, int32_t n, int32_t slot, int32_t* next) {
    RETURN_IF_ERROR(check_loaded());
    if (!tokens || n <= 0) return base::error::invalid_argument("empty prompt");
    if (n > config_.max_seq_len) return base::error::invalid_argument("prompt exceeds max_seq_len");
    const int32_t R = config_.max_rows;
    std::vector<int32_t> pos(static_cast<size_t>(R), 0);
    std::vector<int32_t> slots(static_cast<size_t>(R), slot);
    for (int32_t base_pos = 0; base_pos < n; base_pos += R) {
        const int32_t M = std::min(R, n - base_pos);
        for (int32_t m = 0; m < M; m++) pos[size_t(m)] = base_pos + m;
        RETURN_IF_ERROR(upload_rows(tokens + base_pos, pos.data(), slots.data(), M));
        const bool last = base_pos + M >= n;
        logit_rows_ = last ? 1 : 0;  // only the final token's logits are needed
        RETURN_IF_ERROR(run_pass(M));
        if (last && next) {
            CUDA_OK(cudaMemcpyAsync(host_stage_, get_buffer(ModelBufferType::NextTokens).ptr<int32_t>() + (M - 1), 4,
                                    cudaMemcpyDeviceToHost, stream()));
            CUDA_OK(cudaStreamSynchronize(stream()));
            *next = host_stage_[0];
        }
    }
    return synchronize();
}

// ------------------------------------------------------------------ graph decode loop
base::Status Qwen3Model::ensure_graph(int32_t B) {
    if (graphs_.count(B)) return base::error::success();
    cudaStream_t s = stream();
    logit_rows_ = B;
    // one eager pass first: it configures every kernel variant outside the capture and
    // leaves the same cache contents the captured step will write again
    RETURN_IF_ERROR(run_pass(B, true));
    CUDA_OK(cudaStreamSynchronize(s));

    // capture `steps` consecutive decode steps (pass + advance) into one executable graph
    auto capture = [&](int32_t steps, cudaGraphExec_t* out, int32_t* kernel_nodes) -> base::Status {
        cudaGraph_t graph = nullptr;
        CUDA_OK(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
        base::Status st = base::error::success();
        for (int32_t i = 0; i < steps && st; i++) {
            st = run_pass(B, true);
            if (st) {
                const int rc = kuiper_decode_advance(get_buffer(ModelBufferType::InputTokens).ptr<int32_t>(),
                                                     get_buffer(ModelBufferType::NextTokens).ptr<int32_t>(),
                                                     get_buffer(ModelBufferType::InputPos).ptr<int32_t>(),
                                                     get_buffer(ModelBufferType::SeqLen).ptr<int32_t>(), B,
                                                     config_.max_seq_len, reinterpret_cast<kuiper_stream_t>(s));
                if (rc != 0) st = base::error::internal_error(kuiper_last_error());
            }
        }
        cudaError_t end = cudaStreamEndCapture(s, &graph);
        if (!st) {
            if (graph) cudaGraphDestroy(graph);
            return st;
        }
        CUDA_OK(end);
        if (kernel_nodes) {
            size_t n_nodes = 0;
            CUDA_OK(cudaGraphGetNodes(graph, nullptr, &n_nodes));
            std::vector<cudaGraphNode_t> nodes(n_nodes);
            CUDA_OK(cudaGraphGetNodes(graph, nodes.data(), &n_nodes));
            int32_t kernels = 0;
            for (cudaGraphNode_t node : nodes) {
                cudaGraphNodeType type;
                if (cudaGraphNodeGetType(node, &type) == cudaSuccess && type == cudaGraphNodeTypeKernel) kernels++;
            }
            *kernel_nodes = kernels;
        }
        cudaError_t inst = cudaGraphInstantiate(out, graph, 0);
        cudaGraphDestroy(graph);
        CUDA_OK(inst);
        return base::error::success();
    };
    cudaGraphExec_t single = nullptr, unrolled = nullptr;
    RETURN_IF_ERROR(capture(1, &single, &kernels_per_step_));
    graphs_[B] = single;
    RETURN_IF_ERROR(capture(kGraphUnroll, &unrolled, nullptr));
    graphs_unrolled_[B] = unrolled;
    return base::error::success();
}

base::Status Qwen3Model::decode_begin(const int32_t* tokens, const int32_t* pos, const int32_t* slot, int32_t B) {
    RETURN_IF_ERROR(check_loaded());
    if (!tokens || !pos || !slot) return base::error::invalid_argument("null input pointer");
    if (B <= 0 || B > config_.max_batch) return base::error::invalid_argument("batch exceeds max_batch");
    RETURN_IF_ERROR(upload_rows(tokens, pos, slot, B));
    CUDA_OK(cudaStreamSynchronize(stream()));
    decode_batch_ = B;
    return ensure_graph(B);
}

base::Status Qwen3Model::decode_step(int32_t n_steps) {
    if (decode_batch_ <= 0) return base::error::internal_error("decode_begin() has not been called");
    cudaGraphExec_t exec = graphs_[decode_batch_], exec_unrolled = graphs_unrolled_[decode_batch_];
    int32_t i = 0;
    for (; i + kGraphUnroll <= n_steps; i += kGraphUnroll) CUDA_OK(cudaGraphLaunch(exec_unrolled, stream()));
    for (; i < n_steps; i++) CUDA_OK(cudaGraphLaunch(exec, stream()));
    return base::error::success();
}

base::Status Qwen3Model::decode_read(int32_t* tokens, int32_t B) {
    if (!tokens || B <= 0 || B > config_.max_rows) return base::error::invalid_argument("bad read request");
    CUDA_OK(cudaMemcpyAsync(host_stage_, get_buffer(ModelBufferType::NextTokens).ptr<void>(), size_t(B) * 4,
                            cudaMemcpyDeviceToHost, stream()));
    RETURN_IF_ERROR(synchronize());
    std::memcpy(tokens, host_stage_, size_t(B) * 4);
    return base::error::success();
}

base::Status Qwen3Model::decode_predict(const int32_t* tokens, int32_t B, int32_t* next) {
    if (decode_batch_ != B) return base::error::internal_error("decode_begin() was not called for this batch size");
    if (!tokens || !next) return base::error::invalid_argument("null pointer");
    for (int32_t b = 0; b < B; b++)
        if (tokens[b] < 0 || tokens[b] >= config_.vocab_size) return base::error::invalid_argument("token id out of range");
    cudaStream_t s = stream();
    const int32_t R = config_.max_rows;
    std::memcpy(host_stage_, tokens, size_t(B) * 4);
    CUDA_OK(cudaMemcpyAsync(get_buffer(ModelBufferType::InputTokens).ptr<void>(), host_stage_, size_t(B) * 4,
                            cudaMemcpyHostToDevice, s));
    CUDA_OK(cudaGraphLaunch(graphs_[B], s));
    CUDA_OK(cudaMemcpyAsync(host_stage_ + R, get_buffer(ModelBufferType::NextTokens).ptr<void>(), size_t(B) * 4,
                            cudaMemcpyDeviceToHost, s));
    CUDA_OK(cudaStreamSynchronize(s));
    RETURN_IF_ERROR(check_exchange());
    std::memcpy(next, host_stage_ + R, size_t(B) * 4);
    return base::error::success();
}

base::Status Qwen3Model::read_logits(float* out, int32_t M) {
    if (!out || M <= 0 || M > config_.max_rows) return base::error::invalid_argument("bad read request");
    CUDA_OK(cudaStreamSynchronize(stream()));
    CUDA_OK(cudaMemcpy(out, get_buffer(ModelBufferType::ForwardOutput).ptr<void>(),
                       size_t(M) * config_.vocab_size * 4, cudaMemcpyDeviceToHost));
    return base::error::success();
}

}  // namespace model
