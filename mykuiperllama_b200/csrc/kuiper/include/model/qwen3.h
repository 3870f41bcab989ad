// Qwen3-shaped INT4-AWQ decoder: per layer
//   RMSNorm -> fused QKV matmul -> per-head q/k norm + rotary + KV append -> GQA
//   flash-decoding -> O matmul (+residual) -> RMSNorm -> fused gate|up matmul -> SwiGLU ->
//   down matmul (+residual); then final RMSNorm -> bf16 lm_head -> greedy argmax.
// With tensor parallelism QKV and gate|up are column-split, O and down row-split, and the
// partial rows of O and down are summed with one all-reduce each.
//
// Decode runs as a captured CUDA graph per batch size; the graph also feeds the chosen
// token back as the next input and advances the positions, so a run of decode steps needs
// no host interaction.
#ifndef KUIPER_INCLUDE_MODEL_QWEN3_H
#define KUIPER_INCLUDE_MODEL_QWEN3_H

#include <cuda_runtime_api.h>

#include "model/model.h"
#include "op/add.h"
#include "op/embedding.h"
#include "op/matmul.h"
#include "op/mha.h"
#include "op/rmsnorm.h"
#include "op/rope.h"
#include "op/swiglu.h"
#include "sampler/argmax_sampler.h"

namespace model {

struct Qwen3Layer {
    std::unique_ptr<op::RmsNormLayer> input_norm, post_norm;
    std::unique_ptr<op::MatmulLayer> qkv, o, gate_up, down;
    std::unique_ptr<op::RoPELayer> rope;
    std::unique_ptr<op::MultiHeadAttention> mha;
    std::unique_ptr<op::SwiGLULayer> swiglu;
    tensor::Tensor key_cache, value_cache;  // bf16 [max_batch, local kv heads, max_seq, head_size]
};

class Qwen3Model : public Model {
public:
    explicit Qwen3Model(const ModelConfig& config);
    ~Qwen3Model() override;

    base::Status init(base::DeviceType device_type) override;
    base::Status forward(const int32_t* tokens, const int32_t* pos, const int32_t* slot, int32_t M) override;
    base::Status predict(const int32_t* tokens, const int32_t* pos, const int32_t* slot, int32_t M,
                         int32_t* next) override;

    // weights: copied (and sharded for this rank) into engine-owned device memory
    base::Status load_layer(int32_t layer, const RawLayerWeights& w, bool on_device);
    base::Status load_globals(const void* embed, const void* final_norm, const void* lm_head, bool on_device);

    // Every weight from an AWQ checkpoint in the safetensors container (Hugging Face tensor names of a quantised Qwen3
    // model: separate q / k / v and gate / up projections, which are fused here); the file's tensors enter through
    // LayerParam::set_weight(idx, dims, ptr, DeviceCPU) as borrowed pointers into the mapping and are then copied, and
    // under tensor parallelism sharded, into the model's own device memory.
    base::Status load_checkpoint(const std::string& path);

    // whole prompt of one sequence, in chunks of max_rows; `next` = greedy id after the last token
    base::Status prefill(const int32_t* tokens, int32_t n, int32_t slot, int32_t* next);

    // device-resident decode loop over B sequences: begin() uploads the current token and
    // position of each sequence; step() replays the decode graph n times with no host
    // interaction; read() returns the tokens chosen by the last step (synchronises).
    base::Status decode_begin(const int32_t* tokens, const int32_t* pos, const int32_t* slot, int32_t B);
    base::Status decode_step(int32_t n_steps);
    base::Status decode_read(int32_t* tokens, int32_t B);
    // one end-to-end step of that loop: host tokens in, host tokens out (synchronises)
    base::Status decode_predict(const int32_t* tokens, int32_t B, int32_t* next);

    // copy of the last pass's logits [M, vocab] to the host (synchronises)
    base::Status read_logits(float* out, int32_t M);
    // waits for everything enqueued on the model's stream, then reports a tensor-parallel exchange or a kernel
    // pipeline whose bounded wait ran out since the last check
    base::Status synchronize();
    // number of kernels one decode step launches
    int32_t kernels_per_step() const { return kernels_per_step_; }

private:
    // enqueue one pass over the first M rows of the input buffers; inputs_settled: positions / slots were on the
    // device before anything of this pass was enqueued (the decode graph), not copied in by the pass's own memcpys
    base::Status run_pass(int32_t M, bool inputs_settled = false);
    base::Status upload_rows(const int32_t* tokens, const int32_t* pos, const int32_t* slot, int32_t M);
    base::Status ensure_graph(int32_t B);
    base::Status check_loaded() const;
    base::Status check_exchange() const;
    base::Status check_kernels() const;

    int32_t local_heads() const { return config_.head_num / config_.tp_size; }
    int32_t local_kv_heads() const { return config_.kv_head_num / config_.tp_size; }
    int32_t local_hidden() const { return config_.hidden_dim / config_.tp_size; }

    std::shared_ptr<base::DeviceAllocator> weight_alloc_;  // arena holding weights, caches and step buffers
    std::vector<Qwen3Layer> layers_;
    std::unique_ptr<op::EmbeddingLayer> embedding_;
    std::unique_ptr<op::RmsNormLayer> final_norm_;
    std::unique_ptr<op::MatmulLayer> lm_head_;
    std::unique_ptr<sampler::ArgmaxSampler> sampler_;
    std::vector<bool> layer_loaded_;
    bool globals_loaded_ = false;
    int32_t vocab_local_ = 0;       // rows of the lm_head on this rank (the vocabulary is split under tensor parallelism)
    bool accumulate_ = false;       // every projection runs in accumulate mode (single GPU, see init)
    bool accumulate_cols_ = false;  // the column-split projections (QKV, gate|up) do; true under tensor parallelism too

    // pinned staging for the host <-> device token traffic
    int32_t* host_stage_ = nullptr;
    std::map<int32_t, cudaGraphExec_t> graphs_;  // decode graph per batch size
    // the same step captured kGraphUnroll times in one graph: a run of decode steps then pays the gap between two
    // graph launches once per kGraphUnroll tokens
    std::map<int32_t, cudaGraphExec_t> graphs_unrolled_;
    static constexpr int32_t kGraphUnroll = 4;
    int32_t decode_batch_ = 0;
    int32_t kernels_per_step_ = 0;
    int32_t logit_rows_ = 0;  // rows (counted from the end of a pass) that get logits and a sampled id
    // the rows of the current pass that share a sequence slot lie within `rows` consecutive positions, so the
    // attention kernel may fetch all older cache rows before the rotary kernel has finished
    bool rows_compact_ = false;
    bool slots_distinct_ = false;  // every row of the current pass has its own sequence slot
    // the rows of the current pass are consecutive tokens of one sequence (a prompt chunk): position of the first row,
    // the sequence slot; chunks of at least kPrefillAttentionMinRows rows take the tiled prefill attention kernel
    bool rows_are_chunk_ = false;
    int32_t chunk_pos0_ = 0, chunk_slot_ = 0;
    static constexpr int32_t kPrefillAttentionMinRows = 16;
};

}  // namespace model

#endif  // KUIPER_INCLUDE_MODEL_QWEN3_H
