// Shape of a Qwen3-style decoder and of the engine's runtime limits.
#ifndef KUIPER_INCLUDE_MODEL_CONFIG_H
#define KUIPER_INCLUDE_MODEL_CONFIG_H

#include <cstdint>

namespace model {

struct ModelConfig {
    int32_t layer_num = 0;
    int32_t dim = 0;           // hidden width
    int32_t head_num = 0;      // query heads
    int32_t kv_head_num = 0;
    int32_t head_size = 128;
    int32_t hidden_dim = 0;    // SwiGLU intermediate width
    int32_t vocab_size = 0;
    int32_t group_size = 128;  // AWQ group along the input dimension
    int32_t max_seq_len = 0;   // KV-cache capacity per sequence
    int32_t max_batch = 1;     // sequences held in the KV cache
    int32_t max_rows = 8;      // token rows per forward pass (decode batch or prompt chunk)
    float eps = 1e-6f;
    double rope_theta = 1e6;
    int32_t act_mode = 1;      // INT4 matmul operand rounding: 1 fp16, 0 fp32
    int32_t tp_rank = 0;
    int32_t tp_size = 1;
};

// Unsharded weights of one decoder layer as raw pointers (host or device memory).
// Fused projections: qkv is [dim -> (head_num + 2 kv_head_num) * head_size] with columns
// q heads | k heads | v heads; gate_up is [dim -> 2 hidden_dim] with columns gate | up.
struct RawLayerWeights {
    const void* input_norm = nullptr;  // bf16 [dim]
    const void* post_norm = nullptr;   // bf16 [dim]
    const void* q_norm = nullptr;      // bf16 [head_size]
    const void* k_norm = nullptr;      // bf16 [head_size]
    const void *qkv_qw = nullptr, *qkv_qz = nullptr, *qkv_s = nullptr;
    const void *o_qw = nullptr, *o_qz = nullptr, *o_s = nullptr;
    const void *gu_qw = nullptr, *gu_qz = nullptr, *gu_s = nullptr;
    const void *down_qw = nullptr, *down_qz = nullptr, *down_s = nullptr;
};

}  // namespace model

#endif  // KUIPER_INCLUDE_MODEL_CONFIG_H
