/*
 * kuiper_llama - C ABI of the C++ engine (model::Qwen3Model and the layers under it).
 *
 * The reference drives its model from C++ (Model::forward / predict; the directory is
 * absent in the mounted snapshot, CMakeLists.txt:79).  This header is the same surface
 * for callers that cannot include the C++ headers (Python tests, the benchmark, other
 * language bindings): plain pointers and sizes, int status codes numbered like
 * base::StatusCode (kuiper/include/base/base.h:76-84).
 */
#ifndef KUIPER_LLAMA_H
#define KUIPER_LLAMA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KUIPER_LLAMA_API __attribute__((visibility("default")))

typedef struct kuiper_model kuiper_model;

typedef struct {
    int32_t n_layers, hidden, n_q_heads, n_kv_heads, head_dim, inter, vocab, group;
    int32_t max_seq, max_batch, max_rows;
    float eps;
    double rope_theta;
    int32_t act_mode; /* INT4 matmul operand: 1 rounds x to fp16, 0 keeps fp32, 2 block-scaled 16-bit integers for one-row
                         passes (decode steps of one sequence: the fastest kernel) and fp16 for passes of several rows */
    int32_t tp_rank, tp_size;
} kuiper_model_config;

/* unsharded weights of one layer; the engine copies (and shards) them into its own memory */
typedef struct {
    const void *input_norm, *post_norm, *q_norm, *k_norm;
    const void *qkv_qw, *qkv_qz, *qkv_s;
    const void *o_qw, *o_qz, *o_s;
    const void *gu_qw, *gu_qz, *gu_s;
    const void *down_qw, *down_qz, *down_s;
} kuiper_layer_weights;

KUIPER_LLAMA_API const char* kuiper_llama_last_error(void);

/* creates the model on the current CUDA device; NULL on failure (see kuiper_llama_last_error) */
KUIPER_LLAMA_API kuiper_model* kuiper_model_create(const kuiper_model_config* config);
KUIPER_LLAMA_API void kuiper_model_destroy(kuiper_model* model);

KUIPER_LLAMA_API int kuiper_model_load_layer(kuiper_model* model, int layer, const kuiper_layer_weights* w, int on_device);
KUIPER_LLAMA_API int kuiper_model_load_globals(kuiper_model* model, const void* embed, const void* final_norm,
                                               const void* lm_head, int on_device);

/* Every weight from an AWQ checkpoint in the safetensors container, Hugging Face tensor names of a quantised Qwen3 model
 * (model.layers.<i>.self_attn.{q,k,v,o}_proj.{qweight,qzeros,scales}, mlp.{gate,up,down}_proj..., the norms,
 * model.embed_tokens.weight, model.norm.weight, lm_head.weight or tied).  This is the loader behind the hook the
 * reference leaves empty for quantised layers (LayerParam::set_weight, kuiper/source/op/layer.cpp:256-276). */
KUIPER_LLAMA_API int kuiper_model_load_checkpoint(kuiper_model* model, const char* path);
/* Parses a safetensors file's header (no GPU needed) and writes one line per tensor, "name dtype [shape] bytes", and one
 * per metadata entry into `report`; 0 if the file is well formed. */
KUIPER_LLAMA_API int kuiper_checkpoint_inspect(const char* path, char* report, size_t report_bytes);

/* tensor parallelism: rank 0 makes a 128-byte id, every rank passes it to init_tp */
KUIPER_LLAMA_API int kuiper_tp_unique_id(void* out128);
KUIPER_LLAMA_API int kuiper_model_init_tp(kuiper_model* model, const void* unique_id128);
/* 1 if decode rows are summed by the one-shot exchange over peer memory, 0 if everything goes through NCCL */
KUIPER_LLAMA_API int kuiper_model_tp_one_shot(kuiper_model* model);
/* synchronous health check of that exchange: 5 if a bounded wait on a peer ever ran out */
KUIPER_LLAMA_API int kuiper_model_tp_status(kuiper_model* model);

/* one pass over M host rows; next (M ids) and logits (M x vocab, may be NULL) come back to the host */
KUIPER_LLAMA_API int kuiper_model_predict(kuiper_model* model, const int32_t* tokens, const int32_t* pos,
                                          const int32_t* slot, int M, int32_t* next, float* logits);
/* whole prompt of one sequence; *next = greedy id after its last token */
KUIPER_LLAMA_API int kuiper_model_prefill(kuiper_model* model, const int32_t* tokens, int n, int slot, int32_t* next);

/* device-resident decode loop (CUDA graph per batch size) */
KUIPER_LLAMA_API int kuiper_model_decode_begin(kuiper_model* model, const int32_t* tokens, const int32_t* pos,
                                               const int32_t* slot, int B);
KUIPER_LLAMA_API int kuiper_model_decode_step(kuiper_model* model, int n_steps); /* asynchronous */
KUIPER_LLAMA_API int kuiper_model_decode_read(kuiper_model* model, int32_t* tokens, int B);
/* one end-to-end decode step: host ids in, host ids out */
KUIPER_LLAMA_API int kuiper_model_decode_predict(kuiper_model* model, const int32_t* tokens, int B, int32_t* next);

KUIPER_LLAMA_API int kuiper_model_kernels_per_step(kuiper_model* model);
/* the cudaStream_t all of the model's work is enqueued on */
KUIPER_LLAMA_API void* kuiper_model_stream(kuiper_model* model);
KUIPER_LLAMA_API int kuiper_model_synchronize(kuiper_model* model);

/* runs the built-in checks of the base / tensor / op classes (the behaviour the
 * reference's test/test_tensor and test/test_op suites pin); returns the number of
 * failed checks.  use_cuda = 0 restricts it to the host-only cases. */
KUIPER_LLAMA_API int kuiper_selftest(int use_cuda, char* report, size_t report_bytes);

#ifdef __cplusplus
}
#endif
#endif /* KUIPER_LLAMA_H */
