/*
 * CPU oracle for the INT4-AWQ decode hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This library is the checker that the parity tests, the smoke test and the
 * CPU-baseline leg of the benchmark compare the CUDA path against.  Nothing
 * in the product (the CUDA kernels, the C++ engine) links or calls it.
 *
 * PARITY UNPINNED: the reference repository ships no implementation, golden
 * vector or known-answer test for any function below except the vector add
 * (test/test_op/test_op_add.cpp:7-91 pins 2+3==5 and 2.1+3.3~=5.4).  The
 * numerics here are a restatement of the workload specification (AWQ nibble
 * order [0,2,4,6,1,3,5,7], group 128 along K, fp16 scales, packed zeros,
 * w=(q-z)*s) and of the public Qwen3 block description, in the reference's
 * CPU-kernel idiom (kuiper/source/op/kernel/cpu/add_kernel.cpp:5-26: a free
 * function, fp32 buffers, preconditions checked up front).
 *
 * Conventions: row-major everywhere; fp16/bf16 values travel as uint16_t bit
 * patterns; "acc_double" selects double accumulation (error reference) or
 * fp32 accumulation (timed CPU baseline).
 */
#ifndef KUIPER_ORACLE_H
#define KUIPER_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* how an activation vector is rounded before it enters a matmul */
enum {
    ORC_ROUND_NONE = 0,
    ORC_ROUND_FP16 = 1,
    ORC_ROUND_BF16 = 2,
    /* 16-bit block floating point per 32 consecutive elements: x' = rint(x * 2^e) * 2^-e, |x * 2^e| < 2^14 */
    ORC_ROUND_I16_BLOCK32 = 3,
    /* what an engine with act_mode 2 does: I16_BLOCK32 for a one-row operand, FP16 for several rows */
    ORC_ROUND_ENGINE = 4
};

/* OpenMP threads used by the loops below from now on (n <= 0: only query); returns the value in effect */
int orc_set_num_threads(int n);

/* scalar conversions (round to nearest even) */
uint16_t orc_f32_to_f16(float f);
float orc_f16_to_f32(uint16_t h);
uint16_t orc_f32_to_bf16(float f);
float orc_bf16_to_f32(uint16_t h);
void orc_f32_to_bf16_n(const float* in, uint16_t* out, int64_t n);
void orc_f32_to_f16_n(const float* in, uint16_t* out, int64_t n);
void orc_bf16_to_f32_n(const uint16_t* in, float* out, int64_t n);

/* residual add; mirrors add_kernel_cpu (kernel/cpu/add_kernel.cpp:5-26) */
void orc_add(const float* a, const float* b, float* out, int64_t n);

/* AWQ packing: q is [K,N] uint8 in 0..15, words are [K,N/8] int32 */
void orc_awq_pack(const uint8_t* q, int K, int N, int32_t* words);
void orc_awq_unpack(const int32_t* words, int K, int N, uint8_t* q);
/* W[k,n] = (float)(q[k,n]-z[k/g,n]) * (float)s[k/g,n], exact in fp32 */
void orc_awq_dequant(const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales_f16,
                     int K, int N, int group, float* W);
/* harness quantiser: per (group, column) asymmetric min/max 4-bit */
void orc_awq_quantize(const float* W, int K, int N, int group,
                      int32_t* qweight, int32_t* qzeros, uint16_t* scales_f16);

/* y[M,N] = x[M,K] . W[K,N] on dequantised fp32 weights */
void orc_gemv_f32(const float* x, const float* W, float* y, int M, int K, int N,
                  int acc_double, int act_round);
/* same contraction straight from the packed tensors */
void orc_awq_gemv(const float* x, const int32_t* qweight, const int32_t* qzeros,
                  const uint16_t* scales_f16, float* y, int M, int K, int N, int group,
                  int acc_double, int act_round);
/* y[M,N] = x[M,K] . W[N,K]^T with bf16 W (lm_head layout: one row per output) */
void orc_bf16_gemv(const float* x, const uint16_t* W_bf16, float* y, int M, int K, int N,
                   int acc_double);

/* y = (x * rstd) * w, rstd = 1/sqrt(mean(x^2)+eps); w is bf16 [H] */
void orc_rmsnorm(const float* x, const uint16_t* w_bf16, float* y, int M, int H, float eps);
/* cos/sin tables [max_pos, D/2] for half-split rotary, computed in double */
void orc_rope_tables(int max_pos, int D, double theta, float* cos_t, float* sin_t);
/*
 * qkv is [M, (Nq+2*Nkv)*D] fp32 (q heads, then k heads, then v heads).  Per head:
 * RMSNorm over D with q_norm / k_norm (bf16 [D]), then half-split rotary at pos[m].
 * q_out [M,Nq,D] fp32; k and v are rounded to bf16 and stored at
 * cache[(slot[m]*Nkv + h)*max_seq + pos[m]][D].
 */
void orc_qknorm_rope_kvwrite(const float* qkv, const uint16_t* q_norm_w, const uint16_t* k_norm_w,
                             const float* cos_t, const float* sin_t, const int32_t* pos,
                             const int32_t* slot, int M, int Nq, int Nkv, int D, float eps,
                             int max_seq, float* q_out, uint16_t* kcache, uint16_t* vcache);
/*
 * softmax(q.K^T/sqrt(D)).V per query row m over cache positions [0, seq_len[m]) of
 * sequence slot[m]; GQA: q head h reads kv head h/(Nq/Nkv).  out [M,Nq,D] fp32.
 */
void orc_attention(const float* q, const uint16_t* kcache, const uint16_t* vcache,
                   const int32_t* seq_len, const int32_t* slot, int M, int Nq, int Nkv, int D,
                   int max_seq, float* out);
void orc_swiglu(const float* gate, const float* up, float* out, int64_t n);
void orc_embedding(const int32_t* tokens, const uint16_t* table_bf16, float* out, int M, int H);
/* ties resolve to the lowest index */
void orc_argmax(const float* logits, int M, int V, int32_t* out);

/* ---- whole decoder (Qwen3-shaped) ---- */
typedef struct {
    int32_t n_layers, hidden, n_q_heads, n_kv_heads, head_dim, inter, vocab, group;
    int32_t max_seq, max_batch;
    float eps;
    double rope_theta;
    int32_t act_round; /* ORC_ROUND_* applied to the input of every INT4 matmul */
} orc_config;

typedef struct {
    const uint16_t* input_norm;  /* bf16 [H] */
    const uint16_t* post_norm;   /* bf16 [H] */
    const uint16_t* q_norm;      /* bf16 [D] */
    const uint16_t* k_norm;      /* bf16 [D] */
    /* fused projections: qkv K=H,N=(Nq+2Nkv)*D; o K=Nq*D,N=H; gate_up K=H,N=2*I; down K=I,N=H */
    const int32_t *qkv_qw, *qkv_qz; const uint16_t* qkv_s;
    const int32_t *o_qw, *o_qz;     const uint16_t* o_s;
    const int32_t *gu_qw, *gu_qz;   const uint16_t* gu_s;
    const int32_t *down_qw, *down_qz; const uint16_t* down_s;
} orc_layer_weights;

typedef struct orc_model orc_model;

orc_model* orc_model_create(const orc_config* cfg, const uint16_t* embed_bf16,
                            const uint16_t* final_norm_bf16, const uint16_t* lm_head_bf16,
                            const orc_layer_weights* layers);
void orc_model_destroy(orc_model* m);
/*
 * One forward pass over M tokens (tokens[m] at position pos[m] of sequence slot[m]);
 * rows are processed in order so a prompt chunk sees its own earlier tokens.
 * Logits are computed for the last logit_rows rows only: logits [logit_rows,V] fp32
 * (may be NULL), next [logit_rows] greedy ids (may be NULL).
 */
void orc_model_forward(orc_model* m, const int32_t* tokens, const int32_t* pos, const int32_t* slot,
                       int M, int acc_double, int logit_rows, float* logits, int32_t* next);
/* copies of the bf16 caches for inspection: [L][max_batch][Nkv][max_seq][D] */
const uint16_t* orc_model_kcache(const orc_model* m);
const uint16_t* orc_model_vcache(const orc_model* m);

#ifdef __cplusplus
}
#endif
#endif
