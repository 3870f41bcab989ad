/*
 * kuiper_b200 - C ABI of the sm_100a decode kernels.
 *
 * Every entry point is what the reference's per-device kernel getter would bind for
 * DeviceCUDA: the reference's pattern is one function pointer per op returned by
 * kernel::get_<op>_kernel(base::DeviceType) (kuiper/source/op/kernel/kernel_interface.h:10-11,
 * kernel_interface.cpp:6-14) and the CUDA function behind it
 * (kuiper/source/op/kernel/cuda/add_kernel.cu:14-52).  The hot-path ops other than add
 * have only empty placeholder headers in the reference (kuiper/include/op/matmul.h:1-11,
 * mha.h:1-11, rmsnorm.h:1-10, rope.h:1-10, swiglu.h:1-10, embedding.h:1-10); the entry
 * points below are what their getters bind.
 *
 * Conventions
 *  - plain device pointers and sizes; no allocation, no synchronisation, no host
 *    read-back inside any call: all work is enqueued on `stream` (NULL = default
 *    stream, as add_kernel.cu:31-48) and is CUDA-graph capturable;
 *  - return value: 0 success, 7 invalid argument, 5 internal (launch) error - the
 *    numbering of base::StatusCode (kuiper/include/base/base.h:76-84);
 *  - activations are fp32, row-major [M, width]; fp16 / bf16 tensors travel as
 *    uint16_t bit patterns; M is the number of token rows in the pass;
 *  - INT4-AWQ weight of a K-in x N-out linear layer: qweight int32 [K, N/8], nibble i
 *    (bits 4i..4i+3) of word (k, j) = logical column 8j + {0,2,4,6,1,3,5,7}[i];
 *    qzeros int32 [K/group, N/8] packed the same way; scales fp16 [K/group, N];
 *    w[k,n] = (q[k,n] - z[k/group,n]) * s[k/group,n].
 */
#ifndef KUIPER_B200_H
#define KUIPER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* kuiper_stream_t; /* == cudaStream_t */

#define KUIPER_API __attribute__((visibility("default")))

enum {
    KUIPER_OK = 0,
    KUIPER_INTERNAL_ERROR = 5,
    KUIPER_INVALID_ARGUMENT = 7,
};

/* how the INT4 matmul rounds its activation operand */
enum {
    KUIPER_ACT_FP16 = 1, /* x rounded to fp16, exact products, fp32 accumulation */
    KUIPER_ACT_FP32 = 0, /* x kept in fp32 */
    /* single-row calls of the tensor-core GEMV: per 32 consecutive rows of K, x' = rint(x * 2^e) * 2^-e with e the largest
     * exponent that keeps |x * 2^e| < 2^14 (16-bit block floating point); integer products, exact sums inside a block,
     * fp32 accumulation across blocks.  Calls with more rows round to fp16 as KUIPER_ACT_FP16 does. */
    KUIPER_ACT_INT16_BLOCK = 2,
};

KUIPER_API const char* kuiper_version(void);
/* text of the last error raised on the calling thread ("" if none) */
KUIPER_API const char* kuiper_last_error(void);
/* benchmark sweeps only: override a launch heuristic ("gemv_rows", "gemv_math", "flash_splits"; 0 or -1 restores it) */
KUIPER_API int kuiper_set_tuning(const char* key, int value);

/* ---- residual add: replaces add_kernel_cu (kernel/cuda/add_kernel.cu:14-52) ---- */
KUIPER_API int kuiper_add_f32(const float* a, const float* b, float* out, int64_t n, kuiper_stream_t stream);

/* ---- INT4-AWQ: placeholder kuiper/include/op/matmul.h:1-11, quant fields op/layer.h:151-155 ---- */
/* nibble unpack to uint8 [K, N] (logical column order) */
KUIPER_API int kuiper_awq_unpack_u8(const int32_t* qweight, uint8_t* out, int K, int N, kuiper_stream_t stream);
/* fp32 dequantisation W[K,N] = (q - z) * s, exact */
KUIPER_API int kuiper_awq_dequant_f32(const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales,
                           float* W, int K, int N, int group, kuiper_stream_t stream);
/* bf16 dequantisation (round to nearest even) used by the M>=16 tensor-core path */
KUIPER_API int kuiper_awq_dequant_bf16(const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales,
                            uint16_t* W, int K, int N, int group, kuiper_stream_t stream);

/*
 * Scratch for the split-K GEMV: partial sums plus per-tile arrival counters.  The
 * counters must be zero before the first use (kuiper_workspace_init) and are left
 * zero by every call.  Two calls that overlap on the GPU must not share a workspace.
 */
KUIPER_API size_t kuiper_awq_gemv_workspace_bytes(int M, int K, int N);
KUIPER_API int kuiper_workspace_init(void* workspace, size_t bytes, kuiper_stream_t stream);

/*
 * y[M,N] = x[M,K] . dequant(qweight) (+ residual[M,N] if residual != NULL; y may alias
 * residual).  group must be 128, K % 128 == 0, N % 8 == 0.  M <= 8 runs the SIMT
 * dequant-fused GEMV; larger M is processed in row blocks.
 * act_mode: KUIPER_ACT_FP16, KUIPER_ACT_FP32, or KUIPER_ACT_INT16_BLOCK (N % 32 == 0; applies to M == 1, more rows round to fp16).
 */
KUIPER_API int kuiper_awq_gemv_f32(const float* x, const int32_t* qweight, const int32_t* qzeros,
                        const uint16_t* scales, float* y, const float* residual,
                        int M, int K, int N, int group, int act_mode,
                        void* workspace, size_t workspace_bytes, kuiper_stream_t stream);

/*
 * y[M,N] += x[M,K] . dequant(qweight): the engine's fast path.  The caller guarantees that y already
 * holds the addend (the residual stream, or zeros); partial rows are added with vector float
 * reductions, so no workspace is needed and there is no ordered combine at the end, at the price of
 * a summation order (last bits) that can differ from run to run.  Needs N % 32 == 0.
 */
KUIPER_API int kuiper_awq_gemv_accum_f32(const float* x, const int32_t* qweight, const int32_t* qzeros,
                                         const uint16_t* scales, float* y, int M, int K, int N, int group,
                                         kuiper_stream_t stream);
/*
 * Same, with the RMSNorm of the input fused in: y[M,N] += RMSNorm(h[M,K]; norm_w, eps) . dequant(qweight).
 * h is the un-normalised row (the residual stream); norm_w is bf16 [K].  Replaces an rmsnorm call + a matmul call.
 */
KUIPER_API int kuiper_rmsnorm_awq_gemv_accum_f32(const float* h, const uint16_t* norm_w, float eps,
                                                 const int32_t* qweight, const int32_t* qzeros,
                                                 const uint16_t* scales, float* y, int M, int K, int N, int group,
                                                 kuiper_stream_t stream);
/*
 * Same as kuiper_awq_gemv_accum_f32 with SwiGLU fused in: gate_up is [M, 2K] (gate | up) and the operand is
 * x = silu(gate) * up in fp32 (the formula of kuiper_swiglu_f32), rounded to fp16: y[M,N] += x . dequant(qweight).
 * gate_up is only read.  Replaces a swiglu call + a matmul call.
 */
KUIPER_API int kuiper_swiglu_awq_gemv_accum_f32(const float* gate_up, const int32_t* qweight, const int32_t* qzeros,
                                                const uint16_t* scales, float* y, int M, int K, int N, int group,
                                                kuiper_stream_t stream);
/*
 * The three accumulating calls above in one (the engine's entry): norm_w != NULL selects the fused RMSNorm, swiglu != 0
 * the fused SwiGLU (not both); act_mode KUIPER_ACT_FP16 or KUIPER_ACT_INT16_BLOCK (the faster kernel for M == 1).  tickets: kuiper_awq_gemv_ticket_bytes() bytes of device memory owned by the call site,
 * zeroed once (kuiper_workspace_init) and left at zero by every call; with it the kernel deals only three quarters of
 * the weight stream out statically and hands the rest to whichever CTA is free (an atomic ticket counter), so that
 * all CTAs finish together.  NULL: a fully static deal, as in the calls above.  Launches that may overlap on the
 * GPU (consecutive launches of a stream do, under programmatic dependent launch) must not share tickets; the engine
 * gives every layer object its own.  No counterpart in the reference.
 */
KUIPER_API size_t kuiper_awq_gemv_ticket_bytes(void);
KUIPER_API int kuiper_awq_gemv_accum_balanced_f32(const float* x, const uint16_t* norm_w, float eps, int swiglu,
                                                  const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales,
                                                  float* y, int M, int K, int N, int group, int act_mode, void* tickets,
                                                  kuiper_stream_t stream);
/*
 * A list of independent one-row projections in ONE persistent launch: y_i += x_i . dequant(W_i) for every item, in no
 * particular order (no item may read another's output).  The units of all matrices form one stream, so a list of small
 * matrices (the 2048 x 2048 single-GEMV workload visited over many weight sets) runs at streaming speed instead of
 * paying a launch per 2 MB.  Three steps: kuiper_awq_gemv_group_plan() fills a HOST buffer of
 * kuiper_awq_gemv_group_table_bytes(n) bytes with the table the kernel reads and returns the number of work units in
 * *units; the caller copies the table to 64-byte aligned device memory (it stays valid while the item pointers do);
 * kuiper_awq_gemv_group_f32() launches (act_mode KUIPER_ACT_FP16 or KUIPER_ACT_INT16_BLOCK).  Every item: K % 128 == 0, N % 32 == 0, 16-byte aligned tensors, y holds
 * the addend.  tickets as above (may be NULL).  No counterpart in the reference.
 */
typedef struct kuiper_gemv_item {
    const float* x;          /* [K] */
    const int32_t* qweight;  /* [K, N/8] */
    const int32_t* qzeros;   /* [K/128, N/8] */
    const uint16_t* scales;  /* fp16 [K/128, N] */
    float* y;                /* [N] */
    int32_t K, N;
} kuiper_gemv_item;
KUIPER_API size_t kuiper_awq_gemv_group_table_bytes(int n_items);
KUIPER_API int kuiper_awq_gemv_group_plan(const kuiper_gemv_item* items, int n_items, int group, void* host_table,
                                          int64_t* units);
KUIPER_API int kuiper_awq_gemv_group_f32(const void* device_table, int n_items, int64_t units, int act_mode, void* tickets,
                                         kuiper_stream_t stream);
/* health check (synchronises): 5 if a bounded wait inside the pipelined GEMV ever ran out on this device */
KUIPER_API int kuiper_awq_gemv_status(void);
/*
 * The INT4 GEMV once more, for callers that must not allocate: no counterpart in the reference (its
 * kernels take caller-owned tensors only and it has no split-K scratch at all).  Meant for code that
 * runs after the application has committed all device memory to its own pool, or inside a loop where
 * cudaMalloc and the synchronisation it implies are ruled out.  The scratch of the ordered combine
 * lives in a fixed array inside the library image (kuiper_awq_gemv_noalloc_scratch_bytes(), about
 * 2.1 MiB held per GPU for the life of the process); the call allocates no device or pinned memory.
 * Its first call on a device does one-time set-up on the host (it asks the runtime for the array's address
 * and for the driver's tensor-map encoder, sets the kernel's shared-memory attribute) and an error path may
 * format a message into a thread-local string; later calls only build a tensor map on the stack and launch.
 * Limits: N <= 32768, N % 32 == 0, K % 128 == 0, group 128, M <= 8; other sizes
 * return 7.  Same result as kuiper_awq_gemv_f32 up to fp32 summation order.  The first call on a
 * device resolves the array's device address: issue it before any stream capture.  All calls on a
 * device share the array, so calls that may overlap on the GPU race; its counters are cleared at the
 * start of each call.
 */
KUIPER_API size_t kuiper_awq_gemv_noalloc_scratch_bytes(void);
KUIPER_API int kuiper_awq_gemv_f32_noalloc(const float* x, const int32_t* qweight, const int32_t* qzeros,
                                           const uint16_t* scales, float* y, const float* residual,
                                           int M, int K, int N, int group, kuiper_stream_t stream);

/* ---- INT4-AWQ GEMM on the tcgen05 tensor cores, for M >= 16 token rows (prefill, batched decode).
 * Same placeholder as the GEMV (kuiper/include/op/matmul.h:1-11).  x is rounded to fp16, the weight
 * (q - z) * s is rounded to fp16, accumulation is fp32 in tensor memory.
 *   accumulate == 0, residual == NULL : y  = x . W
 *   accumulate == 0, residual != NULL : y  = x . W + residual   (residual may alias y)
 *   accumulate != 0                   : y += x . W
 * A launch with few output tiles (M <= 128 or so) splits K over several CTAs per tile, which add their sums with
 * reductions: the summation order is then not fixed (differences ~1e-6); larger launches are deterministic.
 * Any M > 0 is accepted (rows are padded to 128 inside the kernel); K % 128 == 0, N % 8 == 0.
 * workspace: kuiper_awq_gemm_workspace_bytes(M, K) bytes (16-byte aligned) for the fp16 copy of x that the
 * pipelined kernel reads (128 x 256 tiles); required.
 * kuiper_awq_gemm_status() synchronously reads the kernel's bounded-wait error word. ---- */
KUIPER_API size_t kuiper_awq_gemm_workspace_bytes(int M, int K);
KUIPER_API int kuiper_awq_gemm_f32(const float* x, const int32_t* qweight, const int32_t* qzeros,
                                   const uint16_t* scales, float* y, const float* residual, int accumulate,
                                   int M, int K, int N, int group, void* workspace, size_t workspace_bytes,
                                   kuiper_stream_t stream);
/* The same call for activations that already are fp16 [M, K] (as kuiper_rmsnorm_f16 / kuiper_swiglu_f16 leave them): no
 * conversion pass, no workspace. */
KUIPER_API int kuiper_awq_gemm_f16in_f32(const uint16_t* x16, const int32_t* qweight, const int32_t* qzeros,
                                         const uint16_t* scales, float* y, const float* residual, int accumulate,
                                         int M, int K, int N, int group, kuiper_stream_t stream);
KUIPER_API int kuiper_awq_gemm_status(void);

/* ---- tensor-parallel exchanges for decode rows over peer-mapped buffers.  No counterpart in the reference (it has no
 * multi-GPU code).
 * Every rank owns an exchange buffer of kuiper_allreduce_buffer_bytes(world, max_count) bytes, zero-initialised once,
 * 128-byte aligned, and mapped into every other rank's process (CUDA IPC); rank_buffers is a HOST array of `world`
 * device pointers, entry r = rank r's buffer as this process sees it (entry `rank` = the own buffer).  state:
 * kuiper_allreduce_state_bytes() zero-initialised bytes on the device, private to the rank (sequence numbers and an
 * error word).  All ranks must issue the same sequence of calls with the same sizes.
 *
 * kuiper_allreduce_sum_f32: out[i] = residual[i] + sum over ranks of partial[i] (residual may be NULL; it must hold the
 * same values on every rank; out may alias residual).  Every value travels as one 8-byte word {value, sequence
 * number} stored straight into the peers' buffers; the receiver polls the words themselves and adds them in rank
 * order, so all ranks get identical bits and there is no flag, fence or barrier between sending and receiving.
 * clear_partial != 0 zeroes `partial` after it has been read (ready for the next accumulating projection).
 * count <= max_count <= 65536, max_count % 16 == 0.
 *
 * kuiper_argmax_allgather: the greedy token over a vocabulary split across ranks.  logits_local is this rank's slice
 * [M, V_local] (rank r holds global indices [r V_local, (r+1) V_local)); next[m] = lowest global index of the maximum
 * over all slices (the tie rule of kuiper_argmax_f32), identical on every rank.  M <= 16.
 *
 * Waits on peers are bounded (default five seconds, tuning key "allreduce_timeout_ms"): when one runs out the call's
 * result is void, an error word is set, and kuiper_allreduce_status (synchronous; clear != 0 resets the word)
 * returns 5. ---- */
KUIPER_API size_t kuiper_allreduce_buffer_bytes(int world, int64_t max_count);
KUIPER_API size_t kuiper_allreduce_state_bytes(void);
KUIPER_API int kuiper_allreduce_sum_f32(const float* partial, const float* residual, float* out, int clear_partial,
                                        int64_t count, int rank, int world, void* const* rank_buffers,
                                        int64_t max_count, uint32_t* state, kuiper_stream_t stream);
KUIPER_API int kuiper_argmax_allgather(const float* logits_local, int32_t* next, int M, int V_local, int rank, int world,
                                       void* const* rank_buffers, int64_t max_count, uint32_t* state,
                                       kuiper_stream_t stream);
KUIPER_API int kuiper_allreduce_status(uint32_t* state, int clear);

/* ---- BF16 GEMV (lm_head): W bf16 [N, K], y[M,N] = x[M,K] . W^T; x stays fp32 in effect (one or two rows: fp32 FMAs;
 * three rows and more: tensor cores with x as three bf16 parts), accumulation fp32 ---- */
KUIPER_API int kuiper_bf16_gemv_f32(const float* x, const uint16_t* W, float* y, int M, int K, int N,
                         kuiper_stream_t stream);

/* ---- RMSNorm: placeholder kuiper/include/op/rmsnorm.h:1-10 ---- */
/* y = (x * rstd) * w, rstd = 1/sqrt(mean(x^2) + eps); w bf16 [H]; y may alias x */
KUIPER_API int kuiper_rmsnorm_f32(const float* x, const uint16_t* w, float* y, int M, int H, float eps,
                       kuiper_stream_t stream);
/* the same row norm with the result rounded to fp16 (the tensor-core GEMM's activation type) */
KUIPER_API int kuiper_rmsnorm_f16(const float* x, const uint16_t* w, uint16_t* y16, int M, int H, float eps,
                                  kuiper_stream_t stream);

/* ---- per-head q/k RMSNorm + rotary + KV-cache write: placeholder kuiper/include/op/rope.h:1-10 ---- */
/*
 * qkv [M, (Nq+2Nkv)*D] fp32 (q heads | k heads | v heads); cos/sin fp32 [max_pos, D/2]
 * (half-split pairing (i, i+D/2)); pos[M], slot[M] int32 on the device.
 * q_out [M, Nq, D] fp32; k, v rounded to bf16 into cache[(slot*Nkv + h)*max_seq + pos][D];
 * the caches hold n_slots sequences; pos and slot are clamped into range on the device.
 * D must be 128.  clear_input != 0 zeroes qkv after it has been read (the buffer is then
 * ready for the next kuiper_awq_gemv_accum_f32 into it).  clear_extra (may be NULL with count 0):
 * clear_extra_count floats (a multiple of 4, 16-byte aligned) that the kernel zeroes on the side - the
 * engine passes the gate|up projection buffer, whose consumer is fused into the down projection and
 * cannot clear it itself.
 */
KUIPER_API int kuiper_qknorm_rope_kvwrite(float* qkv, const uint16_t* q_norm_w, const uint16_t* k_norm_w,
                               const float* cos_t, const float* sin_t, const int32_t* pos,
                               const int32_t* slot, int M, int Nq, int Nkv, int D, float eps,
                               int max_seq, int n_slots, float* q_out, uint16_t* kcache,
                               uint16_t* vcache, int clear_input, float* clear_extra,
                               int64_t clear_extra_count, kuiper_stream_t stream);

/* ---- GQA flash-decoding: placeholder kuiper/include/op/mha.h:1-11 ---- */
/*
 * out[m,h,:] = softmax(q[m,h,:].K^T / sqrt(D)) . V over cache positions [0, seq_len[m]) of
 * sequence slot[m]; q head h reads kv head h / (Nq/Nkv).  The KV range is split across
 * CTAs and the partial (max, sum, out) triples are merged with a log-sum-exp combine.
 * workspace: kuiper_flash_decode_workspace_bytes(M, Nq, D, max_seq) bytes, all of it zeroed once
 * with kuiper_workspace_init (arrival counters, launch numbers and tagged words start from zero).  D must be 128, Nq/Nkv in {1,2,4,8}.
 * fresh_rows: -1 = the kernel touches nothing before the stream's previous kernel has completed.
 * fresh_rows = F >= 0 is a promise by the caller: seq_len, slot and every cache row below
 * seq_len[m] - F were final before the previous kernel on the stream started (that kernel appended
 * at most the newest F rows of a sequence and produced q).  The kernel then fetches those rows
 * under programmatic dependent launch while the previous kernel is still finishing.
 * Two kernels sit behind the call: by default the contractions run on the tensor cores (mma.sync bf16: cache
 * rows as exact operands, q and the probabilities as bf16 high + low parts; agrees with the fp32 oracle to
 * ~1e-5; fresh_rows is accepted and ignored), kuiper_set_tuning("flash_mma", 0) selects the SIMT kernel.
 */
KUIPER_API size_t kuiper_flash_decode_workspace_bytes(int M, int Nq, int D, int max_seq);
/* health check (synchronises): 5 if the bounded wait of a combining CTA (fused decode kernel) ran out on this device
 * since the last call (the outputs of that launch are zeros) */
KUIPER_API int kuiper_flash_decode_status(void);
KUIPER_API int kuiper_flash_decode(const float* q, const uint16_t* kcache, const uint16_t* vcache,
                        const int32_t* seq_len, const int32_t* slot, float* out,
                        int M, int Nq, int Nkv, int D, int max_seq, int n_slots, int fresh_rows,
                        void* workspace, size_t workspace_bytes, kuiper_stream_t stream);

/*
 * Causal attention for a prompt chunk: the M rows are consecutive tokens of ONE sequence (row m at position pos0 + m of
 * sequence `slot`, already appended to the caches) and row m attends to cache positions [0, pos0 + m].  Tiled: every K / V
 * tile is loaded once per block of 64 / (Nq / Nkv) query rows (bf16 mma.sync, fp32 softmax; q and the probabilities as
 * bf16 high + low parts like the decode kernel), no workspace.  Same placeholder (kuiper/include/op/mha.h:1-11).
 * pos0 and slot are host values: a prompt is fed from the host, chunk by chunk.
 */
KUIPER_API int kuiper_flash_prefill(const float* q, const uint16_t* kcache, const uint16_t* vcache, float* out,
                                    int M, int Nq, int Nkv, int D, int max_seq, int n_slots, int pos0, int slot,
                                    kuiper_stream_t stream);

/*
 * The two calls above in one kernel, for decode batches: every token row m must belong to a different
 * sequence slot and seq_len[m] == pos[m] + 1.  Each CTA forms q (per-head RMSNorm + rotary) for its kv
 * head from the raw projection row in qkv; the CTA whose slice ends the sequence appends the new K / V
 * row to the caches and uses it.  With clear_input != 0 the last CTA of a (row, kv head) zeroes the
 * slices of qkv it read; clear_extra / clear_extra_count as in kuiper_qknorm_rope_kvwrite.  fresh_rows
 * as in kuiper_flash_decode (the newest row is never fetched early: it does not exist yet).
 * Like kuiper_flash_decode the call runs its contractions on the tensor cores by default; with
 * kuiper_set_tuning("flash_mma_fused", 0) it uses the SIMT arithmetic and is then bit-identical to
 * kuiper_qknorm_rope_kvwrite followed by kuiper_flash_decode with its SIMT kernel ("flash_mma" = 0).  The two
 * arithmetic paths agree to ~1e-5; the appended cache rows are identical.
 * For one or two sequences at a context of a few thousand rows the call runs eight-warp CTAs whose partial results reach
 * one combining CTA per (row, kv head) as tagged 8-byte words; that CTA's wait for them is bounded (1 s by default) and
 * a run-out is reported by kuiper_flash_decode_status().  The workspace must have been zeroed once, all of it.
 */
KUIPER_API int kuiper_rope_flash_decode(float* qkv, const uint16_t* q_norm_w, const uint16_t* k_norm_w,
                                        const float* cos_t, const float* sin_t, const int32_t* pos,
                                        const int32_t* seq_len, const int32_t* slot, float* out,
                                        uint16_t* kcache, uint16_t* vcache, int M, int Nq, int Nkv, int D,
                                        float eps, int max_seq, int n_slots, int fresh_rows, int clear_input,
                                        float* clear_extra, int64_t clear_extra_count, void* workspace,
                                        size_t workspace_bytes, kuiper_stream_t stream);

#ifdef KUIPER_TRACE
/* Measurement builds only (compiled with -DKUIPER_TRACE; absent from the shipped library): per-CTA clock readings of
 * the last launch of the tensor-core attention kernel, [CTA][10] int64 (slot 0 global timer in ns at entry, then SM
 * clock at 1 entry, 2 early fetches issued, 3 dependency wait passed, 4 q ready, 5 cache rows processed, 6 partial
 * stored, 7 arrival counter answered, 8 slices combined, 9 output stored).  Synchronises; returns the number of values copied or -1. */
KUIPER_API int kuiper_flash_trace_read(int64_t* out, int max_values);
/* The same for the last launch of the tensor-core INT4 GEMV: [CTA][10] (0 global timer at entry, then SM clock at 1 entry,
 * 2 consumers past the dependency wait, 3 first unit ready, 4 last unit consumed, 5 consumer exit, 6 activation warp saw
 * its first descriptor, 7 first fragments written, 8 first weight copy issued, 9 last weight copy issued). */
KUIPER_API int kuiper_gemv_trace_read(int64_t* out, int max_values);
#endif

/* ---- SwiGLU: placeholder kuiper/include/op/swiglu.h:1-10 ---- */
/* out[m,i] = silu(gate_up[m,i]) * gate_up[m,I+i]; gate_up is [M, 2I]; clear_input != 0 zeroes gate_up afterwards */
KUIPER_API int kuiper_swiglu_f32(float* gate_up, float* out, int M, int I, int clear_input, kuiper_stream_t stream);
/* the same with the result rounded to fp16 */
KUIPER_API int kuiper_swiglu_f16(float* gate_up, uint16_t* out16, int M, int I, int clear_input, kuiper_stream_t stream);

/* ---- embedding gather: placeholder kuiper/include/op/embedding.h:1-10 ---- */
KUIPER_API int kuiper_embedding_bf16(const int32_t* tokens, const uint16_t* table, float* out, int M, int H,
                          int vocab, kuiper_stream_t stream);

/* ---- greedy sampler (the reference's sampler directory is absent, CMakeLists.txt:87) ---- */
/* out[m] = lowest index of the maximum of logits[m, 0..V) */
KUIPER_API int kuiper_argmax_f32(const float* logits, int32_t* out, int M, int V, kuiper_stream_t stream);

/*
 * End of a decode step, on the device: feed the chosen ids back as the next input and
 * advance every sequence by one position (clamped to max_seq - 1).
 * tokens[b] = next[b]; pos[b] += 1; seq_len[b] = pos[b] + 1.
 */
KUIPER_API int kuiper_decode_advance(int32_t* tokens, const int32_t* next, int32_t* pos, int32_t* seq_len,
                                     int B, int max_seq, kuiper_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* KUIPER_B200_H */
