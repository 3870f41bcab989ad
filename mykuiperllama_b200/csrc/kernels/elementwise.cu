// Small decode-path kernels for sm_100a: residual add, RMSNorm, SwiGLU, embedding
// gather, greedy argmax, AWQ unpack / dequant, plus the library's error plumbing.
//
// The add kernel replaces add_kernel_cu (kuiper/source/op/kernel/cuda/add_kernel.cu:14-52);
// the others fill empty placeholders of the reference (kuiper/include/op/rmsnorm.h:1-10,
// swiglu.h:1-10, embedding.h:1-10) and its absent sampler (CMakeLists.txt:87).
#include <cstring>

#include "common.cuh"

namespace kuiper {

int g_pdl_enabled = 1;

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

void awq_gemv_set_tuning(const char* key, int value);
void flash_decode_set_tuning(const char* key, int value);
void awq_gemm_set_tuning(const char* key, int value);
void bf16_gemv_set_tuning(const char* key, int value);
void allreduce_set_tuning(const char* key, int value);

namespace {

// ---------------------------------------------------------------- add
// 16-byte vector body plus a scalar tail; the reference kernel is one scalar element
// per thread (add_kernel.cu:4-12).
__global__ void add_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                           int64_t n, int vec_ok) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t tid = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    const int64_t n4 = vec_ok ? n / 4 : 0;
    for (int64_t i = tid; i < n4; i += stride) {
        float4 x = reinterpret_cast<const float4*>(a)[i];
        float4 y = reinterpret_cast<const float4*>(b)[i];
        reinterpret_cast<float4*>(out)[i] = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
    }
    for (int64_t i = n4 * 4 + tid; i < n; i += stride) out[i] = a[i] + b[i];
}

// ---------------------------------------------------------------- rmsnorm
// One CTA of 1024 threads per token row.  The row is read once, with every load of a thread issued
// before the first use (a single CTA is latency bound, so rounds of dependent loads are what costs).
constexpr int kNormThreads = 1024;
constexpr int kNormVec = 4;  // float4 per thread held in registers: rows up to 16384 wide

__device__ __forceinline__ float block_sum_1024(float v, float* s_part) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = v;
    __syncthreads();
    float tot = (threadIdx.x & 31) < (kNormThreads / 32) ? s_part[threadIdx.x & 31] : 0.f;
    return warp_sum(tot);  // every warp reduces the 32 partials itself: same order, same value everywhere
}

// OUT16: the normalised row is written as fp16 (round to nearest: exactly what a conversion of the fp32 result gives),
// for the tensor-core GEMM that takes its activations in that type
__device__ __forceinline__ void norm_store(float* y, int i, float v) { y[i] = v; }
__device__ __forceinline__ void norm_store(__half* y, int i, float v) { y[i] = __float2half_rn(v); }
__device__ __forceinline__ void norm_store4(float* y, int i4, float4 o) { reinterpret_cast<float4*>(y)[i4] = o; }
__device__ __forceinline__ void norm_store4(__half* y, int i4, float4 o) {
    const __half2 a = __floats2half2_rn(o.x, o.y), b = __floats2half2_rn(o.z, o.w);
    reinterpret_cast<uint2*>(y)[i4] = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

template <typename OUT>
__global__ void __launch_bounds__(kNormThreads) rmsnorm_kernel(const float* x, const uint16_t* __restrict__ w, OUT* y, int H,
                                                               float eps) {
    __shared__ float s_part[kNormThreads / 32];
    pdl_launch_dependents();
    pdl_wait();
    const float* xr = x + size_t(blockIdx.x) * H;
    OUT* yr = y + size_t(blockIdx.x) * H;
    const int t = threadIdx.x;
    if ((H & 3) == 0 && H <= kNormThreads * kNormVec * 4 && (reinterpret_cast<uintptr_t>(xr) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(yr) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 7) == 0) {
        const int n4 = H >> 2;
        float4 v[kNormVec];
        uint2 wv[kNormVec];
#pragma unroll
        for (int j = 0; j < kNormVec; j++) {
            const int i = t + j * kNormThreads;
            v[j] = i < n4 ? __ldcg(reinterpret_cast<const float4*>(xr) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            wv[j] = i < n4 ? __ldg(reinterpret_cast<const uint2*>(w) + i) : make_uint2(0, 0);
        }
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < kNormVec; j++) {
            ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
            ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
        }
        const float rstd = 1.0f / sqrtf(block_sum_1024(ss, s_part) / float(H) + eps);
#pragma unroll
        for (int j = 0; j < kNormVec; j++) {
            const int i = t + j * kNormThreads;
            if (i < n4) {
                float4 o;
                o.x = (v[j].x * rstd) * bf16_lo(wv[j].x); o.y = (v[j].y * rstd) * bf16_hi(wv[j].x);
                o.z = (v[j].z * rstd) * bf16_lo(wv[j].y); o.w = (v[j].w * rstd) * bf16_hi(wv[j].y);
                norm_store4(yr, i, o);
            }
        }
        return;
    }
    // any width / alignment: two scalar passes
    float ss = 0.f;
    for (int i = t; i < H; i += kNormThreads) {
        const float a = xr[i];
        ss = fmaf(a, a, ss);
    }
    const float rstd = 1.0f / sqrtf(block_sum_1024(ss, s_part) / float(H) + eps);
    for (int i = t; i < H; i += kNormThreads) norm_store(yr, i, (xr[i] * rstd) * bf16_bits_to_float(w[i]));
}

// ---------------------------------------------------------------- swiglu
template <typename OUT>
__global__ void swiglu_kernel(float* gate_up, OUT* out, int M, int I, int clear_input) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t total = int64_t(M) * I;
    for (int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += int64_t(gridDim.x) * blockDim.x) {
        const int64_t m = idx / I, i = idx - m * I;
        const float g = gate_up[m * 2 * I + i], u = gate_up[m * 2 * I + I + i];
        norm_store(out + idx, 0, (g / (1.0f + expf(-g))) * u);
        if (clear_input) {  // leave the projection buffer zeroed for the next accumulating matmul
            gate_up[m * 2 * I + i] = 0.f;
            gate_up[m * 2 * I + I + i] = 0.f;
        }
    }
}

// ---------------------------------------------------------------- embedding
__global__ void embedding_kernel(const int32_t* tokens, const uint16_t* __restrict__ table, float* out, int H, int vocab) {
    pdl_launch_dependents();
    pdl_wait();
    int tok = tokens[blockIdx.x];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);  // clamp: never read outside the table
    const uint16_t* row = table + size_t(tok) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[size_t(blockIdx.x) * H + i] = bf16_bits_to_float(row[i]);
}

// ---------------------------------------------------------------- argmax
// one CTA of 1024 threads per row; ties go to the lowest index.  Eight 16-byte loads are in flight
// per thread so that the single CTA is bandwidth bound, not latency bound.
__device__ __forceinline__ void argmax_take(float v, int i, float& best, int& bi) {
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
}

__global__ void __launch_bounds__(1024) argmax_kernel(const float* logits, int32_t* out, int V) {
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    pdl_launch_dependents();
    pdl_wait();
    const float* l = logits + size_t(blockIdx.x) * V;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    const int t = threadIdx.x;
    int done = 0;
    if ((reinterpret_cast<uintptr_t>(l) & 15) == 0) {
        const int n4 = V >> 2;
        constexpr int kU = 8;
        int i = t;
        for (; i + (kU - 1) * 1024 < n4; i += kU * 1024) {
            float4 v[kU];
#pragma unroll
            for (int u = 0; u < kU; u++) v[u] = __ldcg(reinterpret_cast<const float4*>(l) + i + u * 1024);
#pragma unroll
            for (int u = 0; u < kU; u++) {
                const int b = (i + u * 1024) * 4;
                argmax_take(v[u].x, b, best, bi); argmax_take(v[u].y, b + 1, best, bi);
                argmax_take(v[u].z, b + 2, best, bi); argmax_take(v[u].w, b + 3, best, bi);
            }
        }
        for (; i < n4; i += 1024) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(l) + i);
            argmax_take(v.x, i * 4, best, bi); argmax_take(v.y, i * 4 + 1, best, bi);
            argmax_take(v.z, i * 4 + 2, best, bi); argmax_take(v.w, i * 4 + 3, best, bi);
        }
        done = n4 * 4;
    }
    for (int i = done + t; i < V; i += 1024) argmax_take(l[i], i, best, bi);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        argmax_take(ov, oi, best, bi);
    }
    if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = best; s_idx[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int nw = blockDim.x >> 5;
        best = threadIdx.x < nw ? s_val[threadIdx.x] : -INFINITY;
        bi = threadIdx.x < nw ? s_idx[threadIdx.x] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, best, o);
            int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            argmax_take(ov, oi, best, bi);
        }
        if (threadIdx.x == 0) out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;  // all-NaN row -> 0
    }
}

// ---------------------------------------------------------------- AWQ unpack / dequant
// one thread per packed word: nibble i holds logical column 8j + {0,2,4,6,1,3,5,7}[i]
__device__ __forceinline__ void unpack8(uint32_t w, int (&q)[8]) {
    q[0] = w & 15; q[2] = (w >> 4) & 15; q[4] = (w >> 8) & 15; q[6] = (w >> 12) & 15;
    q[1] = (w >> 16) & 15; q[3] = (w >> 20) & 15; q[5] = (w >> 24) & 15; q[7] = (w >> 28) & 15;
}

__global__ void awq_unpack_kernel(const int32_t* __restrict__ qw, uint8_t* out, int64_t words) {
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < words; i += int64_t(gridDim.x) * blockDim.x) {
        int q[8];
        unpack8(uint32_t(qw[i]), q);
        uint2 packed;
        packed.x = q[0] | (q[1] << 8) | (q[2] << 16) | (q[3] << 24);
        packed.y = q[4] | (q[5] << 8) | (q[6] << 16) | (q[7] << 24);
        reinterpret_cast<uint2*>(out)[i] = packed;
    }
}

template <bool kBf16>
__global__ void awq_dequant_kernel(const int32_t* __restrict__ qw, const int32_t* __restrict__ qz,
                                   const __half* __restrict__ scales, void* out, int K, int N, int group) {
    const int NW = N / 8;
    const int64_t words = int64_t(K) * NW;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < words; i += int64_t(gridDim.x) * blockDim.x) {
        const int k = int(i / NW), j = int(i - int64_t(k) * NW), g = k / group;
        int q[8], z[8];
        unpack8(uint32_t(qw[i]), q);
        unpack8(uint32_t(qz[size_t(g) * NW + j]), z);
        const uint4 sraw = *reinterpret_cast<const uint4*>(scales + size_t(g) * N + 8 * j);
        const __half2* sh = reinterpret_cast<const __half2*>(&sraw);
        float v[8];
#pragma unroll
        for (int c = 0; c < 4; c++) {
            float2 s = __half22float2(sh[c]);
            v[2 * c] = float(q[2 * c] - z[2 * c]) * s.x;
            v[2 * c + 1] = float(q[2 * c + 1] - z[2 * c + 1]) * s.y;
        }
        if (kBf16) {
            uint4 o;
            o.x = float_to_bf16_bits(v[0]) | (uint32_t(float_to_bf16_bits(v[1])) << 16);
            o.y = float_to_bf16_bits(v[2]) | (uint32_t(float_to_bf16_bits(v[3])) << 16);
            o.z = float_to_bf16_bits(v[4]) | (uint32_t(float_to_bf16_bits(v[5])) << 16);
            o.w = float_to_bf16_bits(v[6]) | (uint32_t(float_to_bf16_bits(v[7])) << 16);
            reinterpret_cast<uint4*>(out)[i] = o;
        } else {
            float4* o = reinterpret_cast<float4*>(out) + 2 * i;
            o[0] = make_float4(v[0], v[1], v[2], v[3]);
            o[1] = make_float4(v[4], v[5], v[6], v[7]);
        }
    }
}

// ---------------------------------------------------------------- decode bookkeeping
__global__ void decode_advance_kernel(int32_t* tokens, const int32_t* next, int32_t* pos, int32_t* seq_len, int B,
                                      int max_seq) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    tokens[b] = next[b];
    int p = pos[b] + 1;
    p = p >= max_seq ? max_seq - 1 : p;
    pos[b] = p;
    seq_len[b] = p + 1;
}

int grid_for(int64_t work_items, int threads) {
    int64_t blocks = (work_items + threads - 1) / threads;
    const int64_t cap = 148 * 16;
    return int(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace
}  // namespace kuiper

using namespace kuiper;

extern "C" const char* kuiper_version(void) { return "kuiper_b200 0.1 (sm_100a)"; }
extern "C" const char* kuiper_last_error(void) { return g_error; }

extern "C" int kuiper_set_tuning(const char* key, int value) {
    if (!key) return KUIPER_INVALID_ARGUMENT;
    if (!strcmp(key, "pdl")) g_pdl_enabled = value;
    awq_gemv_set_tuning(key, value);
    flash_decode_set_tuning(key, value);
    awq_gemm_set_tuning(key, value);
    bf16_gemv_set_tuning(key, value);
    allreduce_set_tuning(key, value);
    return KUIPER_OK;
}

extern "C" int kuiper_workspace_init(void* workspace, size_t bytes, kuiper_stream_t stream) {
    KUIPER_REQUIRE(workspace != nullptr || bytes == 0, "workspace_init: null workspace");
    if (bytes == 0) return KUIPER_OK;
    cudaError_t err = cudaMemsetAsync(workspace, 0, bytes, as_stream(stream));
    if (err != cudaSuccess) {
        set_error("workspace_init: %s", cudaGetErrorString(err));
        return KUIPER_INTERNAL_ERROR;
    }
    return KUIPER_OK;
}

extern "C" int kuiper_add_f32(const float* a, const float* b, float* out, int64_t n, kuiper_stream_t stream) {
    KUIPER_REQUIRE(a && b && out, "add: null tensor pointer");
    KUIPER_REQUIRE(n > 0, "add: empty tensor");
    const int vec_ok = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    return pdl_status(launch_pdl(add_kernel, dim3(grid_for((n + 3) / 4, 256)), dim3(256), 0, as_stream(stream), a, b, out, n, vec_ok), "add");
}

extern "C" int kuiper_rmsnorm_f32(const float* x, const uint16_t* w, float* y, int M, int H, float eps,
                                  kuiper_stream_t stream) {
    KUIPER_REQUIRE(x && w && y, "rmsnorm: null tensor pointer");
    KUIPER_REQUIRE(M > 0 && H > 0, "rmsnorm: empty shape M=%d H=%d", M, H);
    return pdl_status(launch_pdl(rmsnorm_kernel<float>, dim3(M), dim3(kNormThreads), 0, as_stream(stream), x, w, y, H, eps), "rmsnorm");
}

extern "C" int kuiper_rmsnorm_f16(const float* x, const uint16_t* w, uint16_t* y16, int M, int H, float eps,
                                  kuiper_stream_t stream) {
    KUIPER_REQUIRE(x && w && y16, "rmsnorm_f16: null tensor pointer");
    KUIPER_REQUIRE(M > 0 && H > 0, "rmsnorm_f16: empty shape M=%d H=%d", M, H);
    return pdl_status(launch_pdl(rmsnorm_kernel<__half>, dim3(M), dim3(kNormThreads), 0, as_stream(stream), x, w,
                                 reinterpret_cast<__half*>(y16), H, eps), "rmsnorm_f16");
}

extern "C" int kuiper_swiglu_f32(float* gate_up, float* out, int M, int I, int clear_input, kuiper_stream_t stream) {
    KUIPER_REQUIRE(gate_up && out, "swiglu: null tensor pointer");
    KUIPER_REQUIRE(M > 0 && I > 0, "swiglu: empty shape M=%d I=%d", M, I);
    return pdl_status(launch_pdl(swiglu_kernel<float>, dim3(grid_for(int64_t(M) * I, 256)), dim3(256), 0, as_stream(stream), gate_up, out, M, I,
                                 clear_input), "swiglu");
}

extern "C" int kuiper_swiglu_f16(float* gate_up, uint16_t* out16, int M, int I, int clear_input, kuiper_stream_t stream) {
    KUIPER_REQUIRE(gate_up && out16, "swiglu_f16: null tensor pointer");
    KUIPER_REQUIRE(M > 0 && I > 0, "swiglu_f16: empty shape M=%d I=%d", M, I);
    return pdl_status(launch_pdl(swiglu_kernel<__half>, dim3(grid_for(int64_t(M) * I, 256)), dim3(256), 0, as_stream(stream), gate_up,
                                 reinterpret_cast<__half*>(out16), M, I, clear_input), "swiglu_f16");
}

extern "C" int kuiper_embedding_bf16(const int32_t* tokens, const uint16_t* table, float* out, int M, int H,
                                     int vocab, kuiper_stream_t stream) {
    KUIPER_REQUIRE(tokens && table && out, "embedding: null tensor pointer");
    KUIPER_REQUIRE(M > 0 && H > 0 && vocab > 0, "embedding: empty shape M=%d H=%d vocab=%d", M, H, vocab);
    return pdl_status(launch_pdl(embedding_kernel, dim3(M), dim3(256), 0, as_stream(stream), tokens, table, out, H, vocab), "embedding");
}

extern "C" int kuiper_argmax_f32(const float* logits, int32_t* out, int M, int V, kuiper_stream_t stream) {
    KUIPER_REQUIRE(logits && out, "argmax: null tensor pointer");
    KUIPER_REQUIRE(M > 0 && V > 0, "argmax: empty shape M=%d V=%d", M, V);
    return pdl_status(launch_pdl(argmax_kernel, dim3(M), dim3(1024), 0, as_stream(stream), logits, out, V), "argmax");
}

extern "C" int kuiper_awq_unpack_u8(const int32_t* qweight, uint8_t* out, int K, int N, kuiper_stream_t stream) {
    KUIPER_REQUIRE(qweight && out, "awq_unpack: null tensor pointer");
    KUIPER_REQUIRE(K > 0 && N > 0 && N % 8 == 0, "awq_unpack: bad shape K=%d N=%d", K, N);
    KUIPER_REQUIRE((reinterpret_cast<uintptr_t>(out) & 7) == 0, "awq_unpack: output must be 8-byte aligned");
    const int64_t words = int64_t(K) * (N / 8);
    awq_unpack_kernel<<<grid_for(words, 256), 256, 0, as_stream(stream)>>>(qweight, out, words);
    return launch_status("awq_unpack");
}

static int dequant_common(const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales, void* W, int K, int N,
                          int group, bool bf16, kuiper_stream_t stream) {
    KUIPER_REQUIRE(qweight && qzeros && scales && W, "awq_dequant: null tensor pointer");
    KUIPER_REQUIRE(K > 0 && N > 0 && N % 8 == 0, "awq_dequant: bad shape K=%d N=%d", K, N);
    KUIPER_REQUIRE(group > 0 && K % group == 0, "awq_dequant: K=%d is not a multiple of group %d", K, group);
    KUIPER_REQUIRE((reinterpret_cast<uintptr_t>(scales) & 15) == 0 && (reinterpret_cast<uintptr_t>(W) & 15) == 0,
                   "awq_dequant: scales and output must be 16-byte aligned");
    const int64_t words = int64_t(K) * (N / 8);
    if (bf16)
        awq_dequant_kernel<true><<<grid_for(words, 256), 256, 0, as_stream(stream)>>>(
            qweight, qzeros, reinterpret_cast<const __half*>(scales), W, K, N, group);
    else
        awq_dequant_kernel<false><<<grid_for(words, 256), 256, 0, as_stream(stream)>>>(
            qweight, qzeros, reinterpret_cast<const __half*>(scales), W, K, N, group);
    return launch_status("awq_dequant");
}

extern "C" int kuiper_awq_dequant_f32(const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales,
                                      float* W, int K, int N, int group, kuiper_stream_t stream) {
    return dequant_common(qweight, qzeros, scales, W, K, N, group, false, stream);
}

extern "C" int kuiper_awq_dequant_bf16(const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales,
                                       uint16_t* W, int K, int N, int group, kuiper_stream_t stream) {
    return dequant_common(qweight, qzeros, scales, W, K, N, group, true, stream);
}

extern "C" int kuiper_decode_advance(int32_t* tokens, const int32_t* next, int32_t* pos, int32_t* seq_len,
                                     int B, int max_seq, kuiper_stream_t stream) {
    KUIPER_REQUIRE(tokens && next && pos && seq_len, "decode_advance: null tensor pointer");
    KUIPER_REQUIRE(B > 0 && max_seq > 0, "decode_advance: empty shape");
    return pdl_status(launch_pdl(decode_advance_kernel, dim3((B + 127) / 128), dim3(128), 0, as_stream(stream), tokens, next, pos,
                                 seq_len, B, max_seq), "decode_advance");
}
