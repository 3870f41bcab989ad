// Per-head q/k RMSNorm + half-split rotary embedding + KV-cache append for sm_100a.
// Fills the reference's empty rotary placeholder (kuiper/include/op/rope.h:1-10); the
// buffers it touches are the ones model::ModelBufferType names Query / KeyCache /
// ValueCache / SinCache / CosCache / InputPos (kuiper/include/base/base.h:12-31).
//
// One warp per (token row, head).  D = 128: lane l holds elements l, l+32 of the first
// half and l+64, l+96 of the second half, so both rotary partners of an element live in
// the same lane and the only cross-lane step is the sum of squares.
#include "common.cuh"

namespace kuiper {
namespace {

constexpr int kD = 128;

__global__ void __launch_bounds__(128)
qknorm_rope_kvwrite_kernel(float* qkv, const uint16_t* __restrict__ q_norm_w, const uint16_t* __restrict__ k_norm_w,
                           const float* __restrict__ cos_t, const float* __restrict__ sin_t, const int32_t* pos,
                           const int32_t* slot, int M, int Nq, int Nkv, float eps, int max_seq, int n_slots, float* q_out,
                           uint16_t* kcache, uint16_t* vcache, int clear_input, float4* clear_extra, int clear_extra_vec4) {
    pdl_launch_dependents();
    pdl_wait();
    // optional side job: zero another buffer (the gate|up projection output, which nothing uses at this point of a
    // layer and which the next accumulating matmul into it wants zeroed)
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < clear_extra_vec4; i += gridDim.x * blockDim.x)
        clear_extra[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    const int heads = Nq + 2 * Nkv;
    const int wid = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (wid >= M * heads) return;
    const int lane = threadIdx.x & 31;
    const int m = wid / heads, h = wid - m * heads;
    float* src = qkv + (size_t(m) * heads + h) * kD;
    int p = pos[m];
    p = p < 0 ? 0 : (p >= max_seq ? max_seq - 1 : p);  // clamp: never write outside the cache
    int sl = slot[m];
    sl = sl < 0 ? 0 : (sl >= n_slots ? n_slots - 1 : sl);
    const float a0 = src[lane], a1 = src[lane + 32], b0 = src[lane + 64], b1 = src[lane + 96];
    if (clear_input) {  // leave the projection buffer zeroed for the next accumulating matmul
        src[lane] = 0.f; src[lane + 32] = 0.f; src[lane + 64] = 0.f; src[lane + 96] = 0.f;
    }

    if (h >= Nq + Nkv) {  // value head: plain bf16 store
        uint16_t* dst = vcache + ((size_t(sl) * Nkv + (h - Nq - Nkv)) * max_seq + p) * kD;
        dst[lane] = float_to_bf16_bits(a0);
        dst[lane + 32] = float_to_bf16_bits(a1);
        dst[lane + 64] = float_to_bf16_bits(b0);
        dst[lane + 96] = float_to_bf16_bits(b1);
        return;
    }
    const uint16_t* w = h < Nq ? q_norm_w : k_norm_w;
    float ss = a0 * a0;
    ss = fmaf(a1, a1, ss);
    ss = fmaf(b0, b0, ss);
    ss = fmaf(b1, b1, ss);
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / float(kD) + eps);
    const float x0 = (a0 * rstd) * bf16_bits_to_float(w[lane]);
    const float x1 = (a1 * rstd) * bf16_bits_to_float(w[lane + 32]);
    const float y0 = (b0 * rstd) * bf16_bits_to_float(w[lane + 64]);
    const float y1 = (b1 * rstd) * bf16_bits_to_float(w[lane + 96]);
    const float c0 = cos_t[size_t(p) * 64 + lane], s0 = sin_t[size_t(p) * 64 + lane];
    const float c1 = cos_t[size_t(p) * 64 + lane + 32], s1 = sin_t[size_t(p) * 64 + lane + 32];
    // separate multiply and subtract/add, matching (x*c) - (y*s) evaluated without contraction
    const float r0 = __fsub_rn(__fmul_rn(x0, c0), __fmul_rn(y0, s0));
    const float r1 = __fsub_rn(__fmul_rn(x1, c1), __fmul_rn(y1, s1));
    const float t0 = __fadd_rn(__fmul_rn(y0, c0), __fmul_rn(x0, s0));
    const float t1 = __fadd_rn(__fmul_rn(y1, c1), __fmul_rn(x1, s1));
    if (h < Nq) {
        float* dst = q_out + (size_t(m) * Nq + h) * kD;
        dst[lane] = r0; dst[lane + 32] = r1; dst[lane + 64] = t0; dst[lane + 96] = t1;
    } else {
        uint16_t* dst = kcache + ((size_t(sl) * Nkv + (h - Nq)) * max_seq + p) * kD;
        dst[lane] = float_to_bf16_bits(r0);
        dst[lane + 32] = float_to_bf16_bits(r1);
        dst[lane + 64] = float_to_bf16_bits(t0);
        dst[lane + 96] = float_to_bf16_bits(t1);
    }
}

}  // namespace
}  // namespace kuiper

using namespace kuiper;

extern "C" int kuiper_qknorm_rope_kvwrite(float* qkv, const uint16_t* q_norm_w, const uint16_t* k_norm_w,
                                          const float* cos_t, const float* sin_t, const int32_t* pos,
                                          const int32_t* slot, int M, int Nq, int Nkv, int D, float eps,
                                          int max_seq, int n_slots, float* q_out, uint16_t* kcache, uint16_t* vcache,
                                          int clear_input, float* clear_extra, int64_t clear_extra_count,
                                          kuiper_stream_t stream) {
    KUIPER_REQUIRE(clear_extra_count >= 0 && (clear_extra_count == 0 || clear_extra), "qknorm_rope: bad extra buffer");
    KUIPER_REQUIRE(clear_extra_count % 4 == 0 && (reinterpret_cast<uintptr_t>(clear_extra) & 15) == 0 &&
                       clear_extra_count / 4 <= 0x7fffffff,
                   "qknorm_rope: the extra buffer must be 16-byte aligned with a multiple of 4 floats");
    KUIPER_REQUIRE(qkv && q_norm_w && k_norm_w && cos_t && sin_t && pos && slot && q_out && kcache && vcache,
                   "qknorm_rope: null tensor pointer");
    KUIPER_REQUIRE(D == kD, "qknorm_rope: head_dim %d is not supported (128 only)", D);
    KUIPER_REQUIRE(M > 0 && Nq > 0 && Nkv > 0 && max_seq > 0 && n_slots > 0, "qknorm_rope: empty shape");
    const int warps = M * (Nq + 2 * Nkv);
    return pdl_status(launch_pdl(qknorm_rope_kvwrite_kernel, dim3((warps + 3) / 4), dim3(128), 0, as_stream(stream), qkv, q_norm_w,
                                 k_norm_w, cos_t, sin_t, pos, slot, M, Nq, Nkv, eps, max_seq, n_slots, q_out, kcache, vcache,
                                 clear_input, reinterpret_cast<float4*>(clear_extra), int(clear_extra_count / 4)),
                      "qknorm_rope_kvwrite");
}
