// GQA flash-decoding for sm_100a: split-KV attention over a bf16 KV cache with a
// log-sum-exp combine.  Fills the reference's empty attention placeholder
// (kuiper/include/op/mha.h:1-11); the reference's buffer list has a ScoreStorage entry
// (kuiper/include/base/base.h:19), i.e. it intended to materialise the score row - here
// scores never leave registers.
//
// Layout: cache[(slot*Nkv + kv_head)*max_seq + pos][128] bf16, so one KV head of one
// sequence is a contiguous run of 256-byte rows.
//
// grid = (splits, Nkv, M).  A CTA (4 warps) takes one contiguous slice of the KV range of
// one (token row, kv head) and serves all R = Nq/Nkv query heads that share it, so K and V
// are read once.  16 lanes cover one 256-byte row (16 bytes per lane); a warp step loads
// 16 rows (8 per half warp) of K and of V before the first use.  Each warp keeps running
// (max, sum, out) per head; warps merge through shared memory, CTAs through the workspace,
// where the last CTA to arrive at a (row, kv head) does the final combine in slice order.
#include <cstring>

#include "common.cuh"

namespace kuiper {
namespace {

constexpr int kD = 128;
constexpr int kWarps = 4;
constexpr int kMaxSplits = 64;      // slices per (row, kv head)
constexpr int kMaxSplitsMma = 128;  // same for calls of at most kFewRows rows on the four-warp tensor-core kernel
constexpr int kFewRows = 2;
constexpr int kCtasStandalone = 2, kCtasFusedNarrow = 2;  // resident CTAs per SM the four-warp tensor-core kernels are built for
constexpr int kRowsPerStep = 8;  // row slots per half warp per step

int g_force_splits = 0;
int g_flash_drop_slice = -1;  // tuning key "flash_drop_slice" (tests only)
long long g_flash_timeout_ns = 1000000000ll;  // bound of the combining CTA's wait for the other slices (tuning key "flash_timeout_ms")
__device__ int g_flash_wait_error = 0;

__device__ __forceinline__ void st_tagged(uint2* p, float v, unsigned int tag) {
    asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}
__device__ __forceinline__ uint2 ld_tagged(const uint2* p) {
    uint2 v;
    asm volatile("ld.relaxed.gpu.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
int g_flash_early = 1;  // 0: ignore fresh_rows, touch nothing before the dependent-launch wait
int g_flash_mma_fused = 1;  // the fused decode kernel (rotary + append + attention) also uses the tensor cores (0: SIMT)
int g_flash_mma = 1;    // the stand-alone attention call runs its contractions on the tensor cores (0: SIMT kernel)
int g_flash_wide = 1;   // fused tensor-core kernel: eight-warp CTAs when the whole grid is one wave of them (0: always four warps)

// Build flag KUIPER_TRACE (off in the shipped library): every CTA of the tensor-core attention kernel stores clock
// readings at its milestones; kuiper_flash_trace_read() copies those of the last launch to the host.
// slot 0: global timer (ns) at entry; then SM clock at 1 entry, 2 early fetches issued, 3 dependency wait passed,
// 4 q / appended row ready, 5 cache rows processed, 6 partial stored and fenced, 7 arrival counter answered,
// 8 slices combined, 9 output stored (last CTA of a kv head only)
#ifdef KUIPER_TRACE
constexpr int kFlashTraceCtas = 1024, kFlashTraceSlots = 10;
__device__ long long g_flash_trace[kFlashTraceCtas * kFlashTraceSlots];
__device__ __forceinline__ void flash_trace(int slot) {
    if (threadIdx.x == 0) {
        const int cta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
        if (cta < kFlashTraceCtas) g_flash_trace[cta * kFlashTraceSlots + slot] = slot == 0 ? (long long)globaltimer_ns() : clock64();
    }
}
#else
__device__ __forceinline__ void flash_trace(int) {}
#endif

struct FlashParams {
    const float* q;       // [M, Nq, 128]
    const uint16_t* kc;
    const uint16_t* vc;
    const int32_t* seq_len;
    const int32_t* slot;
    float* out;           // [M, Nq, 128]
    float* part_o;        // [M, Nkv, S, R, 128]
    float* part_ml;       // [M, Nkv, S, R, 2]
    int* counters;        // [M * Nkv]
    // eight-warp CTAs: the partials travel as 8-byte words {value, launch number} that the combining CTA polls
    uint2* ll_o;          // [M, Nkv, S, R, 128]
    uint2* ll_ml;         // [M, Nkv, S, R, 2]
    unsigned int* ll_seq; // [M * Nkv] launch number of the last combine
    long long ll_timeout_ns;
    int ll_drop;          // test hook: this slice never sends its words (-1: none), so that the bounded wait can be exercised
    int M, Nq, Nkv, max_seq, n_slots, S;
    int fresh_rows;       // cache rows >= seq_len - fresh_rows may still be in flight from the previous kernel; < 0: all
    // fused rotary prologue (FUSED kernels): q and the newest K / V row are produced here from the raw projection
    float* qkv;                // [M, (Nq + 2 Nkv) * 128] q heads | k heads | v heads
    const uint16_t* q_norm_w;  // bf16 [128]
    const uint16_t* k_norm_w;
    const float* cos_t;        // [max_pos, 64]
    const float* sin_t;
    const int32_t* pos;        // [M], seq_len[m] == pos[m] + 1
    uint16_t* kc_w;            // the caches again, writable
    uint16_t* vc_w;
    float4* clear_extra;       // optional side job: zero this buffer
    int clear_extra_vec4;
    int clear_qkv;             // zero the slices of qkv this (row, kv head) read once nobody needs them any more
    float eps;
};

// q/k RMSNorm over the head + half-split rotary for one head held by one warp: lane l has elements l, l+32 (first
// half) and l+64, l+96 (second half).  Same arithmetic, in the same order, as qknorm_rope_kvwrite_kernel.
__device__ __forceinline__ void head_norm_rope(float a0, float a1, float b0, float b1, const uint16_t* __restrict__ w,
                                               const float* __restrict__ cos_row, const float* __restrict__ sin_row,
                                               float eps, int lane, float (&out)[4]) {
    float ss = a0 * a0;
    ss = fmaf(a1, a1, ss);
    ss = fmaf(b0, b0, ss);
    ss = fmaf(b1, b1, ss);
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / float(128) + eps);
    const float x0 = (a0 * rstd) * bf16_bits_to_float(w[lane]);
    const float x1 = (a1 * rstd) * bf16_bits_to_float(w[lane + 32]);
    const float y0 = (b0 * rstd) * bf16_bits_to_float(w[lane + 64]);
    const float y1 = (b1 * rstd) * bf16_bits_to_float(w[lane + 96]);
    const float c0 = cos_row[lane], s0 = sin_row[lane];
    const float c1 = cos_row[lane + 32], s1 = sin_row[lane + 32];
    out[0] = __fsub_rn(__fmul_rn(x0, c0), __fmul_rn(y0, s0));
    out[1] = __fsub_rn(__fmul_rn(x1, c1), __fmul_rn(y1, s1));
    out[2] = __fadd_rn(__fmul_rn(y0, c0), __fmul_rn(x0, s0));
    out[3] = __fadd_rn(__fmul_rn(y1, c1), __fmul_rn(x1, s1));
}

// a cache row slice; rows this kernel itself wrote must not go through the non-coherent path
__device__ __forceinline__ uint4 ld_row(const uint16_t* ptr, bool coherent) {
    return coherent ? __ldcg(reinterpret_cast<const uint4*>(ptr)) : ld_stream_u4(ptr);
}

template <int R, bool FUSED>
__global__ void __launch_bounds__(kWarps * 32)
flash_decode_kernel(const FlashParams p) {
    __shared__ float s_o[kWarps][R][kD];
    __shared__ float s_q[FUSED ? R : 1][kD];
    __shared__ float s_ml[kWarps][R][2];
    __shared__ int s_last;

    const int split = blockIdx.x, kvh = blockIdx.y, m = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int half = lane >> 4, li = lane & 15;  // half warp and lane within it

    pdl_launch_dependents();
    // With fresh_rows >= 0 the caller vouches that every cache row below seq_len - fresh_rows was final before the
    // work that this grid may overtake under programmatic dependent launch was enqueued, so those rows are fetched
    // while the previous kernel (the one that appends the newest rows and produces q) is still finishing.  seq_len
    // and slot are read early too, but re-read after the wait: if they changed, the kernel starts over.
    // With fresh_rows < 0 nothing is touched before the wait.
    bool waited = p.fresh_rows < 0;
    if (waited) pdl_wait();

    int L, sl, n_active, begin, end, base0, fetched_end;
    const uint16_t *kb, *vb;
    uint4 kraw[kRowsPerStep], vraw[kRowsPerStep];
    while (true) {
        L = __ldcg(p.seq_len + m);
        sl = __ldcg(p.slot + m);
        const int L_seen = L, sl_seen = sl;
        L = L < 0 ? 0 : (L > p.max_seq ? p.max_seq : L);
        sl = sl < 0 ? 0 : (sl >= p.n_slots ? p.n_slots - 1 : sl);
        // slice of the KV range owned by this CTA, in units of 64 rows
        const int blocks = max((L + 63) / 64, 1);
        const int per = (blocks + p.S - 1) / p.S;
        // splits that have rows; the others leave at once and are not waited for
        n_active = (blocks + per - 1) / per;
        begin = split * per * 64;
        end = min(L, begin + per * 64);
        const size_t head_off = (size_t(sl) * p.Nkv + kvh) * p.max_seq * kD;
        kb = p.kc + head_off;
        vb = p.vc + head_off;
        // first step of this warp: rows base0 + half + 2*r; rows below safe_end may be read before the wait
        base0 = begin + warp * 16;
        const bool has_rows = split < n_active;
        // (fused: the newest row is produced by this kernel, so it is never fetched here)
        const int safe_end = waited ? (FUSED ? min(end, L - 1) : end) : min(end, L - (FUSED ? max(p.fresh_rows, 1) : p.fresh_rows));
        fetched_end = safe_end;
#pragma unroll
        for (int r = 0; r < kRowsPerStep; r++) {
            const int row = base0 + half + 2 * r;
            kraw[r] = (has_rows && row < safe_end) ? ld_stream_u4(kb + size_t(row) * kD + li * 8) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int r = 0; r < kRowsPerStep; r++) {
            const int row = base0 + half + 2 * r;
            vraw[r] = (has_rows && row < safe_end) ? ld_stream_u4(vb + size_t(row) * kD + li * 8) : make_uint4(0, 0, 0, 0);
        }
        if (waited) break;
        pdl_wait();
        waited = true;
        // seq_len / slot themselves may have been written by something this grid was allowed to overtake:
        // if they changed, start over with nothing assumed
        if (__ldcg(p.seq_len + m) != L_seen || __ldcg(p.slot + m) != sl_seen) continue;
        break;
    }
    if (FUSED) {
        // side job: zero the buffer the caller named (nothing uses it at this point of a layer)
        const int ctas = gridDim.x * gridDim.y * gridDim.z;
        const int cta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
        for (int i = cta * (kWarps * 32) + threadIdx.x; i < p.clear_extra_vec4; i += ctas * kWarps * 32)
            p.clear_extra[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (split >= n_active) return;

    const int heads = p.Nq + 2 * p.Nkv;
    const int newest = L - 1;  // the row appended by this pass (fused) / by the previous kernel
    if (FUSED) {
        int pp = p.pos[m];
        pp = pp < 0 ? 0 : (pp >= p.max_seq ? p.max_seq - 1 : pp);
        const float* cos_row = p.cos_t + size_t(pp) * 64;
        const float* sin_row = p.sin_t + size_t(pp) * 64;
        // q heads of this kv head: one warp per head
        for (int h = warp; h < R; h += kWarps) {
            const float* src = p.qkv + (size_t(m) * heads + kvh * R + h) * kD;
            float r4[4];
            head_norm_rope(__ldcg(src + lane), __ldcg(src + lane + 32), __ldcg(src + lane + 64), __ldcg(src + lane + 96),
                           p.q_norm_w, cos_row, sin_row, p.eps, lane, r4);
            s_q[h][lane] = r4[0]; s_q[h][lane + 32] = r4[1]; s_q[h][lane + 64] = r4[2]; s_q[h][lane + 96] = r4[3];
        }
        // the CTA whose slice holds the newest row appends it: K through norm + rotary, V as it is, both as bf16
        if (newest >= begin && newest < end) {
            const size_t row_off = ((size_t(sl) * p.Nkv + kvh) * p.max_seq + pp) * kD;
            if (warp == kWarps - 1) {
                const float* src = p.qkv + (size_t(m) * heads + p.Nq + kvh) * kD;
                float r4[4];
                head_norm_rope(__ldcg(src + lane), __ldcg(src + lane + 32), __ldcg(src + lane + 64), __ldcg(src + lane + 96),
                               p.k_norm_w, cos_row, sin_row, p.eps, lane, r4);
                uint16_t* dst = p.kc_w + row_off;
                dst[lane] = float_to_bf16_bits(r4[0]);
                dst[lane + 32] = float_to_bf16_bits(r4[1]);
                dst[lane + 64] = float_to_bf16_bits(r4[2]);
                dst[lane + 96] = float_to_bf16_bits(r4[3]);
            } else if (warp == kWarps - 2) {
                const float* src = p.qkv + (size_t(m) * heads + p.Nq + p.Nkv + kvh) * kD;
                uint16_t* dst = p.vc_w + row_off;
                dst[lane] = float_to_bf16_bits(__ldcg(src + lane));
                dst[lane + 32] = float_to_bf16_bits(__ldcg(src + lane + 32));
                dst[lane + 64] = float_to_bf16_bits(__ldcg(src + lane + 64));
                dst[lane + 96] = float_to_bf16_bits(__ldcg(src + lane + 96));
            }
        }
        __syncthreads();  // s_q is complete; the appended row is visible to the whole CTA
    }
    // rows of the first step that were not fetched ahead of the wait
    {
#pragma unroll
        for (int r = 0; r < kRowsPerStep; r++) {
            const int row = base0 + half + 2 * r;
            if (row >= fetched_end && row < end) {
                const bool coherent = FUSED && row >= newest;
                kraw[r] = ld_row(kb + size_t(row) * kD + li * 8, coherent);
                vraw[r] = ld_row(vb + size_t(row) * kD + li * 8, coherent);
            }
        }
    }

    // q slice of this lane: elements li*8 .. li*8+7 of each of the R heads, pre-scaled
    const float scale = 0.08838834764831845f;  // 1/sqrt(128)
    float qr[R][8];
#pragma unroll
    for (int h = 0; h < R; h++) {
        float4 a, b;
        if (FUSED) {
            a = *reinterpret_cast<const float4*>(&s_q[h][li * 8]);
            b = *reinterpret_cast<const float4*>(&s_q[h][li * 8 + 4]);
        } else {
            const float* qp = p.q + (size_t(m) * p.Nq + kvh * R + h) * kD + li * 8;
            a = __ldcg(reinterpret_cast<const float4*>(qp));
            b = __ldcg(reinterpret_cast<const float4*>(qp + 4));
        }
        qr[h][0] = a.x * scale; qr[h][1] = a.y * scale; qr[h][2] = a.z * scale; qr[h][3] = a.w * scale;
        qr[h][4] = b.x * scale; qr[h][5] = b.y * scale; qr[h][6] = b.z * scale; qr[h][7] = b.w * scale;
    }

    float o[R][8];
    float mx[R], sum[R];
#pragma unroll
    for (int h = 0; h < R; h++) {
        mx[h] = -INFINITY;
        sum[h] = 0.f;
#pragma unroll
        for (int e = 0; e < 8; e++) o[h][e] = 0.f;
    }

    // warp w takes rows begin + w*16 + step*64 + half + 2*r, r = 0..7
    for (int base = base0; base < end; base += kWarps * 16) {
        if (base != base0) {
#pragma unroll
            for (int r = 0; r < kRowsPerStep; r++) {
                const int row = base + half + 2 * r;
                const bool ok = row < end;
                kraw[r] = ok ? ld_row(kb + size_t(row) * kD + li * 8, FUSED && row >= newest) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int r = 0; r < kRowsPerStep; r++) {
                const int row = base + half + 2 * r;
                const bool ok = row < end;
                vraw[r] = ok ? ld_row(vb + size_t(row) * kD + li * 8, FUSED && row >= newest) : make_uint4(0, 0, 0, 0);
            }
        }
        float s[kRowsPerStep][R];
#pragma unroll
        for (int r = 0; r < kRowsPerStep; r++) {
            const float kf[8] = {bf16_lo(kraw[r].x), bf16_hi(kraw[r].x), bf16_lo(kraw[r].y), bf16_hi(kraw[r].y),
                                 bf16_lo(kraw[r].z), bf16_hi(kraw[r].z), bf16_lo(kraw[r].w), bf16_hi(kraw[r].w)};
#pragma unroll
            for (int h = 0; h < R; h++) {
                float d = 0.f;
#pragma unroll
                for (int e = 0; e < 8; e++) d = fmaf(qr[h][e], kf[e], d);
                s[r][h] = d;
            }
        }
        // sum over the 16 lanes of a half warp
#pragma unroll
        for (int off = 8; off > 0; off >>= 1)
#pragma unroll
            for (int r = 0; r < kRowsPerStep; r++)
#pragma unroll
                for (int h = 0; h < R; h++) s[r][h] += __shfl_xor_sync(0xffffffffu, s[r][h], off);

#pragma unroll
        for (int h = 0; h < R; h++) {
            float bm = -INFINITY;
#pragma unroll
            for (int r = 0; r < kRowsPerStep; r++) {
                const bool ok = (base + half + 2 * r) < end;
                s[r][h] = ok ? s[r][h] : -INFINITY;
                bm = fmaxf(bm, s[r][h]);
            }
            const float nm = fmaxf(mx[h], bm);
            // nm is -inf only while this half warp has not seen a valid row yet
            const float corr = (nm == -INFINITY) ? 1.f : __expf(mx[h] - nm);
            mx[h] = nm;
            sum[h] *= corr;
#pragma unroll
            for (int e = 0; e < 8; e++) o[h][e] *= corr;
#pragma unroll
            for (int r = 0; r < kRowsPerStep; r++) {
                const float pexp = (s[r][h] == -INFINITY) ? 0.f : __expf(s[r][h] - nm);
                s[r][h] = pexp;
                sum[h] += pexp;
            }
        }
#pragma unroll
        for (int r = 0; r < kRowsPerStep; r++) {
            const float vf[8] = {bf16_lo(vraw[r].x), bf16_hi(vraw[r].x), bf16_lo(vraw[r].y), bf16_hi(vraw[r].y),
                                 bf16_lo(vraw[r].z), bf16_hi(vraw[r].z), bf16_lo(vraw[r].w), bf16_hi(vraw[r].w)};
#pragma unroll
            for (int h = 0; h < R; h++)
#pragma unroll
                for (int e = 0; e < 8; e++) o[h][e] = fmaf(s[r][h], vf[e], o[h][e]);
        }
    }

    // merge the two half warps (they saw different rows)
#pragma unroll
    for (int h = 0; h < R; h++) {
        const float om = __shfl_xor_sync(0xffffffffu, mx[h], 16);
        const float os = __shfl_xor_sync(0xffffffffu, sum[h], 16);
        const float nm = fmaxf(mx[h], om);
        const float c_self = (mx[h] == -INFINITY) ? 0.f : __expf(mx[h] - nm);
        const float c_other = (om == -INFINITY) ? 0.f : __expf(om - nm);
        sum[h] = sum[h] * c_self + os * c_other;
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const float oo = __shfl_xor_sync(0xffffffffu, o[h][e], 16);
            o[h][e] = o[h][e] * c_self + oo * c_other;
        }
        mx[h] = nm;
    }
    if (half == 0) {
#pragma unroll
        for (int h = 0; h < R; h++) {
#pragma unroll
            for (int e = 0; e < 8; e++) s_o[warp][h][li * 8 + e] = o[h][e];
            if (li == 0) { s_ml[warp][h][0] = mx[h]; s_ml[warp][h][1] = sum[h]; }
        }
    }
    __syncthreads();

    // merge the warps: thread t owns element t of every head
    const int t = threadIdx.x;
    float fo[R], fm[R], fs[R];
#pragma unroll
    for (int h = 0; h < R; h++) {
        float nm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; w++) nm = fmaxf(nm, s_ml[w][h][0]);
        float acc = 0.f, ssum = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; w++) {
            const float wm = s_ml[w][h][0];
            const float c = (wm == -INFINITY) ? 0.f : __expf(wm - nm);
            acc += s_o[w][h][t] * c;
            ssum += s_ml[w][h][1] * c;
        }
        fo[h] = acc; fm[h] = nm; fs[h] = ssum;
    }

    // fused: once every CTA of this (row, kv head) is past its prologue, the raw q / k / v slices can be zeroed for
    // the next projection that accumulates into the buffer
    auto clear_raw = [&]() {
        if (FUSED && p.clear_qkv) {
            float* row = p.qkv + size_t(m) * heads * kD;
#pragma unroll
            for (int h = 0; h < R; h++) row[(kvh * R + h) * kD + t] = 0.f;
            row[(p.Nq + kvh) * kD + t] = 0.f;
            row[(p.Nq + p.Nkv + kvh) * kD + t] = 0.f;
        }
    };
    if (n_active == 1) {
#pragma unroll
        for (int h = 0; h < R; h++)
            p.out[(size_t(m) * p.Nq + kvh * R + h) * kD + t] = fs[h] > 0.f ? fo[h] / fs[h] : 0.f;
        clear_raw();
        return;
    }

    const size_t pbase = (size_t(m) * p.Nkv + kvh) * p.S;
#pragma unroll
    for (int h = 0; h < R; h++) {
        p.part_o[((pbase + split) * R + h) * kD + t] = fo[h];
        if (t == 0) {
            p.part_ml[((pbase + split) * R + h) * 2] = fm[h];
            p.part_ml[((pbase + split) * R + h) * 2 + 1] = fs[h];
        }
    }
    __threadfence();
    __syncthreads();
    if (t == 0) {
        const int prev = atomicAdd(p.counters + m * p.Nkv + kvh, 1);
        s_last = (prev == n_active - 1);
        if (s_last) p.counters[m * p.Nkv + kvh] = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // ---- final combine by the last CTA.  Weights first: warp w takes heads w, w + 4, ...; lane l holds the
    // (max, sum) of slices l and l + 32, so the maximum and the denominator are two warp reductions.
    __shared__ float s_w[64 * R];   // weight of slice sp for head h at [sp * R + h]
    __shared__ float s_den[R];
    for (int h = warp; h < R; h += kWarps) {
        float2 ml0 = make_float2(-INFINITY, 0.f), ml1 = ml0;
        if (lane < n_active) ml0 = __ldcg(reinterpret_cast<const float2*>(p.part_ml + ((pbase + lane) * R + h) * 2));
        if (lane + 32 < n_active) ml1 = __ldcg(reinterpret_cast<const float2*>(p.part_ml + ((pbase + lane + 32) * R + h) * 2));
        const float nm = warp_max(fmaxf(ml0.x, ml1.x));
        const float w0 = (ml0.x == -INFINITY) ? 0.f : __expf(ml0.x - nm);
        const float w1 = (ml1.x == -INFINITY) ? 0.f : __expf(ml1.x - nm);
        const float den = warp_sum(ml0.y * w0 + ml1.y * w1);
        s_w[lane * R + h] = w0;
        s_w[(lane + 32) * R + h] = w1;
        if (lane == 0) s_den[h] = den;
    }
    __syncthreads();
    // then the partial outputs in slice order, eight slices of every head in flight per thread
    float acc[R];
#pragma unroll
    for (int h = 0; h < R; h++) acc[h] = 0.f;
    const float* po = p.part_o + pbase * R * kD + t;
    int sp = 0;
    for (; sp + 8 <= n_active; sp += 8) {
        float a[8][R];
#pragma unroll
        for (int q = 0; q < 8; q++)
#pragma unroll
            for (int h = 0; h < R; h++) a[q][h] = __ldcg(po + (size_t(sp + q) * R + h) * kD);
#pragma unroll
        for (int q = 0; q < 8; q++)
#pragma unroll
            for (int h = 0; h < R; h++) acc[h] = fmaf(a[q][h], s_w[(sp + q) * R + h], acc[h]);
    }
    for (; sp < n_active; sp++) {
        float a[R];
#pragma unroll
        for (int h = 0; h < R; h++) a[h] = __ldcg(po + (size_t(sp) * R + h) * kD);
#pragma unroll
        for (int h = 0; h < R; h++) acc[h] = fmaf(a[h], s_w[sp * R + h], acc[h]);
    }
#pragma unroll
    for (int h = 0; h < R; h++) {
        const float den = s_den[h];
        p.out[(size_t(m) * p.Nq + kvh * R + h) * kD + t] = den > 0.f ? acc[h] / den : 0.f;
    }
    clear_raw();
}

// ---------------------------------------------------------------- the same attention on the tensor cores
//
// For long caches the kernel above is bound by instruction issue (~2 000 SIMT instructions per 16 cache rows and
// kv head), not by the memory system.  This variant keeps its grid, slices, workspace and combine, and moves the
// two contractions of a 16-row step to mma.sync.m16n8k16 (bf16 x bf16 -> fp32), transposed so that the cache rows
// fill the 16-wide dimension and the (up to 8) query heads of the kv head the 8-wide one:
//
//   S^T[row][head] = K[row][dim] . Q^T[dim][head]      A = K as it lies in the cache (row-major), B = q
//   O^T[dim][head] += V^T[dim][row] . P^T[row][head]   A = V^T and B = P^T by movmatrix (8x8 transposes in registers)
//
// K and V are bf16 in the cache, so they are exact operands; q and the probabilities are split into a bf16 high and
// low part (two mma each), which keeps 16 significant bits.  A lane loads 16 contiguous bytes of a row as in the
// kernel above; which head dimension sits at which contraction / fragment index is a fixed permutation that q's
// fragments and the final store follow.
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
// (x, y) as bf16 high parts in one register (x in the low half) and what is left of them as bf16 low parts
__device__ __forceinline__ void split_bf16x2(float x, float y, uint32_t& hi, uint32_t& lo) {
    const uint32_t xh = float_to_bf16_bits(x), yh = float_to_bf16_bits(y);
    hi = xh | (yh << 16);
    const float xr = x - bf16_bits_to_float(uint16_t(xh)), yr = y - bf16_bits_to_float(uint16_t(yh));
    lo = uint32_t(float_to_bf16_bits(xr)) | (uint32_t(float_to_bf16_bits(yr)) << 16);
}

// q/k RMSNorm over the head + half-split rotary with the norm weights and the rotary row already in registers
// (w: elements lane, lane+32, lane+64, lane+96 of the bf16 weight; cs: cos[lane], cos[lane+32], sin[lane], sin[lane+32]).
// Same arithmetic, in the same order, as head_norm_rope.
__device__ __forceinline__ void head_norm_rope_regs(float a0, float a1, float b0, float b1, const float (&w)[4],
                                                    const float (&cs)[4], float eps, float (&out)[4]) {
    float ss = a0 * a0;
    ss = fmaf(a1, a1, ss);
    ss = fmaf(b0, b0, ss);
    ss = fmaf(b1, b1, ss);
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / float(128) + eps);
    const float x0 = (a0 * rstd) * w[0];
    const float x1 = (a1 * rstd) * w[1];
    const float y0 = (b0 * rstd) * w[2];
    const float y1 = (b1 * rstd) * w[3];
    out[0] = __fsub_rn(__fmul_rn(x0, cs[0]), __fmul_rn(y0, cs[2]));
    out[1] = __fsub_rn(__fmul_rn(x1, cs[1]), __fmul_rn(y1, cs[3]));
    out[2] = __fadd_rn(__fmul_rn(y0, cs[0]), __fmul_rn(x0, cs[2]));
    out[3] = __fadd_rn(__fmul_rn(y1, cs[1]), __fmul_rn(x1, cs[3]));
}

// Launch shapes.  Four warps (stand-alone and fused): two CTAs per SM, up to 255 registers - a warp holds two steps of
// cache rows (the one it works on and the next one in flight, 128 registers), which hides the memory latency better
// than the five CTAs per SM of one-step warps did (batch 1, 32 768 rows: 3.0 -> 4.6 TB/s; batch 16: 5.2 -> 5.7 TB/s).
// Fused, eight warps: one CTA per SM and one 128-row step per CTA -
// the shape for a single sequence at a context of a few thousand rows, where the kernel is a chain of latencies and the
// number of slices the last CTA has to combine is what counts.
template <int R, bool FUSED, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, FUSED ? (WARPS == 8 ? 1 : kCtasFusedNarrow) : kCtasStandalone)
flash_decode_mma_kernel(const FlashParams p) {
    constexpr int kBlk = WARPS * 16;  // cache rows per CTA step
    constexpr int kThreads = WARPS * 32;
    __shared__ float s_o[WARPS][R][kD];
    __shared__ float s_q[FUSED ? R : 1][kD];
    __shared__ float s_ml[WARPS][R][2];
    __shared__ __align__(16) uint16_t s_new[FUSED ? 2 : 1][kD];  // fused: the K / V row appended by this CTA
    __shared__ int s_last;
    __shared__ unsigned int s_tag;

    const int split = blockIdx.x, kvh = blockIdx.y, m = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;  // fragment row / column group and thread in group

    flash_trace(0);
    flash_trace(1);
    pdl_launch_dependents();
    if (WARPS == 8 && threadIdx.x == 0 && p.ll_seq != nullptr) {
        // launch number of this (row, kv head): last written by the combining CTA of the previous attention launch, which
        // completed long ago (a whole layer lies between two attention launches)
        unsigned int seq;
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(seq) : "l"(p.ll_seq + m * p.Nkv + kvh) : "memory");
        s_tag = seq + 1u == 0u ? 1u : seq + 1u;
    }
    // fused: rows older than this pass are fetched ahead of the dependency wait, exactly as in the SIMT kernel
    // (fresh_rows, re-check of seq_len / slot after the wait); the stand-alone call waits first
    bool waited = !FUSED || p.fresh_rows < 0;
    if (waited) pdl_wait();

    int L, sl, n_active, begin, end, base0, fetched_end;
    const uint16_t *kb, *vb;
    // first step of this warp: rows base0 + g and base0 + g + 8, 16 bytes of every 32-dimension chunk per lane
    uint4 k0[4], k1[4], v0[4], v1[4];
    // fused: norm weight of the head this warp prepares (q heads: warps 0..R-1 and so on; k: the last warp) and the
    // rotary row of position seq_len - 1, also fetched ahead of the wait (they do not depend on the previous kernel
    // beyond seq_len, which is re-checked)
    float nw[4] = {1.f, 1.f, 1.f, 1.f}, nwk[4] = {1.f, 1.f, 1.f, 1.f}, cs[4] = {1.f, 1.f, 0.f, 0.f};
    // Eight-warp CTAs are chosen when every slice is a single step (seq_len <= S * 128), and decode batches usually keep
    // sequence i in slot i.  Under those two assumptions the rows of this warp are known before seq_len and slot have
    // been read, so they are requested first; the assumptions are checked when the two values arrive (a wrong guess
    // costs a second request, never a wrong result: rows past the end of the slice are zeroed after the wait, the
    // newest rows are fetched after the wait as always).
    bool speculated = false, spec_kept = false;
    int sl_guess = 0;
    if constexpr (FUSED && WARPS == 8) {
        if (!waited) {
            sl_guess = m < p.n_slots ? m : 0;
            const uint16_t* kg = p.kc + (size_t(sl_guess) * p.Nkv + kvh) * p.max_seq * kD;
            const uint16_t* vg = p.vc + (size_t(sl_guess) * p.Nkv + kvh) * p.max_seq * kD;
            const int ra = split * kBlk + warp * 16 + g, rb = ra + 8;
            const bool oa = ra < p.max_seq, ob = rb < p.max_seq;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                k0[i] = oa ? ld_stream_u4(kg + size_t(ra) * kD + 32 * i + 8 * t) : make_uint4(0, 0, 0, 0);
                k1[i] = ob ? ld_stream_u4(kg + size_t(rb) * kD + 32 * i + 8 * t) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                v0[i] = oa ? ld_stream_u4(vg + size_t(ra) * kD + 32 * i + 8 * t) : make_uint4(0, 0, 0, 0);
                v1[i] = ob ? ld_stream_u4(vg + size_t(rb) * kD + 32 * i + 8 * t) : make_uint4(0, 0, 0, 0);
            }
            speculated = true;
        }
    }
    while (true) {
        L = __ldcg(p.seq_len + m);
        sl = __ldcg(p.slot + m);
        const int L_seen = L, sl_seen = sl;
        L = L < 0 ? 0 : (L > p.max_seq ? p.max_seq : L);
        sl = sl < 0 ? 0 : (sl >= p.n_slots ? p.n_slots - 1 : sl);
        const int blocks = max((L + kBlk - 1) / kBlk, 1);
        const int per = (blocks + p.S - 1) / p.S;
        n_active = (blocks + per - 1) / per;
        begin = split * per * kBlk;
        end = min(L, begin + per * kBlk);
        const size_t head_off = (size_t(sl) * p.Nkv + kvh) * p.max_seq * kD;
        kb = p.kc + head_off;
        vb = p.vc + head_off;
        base0 = begin + warp * 16;
        const bool has_rows = split < n_active;
        const int safe_end = waited ? (FUSED ? min(end, L - 1) : end) : min(end, L - max(p.fresh_rows, 1));
        fetched_end = safe_end;
        const bool f0 = FUSED && has_rows && base0 + g < safe_end, f1 = FUSED && has_rows && base0 + g + 8 < safe_end;
        spec_kept = speculated && per == 1 && sl == sl_guess && sl_seen == sl;  // the registers already hold (or await) these rows
        speculated = false;
        if (!spec_kept) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                k0[i] = f0 ? ld_stream_u4(kb + size_t(base0 + g) * kD + 32 * i + 8 * t) : make_uint4(0, 0, 0, 0);
                k1[i] = f1 ? ld_stream_u4(kb + size_t(base0 + g + 8) * kD + 32 * i + 8 * t) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                v0[i] = f0 ? ld_stream_u4(vb + size_t(base0 + g) * kD + 32 * i + 8 * t) : make_uint4(0, 0, 0, 0);
                v1[i] = f1 ? ld_stream_u4(vb + size_t(base0 + g + 8) * kD + 32 * i + 8 * t) : make_uint4(0, 0, 0, 0);
            }
        }
        if (FUSED && has_rows) {
            // the position of a decode row is seq_len - 1 (the caller's contract for the fused call)
            int pp = L - 1;
            pp = pp < 0 ? 0 : pp;
            const float* cos_row = p.cos_t + size_t(pp) * 64;
            const float* sin_row = p.sin_t + size_t(pp) * 64;
            cs[0] = __ldg(cos_row + lane); cs[1] = __ldg(cos_row + lane + 32);
            cs[2] = __ldg(sin_row + lane); cs[3] = __ldg(sin_row + lane + 32);
#pragma unroll
            for (int j = 0; j < 4; j++) nw[j] = bf16_bits_to_float(__ldg(p.q_norm_w + lane + 32 * j));
            if (warp == WARPS - 1) {
#pragma unroll
                for (int j = 0; j < 4; j++) nwk[j] = bf16_bits_to_float(__ldg(p.k_norm_w + lane + 32 * j));
            }
        }
        if (waited) break;
        flash_trace(2);
        pdl_wait();
        flash_trace(3);
        waited = true;
        if (__ldcg(p.seq_len + m) != L_seen || __ldcg(p.slot + m) != sl_seen) continue;
        break;
    }
    if (FUSED) {
        // side job: zero the buffer the caller named (nothing uses it at this point of a layer)
        const int ctas = gridDim.x * gridDim.y * gridDim.z;
        const int cta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
        for (int i = cta * kThreads + threadIdx.x; i < p.clear_extra_vec4; i += ctas * kThreads)
            p.clear_extra[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (split >= n_active) return;

    const int heads = p.Nq + 2 * p.Nkv;
    const int newest = L - 1;  // the row appended by this pass (fused) / by the previous kernel
    const bool appends = FUSED && newest >= begin && newest < end;  // this CTA's slice holds the row this pass adds
    if (FUSED) {
        // q heads of this kv head: one warp per head; the norm weights and the rotary row are in registers already
        for (int h = warp; h < R; h += WARPS) {
            const float* src = p.qkv + (size_t(m) * heads + kvh * R + h) * kD;
            float r4[4];
            head_norm_rope_regs(__ldcg(src + lane), __ldcg(src + lane + 32), __ldcg(src + lane + 64), __ldcg(src + lane + 96),
                                nw, cs, p.eps, r4);
            s_q[h][lane] = r4[0]; s_q[h][lane + 32] = r4[1]; s_q[h][lane + 64] = r4[2]; s_q[h][lane + 96] = r4[3];
        }
        // the CTA whose slice holds the newest row appends it: K through norm + rotary, V as it is, both as bf16;
        // the row also stays in shared memory for the warp that attends to it
        if (appends) {
            const int pp = newest < 0 ? 0 : newest;
            const size_t row_off = ((size_t(sl) * p.Nkv + kvh) * p.max_seq + pp) * kD;
            if (warp == WARPS - 1) {
                const float* src = p.qkv + (size_t(m) * heads + p.Nq + kvh) * kD;
                float r4[4];
                head_norm_rope_regs(__ldcg(src + lane), __ldcg(src + lane + 32), __ldcg(src + lane + 64), __ldcg(src + lane + 96),
                                    nwk, cs, p.eps, r4);
                uint16_t* dst = p.kc_w + row_off;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint16_t b = float_to_bf16_bits(r4[j]);
                    dst[lane + 32 * j] = b;
                    s_new[0][lane + 32 * j] = b;
                }
            } else if (warp == WARPS - 2) {
                const float* src = p.qkv + (size_t(m) * heads + p.Nq + p.Nkv + kvh) * kD;
                uint16_t* dst = p.vc_w + row_off;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint16_t b = float_to_bf16_bits(__ldcg(src + lane + 32 * j));
                    dst[lane + 32 * j] = b;
                    s_new[FUSED ? 1 : 0][lane + 32 * j] = b;
                }
            }
        }
        __syncthreads();  // s_q and the appended row are complete
        flash_trace(4);
    }
    // rows of the first step that were not fetched ahead of the wait (the stand-alone call loads inside the loop)
    if (FUSED) {
        const int r0 = base0 + g, r1 = base0 + g + 8;
        if (spec_kept) {  // requested before the length was known: what lies past the slice's end counts as zeros
            if (r0 >= end) {
#pragma unroll
                for (int i = 0; i < 4; i++) { k0[i] = make_uint4(0, 0, 0, 0); v0[i] = make_uint4(0, 0, 0, 0); }
            }
            if (r1 >= end) {
#pragma unroll
                for (int i = 0; i < 4; i++) { k1[i] = make_uint4(0, 0, 0, 0); v1[i] = make_uint4(0, 0, 0, 0); }
            }
        }
        if (r0 >= fetched_end && r0 < end) {
            if (appends && r0 == newest) {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    k0[i] = *reinterpret_cast<const uint4*>(&s_new[0][32 * i + 8 * t]);
                    v0[i] = *reinterpret_cast<const uint4*>(&s_new[FUSED ? 1 : 0][32 * i + 8 * t]);
                }
            } else {
                const bool coherent = r0 >= newest;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    k0[i] = ld_row(kb + size_t(r0) * kD + 32 * i + 8 * t, coherent);
                    v0[i] = ld_row(vb + size_t(r0) * kD + 32 * i + 8 * t, coherent);
                }
            }
        }
        if (r1 >= fetched_end && r1 < end) {
            if (appends && r1 == newest) {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    k1[i] = *reinterpret_cast<const uint4*>(&s_new[0][32 * i + 8 * t]);
                    v1[i] = *reinterpret_cast<const uint4*>(&s_new[FUSED ? 1 : 0][32 * i + 8 * t]);
                }
            } else {
                const bool coherent = r1 >= newest;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    k1[i] = ld_row(kb + size_t(r1) * kD + 32 * i + 8 * t, coherent);
                    v1[i] = ld_row(vb + size_t(r1) * kD + 32 * i + 8 * t, coherent);
                }
            }
        }
    }

    // q as B fragments.  Contraction step (i, h2), i = 32-dimension chunk, h2 = half of the lane's 16 bytes:
    // index 2t, 2t+1 <-> dimensions 32 i + 8 t + 4 h2 + {0, 1}, index 2t+8, 2t+9 <-> ... + {2, 3}; column g = head g.
    uint32_t qh[4][2][2], ql[4][2][2];
    {
        const float* qp = FUSED ? &s_q[g < R ? g : 0][0] : p.q + (size_t(m) * p.Nq + kvh * R + (g < R ? g : 0)) * kD;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float4 a, b;
            if (FUSED) {
                a = *reinterpret_cast<const float4*>(qp + 32 * i + 8 * t);
                b = *reinterpret_cast<const float4*>(qp + 32 * i + 8 * t + 4);
            } else {
                a = __ldcg(reinterpret_cast<const float4*>(qp + 32 * i + 8 * t));
                b = __ldcg(reinterpret_cast<const float4*>(qp + 32 * i + 8 * t + 4));
            }
            const bool live = g < R;
            split_bf16x2(live ? a.x : 0.f, live ? a.y : 0.f, qh[i][0][0], ql[i][0][0]);
            split_bf16x2(live ? a.z : 0.f, live ? a.w : 0.f, qh[i][0][1], ql[i][0][1]);
            split_bf16x2(live ? b.x : 0.f, live ? b.y : 0.f, qh[i][1][0], ql[i][1][0]);
            split_bf16x2(live ? b.z : 0.f, live ? b.w : 0.f, qh[i][1][1], ql[i][1][1]);
        }
    }

    const float scale = 0.08838834764831845f;  // 1/sqrt(128)
    // this lane's two heads (2t, 2t+1): running maximum, sum over its own rows (rows g and g+8 of every step)
    float mx[2] = {-INFINITY, -INFINITY}, sum[2] = {0.f, 0.f};
    // O^T: block (i, jp) holds dimension rows g -> dim(i, 2jp, g) and g+8 -> dim(i, 2jp+1, g), where
    // dim(i, j, c) = 32 i + 8 (c >> 1) + 2 j + (c & 1); columns 2t, 2t+1 = heads
    float oacc[8][4];
#pragma unroll
    for (int b = 0; b < 8; b++) { oacc[b][0] = oacc[b][1] = oacc[b][2] = oacc[b][3] = 0.f; }

    // One step of a warp = rows base + g and base + g + 8 (16 cache rows, 8 KB of K and V).  The four-warp CTAs run many
    // steps and keep the next step's rows in flight in a second register set while they work on the current one (the
    // per-step chain load -> scores -> softmax -> PV is ~3.5 us long; without the overlap only occupancy hides it);
    // the eight-warp CTAs run a single step.
    auto load_step = [&](int base, uint4 (&K0)[4], uint4 (&K1)[4], uint4 (&V0)[4], uint4 (&V1)[4]) {
        const int r0 = base + g, r1 = base + g + 8;
        const bool ok0 = r0 < end, ok1 = r1 < end;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            K0[i] = ok0 ? ld_row(kb + size_t(r0) * kD + 32 * i + 8 * t, FUSED && r0 >= newest) : make_uint4(0, 0, 0, 0);
            K1[i] = ok1 ? ld_row(kb + size_t(r1) * kD + 32 * i + 8 * t, FUSED && r1 >= newest) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            V0[i] = ok0 ? ld_row(vb + size_t(r0) * kD + 32 * i + 8 * t, FUSED && r0 >= newest) : make_uint4(0, 0, 0, 0);
            V1[i] = ok1 ? ld_row(vb + size_t(r1) * kD + 32 * i + 8 * t, FUSED && r1 >= newest) : make_uint4(0, 0, 0, 0);
        }
    };
    auto compute_step = [&](int base, const uint4 (&K0)[4], const uint4 (&K1)[4], const uint4 (&V0)[4], const uint4 (&V1)[4]) {
        const int r0 = base + g, r1 = base + g + 8;
        const bool ok0 = r0 < end, ok1 = r1 < end;
        // scores S^T[rows g, g+8][heads 2t, 2t+1]
        float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            mma_bf16(s, K0[i].x, K1[i].x, K0[i].y, K1[i].y, qh[i][0][0], qh[i][0][1]);
            mma_bf16(s, K0[i].x, K1[i].x, K0[i].y, K1[i].y, ql[i][0][0], ql[i][0][1]);
            mma_bf16(s, K0[i].z, K1[i].z, K0[i].w, K1[i].w, qh[i][1][0], qh[i][1][1]);
            mma_bf16(s, K0[i].z, K1[i].z, K0[i].w, K1[i].w, ql[i][1][0], ql[i][1][1]);
        }
        s[0] = ok0 ? s[0] * scale : -INFINITY;
        s[1] = ok0 ? s[1] * scale : -INFINITY;
        s[2] = ok1 ? s[2] * scale : -INFINITY;
        s[3] = ok1 ? s[3] * scale : -INFINITY;
        // online softmax per head: maximum over the 16 rows of the step (the 8 lanes with this t)
        float pr[4];
        float corr[2];
#pragma unroll
        for (int e = 0; e < 2; e++) {
            float bm = fmaxf(s[e], s[2 + e]);
            bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 4));
            bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 8));
            bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 16));
            const float nm = fmaxf(mx[e], bm);  // base < end: the step has at least one valid row, so nm is finite
            corr[e] = (mx[e] == -INFINITY) ? 0.f : __expf(mx[e] - nm);
            mx[e] = nm;
            pr[e] = (s[e] == -INFINITY) ? 0.f : __expf(s[e] - nm);
            pr[2 + e] = (s[2 + e] == -INFINITY) ? 0.f : __expf(s[2 + e] - nm);
            sum[e] = sum[e] * corr[e] + pr[e] + pr[2 + e];
        }
#pragma unroll
        for (int b = 0; b < 8; b++) {
            oacc[b][0] *= corr[0]; oacc[b][1] *= corr[1]; oacc[b][2] *= corr[0]; oacc[b][3] *= corr[1];
        }
        // P^T as B fragments: (rows 2t, 2t+1 | rows 2t+8, 2t+9) of head g, by transposing the two 8x8 halves
        uint32_t ph0, pl0, ph1, pl1;
        split_bf16x2(pr[0], pr[1], ph0, pl0);
        split_bf16x2(pr[2], pr[3], ph1, pl1);
        const uint32_t bh0 = movmatrix_trans(ph0), bh1 = movmatrix_trans(ph1);
        const uint32_t bl0 = movmatrix_trans(pl0), bl1 = movmatrix_trans(pl1);
        // V^T as A fragments: the register that holds dimensions (8t + 2j, +1) of row g, transposed, holds rows
        // (2t, 2t+1) of dimension dim(i, j, g)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            {
                const uint32_t a0 = movmatrix_trans(V0[i].x), a1 = movmatrix_trans(V0[i].y);
                const uint32_t a2 = movmatrix_trans(V1[i].x), a3 = movmatrix_trans(V1[i].y);
                mma_bf16(oacc[2 * i], a0, a1, a2, a3, bh0, bh1);
                mma_bf16(oacc[2 * i], a0, a1, a2, a3, bl0, bl1);
            }
            {
                const uint32_t a0 = movmatrix_trans(V0[i].z), a1 = movmatrix_trans(V0[i].w);
                const uint32_t a2 = movmatrix_trans(V1[i].z), a3 = movmatrix_trans(V1[i].w);
                mma_bf16(oacc[2 * i + 1], a0, a1, a2, a3, bh0, bh1);
                mma_bf16(oacc[2 * i + 1], a0, a1, a2, a3, bl0, bl1);
            }
        }
    };
    constexpr bool kPipelined = WARPS == 4;
    if (!FUSED && base0 < end) load_step(base0, k0, k1, v0, v1);  // fused: the first step was fetched above
    if constexpr (kPipelined) {
        uint4 kn0[4], kn1[4], vn0[4], vn1[4];
        for (int base = base0; base < end; base += 2 * kBlk) {
            const bool more = base + kBlk < end;
            if (more) load_step(base + kBlk, kn0, kn1, vn0, vn1);
            compute_step(base, k0, k1, v0, v1);
            if (more) {
                if (base + 2 * kBlk < end) load_step(base + 2 * kBlk, k0, k1, v0, v1);
                compute_step(base + kBlk, kn0, kn1, vn0, vn1);
            }
        }
    } else {
        for (int base = base0; base < end; base += kBlk) {
            if (base != base0) load_step(base, k0, k1, v0, v1);
            compute_step(base, k0, k1, v0, v1);
        }
    }
    flash_trace(5);
    // sums over all rows of the warp: the 8 lanes with this t hold different rows
#pragma unroll
    for (int e = 0; e < 2; e++) {
        sum[e] += __shfl_xor_sync(0xffffffffu, sum[e], 4);
        sum[e] += __shfl_xor_sync(0xffffffffu, sum[e], 8);
        sum[e] += __shfl_xor_sync(0xffffffffu, sum[e], 16);
    }
    // a warp without rows keeps max = -inf and zeros
#pragma unroll
    for (int e = 0; e < 2; e++) {
        const int h = 2 * t + e;
        if (h < R) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
#pragma unroll
                for (int jp = 0; jp < 2; jp++) {
                    const int d_lo = 32 * i + 8 * (g >> 1) + 2 * (2 * jp) + (g & 1);
                    const int d_hi = 32 * i + 8 * (g >> 1) + 2 * (2 * jp + 1) + (g & 1);
                    s_o[warp][h][d_lo] = oacc[2 * i + jp][e];
                    s_o[warp][h][d_hi] = oacc[2 * i + jp][2 + e];
                }
            }
            if (g == 0) { s_ml[warp][h][0] = mx[e]; s_ml[warp][h][1] = sum[e]; }
        }
    }
    __syncthreads();

    // merge the warps: thread (hh, d) owns dimension d of heads hh, hh + HS, ... (HS = threads / 128)
    constexpr int HS = kThreads / kD;            // 1 or 2 head strides
    constexpr int HP = (R + HS - 1) / HS;        // heads per thread
    const int d = threadIdx.x & (kD - 1), hh = threadIdx.x >> 7;
    float fo[HP], fm[HP], fs[HP];
#pragma unroll
    for (int j = 0; j < HP; j++) {
        const int h = hh + j * HS;
        fo[j] = 0.f; fm[j] = -INFINITY; fs[j] = 0.f;
        if (h < R) {
            float nm = -INFINITY;
#pragma unroll
            for (int w = 0; w < WARPS; w++) nm = fmaxf(nm, s_ml[w][h][0]);
            float acc = 0.f, ssum = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; w++) {
                const float wm = s_ml[w][h][0];
                const float c = (wm == -INFINITY) ? 0.f : __expf(wm - nm);
                acc += s_o[w][h][d] * c;
                ssum += s_ml[w][h][1] * c;
            }
            fo[j] = acc; fm[j] = nm; fs[j] = ssum;
        }
    }

    // fused: once every CTA of this (row, kv head) is past its prologue, the raw q / k / v slices can be zeroed for
    // the next projection that accumulates into the buffer
    auto clear_raw = [&]() {
        if (FUSED && p.clear_qkv) {
            float* row = p.qkv + size_t(m) * heads * kD;
#pragma unroll
            for (int j = 0; j < HP; j++)
                if (hh + j * HS < R) row[(kvh * R + hh + j * HS) * kD + d] = 0.f;
            if (hh == 0) {
                row[(p.Nq + kvh) * kD + d] = 0.f;
                row[(p.Nq + p.Nkv + kvh) * kD + d] = 0.f;
            }
        }
    };
    if (n_active == 1) {
#pragma unroll
        for (int j = 0; j < HP; j++)
            if (hh + j * HS < R)
                p.out[(size_t(m) * p.Nq + kvh * R + hh + j * HS) * kD + d] = fs[j] > 0.f ? fo[j] / fs[j] : 0.f;
        clear_raw();
        return;
    }

    const size_t pbase = (size_t(m) * p.Nkv + kvh) * p.S;
    if constexpr (WARPS == 8) {
        // ---- eight-warp CTAs: no arrival counter.  Every partial value travels as one 8-byte word {value, launch
        // number}; the CTA of the last slice (the one that also appends the new row, so the slowest) polls the words of
        // the other slices: a word that carries this launch's number is complete, because an aligned 8-byte store is
        // one transaction - no fence, no atomic, no second trip for the data.  Slice order and a common maximum per
        // head keep the summation order fixed.  The wait is bounded by the wall clock.
        const unsigned int tag = s_tag;  // written before the barrier after the prologue
        uint2* llo = p.ll_o + pbase * R * kD + d;
        uint2* llm = p.ll_ml + pbase * R * 2;
        if (split != n_active - 1) {
            if (split == p.ll_drop) return;
#pragma unroll
            for (int j = 0; j < HP; j++) {
                const int h = hh + j * HS;
                if (h < R) {
                    st_tagged(llo + (size_t(split) * R + h) * kD, fo[j], tag);
                    if (d == 0) {
                        st_tagged(llm + (size_t(split) * R + h) * 2, fm[j], tag);
                        st_tagged(llm + (size_t(split) * R + h) * 2 + 1, fs[j], tag);
                    }
                }
            }
            flash_trace(6);
            return;
        }
        constexpr int kSlices = 20;  // upper bound of n_active here: one CTA per SM and at least 8 slices per kv head
        float acc[HP], den[HP];
        const long long t0 = (long long)globaltimer_ns();
        bool complete = false, gave_up = false;
        uint2 wo[kSlices][HP];
        uint2 wm[HP], wl[HP];  // lane l: (max, sum) of slice l for this thread's heads
        while (true) {
            bool ok = true;
#pragma unroll
            for (int q = 0; q < kSlices; q++)
#pragma unroll
                for (int j = 0; j < HP; j++) {
                    const int h = hh + j * HS;
                    const bool remote = q < n_active - 1 && h < R;
                    wo[q][j] = remote ? ld_tagged(llo + (size_t(q) * R + h) * kD) : make_uint2(0u, tag);
                }
#pragma unroll
            for (int j = 0; j < HP; j++) {
                const int h = hh + j * HS;
                const bool remote = lane < n_active - 1 && h < R;
                wm[j] = remote ? ld_tagged(llm + (size_t(lane) * R + h) * 2) : make_uint2(0u, tag);
                wl[j] = remote ? ld_tagged(llm + (size_t(lane) * R + h) * 2 + 1) : make_uint2(0u, tag);
                ok = ok && wm[j].y == tag && wl[j].y == tag;
            }
#pragma unroll
            for (int q = 0; q < kSlices; q++)
#pragma unroll
                for (int j = 0; j < HP; j++) ok = ok && wo[q][j].y == tag;
            complete = __syncthreads_and(ok ? 1 : 0) != 0;
            if (complete) break;
            if ((long long)globaltimer_ns() - t0 > p.ll_timeout_ns) gave_up = true;
            if (__syncthreads_or(gave_up ? 1 : 0)) {
                if (threadIdx.x == 0) atomicExch(&g_flash_wait_error, 1);
                break;
            }
        }
        flash_trace(7);
#pragma unroll
        for (int j = 0; j < HP; j++) {
            const int h = hh + j * HS;
            // lane l holds slice l (l < n_active - 1) or this CTA's own slice (l == n_active - 1)
            float ml_m = -INFINITY, ml_l = 0.f;
            if (lane < n_active - 1) { ml_m = __uint_as_float(wm[j].x); ml_l = __uint_as_float(wl[j].x); }
            if (lane == n_active - 1) { ml_m = fm[j]; ml_l = fs[j]; }
            if (!complete || h >= R) { ml_m = -INFINITY; ml_l = 0.f; }
            const float gm = warp_max(ml_m);
            const float w = (ml_m == -INFINITY) ? 0.f : __expf(ml_m - gm);
            den[j] = warp_sum(ml_l * w);
            float a = 0.f;
#pragma unroll
            for (int q = 0; q < kSlices; q++) {
                const float wq = __shfl_sync(0xffffffffu, w, q);
                const float v = q < n_active - 1 ? __uint_as_float(wo[q][j].x) : (q == n_active - 1 ? fo[j] : 0.f);
                a = fmaf(v, wq, a);
            }
            acc[j] = a;
        }
        flash_trace(8);
#pragma unroll
        for (int j = 0; j < HP; j++) {
            const int h = hh + j * HS;
            if (h < R) p.out[(size_t(m) * p.Nq + kvh * R + h) * kD + d] = den[j] > 0.f ? acc[j] / den[j] : 0.f;
        }
        if (threadIdx.x == 0) p.ll_seq[m * p.Nkv + kvh] = tag;
        clear_raw();
        flash_trace(9);
        return;
    }
#pragma unroll
    for (int j = 0; j < HP; j++) {
        const int h = hh + j * HS;
        if (h < R) {
            p.part_o[((pbase + split) * R + h) * kD + d] = fo[j];
            if (d == 0) *reinterpret_cast<float2*>(p.part_ml + ((pbase + split) * R + h) * 2) = make_float2(fm[j], fs[j]);
        }
    }
    // Arrival: the barrier orders every thread's partial stores before thread 0's release, and thread 0's acquire
    // before every thread's loads after the second barrier (release / acquire are cumulative over a CTA barrier), so
    // one acq_rel atomic by one thread stands in for a fence by every thread on either side of it.
    __syncthreads();
    flash_trace(6);
    if (threadIdx.x == 0) {
        int prev;
        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(prev) : "l"(p.counters + m * p.Nkv + kvh) : "memory");
        s_last = (prev == n_active - 1);
        if (s_last) p.counters[m * p.Nkv + kvh] = 0;
    }
    __syncthreads();
    flash_trace(7);
    if (!s_last) return;
    float acc[HP], den[HP];
#pragma unroll
    for (int j = 0; j < HP; j++) { acc[j] = 0.f; den[j] = 0.f; }
    const float* po = p.part_o + pbase * R * kD + d;
    const float* pml = p.part_ml + pbase * R * 2;
    {
        // ---- final combine by the last CTA (four warps, one thread per dimension, every head).  Weights first: warp w
        // takes heads w, w + 4, ...; lane l holds the (max, sum) of slices l and l + 32, so the maximum and the
        // denominator are two warp reductions; then the partial outputs in slice order, eight slices of every head in
        // flight per thread.
        __shared__ float s_w[kMaxSplitsMma * R];   // weight of slice sp for head h at [sp * R + h]
        __shared__ float s_den[R];
        constexpr int kPerLane = kMaxSplitsMma / 32;
        for (int h = warp; h < R; h += WARPS) {
            float2 ml[kPerLane];
            float nm = -INFINITY;
#pragma unroll
            for (int i = 0; i < kPerLane; i++) {
                ml[i] = make_float2(-INFINITY, 0.f);
                if (lane + 32 * i < n_active) ml[i] = __ldcg(reinterpret_cast<const float2*>(pml + (size_t(lane + 32 * i) * R + h) * 2));
                nm = fmaxf(nm, ml[i].x);
            }
            nm = warp_max(nm);
            float part = 0.f;
#pragma unroll
            for (int i = 0; i < kPerLane; i++) {
                const float w = (ml[i].x == -INFINITY) ? 0.f : __expf(ml[i].x - nm);
                part = fmaf(ml[i].y, w, part);
                s_w[(lane + 32 * i) * R + h] = w;
            }
            const float dsum = warp_sum(part);
            if (lane == 0) s_den[h] = dsum;
        }
        __syncthreads();
        int sp = 0;
        for (; sp + 8 <= n_active; sp += 8) {
            float a[8][HP];
#pragma unroll
            for (int q = 0; q < 8; q++)
#pragma unroll
                for (int j = 0; j < HP; j++) a[q][j] = __ldcg(po + (size_t(sp + q) * R + j) * kD);
#pragma unroll
            for (int q = 0; q < 8; q++)
#pragma unroll
                for (int j = 0; j < HP; j++) acc[j] = fmaf(a[q][j], s_w[(sp + q) * R + j], acc[j]);
        }
        for (; sp < n_active; sp++) {
#pragma unroll
            for (int j = 0; j < HP; j++) acc[j] = fmaf(__ldcg(po + (size_t(sp) * R + j) * kD), s_w[sp * R + j], acc[j]);
        }
#pragma unroll
        for (int j = 0; j < HP; j++) den[j] = s_den[j];
    }
    flash_trace(8);
#pragma unroll
    for (int j = 0; j < HP; j++) {
        const int h = hh + j * HS;
        if (h < R) p.out[(size_t(m) * p.Nq + kvh * R + h) * kD + d] = den[j] > 0.f ? acc[j] / den[j] : 0.f;
    }
    clear_raw();
    flash_trace(9);
}


// Upper bound of the slices per (row, kv head): 64; 128 for a few rows on the four-warp tensor-core kernel, where a
// long context of one sequence would otherwise leave the SMs short of resident warps (the kernel hides memory latency
// by occupancy: batch 1 at 32 768 rows streams 3.0 TB/s with 64 slices).
int max_splits(int M, int rows_per_step, bool tensor_cores) {
    return (tensor_cores && rows_per_step == 64 && M <= kFewRows) ? kMaxSplitsMma : kMaxSplits;
}

// rows per CTA step: 64 (four warps) or 128 (eight warps)
int pick_splits(int M, int Nkv, int max_seq, int rows_per_step, int ctas_per_sm, bool tensor_cores) {
    const int cap = max_splits(M, rows_per_step, tensor_cores);
    if (g_force_splits > 0) return g_force_splits < cap ? g_force_splits : cap;
    const int by_len = (max_seq + rows_per_step - 1) / rows_per_step;  // a slice is at least one step of the CTA
    int want = (device_sm_count() * 4 + M * Nkv - 1) / (M * Nkv);
    // the tensor-core CTAs are long-lived and few per SM: one wave of them, never a partial second one
    // (batch 16 at 32 768 rows: 6.8 TB/s with 256 CTAs on 296 places, 5.7 TB/s with 640)
    if (tensor_cores) want = device_sm_count() * ctas_per_sm / (M * Nkv);
    int s = want < by_len ? want : by_len;
    if (s < 1) s = 1;
    if (s > cap) s = cap;
    return s;
}

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

// Tagged-word area of the eight-warp CTAs at the end of the workspace: at most one CTA per SM, so at most SMs slices of
// up to 8 heads each are in flight; launch numbers: one per (row, kv head) <= SMs.
constexpr int kWideMaxSlices = 20;  // slices per (row, kv head) the combining CTA of the eight-warp kernel can poll
size_t ll_o_bytes() { return align256(size_t(device_sm_count()) * 8 * kD * sizeof(uint2)); }
size_t ll_ml_bytes() { return align256(size_t(device_sm_count()) * 8 * 2 * sizeof(uint2)); }
size_t ll_seq_bytes() { return align256(size_t(device_sm_count()) * sizeof(unsigned int)); }
size_t ll_area_bytes() { return ll_o_bytes() + ll_ml_bytes() + ll_seq_bytes(); }

// Upper bound of rows x slices of any call with at most M rows: the slice count of a call is sized to the GPU (at most
// four or five CTAs per SM over all rows and kv heads), and a call of one or two rows may use kMaxSplitsMma slices; a
// forced slice count (tuning, tests) is checked against the workspace at launch.
size_t flash_slots(int M) {
    const size_t by_gpu = size_t(M) + 8 * size_t(device_sm_count());
    const size_t by_cap = size_t(M) * kMaxSplits;
    const size_t few = size_t(M < kFewRows ? M : kFewRows) * kMaxSplitsMma;
    const size_t slots = by_gpu < by_cap ? by_gpu : by_cap;
    return slots > few ? slots : few;
}

}  // namespace

void flash_decode_set_tuning(const char* key, int value) {
    if (!strcmp(key, "flash_splits")) g_force_splits = value;
    if (!strcmp(key, "flash_drop_slice")) g_flash_drop_slice = value;
    if (!strcmp(key, "flash_timeout_ms")) g_flash_timeout_ns = (long long)(value < 1 ? 1 : value) * 1000000ll;
    if (!strcmp(key, "flash_early")) g_flash_early = value;
    if (!strcmp(key, "flash_mma")) g_flash_mma = value;
    if (!strcmp(key, "flash_mma_fused")) g_flash_mma_fused = value;
    if (!strcmp(key, "flash_wide")) g_flash_wide = value;
}

}  // namespace kuiper

using namespace kuiper;

#ifdef KUIPER_TRACE
extern "C" KUIPER_API int kuiper_flash_trace_read(int64_t* out, int max_values) {
    KUIPER_REQUIRE(out != nullptr && max_values > 0, "flash_trace_read: empty destination");
    const int n = max_values < kFlashTraceCtas * kFlashTraceSlots ? max_values : kFlashTraceCtas * kFlashTraceSlots;
    if (cudaMemcpyFromSymbol(out, g_flash_trace, size_t(n) * sizeof(long long)) != cudaSuccess) {
        set_error("flash_trace_read: cannot read the trace buffer");
        return -1;
    }
    return n;
}
#endif

extern "C" int kuiper_flash_decode_status(void) {
    int v = 0;
    const int zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_flash_wait_error, sizeof(int)) != cudaSuccess) v = -1;
    if (v == 0) return KUIPER_OK;
    cudaMemcpyToSymbol(g_flash_wait_error, &zero, sizeof(int));  // reported once
    set_error("flash_decode: the combining CTA's bounded wait for the other slices ran out (code %d)", v);
    return KUIPER_INTERNAL_ERROR;
}

extern "C" size_t kuiper_flash_decode_workspace_bytes(int M, int Nq, int D, int max_seq) {
    if (M <= 0 || Nq <= 0 || D <= 0 || max_seq <= 0) return 0;
    // Layout: [tagged-word area of the eight-warp CTAs (fixed size and position, whatever M a call has)]
    // [arrival counters] [partial outputs] [partial (max, sum)].  Slices in flight: a call never runs more than
    // max_slots(M) (row, kv head, slice) triples per kv head count - see flash_slots().
    return ll_area_bytes() + align256(size_t(M) * Nq * sizeof(int)) + align256(flash_slots(M) * Nq * D * sizeof(float)) +
           align256(flash_slots(M) * Nq * 2 * sizeof(float));
}

// argument checks, workspace carving and launch shared by the two entry points; `p` arrives with the tensors set
static int flash_launch(FlashParams& p, bool fused, int M, int Nq, int Nkv, int D, int max_seq, int n_slots, int fresh_rows,
                        void* workspace, size_t workspace_bytes, kuiper_stream_t stream) {
    KUIPER_REQUIRE(D == kD, "flash_decode: head_dim %d is not supported (128 only)", D);
    KUIPER_REQUIRE(M > 0 && Nq > 0 && Nkv > 0 && max_seq > 0 && n_slots > 0, "flash_decode: empty shape");
    KUIPER_REQUIRE(Nq % Nkv == 0, "flash_decode: Nq=%d is not a multiple of Nkv=%d", Nq, Nkv);
    KUIPER_REQUIRE(M <= 65535 && Nkv <= 65535, "flash_decode: grid too large");
    const int R = Nq / Nkv;
    KUIPER_REQUIRE(R == 1 || R == 2 || R == 4 || R == 8, "flash_decode: group size %d is not supported", R);
    p.M = M; p.Nq = Nq; p.Nkv = Nkv; p.max_seq = max_seq; p.n_slots = n_slots;
    p.fresh_rows = g_flash_early ? fresh_rows : -1;
    // one sequence (or a few) at a context of a few thousand rows: eight-warp CTAs, one per SM, one or two 128-row steps
    // each, so that the last CTA of a kv head combines half as many slices; anything larger keeps the four-warp CTAs
    long long wide_slices = device_sm_count() / ((long long)M * Nkv);  // one CTA per SM, a single wave
    if (wide_slices > kWideMaxSlices) wide_slices = kWideMaxSlices;
    const bool wide = fused && g_flash_mma_fused && g_flash_wide && wide_slices >= 8 &&
                      (max_seq + 127) / 128 <= 2 * wide_slices;
    p.S = pick_splits(M, Nkv, max_seq, wide ? 128 : 64, !fused ? kCtasStandalone : wide ? 1 : kCtasFusedNarrow,
                      fused ? g_flash_mma_fused != 0 : g_flash_mma != 0);
    if (wide && p.S > kWideMaxSlices) p.S = kWideMaxSlices;
    if (p.S > 1) {
        KUIPER_REQUIRE(workspace != nullptr, "flash_decode: split KV needs a workspace");
        const size_t need = ll_area_bytes() + align256(size_t(M) * Nq * sizeof(int)) +
                            align256(size_t(M) * Nq * p.S * D * sizeof(float)) + align256(size_t(M) * Nq * p.S * 2 * sizeof(float));
        KUIPER_REQUIRE(workspace_bytes >= need, "flash_decode: workspace of %zu bytes is too small (%zu needed for %d slices)",
                       workspace_bytes, need, p.S);
        // the tagged-word area comes first: a fixed place that the layouts of other row counts never touch
        char* ll = reinterpret_cast<char*>(workspace);
        char* w = ll + ll_area_bytes();
        p.counters = reinterpret_cast<int*>(w);
        w += align256(size_t(M) * Nq * sizeof(int));
        p.part_o = reinterpret_cast<float*>(w);
        w += align256(size_t(M) * Nq * p.S * D * sizeof(float));
        p.part_ml = reinterpret_cast<float*>(w);
        p.ll_o = reinterpret_cast<uint2*>(ll);
        p.ll_ml = reinterpret_cast<uint2*>(ll + ll_o_bytes());
        p.ll_seq = reinterpret_cast<unsigned int*>(ll + ll_o_bytes() + ll_ml_bytes());
        p.ll_timeout_ns = g_flash_timeout_ns;
        p.ll_drop = g_flash_drop_slice;
    } else {
        p.counters = nullptr; p.part_o = nullptr; p.part_ml = nullptr;
        p.ll_o = nullptr; p.ll_ml = nullptr; p.ll_seq = nullptr; p.ll_timeout_ns = 0; p.ll_drop = -1;
    }

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.S, Nkv, M);
    cfg.blockDim = dim3((wide ? 8 : kWarps) * 32, 1, 1);
    cfg.stream = as_stream(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl_enabled ? 1 : 0;
    cudaError_t err;
    if (wide) {
        switch (R) {
            case 1: err = cudaLaunchKernelEx(&cfg, flash_decode_mma_kernel<1, true, 8>, p); break;
            case 2: err = cudaLaunchKernelEx(&cfg, flash_decode_mma_kernel<2, true, 8>, p); break;
            case 4: err = cudaLaunchKernelEx(&cfg, flash_decode_mma_kernel<4, true, 8>, p); break;
            default: err = cudaLaunchKernelEx(&cfg, flash_decode_mma_kernel<8, true, 8>, p); break;
        }
    } else if (fused && g_flash_mma_fused) {
        switch (R) {
            case 1: err = cudaLaunchKernelEx(&cfg, flash_decode_mma_kernel<1, true, 4>, p); break;
            case 2: err = cudaLaunchKernelEx(&cfg, flash_decode_mma_kernel<2, true, 4>, p); break;
            case 4: err = cudaLaunchKernelEx(&cfg, flash_decode_mma_kernel<4, true, 4>, p); break;
            default: err = cudaLaunchKernelEx(&cfg, flash_decode_mma_kernel<8, true, 4>, p); break;
        }
    } else if (fused) {
        switch (R) {
            case 1: err = cudaLaunchKernelEx(&cfg, flash_decode_kernel<1, true>, p); break;
            case 2: err = cudaLaunchKernelEx(&cfg, flash_decode_kernel<2, true>, p); break;
            case 4: err = cudaLaunchKernelEx(&cfg, flash_decode_kernel<4, true>, p); break;
            default: err = cudaLaunchKernelEx(&cfg, flash_decode_kernel<8, true>, p); break;
        }
    } else if (g_flash_mma) {
        switch (R) {
            case 1: err = cudaLaunchKernelEx(&cfg, flash_decode_mma_kernel<1, false, 4>, p); break;
            case 2: err = cudaLaunchKernelEx(&cfg, flash_decode_mma_kernel<2, false, 4>, p); break;
            case 4: err = cudaLaunchKernelEx(&cfg, flash_decode_mma_kernel<4, false, 4>, p); break;
            default: err = cudaLaunchKernelEx(&cfg, flash_decode_mma_kernel<8, false, 4>, p); break;
        }
    } else {
        switch (R) {
            case 1: err = cudaLaunchKernelEx(&cfg, flash_decode_kernel<1, false>, p); break;
            case 2: err = cudaLaunchKernelEx(&cfg, flash_decode_kernel<2, false>, p); break;
            case 4: err = cudaLaunchKernelEx(&cfg, flash_decode_kernel<4, false>, p); break;
            default: err = cudaLaunchKernelEx(&cfg, flash_decode_kernel<8, false>, p); break;
        }
    }
    if (err != cudaSuccess) {
        set_error("flash_decode launch failed: %s", cudaGetErrorString(err));
        return KUIPER_INTERNAL_ERROR;
    }
    return KUIPER_OK;
}

extern "C" int kuiper_flash_decode(const float* q, const uint16_t* kcache, const uint16_t* vcache,
                                   const int32_t* seq_len, const int32_t* slot, float* out,
                                   int M, int Nq, int Nkv, int D, int max_seq, int n_slots, int fresh_rows,
                                   void* workspace, size_t workspace_bytes, kuiper_stream_t stream) {
    KUIPER_REQUIRE(q && kcache && vcache && seq_len && slot && out, "flash_decode: null tensor pointer");
    KUIPER_REQUIRE((reinterpret_cast<uintptr_t>(kcache) & 15) == 0 && (reinterpret_cast<uintptr_t>(vcache) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(q) & 15) == 0,
                   "flash_decode: q and caches must be 16-byte aligned");
    FlashParams p = {};
    p.q = q; p.kc = kcache; p.vc = vcache; p.seq_len = seq_len; p.slot = slot; p.out = out;
    return flash_launch(p, false, M, Nq, Nkv, D, max_seq, n_slots, fresh_rows, workspace, workspace_bytes, stream);
}

extern "C" int kuiper_rope_flash_decode(float* qkv, const uint16_t* q_norm_w, const uint16_t* k_norm_w, const float* cos_t,
                                        const float* sin_t, const int32_t* pos, const int32_t* seq_len, const int32_t* slot,
                                        float* out, uint16_t* kcache, uint16_t* vcache, int M, int Nq, int Nkv, int D,
                                        float eps, int max_seq, int n_slots, int fresh_rows, int clear_input,
                                        float* clear_extra, int64_t clear_extra_count, void* workspace,
                                        size_t workspace_bytes, kuiper_stream_t stream) {
    KUIPER_REQUIRE(qkv && q_norm_w && k_norm_w && cos_t && sin_t && pos && seq_len && slot && out && kcache && vcache,
                   "rope_flash_decode: null tensor pointer");
    KUIPER_REQUIRE((reinterpret_cast<uintptr_t>(kcache) & 15) == 0 && (reinterpret_cast<uintptr_t>(vcache) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(qkv) & 15) == 0,
                   "rope_flash_decode: qkv and caches must be 16-byte aligned");
    KUIPER_REQUIRE(clear_extra_count >= 0 && (clear_extra_count == 0 || clear_extra), "rope_flash_decode: bad extra buffer");
    KUIPER_REQUIRE(clear_extra_count % 4 == 0 && (reinterpret_cast<uintptr_t>(clear_extra) & 15) == 0 &&
                       clear_extra_count / 4 <= 0x7fffffff,
                   "rope_flash_decode: the extra buffer must be 16-byte aligned with a multiple of 4 floats");
    FlashParams p = {};
    p.q = nullptr; p.kc = kcache; p.vc = vcache; p.seq_len = seq_len; p.slot = slot; p.out = out;
    p.qkv = qkv; p.q_norm_w = q_norm_w; p.k_norm_w = k_norm_w; p.cos_t = cos_t; p.sin_t = sin_t; p.pos = pos;
    p.kc_w = kcache; p.vc_w = vcache;
    p.clear_extra = reinterpret_cast<float4*>(clear_extra);
    p.clear_extra_vec4 = int(clear_extra_count / 4);
    p.clear_qkv = clear_input;
    p.eps = eps;
    return flash_launch(p, true, M, Nq, Nkv, D, max_seq, n_slots, fresh_rows, workspace, workspace_bytes, stream);
}
