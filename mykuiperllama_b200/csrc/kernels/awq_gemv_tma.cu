// Persistent, TMA-fed INT4-AWQ GEMV for sm_100a (decode, one or two token rows).
//
// The weight [K, N/8] int32 is cut into units of 32 rows x 1024 columns (16 KB).  Units
// are numbered column-tile major / K minor and dealt out in contiguous runs to a grid of
// one CTA per SM, so every SM streams the same number of bytes (+-1 unit) whatever the
// matrix shape.  Inside a CTA one producer thread keeps a ring of 16 KB shared-memory
// stages full with cp.async.bulk.tensor (2-D tensor map over the native AWQ layout,
// box 32 rows x 128 words, out-of-range columns zero filled), completion tracked by
// mbarriers; 16 consumer warps drain it.  The producer starts before the programmatic
// dependent-launch wait, so the weight stream of this GEMV overlaps the previous kernel.
//
// Consumer thread (cg, rg): columns 16*cg .. 16*cg+15 of the tile (two packed words, one
// 8-byte shared-memory read per row), rows 8*rg .. 8*rg+7 of each unit.  The
// activations of those rows are read from global memory (L2) one unit ahead and rounded to
// fp16; products (q - z) * x are exact and
// are accumulated in fp32 (fma.rn.f32.f16); the fp16 group scale is applied when a
// 128-row group ends.  When a CTA's run leaves a column tile the 8 row groups are reduced
// through shared memory and the CTA's partial row goes to the workspace slot
// (cta + tile); the last CTA to arrive at a tile adds the slots in order (deterministic
// result), adds the residual and writes y.
//
// Every wait on an mbarrier is bounded: after kSpinLimit failed polls the thread records
// an error code in the workspace and leaves the loop.
#include <cuda.h>

#include <cstring>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace kuiper {
namespace {

constexpr int kConsumerWarps = 8;
constexpr int kConsumers = kConsumerWarps * 32;   // 256
constexpr int kRowGroups = kConsumers / 64;       // 4 row groups of 8 rows per unit
constexpr int kCtasPerSm = 2;                     // half an SM per CTA, so that the next kernel can move in early
constexpr int kThreadsTma = kConsumers + 32;      // + producer warp
constexpr int kUnitRows = 32;
constexpr int kTileWords = 128;                   // 1024 columns
constexpr int kTileColsTma = kTileWords * 8;
constexpr int kStageBytes = kUnitRows * kTileWords * 4;  // 16 KB
constexpr uint32_t kMagicTma = 0x64006400u;
constexpr uint32_t kSpinLimit = 1u << 22;

// set when a bounded mbarrier wait ran out (1 producer, 2 consumer); read by kuiper_awq_gemv_status()
__device__ int g_gemv_wait_error = 0;

struct TmaGemvParams {
    const float* x;        // [MT, K]
    float* y;              // [MT, N]
    const float* residual; // [MT, N] or null
    const uint2* qz;       // zeros, 8-byte pairs: [K/128][N/16]
    const __half* scales;  // [K/128][N]
    float* partial;        // [slots][MT][1024]
    int* counters;         // [tiles]
    const uint16_t* norm_w; // bf16 [K]: fused RMSNorm weight of the input (NORM kernels), else null
    float eps;
    int K, N, tiles, upt;  // upt = units per tile = K / 32
    long long U;           // total units
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// bounded wait: false after kSpinLimit unsuccessful polls
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < kSpinLimit; spin++) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory"); }

__device__ __forceinline__ float fma_f16_tma(uint16_t a, uint16_t b, float c) {
    float d;
    asm("fma.rn.f32.f16 %0, %1, %2, %3;" : "=f"(d) : "h"(a), "h"(b), "f"(c));
    return d;
}
__device__ __forceinline__ __half2 u2h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ uint32_t h22u(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }

// (1024 + z) pairs for the low nibbles, -(64 + z) pairs for the high nibbles of one zero word
struct ZeroPairs {
    __half2 lo0, hi0, lo1, hi1;
};
__device__ __forceinline__ ZeroPairs make_zero_pairs(uint32_t zw) {
    ZeroPairs z;
    const __half2 neg_sixteenth = __floats2half2_rn(-0.0625f, -0.0625f);
    z.lo0 = u2h2((zw & 0x000f000fu) | kMagicTma);
    z.hi0 = __hmul2(u2h2((zw & 0x00f000f0u) | kMagicTma), neg_sixteenth);
    const uint32_t z8 = zw >> 8;
    z.lo1 = u2h2((z8 & 0x000f000fu) | kMagicTma);
    z.hi1 = __hmul2(u2h2((z8 & 0x00f000f0u) | kMagicTma), neg_sixteenth);
    return z;
}

// acc[m][base..base+7] += x[m] * (q - z) for the 8 columns of one packed word.  The two halves of a
// dequantised pair are split inside the asm block so that no separate extraction is emitted.
template <int MT>
__device__ __forceinline__ void word_fma(uint32_t w, const ZeroPairs& z, const uint16_t (&xh)[MT], float (*acc)[16], int base) {
    const __half2 sixteenth = __floats2half2_rn(0.0625f, 0.0625f);
    const uint32_t w8 = w >> 8;
    const uint32_t d[4] = {
        h22u(__hsub2(u2h2((w & 0x000f000fu) | kMagicTma), z.lo0)),
        h22u(__hfma2(u2h2((w & 0x00f000f0u) | kMagicTma), sixteenth, z.hi0)),
        h22u(__hsub2(u2h2((w8 & 0x000f000fu) | kMagicTma), z.lo1)),
        h22u(__hfma2(u2h2((w8 & 0x00f000f0u) | kMagicTma), sixteenth, z.hi1)),
    };
#pragma unroll
    for (int i = 0; i < 4; i++) {
#pragma unroll
        for (int m = 0; m < MT; m++) {
            asm("{\n\t.reg .b16 lo, hi;\n\t"
                "mov.b32 {lo, hi}, %2;\n\t"
                "fma.rn.f32.f16 %0, lo, %3, %0;\n\t"
                "fma.rn.f32.f16 %1, hi, %3, %1;\n\t}"
                : "+f"(acc[m][base + 2 * i]), "+f"(acc[m][base + 2 * i + 1])
                : "r"(d[i]), "h"(xh[m]));
        }
    }
}

// NORM: the input row is the residual stream h and the matmul operand is RMSNorm(h) = (h * rstd) * norm_w,
// formed on the fly (every CTA computes rstd from the whole row itself, which is cheaper than a kernel).
// ACCUM: y += x.W with vector float reductions (no cross-CTA ordering, no tail); the caller guarantees
// that y holds the addend (residual stream or zeros).  Otherwise y = x.W (+ residual) with the
// deterministic slot / arrival-counter combine.
template <int MT, int STAGES, bool ACCUM, bool NORM = false>
__global__ void __launch_bounds__(kThreadsTma, (MT == 1 ? kCtasPerSm : 1))
awq_gemv_tma_kernel(const __grid_constant__ CUtensorMap tmap, const TmaGemvParams p) {
    extern __shared__ unsigned char smem_raw[];
    // TMA destinations want 128-byte alignment; the launch reserves 128 spare bytes for this
    unsigned char* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    unsigned char* stages = smem;                                             // STAGES x 16 KB
    float4* red = reinterpret_cast<float4*>(smem + STAGES * kStageBytes);      // [kRowGroups][MT][256] float4
    __shared__ uint64_t full_bar[STAGES];
    __shared__ uint64_t empty_bar[STAGES];
    __shared__ int s_last;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int C = gridDim.x;
    const int u0 = int((long long)blockIdx.x * p.U / C);
    const int u1 = int((long long)(blockIdx.x + 1) * p.U / C);

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], kConsumerWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            int t = u0 / p.upt, kb = u0 - t * p.upt;
            int s = 0;
            uint32_t parity = 0;
            bool ok = true;
            for (int u = u0; u < u1; u++) {
                if (!mbar_wait(&empty_bar[s], parity ^ 1u)) {
                    atomicExch(&g_gemv_wait_error, 1);
                    ok = false;
                    break;
                }
                mbar_expect_tx(&full_bar[s], kStageBytes);
                tma_load_2d(stages + s * kStageBytes, &tmap, t * kTileWords, kb * kUnitRows, &full_bar[s]);
                if (++kb == p.upt) { kb = 0; t++; }
                if (++s == STAGES) { s = 0; parity ^= 1u; }
            }
            if (!ok) {
                // give copies already issued a bounded chance to land before the CTA goes away
                for (int q = 0; q < STAGES; q++) mbar_wait(&full_bar[q], 0);
            }
        }
        return;
    }

    // ---------------------------------------------------------------- consumers
    const int cg = tid & 63;   // 16-column group inside the tile
    const int rg = tid >> 6;   // row group: rows 8*rg .. 8*rg+7 of every unit
    pdl_wait();                // x, y and the workspace belong to the previous kernel until here

    const int groups = p.K >> 7;
    const int zstride = p.N >> 4;  // uint2 per zero row
    const unsigned char* my_stage = stages + rg * 8 * 512 + cg * 8;
    const float* my_x = p.x + rg * 8;

    float rstd[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) rstd[m] = 1.f;
    if (NORM) {
        // sum of squares of the whole input row, by all consumer threads, 4 x 16-byte loads in flight each
        float* s_part = reinterpret_cast<float*>(red);  // [MT][kConsumerWarps], free until the first tile ends
#pragma unroll
        for (int m = 0; m < MT; m++) {
            const float4* hp = reinterpret_cast<const float4*>(p.x + size_t(m) * p.K);
            const int n4 = p.K >> 2;
            float ss = 0.f;
            for (int i = tid; i < n4; i += 4 * kConsumers) {
                float4 v[4];
#pragma unroll
                for (int q = 0; q < 4; q++)
                    v[q] = (i + q * kConsumers < n4) ? __ldcg(hp + i + q * kConsumers) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    ss = fmaf(v[q].x, v[q].x, ss); ss = fmaf(v[q].y, v[q].y, ss);
                    ss = fmaf(v[q].z, v[q].z, ss); ss = fmaf(v[q].w, v[q].w, ss);
                }
            }
            ss = warp_sum(ss);
            if (lane == 0) s_part[m * kConsumerWarps + warp] = ss;
        }
        consumer_sync();
#pragma unroll
        for (int m = 0; m < MT; m++) {
            float tot = 0.f;
#pragma unroll
            for (int q = 0; q < kConsumerWarps; q++) tot += s_part[m * kConsumerWarps + q];
            rstd[m] = 1.0f / sqrtf(tot / float(p.K) + p.eps);
        }
        consumer_sync();  // red is free again
    }

    // raw zero / scale words of a (tile, group) for this thread's 16 columns; zeros outside N
    auto load_consts = [&](int tile, int g, uint2& zraw, uint4& s0, uint4& s1) {
        const int col = tile * kTileColsTma + cg * 16;
        if (col < p.N) {
            zraw = __ldg(p.qz + size_t(g) * zstride + (col >> 4));
            const uint4* sp = reinterpret_cast<const uint4*>(p.scales + size_t(g) * p.N + col);
            s0 = __ldg(sp);
            s1 = __ldg(sp + 1);
        } else {
            zraw = make_uint2(0, 0);
            s0 = make_uint4(0, 0, 0, 0);
            s1 = make_uint4(0, 0, 0, 0);
        }
    };
    // the 8 activations of this thread's rows of unit kb, rounded to fp16 and packed in pairs
    auto load_x = [&](int kb, uint4 (&xr)[MT]) {
#pragma unroll
        for (int m = 0; m < MT; m++) {
            const float4* xp = reinterpret_cast<const float4*>(my_x + size_t(m) * p.K + kb * kUnitRows);
            float4 a = __ldcg(xp), b = __ldcg(xp + 1);
            if (NORM) {
                const uint4 wn = __ldg(reinterpret_cast<const uint4*>(p.norm_w + rg * 8 + kb * kUnitRows));
                a.x = (a.x * rstd[m]) * bf16_lo(wn.x); a.y = (a.y * rstd[m]) * bf16_hi(wn.x);
                a.z = (a.z * rstd[m]) * bf16_lo(wn.y); a.w = (a.w * rstd[m]) * bf16_hi(wn.y);
                b.x = (b.x * rstd[m]) * bf16_lo(wn.z); b.y = (b.y * rstd[m]) * bf16_hi(wn.z);
                b.z = (b.z * rstd[m]) * bf16_lo(wn.w); b.w = (b.w * rstd[m]) * bf16_hi(wn.w);
            }
            xr[m].x = h22u(__floats2half2_rn(a.x, a.y));
            xr[m].y = h22u(__floats2half2_rn(a.z, a.w));
            xr[m].z = h22u(__floats2half2_rn(b.x, b.y));
            xr[m].w = h22u(__floats2half2_rn(b.z, b.w));
        }
    };

    int t = u0 / p.upt, kb = u0 - t * p.upt;
    int units_left = u1 - u0;

    uint2 z_next = make_uint2(0, 0);
    uint4 sa_next = make_uint4(0, 0, 0, 0), sb_next = sa_next, sa_cur, sb_cur;
    load_consts(t, kb >> 2, z_next, sa_cur, sb_cur);
    ZeroPairs z0 = make_zero_pairs(z_next.x), z1 = make_zero_pairs(z_next.y);
    uint4 xr[MT];
    load_x(kb, xr);

    float acc_g[MT][16], acc_t[MT][16];
#pragma unroll
    for (int m = 0; m < MT; m++)
#pragma unroll
        for (int c = 0; c < 16; c++) { acc_g[m][c] = 0.f; acc_t[m][c] = 0.f; }

    int s = 0;
    uint32_t parity = 0;
    bool dead = false;  // a wait ran out: keep walking the barriers so nobody hangs, the result is void
    while (units_left > 0) {
        // ---- one column tile: units kb .. kb + seg - 1 of tile t
        int seg = min(p.upt - kb, units_left);
        units_left -= seg;
        while (seg > 0) {
            // ---- one quantisation group (up to 4 units)
            const int gu = min(4 - (kb & 3), seg);
            seg -= gu;
            const bool more = (seg > 0) || (units_left > 0);
            if (more) {
                // constants of the next group this CTA will visit, fetched while this one is processed
                int ng = (kb >> 2) + 1, nt = t;
                if (ng == groups) { ng = 0; nt++; }
                load_consts(nt, ng, z_next, sa_next, sb_next);
            }
            for (int j = 0; j < gu; j++) {
                if (!dead && !mbar_wait(&full_bar[s], parity)) {
                    atomicExch(&g_gemv_wait_error, 2);
                    dead = true;
                }
                const unsigned char* sp = my_stage + s * kStageBytes;
                uint2 w[8];
#pragma unroll
                for (int i = 0; i < 8; i++) w[i] = *reinterpret_cast<const uint2*>(sp + i * 512);
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty_bar[s]);  // the stage is in registers now
                if (++s == STAGES) { s = 0; parity ^= 1u; }
                // the eight fp16 activations of this thread's rows, one 16-bit register each
                uint16_t x16[8][MT];
#pragma unroll
                for (int m = 0; m < MT; m++) {
                    const uint32_t pr[4] = {xr[m].x, xr[m].y, xr[m].z, xr[m].w};
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        x16[2 * q][m] = uint16_t(pr[q] & 0xffffu);
                        x16[2 * q + 1][m] = uint16_t(pr[q] >> 16);
                    }
                }
                // activations of the next unit this thread will see (same tile or the start of the next one)
                kb++;
                if (j + 1 < gu || more) load_x(kb == p.upt ? 0 : kb, xr);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    word_fma<MT>(w[i].x, z0, x16[i], acc_g, 0);
                    word_fma<MT>(w[i].y, z1, x16[i], acc_g, 8);
                }
            }
            // ---- group done: apply its fp16 scales once
            const uint32_t sraw[8] = {sa_cur.x, sa_cur.y, sa_cur.z, sa_cur.w, sb_cur.x, sb_cur.y, sb_cur.z, sb_cur.w};
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const float2 sc = __half22float2(u2h2(sraw[c]));
#pragma unroll
                for (int m = 0; m < MT; m++) {
                    acc_t[m][2 * c] = fmaf(acc_g[m][2 * c], sc.x, acc_t[m][2 * c]);
                    acc_t[m][2 * c + 1] = fmaf(acc_g[m][2 * c + 1], sc.y, acc_t[m][2 * c + 1]);
                    acc_g[m][2 * c] = 0.f;
                    acc_g[m][2 * c + 1] = 0.f;
                }
            }
            if (more) {
                z0 = make_zero_pairs(z_next.x);
                z1 = make_zero_pairs(z_next.y);
                sa_cur = sa_next;
                sb_cur = sb_next;
            }
        }

        // ---- this CTA's contribution to column tile t is complete: reduce the row groups
#pragma unroll
        for (int m = 0; m < MT; m++)
#pragma unroll
            for (int j = 0; j < 4; j++)
                red[(rg * MT + m) * 256 + cg * 4 + ((j + (cg >> 1)) & 3)] =
                    make_float4(acc_t[m][4 * j], acc_t[m][4 * j + 1], acc_t[m][4 * j + 2], acc_t[m][4 * j + 3]);
#pragma unroll
        for (int m = 0; m < MT; m++)
#pragma unroll
            for (int c = 0; c < 16; c++) acc_t[m][c] = 0.f;
        consumer_sync();

        // thread f owns float4 f of the tile (columns 4f .. 4f+3) for every token row
        const int f = tid;
        const int fcg = f >> 2, fj = f & 3;
        const int col = t * kTileColsTma + f * 4;
        float4 v[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) {
            v[m] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int r = 0; r < kRowGroups; r++) {
                const float4 a = red[(r * MT + m) * 256 + fcg * 4 + ((fj + (fcg >> 1)) & 3)];
                v[m].x += a.x; v[m].y += a.y; v[m].z += a.z; v[m].w += a.w;
            }
        }
        if (ACCUM) {
            if (col < p.N) {
#pragma unroll
                for (int m = 0; m < MT; m++)
                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p.y + size_t(m) * p.N + col),
                                 "f"(v[m].x), "f"(v[m].y), "f"(v[m].z), "f"(v[m].w)
                                 : "memory");
            }
        } else {
            // contributors of this tile: CTAs owning its first and last unit
            const long long first_u = (long long)t * p.upt, last_u = first_u + p.upt - 1;
            const int c_first = int(((first_u + 1) * C - 1) / p.U);
            const int c_last = int(((last_u + 1) * C - 1) / p.U);
            const int n_contrib = c_last - c_first + 1;
            bool finish = true;  // whether this CTA writes y for the tile
            if (n_contrib > 1) {
#pragma unroll
                for (int m = 0; m < MT; m++)
                    *reinterpret_cast<float4*>(p.partial + (size_t(blockIdx.x + t) * MT + m) * kTileColsTma + f * 4) = v[m];
                __threadfence();
                consumer_sync();
                if (tid == 0) {
                    const int prev = atomicAdd(p.counters + t, 1);
                    s_last = (prev == n_contrib - 1);
                    if (s_last) p.counters[t] = 0;
                }
                consumer_sync();
                finish = s_last != 0;
                if (finish) {
                    __threadfence();
                    // slots are added in CTA order (deterministic); loads are issued eight at a time
#pragma unroll
                    for (int m = 0; m < MT; m++) {
                        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                        const float* base = p.partial + (size_t(t) * MT + m) * kTileColsTma + f * 4;
                        int c = c_first;
                        for (; c + 8 <= c_last + 1; c += 8) {
                            float4 a[8];
#pragma unroll
                            for (int q = 0; q < 8; q++)
                                a[q] = __ldcg(reinterpret_cast<const float4*>(base + size_t(c + q) * MT * kTileColsTma));
#pragma unroll
                            for (int q = 0; q < 8; q++) { sum.x += a[q].x; sum.y += a[q].y; sum.z += a[q].z; sum.w += a[q].w; }
                        }
                        for (; c <= c_last; c++) {
                            const float4 a = __ldcg(reinterpret_cast<const float4*>(base + size_t(c) * MT * kTileColsTma));
                            sum.x += a.x; sum.y += a.y; sum.z += a.z; sum.w += a.w;
                        }
                        v[m] = sum;
                    }
                }
            }
            if (finish && col < p.N) {
#pragma unroll
                for (int m = 0; m < MT; m++) {
                    if (p.residual) {
                        const float4 r = __ldcg(reinterpret_cast<const float4*>(p.residual + size_t(m) * p.N + col));
                        v[m].x += r.x; v[m].y += r.y; v[m].z += r.z; v[m].w += r.w;
                    }
                    *reinterpret_cast<float4*>(p.y + size_t(m) * p.N + col) = v[m];
                }
            }
        }
        consumer_sync();  // red is reused by the next tile
        kb = 0;
        t++;
    }
}

// ---------------------------------------------------------------- host side
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

struct MapKey {
    const void* ptr;
    int K, N;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && K == o.K && N == o.N; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.ptr) ^ (size_t(k.K) * 1000003u) ^ (size_t(k.N) * 8191u);
    }
};

// tensor map of a weight matrix: inner dimension N/8 words, outer K rows, box 128 x 32
bool get_tensor_map(const int32_t* qweight, int K, int N, CUtensorMap* out) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key{qweight, K, N};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {cuuint64_t(N / 8), cuuint64_t(K)};
    const cuuint64_t strides[1] = {cuuint64_t(N / 8) * 4};
    const cuuint32_t box[2] = {kTileWords, kUnitRows};
    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap map;
    CUresult rc = fn(&map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<int32_t*>(qweight), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return false;
    if (cache.size() > 16384) cache.clear();
    cache.emplace(key, map);
    *out = map;
    return true;
}

int sm_count() { return device_sm_count(); }

template <int MT, int STAGES, bool ACCUM, bool NORM = false>
int launch_tma(const CUtensorMap& map, const TmaGemvParams& p, int ctas, cudaStream_t stream) {
    auto kern = awq_gemv_tma_kernel<MT, STAGES, ACCUM, NORM>;
    const size_t smem = 128 + size_t(STAGES) * kStageBytes + size_t(kRowGroups) * MT * 1024 * 4;
    static size_t configured[kMaxDevices] = {};  // per instantiation and device
    if (!ensure_dynamic_smem(kern, smem, configured)) {
        set_error("awq_gemv_tma: cannot reserve %zu bytes of shared memory", smem);
        return KUIPER_INTERNAL_ERROR;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas, 1, 1);
    cfg.blockDim = dim3(kThreadsTma, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl_enabled ? 1 : 0;
    cudaError_t err = cudaLaunchKernelEx(&cfg, kern, map, p);
    if (err != cudaSuccess) {
        set_error("awq_gemv_tma launch failed: %s", cudaGetErrorString(err));
        return KUIPER_INTERNAL_ERROR;
    }
    return KUIPER_OK;
}

}  // namespace

// 0 if no bounded wait of the TMA kernel has ever run out on the current device (synchronises)
int awq_gemv_tma_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemv_wait_error, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

void awq_gemv_tma_set_tuning(const char* key, int value) {
    (void)key;
    (void)value;
}

// Workspace layout of the TMA kernel: [counters: tiles ints][error word][partial slots].
size_t awq_gemv_tma_workspace_bytes(int K, int N) {
    const size_t tiles = size_t(N + kTileColsTma - 1) / kTileColsTma;
    const size_t head = ((tiles + 1) * sizeof(int) + 255) / 256 * 256;
    const size_t slots = size_t(sm_count()) * kCtasPerSm + tiles;  // slot index = cta + tile
    return head + slots * 2 * kTileColsTma * sizeof(float);
}

bool awq_gemv_tma_supported(int K, int N) {
    return N % 32 == 0 && K % 128 == 0 && encode_fn() != nullptr;
}

// rows: 1 or 2 token rows starting at x / y / residual
int awq_gemv_tma_launch(const float* x, const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales, float* y,
                        const float* residual, int rows, int K, int N, void* workspace, bool accumulate,
                        const uint16_t* norm_w, float eps, cudaStream_t stream) {
    CUtensorMap map;
    if (!get_tensor_map(qweight, K, N, &map)) {
        set_error("awq_gemv_tma: tensor map encoding failed");
        return KUIPER_INTERNAL_ERROR;
    }
    TmaGemvParams p;
    p.x = x;
    p.y = y;
    p.residual = residual;
    p.qz = reinterpret_cast<const uint2*>(qzeros);
    p.scales = reinterpret_cast<const __half*>(scales);
    p.norm_w = norm_w;
    p.eps = eps;
    p.K = K;
    p.N = N;
    p.tiles = (N + kTileColsTma - 1) / kTileColsTma;
    p.upt = K / kUnitRows;
    p.U = (long long)p.tiles * p.upt;
    const size_t head = ((size_t(p.tiles) + 1) * sizeof(int) + 255) / 256 * 256;
    if (!accumulate && workspace == nullptr) {
        set_error("awq_gemv_tma: the ordered combine needs a workspace");
        return KUIPER_INVALID_ARGUMENT;
    }
    p.counters = reinterpret_cast<int*>(workspace);
    p.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + head);
    long long ctas = (long long)sm_count() * (rows == 1 ? kCtasPerSm : 1);
    if (ctas > p.U) ctas = p.U;
    if (accumulate && norm_w) {
        if (rows == 2) return launch_tma<2, 4, true, true>(map, p, int(ctas), stream);
        return launch_tma<1, 5, true, true>(map, p, int(ctas), stream);
    }
    if (norm_w) {
        set_error("awq_gemv_tma: the fused input norm exists in accumulate mode only");
        return KUIPER_INVALID_ARGUMENT;
    }
    if (accumulate) {
        if (rows == 2) return launch_tma<2, 4, true>(map, p, int(ctas), stream);
        return launch_tma<1, 5, true>(map, p, int(ctas), stream);
    }
    if (rows == 2) return launch_tma<2, 4, false>(map, p, int(ctas), stream);
    return launch_tma<1, 5, false>(map, p, int(ctas), stream);
}

// ---------------------------------------------------------------- entry point that allocates nothing
//
// Some callers cannot hand this library a workspace: code that runs after the host application has
// given every byte of device memory to its own pool, or inside a serving loop where cudaMalloc (and
// the device-wide synchronisation it implies) is not an option.  For them the ordered-combine GEMV is
// offered once more with its scratch (arrival counters + partial-row slots) in a fixed array that is
// part of the library image: every GPU that loads the library holds kNoAllocScratchBytes for it until
// the process exits.
namespace {

constexpr int kNoAllocMaxN = 32768;                       // 32 column tiles
constexpr int kNoAllocMaxCtas = 512;                      // partial-row slots: one per CTA + one per tile
constexpr size_t kNoAllocHeadBytes = 256;                 // arrival counters (32 ints), padded
constexpr size_t kNoAllocScratchBytes =
    kNoAllocHeadBytes + size_t(kNoAllocMaxCtas + kNoAllocMaxN / kTileColsTma) * kTileColsTma * sizeof(float);  // 2 228 480 B

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

void* g_noalloc_ptr[kMaxDevices] = {};  // device address of the array, per device ordinal
std::mutex g_noalloc_mu;

// The array's name is only a host-side stand-in; the address the kernel needs comes from the runtime,
// once per device, with that device current.
int noalloc_scratch(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_error("awq_gemv_noalloc: cannot identify the current device");
        return KUIPER_INTERNAL_ERROR;
    }
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (g_noalloc_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        cudaError_t err = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (err != cudaSuccess || ptr == nullptr) {
            set_error("awq_gemv_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(err));
            return KUIPER_INTERNAL_ERROR;
        }
        g_noalloc_ptr[dev] = ptr;
    }
    *out = g_noalloc_ptr[dev];
    return KUIPER_OK;
}

// tensor map built on the stack: nothing is cached, nothing is allocated
bool encode_tensor_map_once(const int32_t* qweight, int K, int N, CUtensorMap* out) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {cuuint64_t(N / 8), cuuint64_t(K)};
    const cuuint64_t strides[1] = {cuuint64_t(N / 8) * 4};
    const cuuint32_t box[2] = {kTileWords, kUnitRows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<int32_t*>(qweight), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace
}  // namespace kuiper

using namespace kuiper;

extern "C" size_t kuiper_awq_gemv_noalloc_scratch_bytes(void) { return kNoAllocScratchBytes; }

// y[M,N] = x[M,K] . dequant(qweight) (+ residual), same result as kuiper_awq_gemv_f32 up to the order of the
// fp32 partial sums, without a caller workspace and without any allocation.
//  - limits: N <= 32768, N % 32 == 0, K % 128 == 0, group 128, M <= 8; anything else is rejected with status 7;
//  - the first call on a device looks up the scratch array's device address (and sets the kernel's shared
//    memory attribute); make that first call before starting a stream capture;
//  - all calls on a device share the one scratch array: calls that can overlap on the GPU (different streams,
//    or a captured graph replayed concurrently) race on it.  The counters it holds are cleared at the start of
//    every call, so a call that was cut short does not poison the next one.
extern "C" int kuiper_awq_gemv_f32_noalloc(const float* x, const int32_t* qweight, const int32_t* qzeros,
                                           const uint16_t* scales, float* y, const float* residual, int M, int K, int N,
                                           int group, kuiper_stream_t stream) {
    KUIPER_REQUIRE(x && qweight && qzeros && scales && y, "awq_gemv_noalloc: null tensor pointer");
    KUIPER_REQUIRE(M > 0 && K > 0 && N > 0, "awq_gemv_noalloc: empty shape M=%d K=%d N=%d", M, K, N);
    KUIPER_REQUIRE(group == 128, "awq_gemv_noalloc: group size %d is not supported (128 only)", group);
    KUIPER_REQUIRE(K % 128 == 0 && N % 32 == 0, "awq_gemv_noalloc: needs K %% 128 == 0 and N %% 32 == 0 (K=%d N=%d)", K, N);
    KUIPER_REQUIRE(N <= kNoAllocMaxN, "awq_gemv_noalloc: N=%d exceeds the built-in scratch (max N %d)", N, kNoAllocMaxN);
    KUIPER_REQUIRE(M <= 8, "awq_gemv_noalloc: M=%d exceeds the limit of 8 token rows", M);
    KUIPER_REQUIRE(((reinterpret_cast<uintptr_t>(qweight) | reinterpret_cast<uintptr_t>(qzeros) | reinterpret_cast<uintptr_t>(scales) |
                     reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(residual)) & 15) == 0,
                   "awq_gemv_noalloc: tensors must be 16-byte aligned");
    void* scratch = nullptr;
    int rc = noalloc_scratch(&scratch);
    if (rc != KUIPER_OK) return rc;
    CUtensorMap map;
    if (!encode_tensor_map_once(qweight, K, N, &map)) {
        set_error("awq_gemv_noalloc: tensor map encoding failed");
        return KUIPER_INTERNAL_ERROR;
    }
    cudaStream_t st = as_stream(stream);
    TmaGemvParams p;
    p.qz = reinterpret_cast<const uint2*>(qzeros);
    p.scales = reinterpret_cast<const __half*>(scales);
    p.norm_w = nullptr;
    p.eps = 0.f;
    p.K = K;
    p.N = N;
    p.tiles = (N + kTileColsTma - 1) / kTileColsTma;
    p.upt = K / kUnitRows;
    p.U = (long long)p.tiles * p.upt;
    p.counters = reinterpret_cast<int*>(scratch);
    p.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + kNoAllocHeadBytes);
    long long ctas = (long long)sm_count() * kCtasPerSm;
    if (ctas > kNoAllocMaxCtas) ctas = kNoAllocMaxCtas;
    if (ctas > p.U) ctas = p.U;
    for (int m = 0; m < M; m++) {  // one token row per launch: a slot then holds a single partial row
        cudaError_t err = cudaMemsetAsync(scratch, 0, kNoAllocHeadBytes, st);
        if (err != cudaSuccess) {
            set_error("awq_gemv_noalloc: clearing the counters failed: %s", cudaGetErrorString(err));
            return KUIPER_INTERNAL_ERROR;
        }
        p.x = x + size_t(m) * K;
        p.y = y + size_t(m) * N;
        p.residual = residual ? residual + size_t(m) * N : nullptr;
        rc = launch_tma<1, 5, false>(map, p, int(ctas), st);
        if (rc != KUIPER_OK) return rc;
    }
    return KUIPER_OK;
}
