// Persistent, TMA-fed INT4-AWQ GEMV whose dot products run on the tensor cores (decode, 1-4 token rows).
// Placeholder it fills: kuiper/include/op/matmul.h:1-11 of the reference.
//
// Why tensor cores for a GEMV: on B200 the SIMT formulation (unpack, subtract the zero point, eight
// mixed-precision FMAs per packed word) needs about as many issue slots as the memory system leaves
// per word, so it is instruction bound.  Here a packed word costs five integer instructions and
// one eighth of an mma.sync:
//
//   * a nibble is used as it is: (w & 0x000f000f) read as two fp16 values is (q_a, q_b) * 2^-24
//     (subnormals, exact), (w & 0x00f000f0) is (q_c, q_d) * 2^-20; the same two masks on w >> 8 give the
//     other four columns.  No magic-number bias and no zero-point subtraction per weight;
//   * those pairs are the A fragments of mma.sync.m16n8k16 (fp16 in, fp32 accumulate): a fragment row is a
//     pair of adjacent output columns, the contraction index is (weight row, which column of the pair), and
//     the B operand carries x[row] in the matching half and 0 in the other, once per token row - so the
//     eight B columns serve up to four token rows at no extra cost;
//   * the zero point comes back per 128-row group: sum (q - z) x = sum q x - z * sum x, with sum x (of the
//     fp16-rounded activations) produced once per 32 rows by the warp that stages x.  Then the fp16 group
//     scale is applied.  All products are exact; only fp32 additions round.
//
// Data movement: the weight [K, N/8] int32 is cut into units of 32 rows x 1024 columns (16 KB), numbered
// column-tile major / K minor and dealt out in contiguous runs to 2 CTAs per SM.  Warp 8 keeps a ring of
// stages full with cp.async.bulk.tensor (four 32-word x 32-row boxes per unit, 128-byte swizzle so that
// the fragment loads are bank-conflict free); warp 9 writes the unit's 32 activations as ready-made B
// fragments (fused RMSNorm applied here if asked for) and their sum; warps 0-7 each own 128 columns of the
// tile for all rows, so nothing is reduced across warps.  Both producers start ahead of the programmatic
// dependent-launch wait where they may (the weight stream does not depend on the previous kernel).
//
// Every mbarrier wait is bounded: after kSpinLimit failed polls the thread records an error code and
// leaves its loop; kuiper_awq_gemv_status() reports it.
#include <cuda.h>

#include <cstring>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace kuiper {
namespace {

constexpr int kWarpsC = 8;                      // consumer warps
constexpr int kConsumersC = kWarpsC * 32;       // 256
constexpr int kThreadsMma = kConsumersC + 64;   // + TMA warp + activation warp
constexpr int kCtasPerSmMma = 2;
constexpr int kUnitRowsM = 32;
constexpr int kTileWordsM = 128;                // 1024 columns
constexpr int kTileColsM = kTileWordsM * 8;
constexpr int kBoxWords = 32;                   // 128 bytes: the span of the swizzle
constexpr int kBoxBytes = kBoxWords * 4 * kUnitRowsM;   // 4 KB
constexpr int kStageBytesM = 4 * kBoxBytes;             // 16 KB
constexpr int kXRowStride = 160;                // bytes between the B-fragment rows of two column slots
constexpr uint32_t kSpinLimitM = 1u << 22;
constexpr int kStagesM = 3;                     // ring depth: deeper rings measured slower (more queued loads at start)

__device__ int g_gemv_mma_wait_error = 0;

struct MmaGemvParams {
    const float* x;         // [MT, K]
    float* y;               // [MT, N]
    const float* residual;  // [MT, N] or null (ordered mode)
    const uint32_t* qz;     // [K/128][N/8]
    const __half* scales;   // [K/128][N]
    float* partial;         // ordered mode: [slots][MT][1024]
    int* counters;          // ordered mode: [tiles]
    const uint16_t* norm_w; // bf16 [K] or null
    float eps;
    int swiglu;             // != 0: x is a gate|up row [MT, 2K] and the operand is silu(gate) * up
    int K, N, tiles, upt;   // upt = units per tile = K / 32
    long long U;            // total units
};

__device__ __forceinline__ uint32_t sm_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void bar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(sm_u32(bar)), "r"(count));
}
__device__ __forceinline__ void bar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(sm_u32(bar)) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(sm_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = sm_u32(bar);
    for (uint32_t spin = 0; spin < kSpinLimitM; spin++) {
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
// the two producer warps wait with a pause between polls: a spinning warp takes issue slots from the consumers
__device__ __forceinline__ bool bar_wait_relaxed(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = sm_u32(bar);
    for (uint32_t spin = 0; spin < kSpinLimitM; spin++) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        __nanosleep(64);
    }
    return false;
}
__device__ __forceinline__ void tma_box(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(sm_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(sm_u32(bar))
        : "memory");
}
__device__ __forceinline__ void consumers_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumersC) : "memory"); }
// consumers + the activation warp (the fused norm's 1/rms is handed over through shared memory)
__device__ __forceinline__ void norm_sync() { asm volatile("bar.sync 2, %0;" ::"n"(kConsumersC + 32) : "memory"); }

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <int IMM>
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(IMM));
    return v;
}
template <int IMM>
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.b32 {%0, %1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(IMM));
    return v;
}
__device__ __forceinline__ bool bar_try(uint32_t addr, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    return done != 0;
}
__device__ __noinline__ bool bar_wait_addr(uint32_t addr, uint32_t parity) {
    for (uint32_t spin = 0; spin < kSpinLimitM; spin++)
        if (bar_try(addr, parity)) return true;
    return false;
}
__device__ __forceinline__ void bar_arrive_addr(uint32_t addr) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(addr) : "memory");
}
__device__ __forceinline__ float2 halves_to_floats(uint32_t u) { return __half22float2(*reinterpret_cast<__half2*>(&u)); }

// MT token rows (1..4).  ACCUM: y += x.W with vector float reductions, the caller guarantees that y holds the
// addend.  Otherwise y = x.W (+ residual) through workspace slots and arrival counters, summed in CTA order.
// NORM: the operand is RMSNorm(x) = (x * rstd) * norm_w, formed by the activation warp.
template <int MT, int STAGES, bool ACCUM, bool NORM>
__global__ void __launch_bounds__(kThreadsMma, kCtasPerSmMma)
awq_gemv_mma_kernel(const __grid_constant__ CUtensorMap tmap, const MmaGemvParams p) {
    // B-fragment rows of the 2*MT live column slots, one row of zeros for the other lanes, per-token sums
    constexpr int kXStage = (2 * MT + 1) * kXRowStride + 16 * MT;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (sm_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* stages = smem;                                   // STAGES x 16 KB, 1024-byte aligned for the swizzle
    unsigned char* xstages = smem + STAGES * kStageBytesM;          // STAGES x kXStage
    float* red = reinterpret_cast<float*>(xstages + ((STAGES * kXStage + 15) & ~15));  // ordered mode: [MT][1024]
    __shared__ uint64_t full_bar[STAGES];
    __shared__ uint64_t empty_bar[STAGES];
    __shared__ float s_rstd[4];
    __shared__ float s_part[4 * kWarpsC];
    __shared__ int s_last;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int C = gridDim.x;
    const int u0 = int((long long)blockIdx.x * p.U / C);
    const int u1 = int((long long)(blockIdx.x + 1) * p.U / C);

    if (tid < STAGES * 32) {  // the zero rows are written once
        *reinterpret_cast<uint32_t*>(xstages + (tid >> 5) * kXStage + 2 * MT * kXRowStride + (tid & 31) * 4) = 0u;
    }
    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) {
            bar_init(&full_bar[s], 2);          // TMA warp (with the byte count) + activation warp
            bar_init(&empty_bar[s], kWarpsC);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kWarpsC) {
        // ------------------------------------------------------------ weight producer (one thread)
        if (lane == 0) {
            int t = u0 / p.upt, kb = u0 - t * p.upt;
            int s = 0;
            uint32_t parity = 0;
            bool ok = true;
            for (int u = u0; u < u1; u++) {
                if (!bar_wait_relaxed(&empty_bar[s], parity ^ 1u)) {
                    atomicExch(&g_gemv_mma_wait_error, 1);
                    ok = false;
                    break;
                }
                bar_expect_tx(&full_bar[s], kStageBytesM);
#pragma unroll
                for (int b = 0; b < 4; b++)
                    tma_box(stages + s * kStageBytesM + b * kBoxBytes, &tmap, t * kTileWordsM + b * kBoxWords, kb * kUnitRowsM,
                            &full_bar[s]);
                if (++kb == p.upt) { kb = 0; t++; }
                if (++s == STAGES) { s = 0; parity ^= 1u; }
            }
            if (!ok) {
                // give copies already issued a bounded chance to land before the CTA goes away
                for (int q = 0; q < STAGES; q++) bar_wait(&full_bar[q], 0);
            }
        }
        return;
    }

    if (warp == kWarpsC + 1) {
        // ------------------------------------------------------------ activation producer (one warp, lane = row of the unit)
        pdl_wait();  // x belongs to the previous kernel until here
        float rstd[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) rstd[m] = 1.f;
        int kb = u0 % p.upt;
        int s = 0;
        uint32_t parity = 0;
        // raw operand rows (SwiGLU applied, norm not yet) and the norm weight of the row
        auto fetch = [&](int kblock, float (&v)[MT], float& wn) {
#pragma unroll
            for (int m = 0; m < MT; m++) {
                if (p.swiglu) {
                    const float* gp = p.x + size_t(m) * 2 * p.K + kblock * kUnitRowsM + lane;
                    const float gate = __ldcg(gp), up = __ldcg(gp + p.K);
                    v[m] = (gate / (1.0f + expf(-gate))) * up;
                } else {
                    v[m] = __ldcg(p.x + size_t(m) * p.K + kblock * kUnitRowsM + lane);
                }
            }
            wn = NORM ? __uint_as_float(uint32_t(__ldg(p.norm_w + kblock * kUnitRowsM + lane)) << 16) : 1.f;
        };
        float cur[MT], nxt[MT], cur_w = 1.f, nxt_w = 1.f;
        if (u0 < u1) fetch(kb, cur, cur_w);
        bool have_rstd = !NORM;
        for (int u = u0; u < u1; u++) {
            int kb_next = kb + 1;
            if (kb_next == p.upt) kb_next = 0;
            if (u + 1 < u1) fetch(kb_next, nxt, nxt_w);
            if (!have_rstd) {
                // the consumers' sum of squares; the first rows were requested before waiting for it
                norm_sync();
#pragma unroll
                for (int m = 0; m < MT; m++) rstd[m] = s_rstd[m];
                have_rstd = true;
            }
            if (!bar_wait_relaxed(&empty_bar[s], parity ^ 1u)) {
                atomicExch(&g_gemv_mma_wait_error, 3);
                break;
            }
            if (NORM) {
#pragma unroll
                for (int m = 0; m < MT; m++) cur[m] = (cur[m] * rstd[m]) * cur_w;
            }
            unsigned char* xs = xstages + s * kXStage;
#pragma unroll
            for (int m = 0; m < MT; m++) {
                const __half h = __float2half_rn(cur[m]);
                const uint32_t bits = __half_as_ushort(h);
                // column slot 2m carries x in the low half (first column of a pair), slot 2m+1 in the high half
                *reinterpret_cast<uint32_t*>(xs + (2 * m) * kXRowStride + lane * 4) = bits;
                *reinterpret_cast<uint32_t*>(xs + (2 * m + 1) * kXRowStride + lane * 4) = bits << 16;
                const float sum = warp_sum(__half2float(h));
                if (lane == 0) *reinterpret_cast<float*>(xs + (2 * MT + 1) * kXRowStride + m * 4) = sum;
            }
            __syncwarp();
            if (lane == 0) bar_arrive(&full_bar[s]);
#pragma unroll
            for (int m = 0; m < MT; m++) cur[m] = nxt[m];
            cur_w = nxt_w;
            kb = kb_next;
            if (++s == STAGES) { s = 0; parity ^= 1u; }
        }
        return;
    }

    // ---------------------------------------------------------------- consumers
    const int g = lane >> 2, tig = lane & 3;
    pdl_wait();  // y, the workspace and (for the norm) x belong to the previous kernel until here

    if (NORM) {
        // sum of squares of the whole input row, by all consumer threads, 4 x 16-byte loads in flight each
#pragma unroll
        for (int m = 0; m < MT; m++) {
            const float4* hp = reinterpret_cast<const float4*>(p.x + size_t(m) * p.K);
            const int n4 = p.K >> 2;
            float ss = 0.f;
            for (int i = tid; i < n4; i += 4 * kConsumersC) {
                float4 v[4];
#pragma unroll
                for (int q = 0; q < 4; q++)
                    v[q] = (i + q * kConsumersC < n4) ? __ldcg(hp + i + q * kConsumersC) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    ss = fmaf(v[q].x, v[q].x, ss); ss = fmaf(v[q].y, v[q].y, ss);
                    ss = fmaf(v[q].z, v[q].z, ss); ss = fmaf(v[q].w, v[q].w, ss);
                }
            }
            ss = warp_sum(ss);
            if (lane == 0) s_part[m * kWarpsC + warp] = ss;
        }
        consumers_sync();
        if (tid < MT) {
            float tot = 0.f;
#pragma unroll
            for (int q = 0; q < kWarpsC; q++) tot += s_part[tid * kWarpsC + q];
            s_rstd[tid] = 1.0f / sqrtf(tot / float(p.K) + p.eps);
        }
        norm_sync();
    }

    // this warp: word columns 16*warp .. 16*warp+15 of the tile = two blocks of 8 (cb = 2*warp, 2*warp+1), which lie
    // in TMA box warp>>1 at block position cbl = 2*(warp&1) + {0,1}.  Lane (g, tig) reads word g of the block in
    // rows 2*tig and 2*tig+1 of each 8-row step; with the 128-byte swizzle the 16-byte chunk index is XORed with
    // (row & 7), which spreads the 32 lanes over all 32 banks.
    uint32_t off0[2], off1[2];
#pragma unroll
    for (int cbi = 0; cbi < 2; cbi++) {
        const int cbl = 2 * (warp & 1) + cbi;
        const int chunk = 2 * cbl + (g >> 2);
        off0[cbi] = uint32_t((warp >> 1) * kBoxBytes + (2 * tig) * 128 + ((chunk ^ (2 * tig)) << 4) + (g & 3) * 4);
        off1[cbi] = uint32_t((warp >> 1) * kBoxBytes + (2 * tig + 1) * 128 + ((chunk ^ (2 * tig + 1)) << 4) + (g & 3) * 4);
    }
    // lanes whose B-fragment column carries no token row read the row of zeros
    const uint32_t xoff = uint32_t((g < 2 * MT ? g : 2 * MT) * kXRowStride + 2 * tig * 4);
    const bool owner = tig < MT;            // lanes whose accumulator columns are real: token row = tig
    const int groups = p.K >> 7;
    const int NW = p.N >> 3;

    // zero word and eight fp16 scales of (tile, group) for word column block cbi of this lane
    auto load_consts = [&](int tile, int grp, uint32_t (&zw)[2], uint4 (&sc)[2]) {
#pragma unroll
        for (int cbi = 0; cbi < 2; cbi++) {
            const int wcol = tile * kTileWordsM + (2 * warp + cbi) * 8 + g;
            if (wcol < NW) {
                zw[cbi] = __ldg(p.qz + size_t(grp) * NW + wcol);
                sc[cbi] = __ldg(reinterpret_cast<const uint4*>(p.scales + size_t(grp) * p.N + size_t(wcol) * 8));
            } else {
                zw[cbi] = 0u;
                sc[cbi] = make_uint4(0, 0, 0, 0);
            }
        }
    };

    int t = u0 / p.upt, kb = u0 - t * p.upt;

    // constants of the current group and of the one after it (fetched a whole group ahead)
    uint32_t z_cur[2], z_next[2];
    uint4 s_cur[2], s_next[2];
    load_consts(t, kb >> 2, z_cur, s_cur);
    int nt = t, ng = (kb >> 2) + 1;  // the group after the current one on this CTA's path
    if (ng == groups) { ng = 0; nt++; }
    load_consts(nt, ng, z_next, s_next);

    float acc_g[2][2][4];  // [block][mma][fragment]: raw nibble sums of the current group; columns 4*mma + fragment
    float acc_t[2][8];     // scaled total of the current tile
    float gsum = 0.f;      // sum of this token row's activations over the rows of the current group seen so far
#pragma unroll
    for (int cbi = 0; cbi < 2; cbi++) {
#pragma unroll
        for (int i = 0; i < 8; i++) acc_t[cbi][i] = 0.f;
#pragma unroll
        for (int i = 0; i < 4; i++) { acc_g[cbi][0][i] = 0.f; acc_g[cbi][1][i] = 0.f; }
    }

    // 32-bit shared-memory addresses that walk the ring with the stage index
    const uint32_t stage0 = sm_u32(stages), xstage0 = sm_u32(xstages) + xoff;
    const uint32_t full0 = sm_u32(&full_bar[0]), empty0 = sm_u32(&empty_bar[0]);
    const uint32_t sum_rel = uint32_t((2 * MT + 1) * kXRowStride + (owner ? tig : 0) * 4) - xoff;
    uint32_t sbase = stage0, xbase = xstage0, fbar = full0, ebar = empty0;
    int s = 0;
    uint32_t parity = 0;
    bool dead = false;  // a wait ran out: keep walking so that nobody hangs, the result is void
    for (int u = u0; u < u1; u++) {
        if (!dead && !bar_try(fbar, parity) && !bar_wait_addr(fbar, parity)) {
            atomicExch(&g_gemv_mma_wait_error, 2);
            dead = true;
        }
        // the unit is taken in two halves of 16 rows so that only half of it is live in registers at a time;
        // the stage is released after the second half has been read
        const uint32_t a00 = sbase + off0[0], a10 = sbase + off1[0], a01 = sbase + off0[1], a11 = sbase + off1[1];
        uint32_t w0[2][2], w1[2][2];
        uint2 xb[2];
        auto math = [&]() {
#pragma unroll
            for (int rb = 0; rb < 2; rb++) {
#pragma unroll
                for (int cbi = 0; cbi < 2; cbi++) {
                    const uint32_t a = w0[cbi][rb], b = w1[cbi][rb];
                    const uint32_t a8 = a >> 8, b8 = b >> 8;
                    // fragment rows g / g+8 = column pairs (0,1) / (2,3), then (4,5) / (6,7)
                    mma_f16(acc_g[cbi][0], a & 0x000f000fu, a & 0x00f000f0u, b & 0x000f000fu, b & 0x00f000f0u, xb[rb].x, xb[rb].y);
                    mma_f16(acc_g[cbi][1], a8 & 0x000f000fu, a8 & 0x00f000f0u, b8 & 0x000f000fu, b8 & 0x00f000f0u, xb[rb].x, xb[rb].y);
                }
            }
        };
        w0[0][0] = lds32<0>(a00);    w1[0][0] = lds32<0>(a10);    w0[1][0] = lds32<0>(a01);    w1[1][0] = lds32<0>(a11);
        w0[0][1] = lds32<1024>(a00); w1[0][1] = lds32<1024>(a10); w0[1][1] = lds32<1024>(a01); w1[1][1] = lds32<1024>(a11);
        xb[0] = lds64<0>(xbase);
        xb[1] = lds64<32>(xbase);
        {
            const float unit_sum = __uint_as_float(lds32<0>(xbase + sum_rel));
            gsum += owner ? unit_sum : 0.f;
        }
        math();
        w0[0][0] = lds32<2048>(a00); w1[0][0] = lds32<2048>(a10); w0[1][0] = lds32<2048>(a01); w1[1][0] = lds32<2048>(a11);
        w0[0][1] = lds32<3072>(a00); w1[0][1] = lds32<3072>(a10); w0[1][1] = lds32<3072>(a01); w1[1][1] = lds32<3072>(a11);
        xb[0] = lds64<64>(xbase);
        xb[1] = lds64<96>(xbase);
        __syncwarp();
        if (lane == 0) bar_arrive_addr(ebar);  // the stage is in registers now
        if (++s == STAGES) {
            s = 0; parity ^= 1u; sbase = stage0; xbase = xstage0; fbar = full0; ebar = empty0;
        } else {
            sbase += kStageBytesM; xbase += kXStage; fbar += 8; ebar += 8;
        }
        kb++;
        math();
        const bool tile_end = kb == p.upt;
        const bool run_end = u + 1 == u1;
        if ((kb & 3) != 0 && !run_end) continue;

        // ---- group done (or the run ends inside it): take the zero point back out and apply the fp16 scales.  Both
        //      the nibble sums and the zero pairs carry the factor 2^-24 (columns 0,1,4,5 of a word) or 2^-20
        //      (columns 2,3,6,7); it is removed once per tile, which is exact (a power of two).
#pragma unroll
        for (int cbi = 0; cbi < 2; cbi++) {
            const uint32_t zw = z_cur[cbi], z8 = zw >> 8;
            const float2 zf[4] = {halves_to_floats(zw & 0x000f000fu), halves_to_floats(zw & 0x00f000f0u),
                                  halves_to_floats(z8 & 0x000f000fu), halves_to_floats(z8 & 0x00f000f0u)};
            const float2 sf[4] = {halves_to_floats(s_cur[cbi].x), halves_to_floats(s_cur[cbi].y),
                                  halves_to_floats(s_cur[cbi].z), halves_to_floats(s_cur[cbi].w)};
#pragma unroll
            for (int pr = 0; pr < 4; pr++) {
                // pair pr = columns 2pr, 2pr+1 sits in mma pr>>1, fragment entries 2*(pr&1), 2*(pr&1)+1
                float& a0 = acc_g[cbi][pr >> 1][2 * (pr & 1)];
                float& a1 = acc_g[cbi][pr >> 1][2 * (pr & 1) + 1];
                acc_t[cbi][2 * pr] = fmaf(fmaf(-zf[pr].x, gsum, a0), sf[pr].x, acc_t[cbi][2 * pr]);
                acc_t[cbi][2 * pr + 1] = fmaf(fmaf(-zf[pr].y, gsum, a1), sf[pr].y, acc_t[cbi][2 * pr + 1]);
                a0 = 0.f;
                a1 = 0.f;
            }
        }
        gsum = 0.f;
        if (!run_end) {
#pragma unroll
            for (int cbi = 0; cbi < 2; cbi++) { z_cur[cbi] = z_next[cbi]; s_cur[cbi] = s_next[cbi]; }
            if (++ng == groups) { ng = 0; nt++; }
            load_consts(nt, ng, z_next, s_next);  // clamped to zeros past the last tile
        }
        if (!tile_end && !run_end) continue;

        // ---- this CTA's contribution to column tile t is complete
#pragma unroll
        for (int cbi = 0; cbi < 2; cbi++)
#pragma unroll
            for (int i = 0; i < 8; i++) acc_t[cbi][i] *= (i & 2) ? 1048576.f : 16777216.f;
        if (ACCUM) {
            if (owner) {
#pragma unroll
                for (int cbi = 0; cbi < 2; cbi++) {
                    const int col = (t * kTileWordsM + (2 * warp + cbi) * 8 + g) * 8;
                    if (col < p.N) {
                        float* yp = p.y + size_t(tig) * p.N + col;
                        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(yp), "f"(acc_t[cbi][0]),
                                     "f"(acc_t[cbi][1]), "f"(acc_t[cbi][2]), "f"(acc_t[cbi][3])
                                     : "memory");
                        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(yp + 4), "f"(acc_t[cbi][4]),
                                     "f"(acc_t[cbi][5]), "f"(acc_t[cbi][6]), "f"(acc_t[cbi][7])
                                     : "memory");
                    }
                }
            }
        } else {
            if (owner) {
#pragma unroll
                for (int cbi = 0; cbi < 2; cbi++) {
                    float4* rp = reinterpret_cast<float4*>(red + tig * kTileColsM + ((2 * warp + cbi) * 8 + g) * 8);
                    rp[0] = make_float4(acc_t[cbi][0], acc_t[cbi][1], acc_t[cbi][2], acc_t[cbi][3]);
                    rp[1] = make_float4(acc_t[cbi][4], acc_t[cbi][5], acc_t[cbi][6], acc_t[cbi][7]);
                }
            }
            consumers_sync();
            // thread f owns float4 f of the tile (columns 4f .. 4f+3) for every token row
            const int f = tid;
            const int col = t * kTileColsM + f * 4;
            float4 v[MT];
#pragma unroll
            for (int m = 0; m < MT; m++) v[m] = *reinterpret_cast<const float4*>(red + m * kTileColsM + f * 4);
            // contributors of this tile: CTAs owning its first and last unit
            const long long first_u = (long long)t * p.upt, last_u = first_u + p.upt - 1;
            const int c_first = int(((first_u + 1) * C - 1) / p.U);
            const int c_last = int(((last_u + 1) * C - 1) / p.U);
            const int n_contrib = c_last - c_first + 1;
            bool finish = true;  // whether this CTA writes y for the tile
            if (n_contrib > 1) {
#pragma unroll
                for (int m = 0; m < MT; m++)
                    *reinterpret_cast<float4*>(p.partial + (size_t(blockIdx.x + t) * MT + m) * kTileColsM + f * 4) = v[m];
                __threadfence();
                consumers_sync();
                if (tid == 0) {
                    const int prev = atomicAdd(p.counters + t, 1);
                    s_last = (prev == n_contrib - 1);
                    if (s_last) p.counters[t] = 0;
                }
                consumers_sync();
                finish = s_last != 0;
                if (finish) {
                    __threadfence();
                    // slots are added in CTA order (deterministic); loads are issued eight at a time
#pragma unroll
                    for (int m = 0; m < MT; m++) {
                        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                        const float* base = p.partial + (size_t(t) * MT + m) * kTileColsM + f * 4;
                        int c = c_first;
                        for (; c + 8 <= c_last + 1; c += 8) {
                            float4 a[8];
#pragma unroll
                            for (int q = 0; q < 8; q++)
                                a[q] = __ldcg(reinterpret_cast<const float4*>(base + size_t(c + q) * MT * kTileColsM));
#pragma unroll
                            for (int q = 0; q < 8; q++) { sum.x += a[q].x; sum.y += a[q].y; sum.z += a[q].z; sum.w += a[q].w; }
                        }
                        for (; c <= c_last; c++) {
                            const float4 a = __ldcg(reinterpret_cast<const float4*>(base + size_t(c) * MT * kTileColsM));
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
            consumers_sync();  // red is reused by the next tile
        }
#pragma unroll
        for (int cbi = 0; cbi < 2; cbi++)
#pragma unroll
            for (int i = 0; i < 8; i++) acc_t[cbi][i] = 0.f;
        kb = 0;
        t++;
    }
}



// ---------------------------------------------------------------- host side
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn_mma() {
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

// tensor map of a weight matrix: inner dimension N/8 words, outer K rows, box 32 words x 32 rows, 128-byte swizzle
bool encode_map_mma(const int32_t* qweight, int K, int N, CUtensorMap* out) {
    EncodeTiledFn fn = encode_fn_mma();
    if (!fn) return false;
    const cuuint64_t dims[2] = {cuuint64_t(N / 8), cuuint64_t(K)};
    const cuuint64_t strides[1] = {cuuint64_t(N / 8) * 4};
    const cuuint32_t box[2] = {kBoxWords, kUnitRowsM};
    const cuuint32_t estr[2] = {1, 1};
    return fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<int32_t*>(qweight), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct MapKeyM {
    const void* ptr;
    int K, N;
    bool operator==(const MapKeyM& o) const { return ptr == o.ptr && K == o.K && N == o.N; }
};
struct MapKeyMHash {
    size_t operator()(const MapKeyM& k) const {
        return std::hash<const void*>()(k.ptr) ^ (size_t(k.K) * 1000003u) ^ (size_t(k.N) * 8191u);
    }
};

// a tensor map depends on the address and shape only (device pointers of different devices are distinct under
// unified addressing), so one process-wide cache serves every device
bool get_map_mma(const int32_t* qweight, int K, int N, CUtensorMap* out) {
    static std::mutex mu;
    static std::unordered_map<MapKeyM, CUtensorMap, MapKeyMHash> cache;
    const MapKeyM key{qweight, K, N};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    CUtensorMap map;
    if (!encode_map_mma(qweight, K, N, &map)) return false;
    if (cache.size() > 16384) cache.clear();
    cache.emplace(key, map);
    *out = map;
    return true;
}

template <int MT, int STAGES, bool ACCUM, bool NORM>
int launch_mma(const CUtensorMap& map, const MmaGemvParams& p, int ctas, cudaStream_t stream) {
    auto kern = awq_gemv_mma_kernel<MT, STAGES, ACCUM, NORM>;
    constexpr int kXStage = (2 * MT + 1) * kXRowStride + 16 * MT;
    const size_t smem = 1024 + size_t(STAGES) * kStageBytesM + ((size_t(STAGES) * kXStage + 15) & ~size_t(15)) +
                        (ACCUM ? 0 : size_t(MT) * kTileColsM * sizeof(float));
    static size_t configured[kMaxDevices] = {};  // per instantiation and device
    if (!ensure_dynamic_smem(kern, smem, configured)) {
        set_error("awq_gemv_mma: cannot reserve %zu bytes of shared memory", smem);
        return KUIPER_INTERNAL_ERROR;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas, 1, 1);
    cfg.blockDim = dim3(kThreadsMma, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl_enabled ? 1 : 0;
    cudaError_t err = cudaLaunchKernelEx(&cfg, kern, map, p);
    if (err != cudaSuccess) {
        set_error("awq_gemv_mma launch failed: %s", cudaGetErrorString(err));
        return KUIPER_INTERNAL_ERROR;
    }
    return KUIPER_OK;
}

template <bool ACCUM, bool NORM>
int launch_mma_rows(int rows, const CUtensorMap& map, const MmaGemvParams& p, int ctas, cudaStream_t stream) {
    switch (rows) {
        case 1: return launch_mma<1, kStagesM, ACCUM, NORM>(map, p, ctas, stream);
        case 2: return launch_mma<2, kStagesM, ACCUM, NORM>(map, p, ctas, stream);
        case 3: return launch_mma<3, kStagesM, ACCUM, NORM>(map, p, ctas, stream);
        default: return launch_mma<4, kStagesM, ACCUM, NORM>(map, p, ctas, stream);
    }
}

}  // namespace

void awq_gemv_mma_set_tuning(const char* key, int value) {
    (void)key;
    (void)value;
}

int awq_gemv_mma_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemv_mma_wait_error, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

bool awq_gemv_mma_supported(int K, int N) { return N % 32 == 0 && K % 128 == 0 && encode_fn_mma() != nullptr; }

// most token rows one launch takes: 4 when accumulating, 2 through the ordered combine (its workspace slots
// hold two partial rows)
int awq_gemv_mma_max_rows(bool accumulate) { return accumulate ? 4 : 2; }

// Workspace layout of the ordered combine (shared with the SIMT kernel of awq_gemv_tma.cu):
// [counters: tiles ints, padded to 256 bytes][partial slots: (CTAs + tiles) x 2 x 1024 floats].
int awq_gemv_mma_launch(const float* x, const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales, float* y,
                        const float* residual, int rows, int K, int N, void* workspace, bool accumulate,
                        const uint16_t* norm_w, float eps, bool swiglu, cudaStream_t stream) {
    if (rows < 1 || rows > awq_gemv_mma_max_rows(accumulate)) {
        set_error("awq_gemv_mma: %d token rows in one launch", rows);
        return KUIPER_INVALID_ARGUMENT;
    }
    CUtensorMap map;
    if (!get_map_mma(qweight, K, N, &map)) {
        set_error("awq_gemv_mma: tensor map encoding failed");
        return KUIPER_INTERNAL_ERROR;
    }
    MmaGemvParams p;
    p.x = x;
    p.y = y;
    p.residual = residual;
    p.qz = reinterpret_cast<const uint32_t*>(qzeros);
    p.scales = reinterpret_cast<const __half*>(scales);
    p.norm_w = norm_w;
    p.eps = eps;
    p.swiglu = swiglu ? 1 : 0;
    p.K = K;
    p.N = N;
    p.tiles = (N + kTileColsM - 1) / kTileColsM;
    p.upt = K / kUnitRowsM;
    p.U = (long long)p.tiles * p.upt;
    const size_t head = ((size_t(p.tiles) + 1) * sizeof(int) + 255) / 256 * 256;
    if (!accumulate && workspace == nullptr) {
        set_error("awq_gemv_mma: the ordered combine needs a workspace");
        return KUIPER_INVALID_ARGUMENT;
    }
    p.counters = reinterpret_cast<int*>(workspace);
    p.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + head);
    long long ctas = (long long)device_sm_count() * kCtasPerSmMma;
    if (ctas > p.U) ctas = p.U;
    if ((norm_w || swiglu) && !accumulate) {
        set_error("awq_gemv_mma: the fused input norm / SwiGLU exist in accumulate mode only");
        return KUIPER_INVALID_ARGUMENT;
    }
    if (accumulate && norm_w) return launch_mma_rows<true, true>(rows, map, p, int(ctas), stream);
    if (accumulate) return launch_mma_rows<true, false>(rows, map, p, int(ctas), stream);
    if (rows == 2) return launch_mma<2, kStagesM, false, false>(map, p, int(ctas), stream);
    return launch_mma<1, kStagesM, false, false>(map, p, int(ctas), stream);
}

}  // namespace kuiper
