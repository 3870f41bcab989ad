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
// the activation warp tells the consumers that the operand of a chained projection may be read
__device__ __forceinline__ void operand_sync() { asm volatile("bar.sync 3, %0;" ::"n"(kConsumersC + 32) : "memory"); }

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
// w >> 8 as a multiply-high: runs on the FMA pipe and leaves the half-rate integer pipe to the masks
__device__ __forceinline__ uint32_t shr8(uint32_t w) {
    uint32_t v;
    asm("mul.hi.u32 %0, %1, 16777216;" : "=r"(v) : "r"(w));
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
template <int MT, int STAGES, bool ACCUM, bool NORM, int PROBE = 0>
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
                if (PROBE == 2) {  // measurement aid: no weight traffic at all, the consumers run on stale shared memory
                    bar_arrive(&full_bar[s]);
                    if (++kb == p.upt) { kb = 0; t++; }
                    if (++s == STAGES) { s = 0; parity ^= 1u; }
                    continue;
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
            if (PROBE == 1) {  // measurement aid: keep the loads alive, skip the arithmetic
                uint32_t v = 0;
#pragma unroll
                for (int rb = 0; rb < 2; rb++) v ^= w0[0][rb] ^ w1[0][rb] ^ w0[1][rb] ^ w1[1][rb] ^ xb[rb].x ^ xb[rb].y;
                acc_g[0][0][0] += __uint_as_float(v & 0x3fffffffu);
                return;
            }
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

// ---------------------------------------------------------------- one token row on the integer tensor path
//
// Same ring, same units and the same shared-memory layout as the kernel above, other arithmetic: the nibbles are
// used as unsigned bytes and the activations as four signed bytes, so a packed word costs two integer
// instructions and one quarter of an mma.sync.m16n8k32 (s8 x u8 -> s32):
//
//   * (w & 0x0f0f0f0f) holds nibbles 0,2,4,6 of a word as bytes q, (w & 0xf0f0f0f0) holds nibbles 1,3,5,7 as
//     bytes 16 q: both are B operands as they are (contraction index = (weight row, byte position), fragment
//     column = word column), no shift;
//   * the activations of a 128-row group (or of the part of it that this CTA walks) are scaled by a power of
//     two so that the largest is below 2^30, rounded to integers and cut into four signed bytes
//     (x_int = d3 2^24 + d2 2^16 + d1 2^8 + d0, exact).  A-fragment row (digit, byte position c) carries digit d
//     of x[row] at contraction index (row, c) and zeros at the other three positions, which separates the
//     four nibbles of a B byte quadruple into four result rows.  16 fragment rows = 4 digits x 4 positions;
//   * all sums are exact 32-bit integers until the group ends; there the four digit sums are recombined in
//     fp32, the zero point is taken out (sum (q - z) x = sum q x - z sum x) and the fp16 group scale and the
//     power-of-two activation scale are applied.
//
// The activations keep 24+ significant bits relative to the largest of their group (the fp16 B operand of the
// kernel above keeps 11 per element).
//
// Chains.  One launch can run up to kMaxChain projections one after the other, each reading what the one before
// it accumulated (O -> gate|up -> down -> next layer's QKV in the decode step).  Between two projections all
// CTAs meet at a grid barrier (an arrival counter in global memory; every wait on it is bounded).  The weight
// producer does not take part in the barrier: the weights do not depend on the activations, so the ring keeps
// filling with the next projection's units while the consumers drain, meet and fetch their new activations -
// the weight stream does not stop at a projection boundary the way it does between two kernels.  All CTAs of
// the grid are resident at once (2 per SM), which the barrier relies on.
__device__ __forceinline__ void mma_s8u8(int (&d)[4], const uint4& a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

constexpr int kXStageI = 4 * 512 + 16;  // four 8-row steps of ready-made A fragments (16 bytes per lane), sum, scale
constexpr int kMaxChain = 4;
constexpr int kChainSyncInts = 8;       // arrival counters of the barriers + exit counter
constexpr uint32_t kGridSpinLimit = 1u << 21;

struct ChainOp {
    const float* x;          // [K] ([2K] gate|up row with swiglu)
    float* y;                // [N]
    const uint32_t* qz;      // [K/128][N/8]
    const __half* scales;    // [K/128][N]
    const uint16_t* norm_w;  // bf16 [K] or null: the operand is RMSNorm(x)
    float eps;
    int swiglu;              // != 0: the operand is silu(gate) * up
    int K, N, upt, U;        // upt = units per column tile = K / 32, U = total units
};
struct ChainParams {
    CUtensorMap tmap[kMaxChain];
    ChainOp op[kMaxChain];
    const float* residual;   // ordered mode (single projection): [N] or null
    float* partial;          // ordered mode: [slots][1024]
    int* counters;           // ordered mode: [tiles]
    int* sync;               // chains: kChainSyncInts zero-initialised ints, left at zero by every launch
    int n_ops;
    int probe;               // measurement aid: 1 = plain stores instead of the reductions (wrong sums), 2 = neither
};

// TRACE: per-CTA clock readings at the milestones of every projection go to g_gemv_trace (kuiper_gemv_trace_read)
constexpr int kTraceSlots = 24;  // 0 global timer, 1 entry, 2 + 4 op + {0 operand may be read, 1 first unit ready, 2 last unit ready, 3 sums issued}, 18 + op first fragments written
__device__ long long g_gemv_trace[2 * 148 * kTraceSlots];
template <bool TRACE>
__device__ __forceinline__ void trace(int slot) {
    if (TRACE && blockIdx.x < 2 * 148) g_gemv_trace[blockIdx.x * kTraceSlots + slot] = slot == 0 ? (long long)globaltimer_ns() : clock64();
}

// bounded wait until all CTAs of the grid have arrived at barrier `k`
__device__ __noinline__ bool grid_wait(const int* counter, int ctas) {
    for (uint32_t spin = 0; spin < kGridSpinLimit; spin++) {
        int v;
        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
        if (v >= ctas) return true;
        __nanosleep(32);
    }
    atomicExch(&g_gemv_mma_wait_error, 4);
    return false;
}

template <int STAGES, bool ACCUM, bool TRACE = false>
__global__ void __launch_bounds__(kThreadsMma, kCtasPerSmMma)
awq_gemv_imma_kernel(const __grid_constant__ ChainParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (sm_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* stages = smem;                                   // STAGES x 16 KB, 1024-byte aligned for the swizzle
    unsigned char* xstages = smem + STAGES * kStageBytesM;          // STAGES x kXStageI
    // accumulate mode: 128 floats per consumer warp (transpose before the vector reductions);
    // ordered mode: the 1024 columns of the tile
    float* red = reinterpret_cast<float*>(xstages + STAGES * kXStageI);
    __shared__ uint64_t full_bar[STAGES];
    __shared__ uint64_t empty_bar[STAGES];
    __shared__ float s_rstd;
    __shared__ float s_part[kWarpsC];
    __shared__ int s_last;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int C = gridDim.x;
    // fragment coordinates: g = fragment row / column, t = thread in group; as an A row, g = (digit pair, byte position)
    const int g = lane >> 2, t = lane & 3;
    const int c = g & 3, plo = g >> 2;

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) {
            bar_init(&full_bar[s], 2);          // TMA warp (with the byte count) + activation warp
            bar_init(&empty_bar[s], kWarpsC);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        trace<TRACE>(0);
        trace<TRACE>(1);
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kWarpsC) {
        // ------------------------------------------------------------ weight producer (one thread)
        if (lane == 0) {
            int s = 0;
            uint32_t parity = 0;
            bool ok = true;
            for (int op = 0; op < p.n_ops && ok; op++) {
                const ChainOp& o = p.op[op];
                const int u0 = int((long long)blockIdx.x * o.U / C), u1 = int((long long)(blockIdx.x + 1) * o.U / C);
                int tl = u0 / o.upt, kb = u0 - tl * o.upt;
                for (int u = u0; u < u1; u++) {
                    if (!bar_wait_relaxed(&empty_bar[s], parity ^ 1u)) {
                        atomicExch(&g_gemv_mma_wait_error, 1);
                        ok = false;
                        break;
                    }
                    bar_expect_tx(&full_bar[s], kStageBytesM);
#pragma unroll
                    for (int b = 0; b < 4; b++)
                        tma_box(stages + s * kStageBytesM + b * kBoxBytes, &p.tmap[op], tl * kTileWordsM + b * kBoxWords,
                                kb * kUnitRowsM, &full_bar[s]);
                    if (++kb == o.upt) { kb = 0; tl++; }
                    if (++s == STAGES) { s = 0; parity ^= 1u; }
                }
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
        // byte selectors that put digit plo (plo + 2) of a word at byte position c and zeros elsewhere
        const uint32_t sel_keep = 0x4444u & ~(0xfu << (4 * c));
        const uint32_t sel_lo = sel_keep | (uint32_t(plo) << (4 * c));
        const uint32_t sel_hi = sel_keep | (uint32_t(plo + 2) << (4 * c));
        int s = 0;
        uint32_t parity = 0;
        bool alive = true;  // false once a wait ran out: keep walking without waiting so that nobody hangs, the result is void
        for (int op = 0; op < p.n_ops; op++) {
            const ChainOp& o = p.op[op];
            const int u0 = int((long long)blockIdx.x * o.U / C), u1 = int((long long)(blockIdx.x + 1) * o.U / C);
            const bool norm = o.norm_w != nullptr;
            if (op > 0 && alive) {
                // the operand is what all CTAs accumulated in the projection before
                int ok = 1;
                if (lane == 0) ok = grid_wait(p.sync + (op - 1), C) ? 1 : 0;
                alive = __shfl_sync(0xffffffffu, ok, 0) != 0;
            }
            if (op > 0 && norm) operand_sync();  // lets the consumers start the sum of squares
            if (TRACE && lane == 0 && !norm) trace<TRACE>(2 + 4 * op);
            float rstd = 1.f;
            int kb = u0 % o.upt;
            // Rows are requested a segment ahead and only loaded here: the arithmetic on them (SwiGLU, norm weight)
            // happens when the segment becomes current, so that the warp does not stall on the loads it has just issued.
            // a = x (or gate), b = up (SwiGLU) or the bf16 norm weight's bits
            auto fetch = [&](int kblock, float& a, uint32_t& b) {
                const float* xp = o.x + kblock * kUnitRowsM + lane;
                a = __ldcg(xp);
                b = 0u;
                if (o.swiglu) b = __float_as_uint(__ldcg(xp + o.K));
                else if (norm) b = uint32_t(__ldg(o.norm_w + kblock * kUnitRowsM + lane));
            };
            // a segment = the units of one 128-row group that lie in this CTA's run; they share one activation scale
            auto seg_len = [&](int u, int kblock) {
                const int n = 4 - (kblock & 3);
                return n < u1 - u ? n : u1 - u;
            };
            float cur[4], nxt[4];
            uint32_t cur_b[4], nxt_b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { cur[i] = nxt[i] = 0.f; cur_b[i] = nxt_b[i] = 0u; }
            int u = u0;
            int n_cur = u0 < u1 ? seg_len(u0, kb) : 0;
#pragma unroll
            for (int i = 0; i < 4; i++)
                if (i < n_cur) fetch(kb + i, cur[i], cur_b[i]);
            if (norm) {
                // the consumers' sum of squares; the first rows were requested before waiting for it
                norm_sync();
                rstd = s_rstd;
            }
            while (u < u1) {
                const int u_next = u + n_cur;
                int kb_next = kb + n_cur;
                if (kb_next == o.upt) kb_next = 0;
                const int n_next = u_next < u1 ? seg_len(u_next, kb_next) : 0;
#pragma unroll
                for (int i = 0; i < 4; i++)
                    if (i < n_next) fetch(kb_next + i, nxt[i], nxt_b[i]);
                float amax = 0.f;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    if (i < n_cur) {
                        if (o.swiglu) cur[i] = (cur[i] / (1.0f + expf(-cur[i]))) * __uint_as_float(cur_b[i]);
                        else if (norm) cur[i] = (cur[i] * rstd) * __uint_as_float(cur_b[i] << 16);
                        amax = fmaxf(amax, fabsf(cur[i]));
                    }
                }
                // amax < 2^(eb - 126): scaling by 2^(156 - eb) puts every value of the segment below 2^30
                uint32_t eb = __reduce_max_sync(0xffffffffu, __float_as_uint(amax)) >> 23;
                eb = eb < 30u ? 30u : eb;
                const float to_int = __uint_as_float((283u - eb) << 23);
                const float from_int = __uint_as_float((eb - 29u) << 23);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    if (i < n_cur) {
                        if (alive && !bar_wait_relaxed(&empty_bar[s], parity ^ 1u)) {
                            atomicExch(&g_gemv_mma_wait_error, 3);
                            alive = false;
                        }
                        {
                            const int xi = __float2int_rn(cur[i] * to_int);
                            // bytes of `digits` read as signed: d0, d1, d2, d3 with xi = d3 2^24 + d2 2^16 + d1 2^8 + d0
                            const uint32_t digits = (uint32_t(xi) + 0x00808080u) ^ 0x00808080u;
                            // sum of the unit's integers, exact: low and high halves are reduced separately
                            const int sum_lo = __reduce_add_sync(0xffffffffu, xi & 0xffff);
                            const int sum_hi = __reduce_add_sync(0xffffffffu, xi >> 16);
                            const float sum = fmaf(__int2float_rn(sum_hi), 65536.f, __int2float_rn(sum_lo));
                            unsigned char* xs = xstages + s * kXStageI;
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                // fragment of rows 8j .. 8j+7: contraction slots (t, first half) / (t, second half) = rows 8j+2t / 8j+2t+1
                                const uint32_t d0 = __shfl_sync(0xffffffffu, digits, 8 * j + 2 * t);
                                const uint32_t d1 = __shfl_sync(0xffffffffu, digits, 8 * j + 2 * t + 1);
                                uint4 frag;
                                frag.x = __byte_perm(d0, 0u, sel_lo);   // fragment row g,     first half
                                frag.y = __byte_perm(d0, 0u, sel_hi);   // fragment row g + 8, first half
                                frag.z = __byte_perm(d1, 0u, sel_lo);   // fragment row g,     second half
                                frag.w = __byte_perm(d1, 0u, sel_hi);   // fragment row g + 8, second half
                                *reinterpret_cast<uint4*>(xs + j * 512 + lane * 16) = frag;
                            }
                            if (lane == 0) *reinterpret_cast<float2*>(xs + 2048) = make_float2(sum, from_int);
                            __syncwarp();
                            if (lane == 0) bar_arrive(&full_bar[s]);
                            if (TRACE && lane == 0 && u == u0 && i == 0) trace<TRACE>(18 + op);
                            if (++s == STAGES) { s = 0; parity ^= 1u; }
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; i++) { cur[i] = nxt[i]; cur_b[i] = nxt_b[i]; }
                kb = kb_next;
                u = u_next;
                n_cur = n_next;
            }
        }
        return;
    }

    // ---------------------------------------------------------------- consumers
    pdl_wait();  // y, the workspace and (for the norm) x belong to the previous kernel until here

    // this warp: word columns 16*warp .. 16*warp+15 of the tile = two blocks of 8 (cb = 2*warp, 2*warp+1), which lie
    // in TMA box warp>>1 at block position cbl = 2*(warp&1) + {0,1}.  Lane (g, t) reads word g of the block in
    // rows 2t and 2t+1 of each 8-row step (the two halves of its B fragment); with the 128-byte swizzle the
    // 16-byte chunk index is XORed with (row & 7), which spreads the 32 lanes over all 32 banks.
    uint32_t off0[2], off1[2];
#pragma unroll
    for (int cbi = 0; cbi < 2; cbi++) {
        const int cbl = 2 * (warp & 1) + cbi;
        const int chunk = 2 * cbl + (g >> 2);
        off0[cbi] = uint32_t((warp >> 1) * kBoxBytes + (2 * t) * 128 + ((chunk ^ (2 * t)) << 4) + (g & 3) * 4);
        off1[cbi] = uint32_t((warp >> 1) * kBoxBytes + (2 * t + 1) * 128 + ((chunk ^ (2 * t + 1)) << 4) + (g & 3) * 4);
    }
    const float digit_lo = plo ? 256.f : 1.f, digit_hi = digit_lo * 65536.f;   // weights of this lane's two digits
    const int zshift = 8 * c, sshift = 16 * (c >> 1);
    // column of this lane's results inside a word: [0,4,1,5][c] for the low nibbles, two further for the high ones
    const int col_in_word = ((c & 1) << 2) + (c >> 1) + 2 * plo;

    // 32-bit shared-memory addresses that walk the ring with the stage index
    const uint32_t stage0 = sm_u32(stages), xstage0 = sm_u32(xstages) + uint32_t(lane) * 16u;
    const uint32_t full0 = sm_u32(&full_bar[0]), empty0 = sm_u32(&empty_bar[0]);
    const uint32_t sum_rel = 2048u - uint32_t(lane) * 16u;
    uint32_t sbase = stage0, xbase = xstage0, fbar = full0, ebar = empty0;
    int s = 0;
    uint32_t parity = 0;
    bool dead = false;  // a wait ran out: keep walking so that nobody hangs, the result is void

    for (int op = 0; op < p.n_ops; op++) {
        const ChainOp& o = p.op[op];
        const int u0 = int((long long)blockIdx.x * o.U / C), u1 = int((long long)(blockIdx.x + 1) * o.U / C);
        const int groups = o.K >> 7;
        const int NW = o.N >> 3;
        const bool last_op = op + 1 == p.n_ops;

        // This lane's results: fragment rows g and g + 8 (digits plo and plo + 2 at byte position c), fragment columns
        // 2t and 2t + 1 = word columns 2t + ni of each block.  Byte position c of the low-nibble operand is nibble 2c =
        // column [0,4,1,5][c] of the word; the high-nibble operand is two columns further.  The group constants it
        // needs: the zero word of its four word columns and, of each one's eight fp16 scales, the 8-byte half that
        // holds those two columns (.x -> low-nibble column, .y -> high-nibble column, 16-bit lane c >> 1).
        auto load_consts = [&](int tile, int grp, uint32_t (&zw)[2][2], uint2 (&sc)[2][2]) {
#pragma unroll
            for (int cbi = 0; cbi < 2; cbi++) {
#pragma unroll
                for (int ni = 0; ni < 2; ni++) {
                    const int wcol = tile * kTileWordsM + (2 * warp + cbi) * 8 + 2 * t + ni;
                    if (wcol < NW) {
                        zw[cbi][ni] = __ldg(o.qz + size_t(grp) * NW + wcol);
                        sc[cbi][ni] = __ldg(reinterpret_cast<const uint2*>(o.scales + size_t(grp) * o.N + size_t(wcol) * 8 + 4 * (c & 1)));
                    } else {
                        zw[cbi][ni] = 0u;
                        sc[cbi][ni] = make_uint2(0u, 0u);
                    }
                }
            }
        };

        int tl = u0 / o.upt, kb = u0 - tl * o.upt;
        // constants of the current group and of the one after it (fetched a whole group ahead); they belong to
        // the weights, so they are requested before the barrier
        uint32_t z_cur[2][2], z_next[2][2];
        uint2 s_cur[2][2], s_next[2][2];
        load_consts(tl, kb >> 2, z_cur, s_cur);
        int nt = tl, ng = (kb >> 2) + 1;  // the group after the current one on this CTA's path
        if (ng == groups) { ng = 0; nt++; }
        load_consts(nt, ng, z_next, s_next);

        // The consumers do not wait at the grid barrier themselves: they only ever see the new operand through the
        // fragments of the activation warp, which does (a poll with acquire semantics has to wait for the loads
        // above, which go to DRAM).  Only the norm's sum of squares reads the operand directly.
        if (o.norm_w != nullptr) {
            if (op > 0) operand_sync();  // the activation warp has passed the barrier
            if (TRACE && tid == 0) trace<TRACE>(2 + 4 * op);
            // sum of squares of the whole input row, by all consumer threads, 4 x 16-byte loads in flight each
            const float4* hp = reinterpret_cast<const float4*>(o.x);
            const int n4 = o.K >> 2;
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
            if (lane == 0) s_part[warp] = ss;
            consumers_sync();
            if (tid == 0) {
                float tot = 0.f;
#pragma unroll
                for (int q = 0; q < kWarpsC; q++) tot += s_part[q];
                s_rstd = 1.0f / sqrtf(tot / float(o.K) + o.eps);
            }
            norm_sync();
        }

        int acc_lo[2][4], acc_hi[2][4];  // [block][fragment]: integer sums of the current group, low / high nibbles (x 16)
        float acc_t[2][2][2];            // [block][low / high nibble][ni]: this lane's share of the current tile
        float gsum = 0.f;                // sum of the integer activations over the rows of the current group seen so far
        float from_int = 0.f;            // what one integer step of the current group's activations is worth
#pragma unroll
        for (int cbi = 0; cbi < 2; cbi++) {
#pragma unroll
            for (int i = 0; i < 4; i++) { acc_lo[cbi][i] = 0; acc_hi[cbi][i] = 0; }
            acc_t[cbi][0][0] = acc_t[cbi][0][1] = acc_t[cbi][1][0] = acc_t[cbi][1][1] = 0.f;
        }

        for (int u = u0; u < u1; u++) {
            if (!dead && !bar_try(fbar, parity) && !bar_wait_addr(fbar, parity)) {
                atomicExch(&g_gemv_mma_wait_error, 2);
                dead = true;
            }
            if (TRACE && tid == 0) {
                if (u == u0) trace<TRACE>(3 + 4 * op);
                if (u + 1 == u1) trace<TRACE>(4 + 4 * op);
            }
            // the unit is taken in two halves of 16 rows so that only half of it is live in registers at a time;
            // the stage is released after the second half has been read
            const uint32_t a00 = sbase + off0[0], a10 = sbase + off1[0], a01 = sbase + off0[1], a11 = sbase + off1[1];
            uint32_t w0[2][2], w1[2][2];
            uint4 xa[2];
            auto math = [&]() {
#pragma unroll
                for (int rb = 0; rb < 2; rb++) {
#pragma unroll
                    for (int cbi = 0; cbi < 2; cbi++) {
                        const uint32_t a = w0[cbi][rb], b = w1[cbi][rb];
                        mma_s8u8(acc_lo[cbi], xa[rb], a & 0x0f0f0f0fu, b & 0x0f0f0f0fu);
                        mma_s8u8(acc_hi[cbi], xa[rb], a & 0xf0f0f0f0u, b & 0xf0f0f0f0u);
                    }
                }
            };
            w0[0][0] = lds32<0>(a00);    w1[0][0] = lds32<0>(a10);    w0[1][0] = lds32<0>(a01);    w1[1][0] = lds32<0>(a11);
            w0[0][1] = lds32<1024>(a00); w1[0][1] = lds32<1024>(a10); w0[1][1] = lds32<1024>(a01); w1[1][1] = lds32<1024>(a11);
            xa[0] = lds128(xbase);
            xa[1] = lds128(xbase + 512u);
            {
                const uint2 sv = lds64<0>(xbase + sum_rel);
                gsum += __uint_as_float(sv.x);
                from_int = __uint_as_float(sv.y);
            }
            math();
            w0[0][0] = lds32<2048>(a00); w1[0][0] = lds32<2048>(a10); w0[1][0] = lds32<2048>(a01); w1[1][0] = lds32<2048>(a11);
            w0[0][1] = lds32<3072>(a00); w1[0][1] = lds32<3072>(a10); w0[1][1] = lds32<3072>(a01); w1[1][1] = lds32<3072>(a11);
            xa[0] = lds128(xbase + 1024u);
            xa[1] = lds128(xbase + 1536u);
            __syncwarp();
            if (lane == 0) bar_arrive_addr(ebar);  // the stage is in registers now
            if (++s == STAGES) {
                s = 0; parity ^= 1u; sbase = stage0; xbase = xstage0; fbar = full0; ebar = empty0;
            } else {
                sbase += kStageBytesM; xbase += kXStageI; fbar += 8; ebar += 8;
            }
            kb++;
            math();
            const bool tile_end = kb == o.upt;
            const bool run_end = u + 1 == u1;
            if ((kb & 3) != 0 && !run_end) continue;

            // ---- group done (or the run ends inside it): recombine the digits, take the zero point out, apply the scales
            {
                const float zsum = plo ? 0.f : gsum;  // the zero point is subtracted once, by the lane with digits 0 and 2
#pragma unroll
                for (int cbi = 0; cbi < 2; cbi++) {
#pragma unroll
                    for (int ni = 0; ni < 2; ni++) {
                        const uint32_t zw = z_cur[cbi][ni] >> zshift;
                        const float z_lo = float(zw & 15u), z_hi = float(zw & 0xf0u);  // the high nibble keeps its factor 16
                        const float s_lo = __half2float(__ushort_as_half((unsigned short)(s_cur[cbi][ni].x >> sshift)));
                        const float s_hi = __half2float(__ushort_as_half((unsigned short)(s_cur[cbi][ni].y >> sshift)));
                        const float v_lo = fmaf(__int2float_rn(acc_lo[cbi][2 + ni]), digit_hi, __int2float_rn(acc_lo[cbi][ni]) * digit_lo);
                        const float v_hi = fmaf(__int2float_rn(acc_hi[cbi][2 + ni]), digit_hi, __int2float_rn(acc_hi[cbi][ni]) * digit_lo);
                        acc_t[cbi][0][ni] = fmaf(fmaf(-z_lo, zsum, v_lo), s_lo * from_int, acc_t[cbi][0][ni]);
                        acc_t[cbi][1][ni] = fmaf(fmaf(-z_hi, zsum, v_hi), s_hi * (from_int * 0.0625f), acc_t[cbi][1][ni]);
                    }
#pragma unroll
                    for (int i = 0; i < 4; i++) { acc_lo[cbi][i] = 0; acc_hi[cbi][i] = 0; }
                }
            }
            gsum = 0.f;
            if (!run_end) {
#pragma unroll
                for (int cbi = 0; cbi < 2; cbi++)
#pragma unroll
                    for (int ni = 0; ni < 2; ni++) { z_cur[cbi][ni] = z_next[cbi][ni]; s_cur[cbi][ni] = s_next[cbi][ni]; }
                if (++ng == groups) { ng = 0; nt++; }
                load_consts(nt, ng, z_next, s_next);  // clamped to zeros past the last tile
            }
            if (!tile_end && !run_end) continue;

            // ---- this CTA's contribution to column tile tl is complete: add the two digit halves (lanes g and g ^ 4),
            //      then lanes with plo = 0 place the low-nibble columns and lanes with plo = 1 the high-nibble columns
            float mine[2][2];  // [block][ni]
#pragma unroll
            for (int cbi = 0; cbi < 2; cbi++) {
#pragma unroll
                for (int ni = 0; ni < 2; ni++) {
                    const float lo = acc_t[cbi][0][ni] + __shfl_xor_sync(0xffffffffu, acc_t[cbi][0][ni], 16);
                    const float hi = acc_t[cbi][1][ni] + __shfl_xor_sync(0xffffffffu, acc_t[cbi][1][ni], 16);
                    mine[cbi][ni] = plo ? hi : lo;
                    acc_t[cbi][0][ni] = 0.f;
                    acc_t[cbi][1][ni] = 0.f;
                }
            }
            if (ACCUM) {
                float* wred = red + warp * 128;
                __syncwarp();
#pragma unroll
                for (int cbi = 0; cbi < 2; cbi++)
#pragma unroll
                    for (int ni = 0; ni < 2; ni++) wred[(cbi * 8 + 2 * t + ni) * 8 + col_in_word] = mine[cbi][ni];
                __syncwarp();
                const float4 v = *reinterpret_cast<const float4*>(wred + lane * 4);
                const int col = (tl * kTileWordsM + warp * 16) * 8 + lane * 4;
                if (col < o.N) {
                    if (p.probe == 0)
                        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o.y + col), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                                     : "memory");
                    else if (p.probe == 1)
                        *reinterpret_cast<float4*>(o.y + col) = v;
                }
            } else {
#pragma unroll
                for (int cbi = 0; cbi < 2; cbi++)
#pragma unroll
                    for (int ni = 0; ni < 2; ni++) red[((2 * warp + cbi) * 8 + 2 * t + ni) * 8 + col_in_word] = mine[cbi][ni];
                consumers_sync();
                // thread f owns float4 f of the tile (columns 4f .. 4f+3)
                const int f = tid;
                const int col = tl * kTileColsM + f * 4;
                float4 v = *reinterpret_cast<const float4*>(red + f * 4);
                // contributors of this tile: CTAs owning its first and last unit
                const long long first_u = (long long)tl * o.upt, last_u = first_u + o.upt - 1;
                const int c_first = int(((first_u + 1) * C - 1) / o.U);
                const int c_last = int(((last_u + 1) * C - 1) / o.U);
                const int n_contrib = c_last - c_first + 1;
                bool finish = true;  // whether this CTA writes y for the tile
                if (n_contrib > 1) {
                    *reinterpret_cast<float4*>(p.partial + size_t(blockIdx.x + tl) * kTileColsM + f * 4) = v;
                    __threadfence();
                    consumers_sync();
                    if (tid == 0) {
                        const int prev = atomicAdd(p.counters + tl, 1);
                        s_last = (prev == n_contrib - 1);
                        if (s_last) p.counters[tl] = 0;
                    }
                    consumers_sync();
                    finish = s_last != 0;
                    if (finish) {
                        __threadfence();
                        // slots are added in CTA order (deterministic); loads are issued eight at a time
                        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                        const float* base = p.partial + size_t(tl) * kTileColsM + f * 4;
                        int cc = c_first;
                        for (; cc + 8 <= c_last + 1; cc += 8) {
                            float4 a[8];
#pragma unroll
                            for (int q = 0; q < 8; q++) a[q] = __ldcg(reinterpret_cast<const float4*>(base + size_t(cc + q) * kTileColsM));
#pragma unroll
                            for (int q = 0; q < 8; q++) { sum.x += a[q].x; sum.y += a[q].y; sum.z += a[q].z; sum.w += a[q].w; }
                        }
                        for (; cc <= c_last; cc++) {
                            const float4 a = __ldcg(reinterpret_cast<const float4*>(base + size_t(cc) * kTileColsM));
                            sum.x += a.x; sum.y += a.y; sum.z += a.z; sum.w += a.w;
                        }
                        v = sum;
                    }
                }
                if (finish && col < o.N) {
                    if (p.residual) {
                        const float4 r = __ldcg(reinterpret_cast<const float4*>(p.residual + col));
                        v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w;
                    }
                    *reinterpret_cast<float4*>(o.y + col) = v;
                }
                consumers_sync();  // red is reused by the next tile
            }
            kb = 0;
            tl++;
        }

        if (TRACE && tid == 0) trace<TRACE>(5 + 4 * op);
        if (!last_op) {
            // arrive at the grid barrier once this CTA's sums are visible to the whole device
            __threadfence();
            consumers_sync();
            if (tid == 0) {
                __threadfence();
                asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(p.sync + op) : "memory");
            }
        }
    }
    if (tid == 0) {
        if (p.n_ops > 1) {
            // the last CTA to leave puts the counters back to zero for the next launch
            const int prev = atomicAdd(p.sync + (kChainSyncInts - 1), 1);
            if (prev == C - 1) {
#pragma unroll
                for (int i = 0; i < kChainSyncInts; i++) p.sync[i] = 0;
            }
        }
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

int sm_count_mma() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

int g_mma_nomath = 0;
int g_mma_stages = 0;
int g_mma_trace = 0;
int g_chain_stages = 0;
int g_mma_int8 = 0;  // 1: one-row launches take the integer kernel (measured slower inside the decode step; chains always use it)

template <int MT, int STAGES, bool ACCUM, bool NORM, int PROBE = 0>
int launch_mma(const CUtensorMap& map, const MmaGemvParams& p, int ctas, cudaStream_t stream) {
    auto kern = awq_gemv_mma_kernel<MT, STAGES, ACCUM, NORM, PROBE>;
    constexpr int kXStage = (2 * MT + 1) * kXRowStride + 16 * MT;
    const size_t smem = 1024 + size_t(STAGES) * kStageBytesM + ((size_t(STAGES) * kXStage + 15) & ~size_t(15)) +
                        (ACCUM ? 0 : size_t(MT) * kTileColsM * sizeof(float));
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) {
            set_error("awq_gemv_mma: cannot reserve %zu bytes of shared memory", smem);
            return KUIPER_INTERNAL_ERROR;
        }
        configured = true;
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

template <int STAGES, bool ACCUM, bool TRACE = false>
int launch_imma(const ChainParams& p, int ctas, cudaStream_t stream) {
    auto kern = awq_gemv_imma_kernel<STAGES, ACCUM, TRACE>;
    const size_t smem = 1024 + size_t(STAGES) * (kStageBytesM + kXStageI) + size_t(kTileColsM) * sizeof(float);
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) {
            set_error("awq_gemv_imma: cannot reserve %zu bytes of shared memory", smem);
            return KUIPER_INTERNAL_ERROR;
        }
        configured = true;
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
    cudaError_t err = cudaLaunchKernelEx(&cfg, kern, p);
    if (err != cudaSuccess) {
        set_error("awq_gemv_imma launch failed: %s", cudaGetErrorString(err));
        return KUIPER_INTERNAL_ERROR;
    }
    return KUIPER_OK;
}

// one projection of a chain (or the only one of a plain launch)
bool fill_chain_op(ChainParams& cp, int i, const float* x, const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales,
                   float* y, int K, int N, const uint16_t* norm_w, float eps, bool swiglu) {
    if (!get_map_mma(qweight, K, N, &cp.tmap[i])) return false;
    ChainOp& o = cp.op[i];
    o.x = x;
    o.y = y;
    o.qz = reinterpret_cast<const uint32_t*>(qzeros);
    o.scales = reinterpret_cast<const __half*>(scales);
    o.norm_w = norm_w;
    o.eps = eps;
    o.swiglu = swiglu ? 1 : 0;
    o.K = K;
    o.N = N;
    o.upt = K / kUnitRowsM;
    o.U = ((N + kTileColsM - 1) / kTileColsM) * o.upt;
    return true;
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
    if (!strcmp(key, "gemv_nomath")) g_mma_nomath = value;
    if (!strcmp(key, "gemv_stages")) g_mma_stages = value;
    if (!strcmp(key, "gemv_int8")) g_mma_int8 = value;
    if (!strcmp(key, "gemv_trace")) g_mma_trace = value;
    if (!strcmp(key, "gemv_chain_stages")) g_chain_stages = value;
}

int awq_gemv_mma_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemv_mma_wait_error, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

// copies the clock readings of the last traced launch: [CTA][8] (slot 0: global timer in ns, slots 1..: SM clock)
int awq_gemv_trace_read(long long* out, int max_values) {
    const int n = max_values < 2 * 148 * kTraceSlots ? max_values : 2 * 148 * kTraceSlots;
    return cudaMemcpyFromSymbol(out, g_gemv_trace, size_t(n) * sizeof(long long)) == cudaSuccess ? n : -1;
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
    long long ctas = (long long)sm_count_mma() * kCtasPerSmMma;
    if (ctas > p.U) ctas = p.U;
    if ((norm_w || swiglu) && !accumulate) {
        set_error("awq_gemv_mma: the fused input norm / SwiGLU exist in accumulate mode only");
        return KUIPER_INVALID_ARGUMENT;
    }
    if (rows == 1 && g_mma_int8 && g_mma_nomath == 0 && g_mma_stages == 0) {
        ChainParams cp;
        memset(&cp, 0, sizeof(cp));
        if (!fill_chain_op(cp, 0, x, qweight, qzeros, scales, y, K, N, norm_w, eps, swiglu)) {
            set_error("awq_gemv_mma: tensor map encoding failed");
            return KUIPER_INTERNAL_ERROR;
        }
        cp.n_ops = 1;
        cp.residual = residual;
        cp.partial = p.partial;
        cp.counters = p.counters;
        if (accumulate && g_mma_trace) return launch_imma<kStagesM, true, true>(cp, int(ctas), stream);
        if (accumulate) return launch_imma<kStagesM, true>(cp, int(ctas), stream);
        return launch_imma<kStagesM, false>(cp, int(ctas), stream);
    }
    if (accumulate && norm_w) return launch_mma_rows<true, true>(rows, map, p, int(ctas), stream);
    if (accumulate && g_mma_nomath == 1 && rows == 1) return launch_mma<1, kStagesM, true, false, 1>(map, p, int(ctas), stream);
    if (accumulate && g_mma_nomath == 2 && rows == 1) return launch_mma<1, kStagesM, true, false, 2>(map, p, int(ctas), stream);
    if (accumulate && !norm_w && rows == 1 && g_mma_stages == 5) return launch_mma<1, 5, true, false>(map, p, int(ctas), stream);
    if (accumulate && !norm_w && rows == 1 && g_mma_stages == 4) return launch_mma<1, 4, true, false>(map, p, int(ctas), stream);
    if (accumulate && !norm_w && rows == 1 && g_mma_stages == 6) return launch_mma<1, 6, true, false>(map, p, int(ctas), stream);
    if (accumulate) return launch_mma_rows<true, false>(rows, map, p, int(ctas), stream);
    if (rows == 2) return launch_mma<2, kStagesM, false, false>(map, p, int(ctas), stream);
    return launch_mma<1, kStagesM, false, false>(map, p, int(ctas), stream);
}


// A chain of one-row projections in one launch: operand i + 1 is read after every CTA's sums of projection i have
// landed (grid barrier).  `sync`: kChainSyncInts zero-initialised ints that every launch leaves at zero.
int awq_gemv_chain_max_ops() { return kMaxChain; }
size_t awq_gemv_chain_sync_bytes() { return kChainSyncInts * sizeof(int); }
int awq_gemv_chain_launch(const kuiper_gemv_chain_op* ops, int n_ops, int* sync, cudaStream_t stream) {
    if (n_ops < 1 || n_ops > kMaxChain) {
        set_error("awq_gemv_chain: %d projections in one chain (1..%d)", n_ops, kMaxChain);
        return KUIPER_INVALID_ARGUMENT;
    }
    if (n_ops > 1 && sync == nullptr) {
        set_error("awq_gemv_chain: a chain needs the barrier counters");
        return KUIPER_INVALID_ARGUMENT;
    }
    ChainParams cp;
    memset(&cp, 0, sizeof(cp));
    for (int i = 0; i < n_ops; i++) {
        const kuiper_gemv_chain_op& o = ops[i];
        if (!fill_chain_op(cp, i, o.x, o.qweight, o.qzeros, o.scales, o.y, o.K, o.N, o.norm_w, o.eps, o.swiglu != 0)) {
            set_error("awq_gemv_chain: tensor map encoding failed");
            return KUIPER_INTERNAL_ERROR;
        }
    }
    cp.n_ops = n_ops;
    cp.sync = sync;
    cp.probe = g_mma_nomath;
    // every CTA takes part in the barriers, also those without units in one of the projections
    const int ctas = sm_count_mma() * kCtasPerSmMma;
    if (g_mma_trace) return launch_imma<5, true, true>(cp, ctas, stream);
    if (g_chain_stages == 3) return launch_imma<3, true>(cp, ctas, stream);
    if (g_chain_stages == 4) return launch_imma<4, true>(cp, ctas, stream);
    return launch_imma<5, true>(cp, ctas, stream);
}

}  // namespace kuiper

using namespace kuiper;

extern "C" size_t kuiper_awq_gemv_chain_sync_bytes(void) { return awq_gemv_chain_sync_bytes(); }

extern "C" int kuiper_awq_gemv_chain_f32(const kuiper_gemv_chain_op* ops, int n_ops, int group, void* sync, kuiper_stream_t stream) {
    KUIPER_REQUIRE(ops != nullptr, "awq_gemv_chain: null projection list");
    KUIPER_REQUIRE(group == 128, "awq_gemv_chain: group size %d is not supported (128 only)", group);
    KUIPER_REQUIRE(n_ops >= 1 && n_ops <= awq_gemv_chain_max_ops(), "awq_gemv_chain: %d projections in one chain (1..%d)", n_ops,
                   awq_gemv_chain_max_ops());
    for (int i = 0; i < n_ops; i++) {
        const kuiper_gemv_chain_op& o = ops[i];
        KUIPER_REQUIRE(o.x && o.qweight && o.qzeros && o.scales && o.y, "awq_gemv_chain: null tensor pointer in projection %d", i);
        KUIPER_REQUIRE(o.K > 0 && o.N > 0 && o.K % 128 == 0 && o.N % 32 == 0,
                       "awq_gemv_chain: projection %d needs K %% 128 == 0 and N %% 32 == 0 (K=%d N=%d)", i, o.K, o.N);
        KUIPER_REQUIRE(((reinterpret_cast<uintptr_t>(o.qweight) | reinterpret_cast<uintptr_t>(o.qzeros) |
                         reinterpret_cast<uintptr_t>(o.scales) | reinterpret_cast<uintptr_t>(o.y) | reinterpret_cast<uintptr_t>(o.x) |
                         reinterpret_cast<uintptr_t>(o.norm_w)) & 15) == 0,
                       "awq_gemv_chain: tensors of projection %d must be 16-byte aligned", i);
        KUIPER_REQUIRE(!(o.norm_w && o.swiglu), "awq_gemv_chain: projection %d asks for both the fused norm and the fused SwiGLU", i);
    }
    KUIPER_REQUIRE(n_ops == 1 || (sync != nullptr && (reinterpret_cast<uintptr_t>(sync) & 15) == 0),
                   "awq_gemv_chain: a chain needs 16-byte aligned barrier counters");
    KUIPER_REQUIRE(awq_gemv_mma_supported(128, 32), "awq_gemv_chain: tensor-map support is unavailable");
    return awq_gemv_chain_launch(ops, n_ops, static_cast<int*>(sync), as_stream(stream));
}
