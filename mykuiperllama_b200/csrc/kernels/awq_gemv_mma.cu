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
// Data movement: a weight [K, N/8] int32 is cut into units of 32 rows x 1024 columns (16 KB), numbered
// column-tile major / K minor (over all matrices of a grouped call) and dealt out in contiguous runs to 2 CTAs
// per SM (3 for large one-row integer-operand launches, see g_int8_ctas); optionally a tail of 128-row groups is handed out through an atomic ticket counter instead (off by
// default, see g_dyn_pct).  Warp 8 keeps a ring of stages full: per unit a descriptor (item, tile, row block,
// first-of-group / last-of-run flags) that the other warps follow, four cp.async.bulk.tensor boxes (32 words x 32
// rows, 128-byte swizzle so that the fragment loads are bank-conflict free) and, for the first unit of a 128-row
// group on the CTA's path, the group's zero words and fp16 scales of the tile (two plain bulk copies).  Warp 9
// writes the unit's 32 activations as ready-made B fragments (fused RMSNorm / SwiGLU applied here) with their sum.
// Warps 0-7 each own 128 columns of the tile for all rows, so nothing is reduced across warps.  The weight
// producer never waits for the previous kernel (the weights do not depend on it), so under programmatic dependent
// launch the ring is full by the time the operand may be read.
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
constexpr int kThreadsMma = kConsumersC + 64;   // + weight producer warp + activation warp
constexpr int kCtasPerSmMma = 2;
constexpr int kCtasPerSmInt8 = 3;  // the integer-operand consumers fit in 64 registers: a third CTA per SM is possible
constexpr int kUnitRowsM = 32;
constexpr int kTileWordsM = 128;                // 1024 columns
constexpr int kTileColsM = kTileWordsM * 8;
constexpr int kBoxWords = 32;                   // 128 bytes: the span of the swizzle
constexpr int kBoxBytes = kBoxWords * 4 * kUnitRowsM;   // 4 KB
constexpr int kUnitBytes = 4 * kBoxBytes;               // 16 KB of packed weights
constexpr int kZeroBytes = kTileWordsM * 4;             // zero words of one (group, tile)
constexpr int kScaleBytes = kTileColsM * 2;             // fp16 scales of one (group, tile)
constexpr int kXRowStride = 160;                // bytes between the B-fragment rows of two column slots
constexpr uint32_t kSpinLimitM = 1u << 22;
constexpr int kStagesM = 3;                     // ring depth: deeper rings measured slower (more queued loads at start)

// stage layout: weights | zero words | scales | activation fragments | descriptor (16 bytes)
constexpr int kOffZero = kUnitBytes;
constexpr int kOffScale = kOffZero + kZeroBytes;
constexpr int kOffX = kOffScale + kScaleBytes;
// fp16 operand: B-fragment rows of the 2*MT live column slots, one row of zeros, per-token sums;
// integer operand (one token row): 4 steps x 32 lanes x 8 bytes of ready-made B fragments, then 1 / scale and the unit's sum
constexpr int kXBytesInt8 = 4 * 32 * 8;
constexpr int x_stage_bytes(int MT, bool int8) { return int8 ? kXBytesInt8 + 16 : (2 * MT + 1) * kXRowStride + 16 * MT; }
constexpr int stage_bytes(int MT, bool int8) { return (kOffX + x_stage_bytes(MT, int8) + 16 + 1023) / 1024 * 1024; }

constexpr int kFlagFirst = 1;   // first unit of a 128-row group on this CTA's path: the stage carries the group's zeros and scales
constexpr int kFlagLast = 2;    // the next unit is not the next row block of the same tile: finish the tile after this one

__device__ int g_gemv_mma_wait_error = 0;

// Build flag KUIPER_TRACE (off in the shipped library): per-CTA clock readings of the last launch, read back with
// kuiper_gemv_trace_read().  Slot 0: global timer (ns) at entry; then SM clock at 1 entry, 2 consumers past the dependency
// wait, 3 first unit ready, 4 last unit consumed, 5 consumer exit, 6 activation warp saw its first descriptor,
// 7 first fragments written, 8 first weight copy issued, 9 last weight copy issued
#ifdef KUIPER_TRACE
constexpr int kGemvTraceCtas = 304, kGemvTraceSlots = 10;
__device__ long long g_gemv_trace[kGemvTraceCtas * kGemvTraceSlots];
__device__ __forceinline__ void gemv_trace(int slot) {
    if (blockIdx.x < kGemvTraceCtas) g_gemv_trace[blockIdx.x * kGemvTraceSlots + slot] = slot == 0 ? (long long)globaltimer_ns() : clock64();
}
#else
__device__ __forceinline__ void gemv_trace(int) {}
#endif

// one projection; 64-byte aligned because the TMA unit reads the tensor map in place
struct __align__(64) GemvItem {
    CUtensorMap tmap;        // over qweight: [K rows][N/8 words], box 32 x 32, 128-byte swizzle
    const float* x;          // [MT, K] ([MT, 2K] gate|up rows with swiglu)
    float* y;                // [MT, N]
    const uint32_t* qz;      // [K/128][N/8]
    const __half* scales;    // [K/128][N]
    const uint16_t* norm_w;  // bf16 [K] or null
    float eps;
    int swiglu;              // != 0: the operand is silu(gate) * up
    int K, N, tiles, upt;    // upt = units per tile = K / 32
    int unit0;               // index of the item's first unit in the call's numbering
    int pad_[13];
};
static_assert(sizeof(GemvItem) == 256, "GemvItem is laid out for a 256-byte table stride");

struct GemvCall {
    const GemvItem* items;   // grouped calls: table in device memory; otherwise null (the item is a kernel parameter)
    int n_items;
    int U;                   // units of the whole call
    int U_static;            // units [0, U_static) are dealt out in contiguous runs, the rest through tickets
    int chunk;               // units per ticket
    int n_chunks;
    int* tickets;            // [0] ticket counter, [1] exit counter, both zero between launches; null: no tickets
    // ordered mode (single item, no tickets)
    const float* residual;   // [MT, N] or null
    float* partial;          // [slots][MT][1024]
    int* counters;           // [tiles]
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
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = sm_u32(bar);
    for (uint32_t spin = 0; spin < kSpinLimitM; spin++)
        if (bar_try(addr, parity)) return true;
    return false;
}
// the producer waits with a pause between polls: a spinning warp takes issue slots from the consumers
__device__ __forceinline__ bool bar_wait_relaxed(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = sm_u32(bar);
    for (uint32_t spin = 0; spin < kSpinLimitM; spin++) {
        if (bar_try(addr, parity)) return true;
        __nanosleep(64);
    }
    return false;
}
__device__ __noinline__ bool bar_wait_addr(uint32_t addr, uint32_t parity) {
    for (uint32_t spin = 0; spin < kSpinLimitM; spin++)
        if (bar_try(addr, parity)) return true;
    return false;
}
__device__ __forceinline__ void bar_arrive_addr(uint32_t addr) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(addr) : "memory");
}
__device__ __forceinline__ void tma_box(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(sm_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(sm_u32(bar))
        : "memory");
}
// plain bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completion on the mbarrier
__device__ __forceinline__ void bulk_copy(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(sm_u32(dst)), "l"(src), "r"(bytes), "r"(sm_u32(bar))
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
// unsigned weight bytes (A) x signed activation digits (B) -> exact 32-bit sums
__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float lds_f16(uint32_t addr) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return __half2float(__ushort_as_half(v));
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
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float2 halves_to_floats(uint32_t u) { return __half22float2(*reinterpret_cast<__half2*>(&u)); }

// a unit of the call as the producer sees it
struct UnitRef {
    const GemvItem* it;  // grouped calls: the item's table entry
    int item, t, kb, flags;
};

// MT token rows (1..4).  ACCUM: y += x.W with vector float reductions, the caller guarantees that y holds the
// addend.  Otherwise y = x.W (+ residual) through workspace slots and arrival counters, summed in CTA order.
// NORM: the operand is RMSNorm(x) = (x * rstd) * norm_w, formed by the producer warp.
// GROUPED: the call is a list of independent projections (table in device memory) whose units form one numbering.
// INT8 (one token row): the operand is block-scaled to 16-bit integers per 32 rows (x' = rint(x * 2^e) * 2^-e with
// |x * 2^e| < 2^14 for the largest of the 32) and enters mma.sync.m16n8k32 (u8 x s8 -> s32) as two signed byte
// digits; the nibbles are used as unsigned bytes: (w & 0x0f0f0f0f) holds nibbles 0,2,4,6 of a word as bytes q,
// (w & 0xf0f0f0f0) nibbles 1,3,5,7 as bytes 16 q - two masks per word, no shift.  Fragment row = (word column,
// low / high nibbles), contraction index = (weight row, byte position c), B column = (byte position c', digit):
// B[(r, c)][(c', d)] = digit d of x'[r] when c == c', else 0, which separates the four bytes of a word into four
// result columns.  All sums are exact integers inside a unit; 512 weights per mma, 2 integer instructions per word.
template <int MT, int STAGES, bool ACCUM, bool NORM, bool GROUPED, bool INT8, int OCC>
__global__ void __launch_bounds__(kThreadsMma, OCC)
awq_gemv_mma_kernel(const __grid_constant__ GemvItem item0, const GemvCall p) {
    static_assert(!INT8 || MT == 1, "the integer operand path takes one token row");
    constexpr int kXStage = x_stage_bytes(MT, INT8);
    constexpr int kStage = stage_bytes(MT, INT8);
    constexpr int kOffMeta = kOffX + kXStage;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (sm_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* stages = smem;                                   // STAGES x kStage, 1024-byte aligned for the swizzle
    float* red = reinterpret_cast<float*>(smem + STAGES * kStage);  // ordered mode: [MT][1024]
    __shared__ uint64_t full_bar[STAGES];
    __shared__ uint64_t empty_bar[STAGES];
    __shared__ uint64_t meta_bar[STAGES];   // the stage's descriptor is written (weight producer -> activation warp)
    __shared__ float s_rstd[4];
    __shared__ float s_part[4 * kWarpsC];
    __shared__ int s_last;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int C = gridDim.x;

    if (!INT8 && tid < STAGES * 32) {  // the zero rows of the activation fragments are written once
        *reinterpret_cast<uint32_t*>(stages + (tid >> 5) * kStage + kOffX + 2 * MT * kXRowStride + (tid & 31) * 4) = 0u;
    }
    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) {
            bar_init(&full_bar[s], 2);          // weight producer (with the byte count) + activation warp
            bar_init(&empty_bar[s], kWarpsC);
            bar_init(&meta_bar[s], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();
    if (tid == 0) { gemv_trace(0); gemv_trace(1); }

    if (warp == kWarpsC) {
        // ------------------------------------------------------------ weight producer (one warp, lane 0 issues)
        // The sequence of units this CTA works through: its static run, then chunks taken by ticket.  Every lane keeps
        // the same cursor (tickets are taken by lane 0 and broadcast).
        int run_u = int((long long)blockIdx.x * p.U_static / C);
        int run_end = int((long long)(blockIdx.x + 1) * p.U_static / C);
        bool tickets_open = p.tickets != nullptr && p.n_chunks > 0;
        int next_ticket = -1;   // lane 0: a ticket requested ahead of need
        bool ticket_pending = false;
        auto request_ticket = [&]() {
            if (tickets_open && !ticket_pending) {
                if (lane == 0) next_ticket = atomicAdd(p.tickets, 1);
                ticket_pending = true;
            }
        };
        auto next_unit = [&]() -> int {  // next unit of the sequence or -1
            while (true) {
                if (run_u < run_end) return run_u++;
                if (!tickets_open) return -1;
                request_ticket();
                const int tk = __shfl_sync(0xffffffffu, next_ticket, 0);
                ticket_pending = false;
                if (tk >= p.n_chunks) {
                    // no work left: sign out; the last CTA to do so puts both counters back to zero for the next launch
                    tickets_open = false;
                    if (lane == 0) {
                        const int prev = atomicAdd(p.tickets + 1, 1);
                        if (prev == C - 1) {
                            p.tickets[0] = 0;
                            p.tickets[1] = 0;
                        }
                    }
                    return -1;
                }
                run_u = p.U_static + tk * p.chunk;
                run_end = min(run_u + p.chunk, p.U);
                request_ticket();  // the one after, so that its round trip overlaps this chunk
            }
        };
        request_ticket();

        // which item a unit belongs to (grouped calls): items are few and their first units ascend
        const GemvItem* it = GROUPED ? p.items : &item0;
        int it_idx = 0, it_unit0 = 0;
        int it_upt = GROUPED ? __ldg(&p.items[0].upt) : item0.upt;
        int it_units = GROUPED ? __ldg(&p.items[0].tiles) * it_upt : p.U;
        bool prev_last = true;  // the unit before (in this CTA's sequence) ended a run, or there was none
        // place `u` (with `nxt` the unit after it in the sequence, or -1): item, tile, row block, flags
        auto place = [&](int u, int nxt) -> UnitRef {
            if (GROUPED && (u < it_unit0 || u >= it_unit0 + it_units)) {
                int found = 0;
                for (int base = 0; base < p.n_items; base += 32) {
                    const int i = base + lane;
                    const int first = i < p.n_items ? __ldg(&p.items[i].unit0) : 0x7fffffff;
                    const unsigned below = __ballot_sync(0xffffffffu, first <= u);
                    if (below == 0u) break;
                    found = base + 31 - __clz(below);
                    if (below != 0xffffffffu) break;
                }
                it_idx = found;
                it = p.items + found;
                it_unit0 = __ldg(&it->unit0);
                it_upt = __ldg(&it->upt);
                it_units = __ldg(&it->tiles) * it_upt;
            }
            UnitRef r;
            r.it = it;
            r.item = it_idx;
            const int rel = u - it_unit0;
            r.t = rel / it_upt;
            r.kb = rel - r.t * it_upt;
            r.flags = 0;
            if (prev_last || (r.kb & 3) == 0) r.flags |= kFlagFirst;
            const bool contiguous = nxt == u + 1 && r.kb + 1 < it_upt;
            if (!contiguous) r.flags |= kFlagLast;
            prev_last = !contiguous;
            return r;
        };
        int s = 0;
        uint32_t parity = 0;
        bool ok = true;
        int cur = next_unit();
        bool first_issue = true;
        while (cur >= 0) {
            const int nxt = next_unit();
            const UnitRef r = place(cur, nxt);
            if (!bar_wait_relaxed(&empty_bar[s], parity ^ 1u)) {
                atomicExch(&g_gemv_mma_wait_error, 1);
                ok = false;
                break;
            }
            if (lane == 0) {
                // descriptor, then the weight stream of the unit; a first-of-group unit also brings the group's constants
                unsigned char* st = stages + s * kStage;
                *reinterpret_cast<int4*>(st + kOffMeta) = make_int4(r.item, r.t, r.kb, r.flags);
                bar_arrive(&meta_bar[s]);
                const int N = GROUPED ? __ldg(&r.it->N) : item0.N;
                const int NW = N >> 3;
                const int words = min(kTileWordsM, NW - r.t * kTileWordsM);
                uint32_t bytes = kUnitBytes;
                if (r.flags & kFlagFirst) bytes += uint32_t(words) * 20u;
                bar_expect_tx(&full_bar[s], bytes);
                const CUtensorMap* map = GROUPED ? &r.it->tmap : &item0.tmap;
#pragma unroll
                for (int b = 0; b < 4; b++)
                    tma_box(st + b * kBoxBytes, map, r.t * kTileWordsM + b * kBoxWords, r.kb * kUnitRowsM, &full_bar[s]);
                if (r.flags & kFlagFirst) {
                    const uint32_t* qz = GROUPED ? r.it->qz : item0.qz;
                    const __half* sc = GROUPED ? r.it->scales : item0.scales;
                    const int grp = r.kb >> 2;
                    bulk_copy(st + kOffZero, qz + size_t(grp) * NW + r.t * kTileWordsM, uint32_t(words) * 4u, &full_bar[s]);
                    bulk_copy(st + kOffScale, sc + size_t(grp) * N + size_t(r.t) * kTileColsM, uint32_t(words) * 16u, &full_bar[s]);
                }
                if (first_issue) gemv_trace(8);
                gemv_trace(9);
            }
            first_issue = false;
            if (++s == STAGES) { s = 0; parity ^= 1u; }
            cur = nxt;
        }
        if (ok) {
            // end marker: a stage whose descriptor says "no unit"
            if (bar_wait_relaxed(&empty_bar[s], parity ^ 1u)) {
                if (lane == 0) {
                    *reinterpret_cast<int4*>(stages + s * kStage + kOffMeta) = make_int4(-1, 0, 0, 0);
                    bar_arrive(&meta_bar[s]);
                    bar_arrive(&full_bar[s]);
                }
            } else {
                atomicExch(&g_gemv_mma_wait_error, 3);
            }
        } else if (lane == 0) {
            // give copies already issued a bounded chance to land before the CTA goes away
            for (int q = 0; q < STAGES; q++) bar_wait(&full_bar[q], 0);
        }
        return;
    }

    if (warp == kWarpsC + 1) {
        // ------------------------------------------------------------ activation producer (one warp, lane = row of the unit)
        pdl_wait();  // x belongs to the previous kernel until here
        float rstd[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) rstd[m] = 1.f;
        bool have_rstd = !NORM;
        // raw operand rows of a unit (SwiGLU applied, norm not yet) and the norm weight of the lane's row
        auto fetch = [&](int item, int kblock, float (&v)[MT], float& wn) {
            const float* xp = GROUPED ? p.items[item].x : item0.x;
            const int K = GROUPED ? __ldg(&p.items[item].K) : item0.K;
            const int sw = GROUPED ? 0 : item0.swiglu;
#pragma unroll
            for (int m = 0; m < MT; m++) {
                if (sw) {
                    const float* gp = xp + size_t(m) * 2 * K + kblock * kUnitRowsM + lane;
                    const float gate = __ldcg(gp), up = __ldcg(gp + K);
                    v[m] = (gate / (1.0f + expf(-gate))) * up;
                } else {
                    v[m] = __ldcg(xp + size_t(m) * K + kblock * kUnitRowsM + lane);
                }
            }
            wn = NORM ? __uint_as_float(uint32_t(__ldg(item0.norm_w + kblock * kUnitRowsM + lane)) << 16) : 1.f;
        };
        int s = 0;
        uint32_t parity = 0;
        float cur[MT], nxt[MT], cur_w = 1.f, nxt_w = 1.f;
        bool have_cur = false, done = false, first_fill = true;
        while (!done) {
            if (!have_cur) {
                // the descriptor of this stage tells which rows of which operand it needs
                if (!bar_wait_relaxed(&meta_bar[s], parity)) {
                    atomicExch(&g_gemv_mma_wait_error, 4);
                    break;
                }
                const int4 meta = *reinterpret_cast<const int4*>(stages + s * kStage + kOffMeta);
                if (meta.x < 0) {
                    done = true;
                } else {
                    fetch(meta.x, meta.z, cur, cur_w);
                }
                if (first_fill && lane == 0) gemv_trace(6);
            }
            if (done) {
                if (lane == 0) bar_arrive(&full_bar[s]);  // second arrival of the end marker
                break;
            }
            // the unit after this one, if the weight producer is already past it: its rows are requested now
            int s1 = s + 1;
            uint32_t parity1 = parity;
            if (s1 == STAGES) { s1 = 0; parity1 ^= 1u; }
            bool have_next = false, next_is_end = false;
            if (bar_try(sm_u32(&meta_bar[s1]), parity1)) {
                const int4 meta = *reinterpret_cast<const int4*>(stages + s1 * kStage + kOffMeta);
                if (meta.x < 0) {
                    next_is_end = true;
                } else {
                    fetch(meta.x, meta.z, nxt, nxt_w);
                    have_next = true;
                }
            }
            if (!have_rstd) {
                norm_sync();  // the consumers' sum of squares; the first rows were requested before waiting for it
#pragma unroll
                for (int m = 0; m < MT; m++) rstd[m] = s_rstd[m];
                have_rstd = true;
            }
            unsigned char* xs = stages + s * kStage + kOffX;
            if (INT8) {
                // block scale of the unit: the largest magnitude lands in [2^13, 2^14)
                const float val = NORM ? (cur[0] * rstd[0]) * cur_w : cur[0];
                const float amax = warp_max(fabsf(val));
                const int ea = int((__float_as_uint(amax) >> 23) & 0xffu) - 127;  // floor(log2 amax); -127 for zero / subnormal
                int e = 13 - ea;
                e = e > 126 ? 126 : e;
                const float scale = __uint_as_float(uint32_t(127 + e) << 23);
                const float inv = __uint_as_float(uint32_t(127 - e) << 23);
                const int xi = __float2int_rn(val * scale);
                const int d0 = (xi << 24) >> 24;   // signed low byte
                const int d1 = (xi - d0) >> 8;     // signed high byte: xi = 256 d1 + d0
                int isum = xi;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) isum += __shfl_xor_sync(0xffffffffu, isum, o);
                // consumer lane (g, tig) of 8-row step st reads 8 bytes at ((st * 4 + tig) * 8 + g) * 8: the fragment
                // words of rows 8 st + 2 tig and 8 st + 2 tig + 1; column g = (byte position g >> 1, digit g & 1)
                const int st = lane >> 3, hi_row = lane & 1, tq = (lane >> 1) & 3;
                unsigned char* base = xs + ((st * 4 + tq) * 8) * 8 + 4 * hi_row;
#pragma unroll
                for (int gg = 0; gg < 8; gg++) {
                    const uint32_t dig = uint32_t((gg & 1) ? d1 : d0) & 0xffu;
                    *reinterpret_cast<uint32_t*>(base + gg * 8) = dig << (8 * (gg >> 1));
                }
                if (lane == 0) *reinterpret_cast<float2*>(xs + kXBytesInt8) = make_float2(inv, float(isum));
            } else {
#pragma unroll
            for (int m = 0; m < MT; m++) {
                const float val = NORM ? (cur[m] * rstd[m]) * cur_w : cur[m];
                const __half h = __float2half_rn(val);
                const uint32_t bits = __half_as_ushort(h);
                // column slot 2m carries x in the low half (first column of a pair), slot 2m+1 in the high half
                *reinterpret_cast<uint32_t*>(xs + (2 * m) * kXRowStride + lane * 4) = bits;
                *reinterpret_cast<uint32_t*>(xs + (2 * m + 1) * kXRowStride + lane * 4) = bits << 16;
                const float sum = warp_sum(__half2float(h));
                if (lane == 0) *reinterpret_cast<float*>(xs + (2 * MT + 1) * kXRowStride + m * 4) = sum;
            }
            }
            __syncwarp();
            if (lane == 0) bar_arrive(&full_bar[s]);
            if (first_fill && lane == 0) gemv_trace(7);
            first_fill = false;
            s = s1;
            parity = parity1;
            if (next_is_end) {
                if (lane == 0) bar_arrive(&full_bar[s]);  // second arrival of the end marker
                break;
            }
            have_cur = have_next;
#pragma unroll
            for (int m = 0; m < MT; m++) cur[m] = nxt[m];
            cur_w = nxt_w;
        }
        if (!have_rstd) norm_sync();  // a CTA without units still meets the consumers at the barrier
        return;
    }

    // ---------------------------------------------------------------- consumers
    const int g = lane >> 2, tig = lane & 3;
    pdl_wait();  // y, the workspace and (for the norm) x belong to the previous kernel until here
    if (tid == 0) gemv_trace(2);

    if (NORM) {
        // sum of squares of the whole input row, by all consumer threads, 4 x 16-byte loads in flight each
#pragma unroll
        for (int m = 0; m < MT; m++) {
            const float4* hp = reinterpret_cast<const float4*>(item0.x + size_t(m) * item0.K);
            const int n4 = item0.K >> 2;
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
            s_rstd[tid] = 1.0f / sqrtf(tot / float(item0.K) + item0.eps);
        }
        norm_sync();
    }

    if constexpr (INT8) {
        // This warp: word columns 16*warp .. 16*warp+15 of the tile = two blocks of 8 (cb = 2*warp, 2*warp+1) in TMA box
        // warp>>1.  Lane (g, tig) reads word g of the block in rows 2 tig and 2 tig + 1 of each 8-row step (the 128-byte
        // swizzle XORs the 16-byte chunk index with row & 7, which spreads the 32 lanes over all banks).  The first
        // half of the contraction index (k < 16) therefore stands for the even rows of the step, the second for the odd ones.
        uint32_t offA[2], offB[2];
#pragma unroll
        for (int cbi = 0; cbi < 2; cbi++) {
            const int cbl = 2 * (warp & 1) + cbi;
            const int chunk = 2 * cbl + (g >> 2);
            offA[cbi] = uint32_t((warp >> 1) * kBoxBytes + (2 * tig) * 128 + ((chunk ^ (2 * tig)) << 4) + (g & 3) * 4);
            offB[cbi] = uint32_t((warp >> 1) * kBoxBytes + (2 * tig + 1) * 128 + ((chunk ^ (2 * tig + 1)) << 4) + (g & 3) * 4);
        }
        const uint32_t xoff8 = uint32_t(kOffX + tig * 64 + g * 8);
        const uint32_t inv_off = uint32_t(kOffX + kXBytesInt8);
        // The lane's results: byte position tig of the low-nibble bytes is nibble 2 tig = column ord[2 tig] of the word,
        // of the high-nibble bytes nibble 2 tig + 1 = column ord[2 tig + 1], ord = {0,2,4,6,1,3,5,7}.
        const int c_lo = (tig < 2) ? 4 * tig : 4 * tig - 7;        // 0, 4, 1, 5
        const int c_hi = c_lo + 2;                                  // 2, 6, 3, 7
        const uint32_t zoff = uint32_t(kOffZero + (2 * warp * 8 + g) * 4);
        const uint32_t soff = uint32_t(kOffScale + (2 * warp * 8 + g) * 16);
        float* y = item0.y;
        int N = item0.N;
        int cur_item = GROUPED ? -1 : 0;
        float zf[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, sf[2][2] = {{0.f, 0.f}, {0.f, 0.f}};  // [block][low / high nibble column]
        float accf[2][2] = {{0.f, 0.f}, {0.f, 0.f}};   // sums of the current group, in units of x
        float acc_t[2][2] = {{0.f, 0.f}, {0.f, 0.f}};  // scaled total of the current tile
        float gsum = 0.f;                               // sum of the activations over the rows of the current group seen so far
        int acc[2][4];
#pragma unroll
        for (int cbi = 0; cbi < 2; cbi++) { acc[cbi][0] = acc[cbi][1] = acc[cbi][2] = acc[cbi][3] = 0; }

        const uint32_t stage0 = sm_u32(stages);
        const uint32_t full0 = sm_u32(&full_bar[0]), empty0 = sm_u32(&empty_bar[0]);
        uint32_t sbase = stage0, fbar = full0, ebar = empty0;
        int s = 0;
        uint32_t parity = 0;
        bool first_unit = true;
        while (true) {
            if (!bar_try(fbar, parity) && !bar_wait_addr(fbar, parity)) {
                atomicExch(&g_gemv_mma_wait_error, 2);
                break;  // the result is void; the host sees the error word
            }
            // two halves of 16 rows; all loads of the first half are issued before the descriptor is looked at
            const uint32_t a0 = sbase + offA[0], b0 = sbase + offB[0], a1 = sbase + offA[1], b1 = sbase + offB[1];
            const uint32_t xbase = sbase + xoff8;
            uint32_t wA[2][2], wB[2][2];
            uint2 xb[2];
            auto math = [&]() {
#pragma unroll
                for (int st = 0; st < 2; st++) {
#pragma unroll
                    for (int cbi = 0; cbi < 2; cbi++) {
                        const uint32_t a = wA[cbi][st], b = wB[cbi][st];
                        // fragment rows g / g+8 = low / high nibbles of word g; contraction halves = weight rows 2 tig / 2 tig + 1
                        mma_u8s8(acc[cbi], a & 0x0f0f0f0fu, a & 0xf0f0f0f0u, b & 0x0f0f0f0fu, b & 0xf0f0f0f0u, xb[st].x, xb[st].y);
                    }
                }
            };
            wA[0][0] = lds32<0>(a0);    wB[0][0] = lds32<0>(b0);    wA[1][0] = lds32<0>(a1);    wB[1][0] = lds32<0>(b1);
            wA[0][1] = lds32<1024>(a0); wB[0][1] = lds32<1024>(b0); wA[1][1] = lds32<1024>(a1); wB[1][1] = lds32<1024>(b1);
            xb[0] = lds64<0>(xbase);
            xb[1] = lds64<256>(xbase);
            const uint2 unit_consts = lds64<0>(sbase + inv_off);  // 1 / scale, sum of the unit's integer activations
            const uint4 meta = lds128(sbase + kOffMeta);
            if (int(meta.x) < 0) break;  // end marker
            if (first_unit && tid == 0) gemv_trace(3);
            first_unit = false;
            const int t = int(meta.y);
            int kb = int(meta.z);
            const int flags = int(meta.w);
            if (GROUPED && int(meta.x) != cur_item) {
                cur_item = int(meta.x);
                y = p.items[cur_item].y;
                N = __ldg(&p.items[cur_item].N);
            }
            if (flags & kFlagFirst) {
#pragma unroll
                for (int cbi = 0; cbi < 2; cbi++) {
                    const uint32_t zw = cbi ? lds32<32>(sbase + zoff) : lds32<0>(sbase + zoff);
                    zf[cbi][0] = float((zw >> (8 * tig)) & 0xfu);
                    zf[cbi][1] = float((zw >> (8 * tig + 4)) & 0xfu);
                    sf[cbi][0] = lds_f16(sbase + soff + cbi * 128 + c_lo * 2);
                    sf[cbi][1] = lds_f16(sbase + soff + cbi * 128 + c_hi * 2);
                }
            }
            math();
            wA[0][0] = lds32<2048>(a0); wB[0][0] = lds32<2048>(b0); wA[1][0] = lds32<2048>(a1); wB[1][0] = lds32<2048>(b1);
            wA[0][1] = lds32<3072>(a0); wB[0][1] = lds32<3072>(b0); wA[1][1] = lds32<3072>(a1); wB[1][1] = lds32<3072>(b1);
            xb[0] = lds64<512>(xbase);
            xb[1] = lds64<768>(xbase);
            __syncwarp();
            if (lane == 0) bar_arrive_addr(ebar);  // the stage is in registers now
            if (++s == STAGES) {
                s = 0; parity ^= 1u; sbase = stage0; fbar = full0; ebar = empty0;
            } else {
                sbase += kStage; fbar += 8; ebar += 8;
            }
            kb++;
            math();
            // ---- unit done: the two digit sums become one exact integer, scaled back to units of x
            const float inv = __uint_as_float(unit_consts.x);
#pragma unroll
            for (int cbi = 0; cbi < 2; cbi++) {
                const int lo = acc[cbi][0] + (acc[cbi][1] << 8);
                const int hi = (acc[cbi][2] + (acc[cbi][3] << 8)) >> 4;  // the high-nibble bytes are 16 q: exact shift
                accf[cbi][0] = fmaf(float(lo), inv, accf[cbi][0]);
                accf[cbi][1] = fmaf(float(hi), inv, accf[cbi][1]);
                acc[cbi][0] = acc[cbi][1] = acc[cbi][2] = acc[cbi][3] = 0;
            }
            gsum = fmaf(__uint_as_float(unit_consts.y), inv, gsum);
            const bool last = (flags & kFlagLast) != 0;
            if ((kb & 3) != 0 && !last) continue;

            // ---- group done (or the run ends inside it): take the zero point back out, apply the fp16 scales
#pragma unroll
            for (int cbi = 0; cbi < 2; cbi++) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    acc_t[cbi][h] = fmaf(fmaf(-zf[cbi][h], gsum, accf[cbi][h]), sf[cbi][h], acc_t[cbi][h]);
                    accf[cbi][h] = 0.f;
                }
            }
            gsum = 0.f;
            if (!last) continue;

            // ---- this CTA's contribution to column tile t is complete.  Lane (g, tig) holds columns c_lo, c_hi of words
            // 16 warp + g and 16 warp + 8 + g; lanes tig and tig ^ 2 hold the other two columns of the same quartet
            // (tig 0: 0,2 / tig 2: 1,3 / tig 1: 4,6 / tig 3: 5,7), so after one exchange every lane owns four consecutive
            // columns of one word: tig < 2 of block 0, tig >= 2 of block 1.
            {
                const bool upper = tig >= 2;
                const float send0 = upper ? acc_t[0][0] : acc_t[1][0], send1 = upper ? acc_t[0][1] : acc_t[1][1];
                const float recv0 = __shfl_xor_sync(0xffffffffu, send0, 2), recv1 = __shfl_xor_sync(0xffffffffu, send1, 2);
                const float own0 = upper ? acc_t[1][0] : acc_t[0][0], own1 = upper ? acc_t[1][1] : acc_t[0][1];
                // ascending columns: the lane with the even pair (tig < 2) has columns q+0, q+2; its partner q+1, q+3
                const float4 v = upper ? make_float4(recv0, own0, recv1, own1) : make_float4(own0, recv0, own1, recv1);
                const int word = (2 * warp + (upper ? 1 : 0)) * 8 + g;
                const int col_in_tile = word * 8 + ((tig & 1) ? 4 : 0);
                const int col = t * kTileColsM + col_in_tile;
                if (ACCUM) {
                    if (col < N)
                        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(y + col), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                                     : "memory");
                } else {
                    *reinterpret_cast<float4*>(red + col_in_tile) = v;
                }
            }
            if (!ACCUM) {
                consumers_sync();
                // thread f owns float4 f of the tile (columns 4f .. 4f+3)
                const int f = tid;
                const int col = t * kTileColsM + f * 4;
                float4 v = *reinterpret_cast<const float4*>(red + f * 4);
                const long long first_u = (long long)t * item0.upt, last_u = first_u + item0.upt - 1;
                const int c_first = int(((first_u + 1) * C - 1) / p.U);
                const int c_last = int(((last_u + 1) * C - 1) / p.U);
                const int n_contrib = c_last - c_first + 1;
                bool finish = true;
                if (n_contrib > 1) {
                    *reinterpret_cast<float4*>(p.partial + size_t(blockIdx.x + t) * kTileColsM + f * 4) = v;
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
                        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                        const float* base = p.partial + size_t(t) * kTileColsM + f * 4;
                        int c = c_first;
                        for (; c + 8 <= c_last + 1; c += 8) {
                            float4 a[8];
#pragma unroll
                            for (int q = 0; q < 8; q++) a[q] = __ldcg(reinterpret_cast<const float4*>(base + size_t(c + q) * kTileColsM));
#pragma unroll
                            for (int q = 0; q < 8; q++) { sum.x += a[q].x; sum.y += a[q].y; sum.z += a[q].z; sum.w += a[q].w; }
                        }
                        for (; c <= c_last; c++) {
                            const float4 a = __ldcg(reinterpret_cast<const float4*>(base + size_t(c) * kTileColsM));
                            sum.x += a.x; sum.y += a.y; sum.z += a.z; sum.w += a.w;
                        }
                        v = sum;
                    }
                }
                if (finish && col < N) {
                    if (p.residual) {
                        const float4 r = __ldcg(reinterpret_cast<const float4*>(p.residual + col));
                        v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w;
                    }
                    *reinterpret_cast<float4*>(y + col) = v;
                }
                consumers_sync();  // red is reused by the next tile
            }
#pragma unroll
            for (int cbi = 0; cbi < 2; cbi++) { acc_t[cbi][0] = 0.f; acc_t[cbi][1] = 0.f; }
            if (tid == 0) gemv_trace(4);
        }
        if (tid == 0) gemv_trace(5);
        return;
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
    const uint32_t xoff = uint32_t(kOffX + (g < 2 * MT ? g : 2 * MT) * kXRowStride + 2 * tig * 4);
    const bool owner = tig < MT;            // lanes whose accumulator columns are real: token row = tig
    const uint32_t sum_off = uint32_t(kOffX + (2 * MT + 1) * kXRowStride + (owner ? tig : 0) * 4);
    // zero word and eight fp16 scales of this lane's word column of block 0 (block 1: eight word columns further)
    const uint32_t zoff = uint32_t(kOffZero + (2 * warp * 8 + g) * 4);
    const uint32_t soff = uint32_t(kOffScale + (2 * warp * 8 + g) * 16);

    // what the current tile belongs to (grouped calls switch between items)
    float* y = item0.y;
    int N = item0.N;
    int cur_item = GROUPED ? -1 : 0;

    uint32_t z_cur[2] = {0u, 0u};
    uint4 s_cur[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
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

    const uint32_t stage0 = sm_u32(stages);
    const uint32_t full0 = sm_u32(&full_bar[0]), empty0 = sm_u32(&empty_bar[0]);
    uint32_t sbase = stage0, fbar = full0, ebar = empty0;
    int s = 0;
    uint32_t parity = 0;
    bool first_unit = true;
    while (true) {
        if (!bar_try(fbar, parity) && !bar_wait_addr(fbar, parity)) {
            atomicExch(&g_gemv_mma_wait_error, 2);
            break;  // the result is void; the host sees the error word
        }
        // the unit is taken in two halves of 16 rows so that only half of it is live in registers at a time;
        // the stage is released after the second half has been read.  All loads of the first half are issued before
        // the descriptor is looked at (for the end marker they read stale bytes that nobody uses).
        const uint32_t a00 = sbase + off0[0], a10 = sbase + off1[0], a01 = sbase + off0[1], a11 = sbase + off1[1];
        const uint32_t xbase = sbase + xoff;
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
        const float unit_sum = __uint_as_float(lds32<0>(sbase + sum_off));
        const uint4 meta = lds128(sbase + kOffMeta);
        if (int(meta.x) < 0) break;  // end marker
        if (first_unit && tid == 0) gemv_trace(3);
        first_unit = false;
        const int t = int(meta.y);
        int kb = int(meta.z);
        const int flags = int(meta.w);
        if (GROUPED && int(meta.x) != cur_item) {
            cur_item = int(meta.x);
            y = p.items[cur_item].y;
            N = __ldg(&p.items[cur_item].N);
        }
        if (flags & kFlagFirst) {
            z_cur[0] = lds32<0>(sbase + zoff);
            z_cur[1] = lds32<32>(sbase + zoff);
            s_cur[0] = lds128(sbase + soff);
            s_cur[1] = lds128(sbase + soff + 128);
        }
        gsum += owner ? unit_sum : 0.f;
        math();
        w0[0][0] = lds32<2048>(a00); w1[0][0] = lds32<2048>(a10); w0[1][0] = lds32<2048>(a01); w1[1][0] = lds32<2048>(a11);
        w0[0][1] = lds32<3072>(a00); w1[0][1] = lds32<3072>(a10); w0[1][1] = lds32<3072>(a01); w1[1][1] = lds32<3072>(a11);
        xb[0] = lds64<64>(xbase);
        xb[1] = lds64<96>(xbase);
        __syncwarp();
        if (lane == 0) bar_arrive_addr(ebar);  // the stage is in registers now
        if (++s == STAGES) {
            s = 0; parity ^= 1u; sbase = stage0; fbar = full0; ebar = empty0;
        } else {
            sbase += kStage; fbar += 8; ebar += 8;
        }
        kb++;
        math();
        const bool last = (flags & kFlagLast) != 0;
        if ((kb & 3) != 0 && !last) continue;

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
        if (!last) continue;

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
                    if (col < N) {
                        float* yp = y + size_t(tig) * N + col;
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
            // contributors of this tile: CTAs owning its first and last unit (the ordered mode deals every unit statically)
            const long long first_u = (long long)t * item0.upt, last_u = first_u + item0.upt - 1;
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
            if (finish && col < N) {
#pragma unroll
                for (int m = 0; m < MT; m++) {
                    if (p.residual) {
                        const float4 r = __ldcg(reinterpret_cast<const float4*>(p.residual + size_t(m) * N + col));
                        v[m].x += r.x; v[m].y += r.y; v[m].z += r.z; v[m].w += r.w;
                    }
                    *reinterpret_cast<float4*>(y + size_t(m) * N + col) = v[m];
                }
            }
            consumers_sync();  // red is reused by the next tile
        }
#pragma unroll
        for (int cbi = 0; cbi < 2; cbi++)
#pragma unroll
            for (int i = 0; i < 8; i++) acc_t[cbi][i] = 0.f;
        if (tid == 0) gemv_trace(4);
    }
    if (tid == 0) gemv_trace(5);
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

// Share of the units handed out through tickets when the caller provides counters (tuning key "gemv_dyn_pct").  Off by
// default: inside a chain of dependent launches the early finishers of a static deal are what lets the next launch's
// CTAs start their weight stream early, and a ticketed tail (measured at 10 - 60 % on the Qwen3-8B shapes) took that
// away without finishing sooner; it pays for a launch that nothing follows closely.
int g_dyn_pct = 0;
int g_dyn_chunk = 0;   // 128-row groups per ticket; 0: one (tuning key "gemv_dyn_chunk")
// One-row integer-operand launches in accumulate mode: a matrix of at least g_int8_ctas3_units units runs three CTAs
// per SM (consumers held to 64 registers: more loads in flight, 4096 x 24576 goes from 11.7 to 10.5 us), a smaller one
// two CTAs per SM of the 96-register build (4096 x 4096: 3.6 us against 3.9).  Tuning keys "gemv_ctas" (2 switches the
// three-CTA build off) and "gemv_ctas3_units".
int g_int8_ctas = kCtasPerSmInt8;
int g_int8_ctas3_units = 1024;

template <int MT, int STAGES, bool ACCUM, bool NORM, bool GROUPED, bool INT8 = false, int OCC = kCtasPerSmMma>
int launch_mma(const GemvItem& item, const GemvCall& call, int ctas, cudaStream_t stream) {
    auto kern = awq_gemv_mma_kernel<MT, STAGES, ACCUM, NORM, GROUPED, INT8, OCC>;
    const size_t smem = 1024 + size_t(STAGES) * stage_bytes(MT, INT8) + (ACCUM ? 0 : size_t(MT) * kTileColsM * sizeof(float));
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
    cudaError_t err = cudaLaunchKernelEx(&cfg, kern, item, call);
    if (err != cudaSuccess) {
        set_error("awq_gemv_mma launch failed: %s", cudaGetErrorString(err));
        return KUIPER_INTERNAL_ERROR;
    }
    return KUIPER_OK;
}

template <bool ACCUM, bool NORM>
int launch_mma_rows(int rows, const GemvItem& item, const GemvCall& call, int ctas, cudaStream_t stream) {
    switch (rows) {
        case 1: return launch_mma<1, kStagesM, ACCUM, NORM, false>(item, call, ctas, stream);
        case 2: return launch_mma<2, kStagesM, ACCUM, NORM, false>(item, call, ctas, stream);
        case 3: return launch_mma<3, kStagesM, ACCUM, NORM, false>(item, call, ctas, stream);
        default: return launch_mma<4, kStagesM, ACCUM, NORM, false>(item, call, ctas, stream);
    }
}

bool fill_item(GemvItem& it, const float* x, const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales, float* y,
               int K, int N, const uint16_t* norm_w, float eps, bool swiglu, int unit0) {
    memset(&it, 0, sizeof(it));
    if (!get_map_mma(qweight, K, N, &it.tmap)) return false;
    it.x = x;
    it.y = y;
    it.qz = reinterpret_cast<const uint32_t*>(qzeros);
    it.scales = reinterpret_cast<const __half*>(scales);
    it.norm_w = norm_w;
    it.eps = eps;
    it.swiglu = swiglu ? 1 : 0;
    it.K = K;
    it.N = N;
    it.tiles = (N + kTileColsM - 1) / kTileColsM;
    it.upt = K / kUnitRowsM;
    it.unit0 = unit0;
    return true;
}

// Splits the U units of a call into the statically dealt part and the ticketed tail.  A ticket is one 128-row group
// of one column tile (4 units; every tile is a whole number of groups), so a ticketed chunk costs one set of group
// constants and one flush of its tile, like a group inside a static run.
void plan_tickets(GemvCall& call, int ctas, int* tickets) {
    call.U_static = call.U;
    call.chunk = 4;
    call.n_chunks = 0;
    call.tickets = nullptr;
    if (tickets == nullptr || g_dyn_pct <= 0 || call.U < 4 * ctas) return;
    const int chunk = g_dyn_chunk > 0 ? 4 * g_dyn_chunk : 4;
    long long dyn = (long long)call.U * (g_dyn_pct > 90 ? 90 : g_dyn_pct) / 100;
    dyn -= dyn % chunk;
    if (dyn <= 0) return;
    // the tail starts at a group boundary: U is a multiple of 4 and so is dyn
    call.U_static = call.U - int(dyn);
    call.chunk = chunk;
    call.n_chunks = int(dyn / chunk);
    call.tickets = tickets;
}

}  // namespace

#ifdef KUIPER_TRACE
int awq_gemv_trace_read(long long* out, int max_values) {
    const int n = max_values < kGemvTraceCtas * kGemvTraceSlots ? max_values : kGemvTraceCtas * kGemvTraceSlots;
    return cudaMemcpyFromSymbol(out, g_gemv_trace, size_t(n) * sizeof(long long)) == cudaSuccess ? n : -1;
}
#endif

void awq_gemv_mma_set_tuning(const char* key, int value) {
    if (!strcmp(key, "gemv_dyn_pct")) g_dyn_pct = value < 0 ? 0 : value;
    if (!strcmp(key, "gemv_dyn_chunk")) g_dyn_chunk = value < 0 ? 0 : value;
    if (!strcmp(key, "gemv_ctas3_units")) g_int8_ctas3_units = value < 1 ? 1 : value;
    if (!strcmp(key, "gemv_ctas")) g_int8_ctas = value >= kCtasPerSmInt8 ? kCtasPerSmInt8 : kCtasPerSmMma;
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
// tickets (accumulate mode): two zero-initialised ints owned by this call site, or null for a fully static deal.
// int_operand: a one-row launch rounds its operand to block-scaled 16-bit integers (INT8 kernel) instead of fp16.
int awq_gemv_mma_launch(const float* x, const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales, float* y,
                        const float* residual, int rows, int K, int N, void* workspace, bool accumulate,
                        const uint16_t* norm_w, float eps, bool swiglu, int* tickets, bool int_operand, cudaStream_t stream) {
    if (rows < 1 || rows > awq_gemv_mma_max_rows(accumulate)) {
        set_error("awq_gemv_mma: %d token rows in one launch", rows);
        return KUIPER_INVALID_ARGUMENT;
    }
    GemvItem item;
    if (!fill_item(item, x, qweight, qzeros, scales, y, K, N, norm_w, eps, swiglu, 0)) {
        set_error("awq_gemv_mma: tensor map encoding failed");
        return KUIPER_INTERNAL_ERROR;
    }
    GemvCall call;
    memset(&call, 0, sizeof(call));
    call.n_items = 1;
    call.U = item.tiles * item.upt;
    call.residual = residual;
    const size_t head = ((size_t(item.tiles) + 1) * sizeof(int) + 255) / 256 * 256;
    if (!accumulate && workspace == nullptr) {
        set_error("awq_gemv_mma: the ordered combine needs a workspace");
        return KUIPER_INVALID_ARGUMENT;
    }
    call.counters = reinterpret_cast<int*>(workspace);
    call.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + head);
    const bool three = int_operand && rows == 1 && accumulate && g_int8_ctas == kCtasPerSmInt8 && call.U >= g_int8_ctas3_units;
    long long ctas = (long long)device_sm_count() * (three ? kCtasPerSmInt8 : kCtasPerSmMma);
    if (ctas > call.U) ctas = call.U;
    if ((norm_w || swiglu) && !accumulate) {
        set_error("awq_gemv_mma: the fused input norm / SwiGLU exist in accumulate mode only");
        return KUIPER_INVALID_ARGUMENT;
    }
    plan_tickets(call, int(ctas), accumulate ? tickets : nullptr);
    if (int_operand && rows == 1) {
        if (accumulate && three) {
            if (norm_w) return launch_mma<1, kStagesM, true, true, false, true, kCtasPerSmInt8>(item, call, int(ctas), stream);
            return launch_mma<1, kStagesM, true, false, false, true, kCtasPerSmInt8>(item, call, int(ctas), stream);
        }
        if (accumulate && norm_w) return launch_mma<1, kStagesM, true, true, false, true>(item, call, int(ctas), stream);
        if (accumulate) return launch_mma<1, kStagesM, true, false, false, true>(item, call, int(ctas), stream);
        return launch_mma<1, kStagesM, false, false, false, true>(item, call, int(ctas), stream);
    }
    if (accumulate && norm_w) return launch_mma_rows<true, true>(rows, item, call, int(ctas), stream);
    if (accumulate) return launch_mma_rows<true, false>(rows, item, call, int(ctas), stream);
    if (rows == 2) return launch_mma<2, kStagesM, false, false, false>(item, call, int(ctas), stream);
    return launch_mma<1, kStagesM, false, false, false>(item, call, int(ctas), stream);
}

// ---- grouped call: a list of independent one-row accumulate-mode projections in one persistent launch
size_t awq_gemv_group_table_bytes(int n_items) { return n_items > 0 ? size_t(n_items) * sizeof(GemvItem) : 0; }

// Fills `host_table` (awq_gemv_group_table_bytes(n) bytes of host memory) with the table the kernel reads; the
// caller copies it to 64-byte aligned device memory.  Returns the number of units of the call, or -1.
long long awq_gemv_group_fill(const kuiper_gemv_item* items, int n_items, void* host_table) {
    GemvItem* table = reinterpret_cast<GemvItem*>(host_table);
    long long unit0 = 0;
    for (int i = 0; i < n_items; i++) {
        const kuiper_gemv_item& o = items[i];
        if (unit0 > 0x3fffffff) return -1;
        GemvItem it;
        if (!fill_item(it, o.x, o.qweight, o.qzeros, o.scales, o.y, o.K, o.N, nullptr, 0.f, false, int(unit0))) return -1;
        memcpy(&table[i], &it, sizeof(it));
        unit0 += (long long)it.tiles * it.upt;
    }
    return unit0 > 0x3fffffff ? -1 : unit0;
}

int awq_gemv_group_launch(const void* device_table, int n_items, long long units, int* tickets, bool int_operand,
                          cudaStream_t stream) {
    GemvItem none;
    memset(&none, 0, sizeof(none));
    GemvCall call;
    memset(&call, 0, sizeof(call));
    call.items = reinterpret_cast<const GemvItem*>(device_table);
    call.n_items = n_items;
    call.U = int(units);
    const bool three = int_operand && g_int8_ctas == kCtasPerSmInt8 && call.U >= g_int8_ctas3_units;
    long long ctas = (long long)device_sm_count() * (three ? kCtasPerSmInt8 : kCtasPerSmMma);
    if (ctas > call.U) ctas = call.U;
    plan_tickets(call, int(ctas), tickets);
    if (three) return launch_mma<1, kStagesM, true, false, true, true, kCtasPerSmInt8>(none, call, int(ctas), stream);
    if (int_operand) return launch_mma<1, kStagesM, true, false, true, true>(none, call, int(ctas), stream);
    return launch_mma<1, kStagesM, true, false, true>(none, call, int(ctas), stream);
}

}  // namespace kuiper
