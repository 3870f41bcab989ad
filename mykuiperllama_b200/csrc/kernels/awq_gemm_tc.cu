// INT4-AWQ GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) for M >= 16 token rows:
// prefill chunks and batched decode, where the operation is a dense contraction.
// Same placeholder as the GEMV: kuiper/include/op/matmul.h:1-11 of the reference.
//
// y[M,N] (+)= x[M,K] . dequant(qweight)[K,N]
//
// One CTA owns a 128 x 256 output tile; its fp32 accumulator lives in tensor memory (128 lanes x 256
// columns), two CTAs share an SM.  The activations are converted to fp16 once per call (the same operand
// rounding as the GEMV) and reach shared memory with cp.async; every thread dequantises one packed word
// column and one K octet of the weight tile: the nibble pairs come out of the LOP3 / 0x6400 trick exactly
// as in the GEMV, the fp16 group scale is applied, and register transposes (PRMT) turn "two columns of one
// row" into "two rows of one column", so that each column's eight K values are one 16-byte shared-memory
// store.  Both operands are stored K-major with the 128-byte swizzle: a tile row is the 64 K values (128
// bytes) of one token row / weight column, eight rows form a 1024-byte atom, and the 16-byte chunk c of row
// r sits at chunk position c ^ (r % 8).  One thread issues four tcgen05.mma (K = 16 each) per stage and a
// tcgen05.commit onto the stage's mbarrier; a stage is refilled only after that commit.  In the default kernel
// (awq_gemm_tc3_kernel) that thread belongs to a warp of its own and learns through a second mbarrier that the
// producer warps have filled the stage; awq_gemm_tc2_kernel hands the stage over at a block-wide barrier.  The
// epilogue reads the accumulator with tcgen05.ld (one TMEM lane = one output row per thread).
//
// Every mbarrier wait is bounded; on a timeout the CTA records an error word, stops issuing work,
// still frees its tensor memory and returns.
#include <cstring>

#include "common.cuh"

namespace kuiper {
namespace {

constexpr int kBM = 128, kBK = 64;
constexpr int kGemmThreads = 256;
constexpr uint32_t kMagicTc = 0x64006400u;
constexpr uint32_t kSpinLimitTc = 1u << 22;

__device__ int g_gemm_wait_error = 0;

constexpr uint32_t kDescLayoutSw128 = 2;  // layout field of the matrix descriptor: 128-byte swizzle
constexpr uint32_t kDescVersion = 1;

struct GemmParams {
    const float* x;        // [M, K]
    const uint32_t* qw;    // [K, N/8]
    const uint32_t* qz;    // [K/128, N/8]
    const __half* scales;  // [K/128, N]
    float* y;              // [M, N]
    const float* residual; // mode 1
    int M, K, N;
    int mode;              // 0: y = acc, 1: y = acc + residual, 2: y += acc
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ __half2 tc_u2h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ uint32_t tc_h22u(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }

__device__ __forceinline__ bool tc_mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_addr(bar);
    for (uint32_t spin = 0; spin < kSpinLimitTc; spin++) {
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

// 64-bit shared-memory matrix descriptor: start address, leading / stride byte offsets (all >> 4),
// descriptor version, swizzle mode
// K-major, 128-byte swizzle: 8-row atoms are 1024 B apart; the leading offset is unused because one
// atom spans the whole K tile
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= uint64_t((saddr >> 4) & 0x3fffu);
    d |= uint64_t((1024u >> 4) & 0x3fffu) << 32;
    d |= uint64_t(kDescVersion) << 46;
    d |= uint64_t(kDescLayoutSw128) << 61;
    return d;
}

struct TileConsts {
    __half2 z0, z1, z2, z3;  // (1024 + z) pairs for the low nibbles, -(64 + z) pairs for the high nibbles
    __half2 s0, s1, s2, s3;  // fp16 scales of column pairs (0,1) (2,3) (4,5) (6,7)
};
__device__ __forceinline__ TileConsts make_tile_consts(uint32_t zw, const uint4& sraw) {
    const __half2 neg_sixteenth = __floats2half2_rn(-0.0625f, -0.0625f);
    const uint32_t z8 = zw >> 8;
    TileConsts c;
    c.z0 = tc_u2h2((zw & 0x000f000fu) | kMagicTc);
    c.z1 = __hmul2(tc_u2h2((zw & 0x00f000f0u) | kMagicTc), neg_sixteenth);
    c.z2 = tc_u2h2((z8 & 0x000f000fu) | kMagicTc);
    c.z3 = __hmul2(tc_u2h2((z8 & 0x00f000f0u) | kMagicTc), neg_sixteenth);
    c.s0 = tc_u2h2(sraw.x); c.s1 = tc_u2h2(sraw.y); c.s2 = tc_u2h2(sraw.z); c.s3 = tc_u2h2(sraw.w);
    return c;
}
__device__ __forceinline__ void dequant_word_consts(uint32_t w, const TileConsts& c, uint32_t (&out)[4]) {
    const __half2 sixteenth = __floats2half2_rn(0.0625f, 0.0625f);
    const uint32_t w8 = w >> 8;
    out[0] = tc_h22u(__hmul2(__hsub2(tc_u2h2((w & 0x000f000fu) | kMagicTc), c.z0), c.s0));
    out[1] = tc_h22u(__hmul2(__hfma2(tc_u2h2((w & 0x00f000f0u) | kMagicTc), sixteenth, c.z1), c.s1));
    out[2] = tc_h22u(__hmul2(__hsub2(tc_u2h2((w8 & 0x000f000fu) | kMagicTc), c.z2), c.s2));
    out[3] = tc_h22u(__hmul2(__hfma2(tc_u2h2((w8 & 0x00f000f0u) | kMagicTc), sixteenth, c.z3), c.s3));
}

// ---------------------------------------------------------------------------------------------
// Second generation: 128 x 256 tiles, two CTAs per SM, no global-memory latency on the critical path.
//   * the activations are converted to fp16 once per call (convert_f16_kernel) and reach shared memory with
//     cp.async, 16 bytes per (row, K octet), straight into their swizzled position, one tile ahead;
//   * the packed weights of the next tile are already in registers while the current tile is dequantised;
//   * a stage is reused only after the tcgen05.commit of the MMAs that read it; two stages of 48 KB, so that two
//     CTAs share an SM and one's dequantisation overlaps the other's MMAs.
constexpr int kBN2 = 256;
constexpr int kStages2 = 2;   // 96 KB per CTA: two CTAs (16 warps, 2 x 256 TMEM columns) share an SM
constexpr int kStageA2 = kBM * kBK * 2;   // 16 KB
constexpr int kStageB2 = kBN2 * kBK * 2;  // 32 KB

// x -> fp16 copy; optionally zeroes the output of a split-K call (zero4 float4s), so that the zeroing is a kernel of
// the programmatic-dependent-launch chain like everything else (the GEMM's dependency wait covers it)
__global__ void convert_f16_kernel(const float4* __restrict__ x, uint2* __restrict__ out, int64_t n4, float4* __restrict__ zero,
                                   int64_t zero4) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 v = __ldcg(x + i);
        out[i] = make_uint2(tc_h22u(__floats2half2_rn(v.x, v.y)), tc_h22u(__floats2half2_rn(v.z, v.w)));
    }
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < zero4; i += stride) zero[i] = make_float4(0.f, 0.f, 0.f, 0.f);
}

struct GemmParams2 {
    GemmParams g;
    const __half* x16;  // [M, K] fp16 copy of x
    int tiles_per_split; // third generation: 64-row K tiles of one CTA (grid.z CTAs share an output tile); 0 = all of K
};

__global__ void __launch_bounds__(kGemmThreads, 2) awq_gemm_tc2_kernel(const GemmParams2 pp) {
    const GemmParams& p = pp.g;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    unsigned char* sA = smem;                          // kStages2 x 16 KB
    unsigned char* sB = smem + kStages2 * kStageA2;    // kStages2 x 32 KB
    __shared__ uint64_t mma_bar[kStages2];
    __shared__ uint32_t s_tmem;
    __shared__ int s_dead;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * kBN2, m0 = blockIdx.y * kBM;
    const int NW = p.N >> 3;

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < kStages2; i++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&mma_bar[i])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_dead = 0;
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&s_tmem)), "r"(uint32_t(kBN2))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    pdl_launch_dependents();
    pdl_wait();

    const uint32_t idesc = (1u << 4) | (uint32_t(kBN2 >> 3) << 17) | (uint32_t(kBM >> 4) << 24);
    const int nk = p.K / kBK;
    bool dead = false;

    // ---- this thread's share of a tile; everything that does not depend on the tile is computed here
    // activations: four 16-byte chunks (row m, K octet koct), global fp16 -> swizzled shared memory
    const __half* a_src[4];
    uint32_t a_dst[4], a_bytes[4];
#pragma unroll
    for (int q = 0; q < 4; q++) {
        const int item = q * kGemmThreads + tid;
        const int koct = item & 7, m = item >> 3;
        const bool ok = m0 + m < p.M;
        a_src[q] = pp.x16 + size_t(ok ? m0 + m : 0) * p.K + koct * 8;
        a_dst[q] = smem_addr(sA) + (m >> 3) * 1024 + (m & 7) * 128 + ((koct ^ (m & 7)) << 4);
        a_bytes[q] = ok ? 16u : 0u;  // 0: the chunk is zero filled
    }
    auto issue_a = [&](int tile, int stage) {
#pragma unroll
        for (int q = 0; q < 4; q++)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(a_dst[q] + stage * kStageA2),
                         "l"(a_src[q] + tile * kBK), "r"(a_bytes[q])
                         : "memory");
    };
    // weights: packed word column j of the tile (8 output columns), K octet koct (8 rows)
    const int koct_b = tid & 7, j_b = tid >> 3;
    const int wcol = (n0 >> 3) + j_b;
    const bool col_ok = wcol < NW;
    const uint32_t* w_src = p.qw + (col_ok ? size_t(koct_b * 8) * NW + wcol : 0);  // + tile * kBK * NW + r * NW
    const uint32_t* z_src = p.qz + (col_ok ? wcol : 0);                            // + group * NW
    const uint4* s_src = reinterpret_cast<const uint4*>(p.scales + (col_ok ? n0 + j_b * 8 : 0));  // + group * N halves
    const int tile_words = kBK * NW;
    auto load_b = [&](int tile, uint32_t (&w)[8], uint32_t& zw, uint4& sraw) {
        const uint32_t* wp = w_src + size_t(tile) * tile_words;
        const int g = tile >> 1;  // two 64-row tiles per 128-row group
#pragma unroll
        for (int r = 0; r < 8; r++) w[r] = col_ok ? __ldg(wp + r * NW) : 0u;
        zw = col_ok ? __ldg(z_src + size_t(g) * NW) : 0u;
        sraw = col_ok ? __ldg(s_src + size_t(g) * (p.N >> 3)) : make_uint4(0, 0, 0, 0);
    };

    // one tile of the K loop; the packed words of tile `it` are in (w, zw, sraw) and the same registers are
    // refilled with tile it + 2 as soon as they have been consumed, so a load has two tiles of time to land
    auto tile_step = [&](int it, uint32_t (&w)[8], uint32_t& zw, uint4& sraw) {
        const int s = it % kStages2;
        // ---- dequantise the weight tile into stage s (free: checked one tile ago, when its activations were requested)
        {
            uint32_t d[8][4];  // [row][column pair]
            const TileConsts tc = make_tile_consts(zw, sraw);
#pragma unroll
            for (int r = 0; r < 8; r++) dequant_word_consts(w[r], tc, d[r]);
            if (it + 2 < nk) load_b(it + 2, w, zw, sraw);
            unsigned char* dst = sB + s * kStageB2 + j_b * 1024;
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const int pr = c >> 1;
                const uint32_t sel = (c & 1) ? 0x7632u : 0x5410u;
                uint4 o;  // rows (0,1) (2,3) (4,5) (6,7) of column c
                o.x = __byte_perm(d[0][pr], d[1][pr], sel);
                o.y = __byte_perm(d[2][pr], d[3][pr], sel);
                o.z = __byte_perm(d[4][pr], d[5][pr], sel);
                o.w = __byte_perm(d[6][pr], d[7][pr], sel);
                *reinterpret_cast<uint4*>(dst + c * 128 + ((koct_b ^ c) << 4)) = o;
            }
        }
        // ---- request the next tile's activations; its stage is free once the MMAs that last read it have finished
        //      (by now they had the whole dequantisation above to do so)
        if (it + 1 < nk) {
            const int sn = (it + 1) % kStages2;
            if (it + 1 >= kStages2 && !dead) {
                if (!tc_mbar_wait(&mma_bar[sn], uint32_t((it + 1) / kStages2 - 1) & 1u)) {
                    atomicExch(&g_gemm_wait_error, 3);
                    s_dead = 1;
                    dead = true;
                }
            }
            issue_a(it + 1, sn);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");  // everything but the newest group: this tile's activations
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        dead = dead || (s_dead != 0);
        if (tid == 0 && !dead) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_base = smem_addr(sA + s * kStageA2), b_base = smem_addr(sB + s * kStageB2);
#pragma unroll
            for (int kk = 0; kk < kBK / 16; kk++) {
                const uint64_t adesc = make_desc(a_base + kk * 32);
                const uint64_t bdesc = make_desc(b_base + kk * 32);
                const uint32_t accumulate = (it > 0 || kk > 0) ? 1u : 0u;
                asm volatile(
                    "{\n\t.reg .pred p;\n\t"
                    "setp.ne.b32 p, %4, 0;\n\t"
                    "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                    ::"r"(tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
                    : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(&mma_bar[s]))
                         : "memory");
        }
    };

    uint32_t w_even[8], w_odd[8], zw_even, zw_odd = 0;
    uint4 s_even, s_odd = make_uint4(0, 0, 0, 0);
    issue_a(0, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    load_b(0, w_even, zw_even, s_even);
    if (nk > 1) load_b(1, w_odd, zw_odd, s_odd);
    for (int it = 0; it < nk; it += 2) {
        tile_step(it, w_even, zw_even, s_even);
        if (it + 1 < nk) tile_step(it + 1, w_odd, zw_odd, s_odd);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // ---- all MMAs done?  (they complete in order: the last commit covers everything)
    if (!dead) {
        const int last = nk - 1;
        if (!tc_mbar_wait(&mma_bar[last % kStages2], uint32_t(last / kStages2) & 1u)) {
            atomicExch(&g_gemm_wait_error, 4);
            dead = true;
        }
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    if (!dead) {
        // ---- epilogue: warp w reads TMEM lanes 32*(w&3).., columns 128*(w>>2)..; one output row per thread
        const int row = m0 + (warp & 3) * 32 + lane;
        const int cbase = (warp >> 2) * 128;
#pragma unroll 1
        for (int ch = 0; ch < 4; ch++) {
            uint32_t r[32];
            const uint32_t taddr = tmem + (uint32_t((warp & 3) * 32) << 16) + uint32_t(cbase + ch * 32);
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                  "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
                  "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
                  "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                : "r"(taddr)
                : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (row < p.M) {
                const int col0 = n0 + cbase + ch * 32;
                float* yp = p.y + size_t(row) * p.N + col0;
                const float* rp = p.mode == 1 ? p.residual + size_t(row) * p.N + col0 : (p.mode == 2 ? yp : nullptr);
#pragma unroll
                for (int v = 0; v < 8; v++) {
                    if (col0 + v * 4 < p.N) {
                        float4 o = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                               __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                        if (rp) {
                            const float4 a = __ldcg(reinterpret_cast<const float4*>(rp) + v);
                            o.x += a.x; o.y += a.y; o.z += a.z; o.w += a.w;
                        }
                        reinterpret_cast<float4*>(yp)[v] = o;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(uint32_t(kBN2)) : "memory");
    }
}


// ---------------------------------------------------------------------------------------------
// Third generation: the same tiles, stages and dequantisation, but nobody waits at a block-wide barrier per stage.
//   * eight producer warps fill the stages (weights dequantised into stage s, activations of the next tile by cp.async);
//     each thread arrives on the stage's "full" mbarrier once its own copies have landed and its stores are visible to
//     the tensor-core proxy;
//   * a ninth warp only waits for "full", issues the four tcgen05.mma of the stage and commits them onto the stage's
//     "free" mbarrier, which the producers check before they overwrite the stage - so a producer warp that is ahead
//     keeps working on the next tile instead of waiting for the slowest warp of the block;
//   * zero words and scales are loaded and prepared once per 128-row group (two stages), addresses are carried as running
//     pointers, and the swizzled store offsets are computed once.
constexpr int kProducerThreads3 = 256;
constexpr int kGemmThreads3 = kProducerThreads3 + 32;

__global__ void __launch_bounds__(kGemmThreads3, 2) awq_gemm_tc3_kernel(const GemmParams2 pp) {
    const GemmParams& p = pp.g;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    unsigned char* sA = smem;                          // kStages2 x 16 KB
    unsigned char* sB = smem + kStages2 * kStageA2;    // kStages2 x 32 KB
    __shared__ uint64_t full_bar[kStages2];            // producers -> MMA warp
    __shared__ uint64_t free_bar[kStages2];            // tcgen05.commit -> producers
    __shared__ uint32_t s_tmem;
    __shared__ int s_dead;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * kBN2, m0 = blockIdx.y * kBM;
    const int NW = p.N >> 3;

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < kStages2; i++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&full_bar[i])), "r"(uint32_t(kProducerThreads3)));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&free_bar[i])));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_dead = 0;
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&s_tmem)), "r"(uint32_t(kBN2))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    pdl_launch_dependents();
    pdl_wait();

    // split K: grid.z CTAs work on consecutive runs of K tiles of the same output tile and add their sums with reductions
    const int nk = pp.tiles_per_split > 0 ? pp.tiles_per_split : p.K / kBK;
    const int tile0 = int(blockIdx.z) * nk;
    const bool split_k = gridDim.z > 1;
    bool dead = false;

    if (warp == kProducerThreads3 / 32) {
        // ------------------------------------------------------------ MMA warp: one lane issues
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (uint32_t(kBN2 >> 3) << 17) | (uint32_t(kBM >> 4) << 24);
            for (int it = 0; it < nk && !dead; it++) {
                const int s = it % kStages2;
                if (!tc_mbar_wait(&full_bar[s], uint32_t(it / kStages2) & 1u)) {
                    atomicExch(&g_gemm_wait_error, 5);
                    s_dead = 1;
                    dead = true;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_base = smem_addr(sA + s * kStageA2), b_base = smem_addr(sB + s * kStageB2);
#pragma unroll
                for (int kk = 0; kk < kBK / 16; kk++) {
                    const uint64_t adesc = make_desc(a_base + kk * 32);
                    const uint64_t bdesc = make_desc(b_base + kk * 32);
                    const uint32_t accumulate = (it > 0 || kk > 0) ? 1u : 0u;
                    asm volatile(
                        "{\n\t.reg .pred p;\n\t"
                        "setp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                        ::"r"(tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
                        : "memory");
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(&free_bar[s]))
                             : "memory");
            }
        }
    } else {
        // ------------------------------------------------------------ producers
        // activations: four 16-byte chunks (row m, K octet koct), global fp16 -> swizzled shared memory, one tile ahead
        const unsigned char* a_src[4];
        uint32_t a_dst[4], a_bytes[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int item = q * kProducerThreads3 + tid;
            const int koct = item & 7, m = item >> 3;
            const bool ok = m0 + m < p.M;
            a_src[q] = reinterpret_cast<const unsigned char*>(pp.x16 + size_t(ok ? m0 + m : 0) * p.K + koct * 8 + size_t(tile0) * kBK);
            a_dst[q] = smem_addr(sA) + (m >> 3) * 1024 + (m & 7) * 128 + ((koct ^ (m & 7)) << 4);
            a_bytes[q] = ok ? 16u : 0u;  // 0: the chunk is zero filled
        }
        auto issue_a = [&](int stage) {  // the next tile along K; the sources advance by one tile
#pragma unroll
            for (int q = 0; q < 4; q++) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(a_dst[q] + stage * kStageA2), "l"(a_src[q]),
                             "r"(a_bytes[q])
                             : "memory");
                a_src[q] += kBK * sizeof(__half);
            }
        };
        // weights: packed word column j of the tile (8 output columns), K octet koct (8 rows)
        const int koct_b = tid & 7, j_b = tid >> 3;
        const int wcol = (n0 >> 3) + j_b;
        const bool col_ok = wcol < NW;
        const size_t tile_words = size_t(kBK) * NW;
        const size_t row_words = size_t(NW);
        const size_t scale_vecs = size_t(p.N >> 3);
        const size_t group0 = size_t(tile0 >> 1);  // a split starts at a 128-row group
        const uint32_t* w_next = p.qw + (col_ok ? size_t(koct_b * 8) * NW + wcol + size_t(tile0) * tile_words : 0);  // next tile to load
        const uint32_t* z_next = p.qz + (col_ok ? wcol + group0 * row_words : 0);       // zero word of the next group to load
        const uint4* s_next = reinterpret_cast<const uint4*>(p.scales + (col_ok ? n0 + j_b * 8 : 0)) + (col_ok ? group0 * scale_vecs : 0);
        auto load_w = [&](uint32_t (&w)[8]) {
#pragma unroll
            for (int r = 0; r < 8; r++) w[r] = col_ok ? __ldg(w_next + r * row_words) : 0u;
            w_next += tile_words;
        };
        auto load_consts = [&](uint32_t& zw, uint4& sraw) {
            zw = col_ok ? __ldg(z_next) : 0u;
            sraw = col_ok ? __ldg(s_next) : make_uint4(0, 0, 0, 0);
            z_next += row_words;
            s_next += scale_vecs;
        };
        // swizzled 16-byte store slots of this thread inside its 1024-byte column block
        uint32_t b_off[8];
#pragma unroll
        for (int c = 0; c < 8; c++) b_off[c] = uint32_t(c * 128 + ((koct_b ^ c) << 4));
        const uint32_t b_dst = smem_addr(sB) + j_b * 1024;

        TileConsts tc;
        auto tile_step = [&](int it, uint32_t (&w)[8]) {
            const int s = it % kStages2;
            {
                uint32_t d[8][4];  // [row][column pair]
#pragma unroll
                for (int r = 0; r < 8; r++) dequant_word_consts(w[r], tc, d[r]);
                if (it + 2 < nk) load_w(w);
                const uint32_t dst = b_dst + s * kStageB2;
#pragma unroll
                for (int c = 0; c < 8; c++) {
                    const int pr = c >> 1;
                    const uint32_t sel = (c & 1) ? 0x7632u : 0x5410u;
                    const uint32_t o0 = __byte_perm(d[0][pr], d[1][pr], sel), o1 = __byte_perm(d[2][pr], d[3][pr], sel);
                    const uint32_t o2 = __byte_perm(d[4][pr], d[5][pr], sel), o3 = __byte_perm(d[6][pr], d[7][pr], sel);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + b_off[c]), "r"(o0), "r"(o1), "r"(o2), "r"(o3)
                                 : "memory");
                }
            }
            // the next tile's activations go into the other stage once the MMAs that last read it have finished
            if (it + 1 < nk) {
                const int sn = (it + 1) % kStages2;
                if (it + 1 >= kStages2 && !dead) {
                    if (!tc_mbar_wait(&free_bar[sn], uint32_t((it + 1) / kStages2 - 1) & 1u)) {
                        atomicExch(&g_gemm_wait_error, 3);
                        s_dead = 1;
                        dead = true;
                    }
                }
                issue_a(sn);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 1;" ::: "memory");  // everything but the newest group: this tile's activations
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(&full_bar[s])) : "memory");
        };

        uint32_t w_even[8], w_odd[8], zw;
        uint4 sraw;
        issue_a(0);
        asm volatile("cp.async.commit_group;" ::: "memory");
        load_w(w_even);
        if (nk > 1) load_w(w_odd);
        load_consts(zw, sraw);
        for (int it = 0; it < nk; it += 2) {  // two 64-row tiles = one 128-row group: one set of constants
            tc = make_tile_consts(zw, sraw);
            if (it + 2 < nk) load_consts(zw, sraw);
            tile_step(it, w_even);
            if (it + 1 < nk) tile_step(it + 1, w_odd);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");

        // ---- all MMAs done?  (they complete in order: the last commit covers everything)
        if (!dead) {
            const int last = nk - 1;
            if (!tc_mbar_wait(&free_bar[last % kStages2], uint32_t(last / kStages2) & 1u)) {
                atomicExch(&g_gemm_wait_error, 4);
                dead = true;
            }
        }
        dead = dead || (s_dead != 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

        if (!dead) {
            // ---- epilogue: warp w reads TMEM lanes 32*(w&3).., columns 128*(w>>2)..; one output row per thread
            const int row = m0 + (warp & 3) * 32 + lane;
            const int cbase = (warp >> 2) * 128;
#pragma unroll 1
            for (int ch = 0; ch < 4; ch++) {
                uint32_t r[32];
                const uint32_t taddr = tmem + (uint32_t((warp & 3) * 32) << 16) + uint32_t(cbase + ch * 32);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                      "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
                      "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
                      "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < p.M) {
                    const int col0 = n0 + cbase + ch * 32;
                    float* yp = p.y + size_t(row) * p.N + col0;
                    // split K: every CTA adds into y (zeroed by the host unless the call accumulates); the residual rides
                    // with the first split
                    const float* rp = p.mode == 1 ? (split_k && blockIdx.z != 0 ? nullptr : p.residual + size_t(row) * p.N + col0)
                                                  : (p.mode == 2 && !split_k ? yp : nullptr);
#pragma unroll
                    for (int v = 0; v < 8; v++) {
                        if (col0 + v * 4 < p.N) {
                            float4 o = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                                   __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                            if (rp) {
                                const float4 a = __ldcg(reinterpret_cast<const float4*>(rp) + v);
                                o.x += a.x; o.y += a.y; o.z += a.z; o.w += a.w;
                            }
                            if (split_k)
                                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(yp + 4 * v), "f"(o.x), "f"(o.y), "f"(o.z),
                                             "f"(o.w)
                                             : "memory");
                            else
                                reinterpret_cast<float4*>(yp)[v] = o;
                        }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(uint32_t(kBN2)) : "memory");
    }
}

constexpr int kMaxSplitK = 8;
int g_gemm_split_k = 1;  // tuning key "gemm_split_k": 0 switches the K split of the third generation off
int g_gemm_impl = 3;  // 3: mbarrier hand-over to a dedicated MMA warp (default); 2: stages handed over at a block-wide barrier (tuning key "gemm_impl")

}  // namespace

void awq_gemm_set_tuning(const char* key, int value) {
    if (!strcmp(key, "gemm_impl")) g_gemm_impl = value == 3 ? 3 : 2;
    if (!strcmp(key, "gemm_split_k")) g_gemm_split_k = value < 0 ? 0 : value;
}

}  // namespace kuiper

using namespace kuiper;

extern "C" int kuiper_awq_gemm_status(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_wait_error, sizeof(int)) != cudaSuccess) v = -1;
    if (v == 0) return KUIPER_OK;
    set_error("awq_gemm: a bounded tensor-core pipeline wait ran out (code %d)", v);
    return KUIPER_INTERNAL_ERROR;
}

extern "C" size_t kuiper_awq_gemm_workspace_bytes(int M, int K) {
    if (M <= 0 || K <= 0) return 0;
    return (size_t(M) * size_t(K) * sizeof(__half) + 255) / 256 * 256;  // fp16 copy of the activations
}

// Shared by the two entry points: x is fp32 (converted into the workspace first) or already fp16 (x16, no workspace).
static int gemm_common(const float* x, const __half* x16_in, const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales,
                       float* y, const float* residual, int accumulate, int M, int K, int N, int group, void* workspace,
                       size_t workspace_bytes, kuiper_stream_t stream) {
    KUIPER_REQUIRE((x || x16_in) && qweight && qzeros && scales && y, "awq_gemm: null tensor pointer");
    KUIPER_REQUIRE(M > 0 && K > 0 && N > 0, "awq_gemm: empty shape M=%d K=%d N=%d", M, K, N);
    KUIPER_REQUIRE(group == 128, "awq_gemm: group size %d is not supported (128 only)", group);
    KUIPER_REQUIRE(K % 128 == 0 && N % 8 == 0, "awq_gemm: needs K %% 128 == 0 and N %% 8 == 0 (K=%d N=%d)", K, N);
    KUIPER_REQUIRE(!(accumulate && residual), "awq_gemm: accumulate and residual are exclusive");
    KUIPER_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(x16_in) | reinterpret_cast<uintptr_t>(y) |
                     reinterpret_cast<uintptr_t>(scales) | reinterpret_cast<uintptr_t>(residual)) & 15) == 0 && (N % 4 == 0),
                   "awq_gemm: x, y, scales and residual must be 16-byte aligned");
    GemmParams p;
    p.x = x;
    p.qw = reinterpret_cast<const uint32_t*>(qweight);
    p.qz = reinterpret_cast<const uint32_t*>(qzeros);
    p.scales = reinterpret_cast<const __half*>(scales);
    p.y = y;
    p.residual = residual;
    p.M = M; p.K = K; p.N = N;
    p.mode = accumulate ? 2 : (residual ? (residual == y ? 2 : 1) : 0);  // y + residual with residual == y is y += 
    KUIPER_REQUIRE(x16_in != nullptr || (workspace != nullptr && workspace_bytes >= kuiper_awq_gemm_workspace_bytes(M, K) &&
                                         (reinterpret_cast<uintptr_t>(workspace) & 15) == 0),
                   "awq_gemm: needs a 16-byte aligned workspace of kuiper_awq_gemm_workspace_bytes(M, K) bytes (got %zu)",
                   workspace_bytes);
    // Few output tiles (a decode batch, a short chunk: one row of tiles is N / 256 CTAs) leave most SMs without work while
    // every CTA streams a whole column panel of the weight: the third generation then splits K so that about two CTAs
    // per SM are busy.  A split is a whole number of 128-row groups; the sums meet through reductions, so y starts from
    // zero (or from its content when the call accumulates) and the summation order is no longer fixed.
    const dim3 grid2((N + kBN2 - 1) / kBN2, (M + kBM - 1) / kBM, 1);
    int splits = 1;
    if (g_gemm_impl == 3 && g_gemm_split_k) {
        // up to a third of a second wave is still a gain (measured: 96 tiles run 48 us with 4 splits, 55 us with 2)
        const int tiles = int(grid2.x * grid2.y), groups = K / 128, want = (2 * device_sm_count() * 4 / 3 + tiles - 1) / tiles;
        for (int sdiv = 2; sdiv <= groups && sdiv <= kMaxSplitK && sdiv <= want; sdiv++)
            if (groups % sdiv == 0) splits = sdiv;
        if (g_gemm_split_k > 1 && groups % g_gemm_split_k == 0) splits = g_gemm_split_k;  // forced (measurement aid)
    }
    const bool zero_y = splits > 1 && p.mode != 2;
    // activations converted to fp16 once (the same launch zeroes y for a split call), then 128 x 256 output tiles
    const int64_t n4 = x16_in ? 0 : int64_t(M) * K / 4;  // activations that arrive as fp16 need no conversion
    const int64_t zero4 = zero_y ? int64_t(M) * N / 4 : 0;
    if (n4 > 0 || zero4 > 0) {
        int blocks = int(((n4 > zero4 ? n4 : zero4) + 255) / 256);
        if (blocks > 148 * 8) blocks = 148 * 8;
        int rc = pdl_status(launch_pdl(convert_f16_kernel, dim3(blocks), dim3(256), 0, as_stream(stream),
                                       reinterpret_cast<const float4*>(x), reinterpret_cast<uint2*>(workspace), n4,
                                       reinterpret_cast<float4*>(y), zero4),
                            "awq_gemm convert");
        if (rc != KUIPER_OK) return rc;
    }
    GemmParams2 p2;
    p2.g = p;
    p2.x16 = x16_in ? x16_in : reinterpret_cast<const __half*>(workspace);
    p2.tiles_per_split = 0;
    const size_t smem2 = 1024 + size_t(kStages2) * (kStageA2 + kStageB2);
    if (g_gemm_impl == 3) {
        static size_t configured3[kMaxDevices] = {};
        if (!ensure_dynamic_smem(awq_gemm_tc3_kernel, smem2, configured3)) {
            set_error("awq_gemm: cannot reserve %zu bytes of shared memory", smem2);
            return KUIPER_INTERNAL_ERROR;
        }
        dim3 grid3 = grid2;
        if (splits > 1) {
            grid3.z = splits;
            p2.tiles_per_split = (K / kBK) / splits;
        }
        return pdl_status(launch_pdl(awq_gemm_tc3_kernel, grid3, dim3(kGemmThreads3), smem2, as_stream(stream), p2), "awq_gemm");
    }
    static size_t configured[kMaxDevices] = {};
    if (!ensure_dynamic_smem(awq_gemm_tc2_kernel, smem2, configured)) {
        set_error("awq_gemm: cannot reserve %zu bytes of shared memory", smem2);
        return KUIPER_INTERNAL_ERROR;
    }
    return pdl_status(launch_pdl(awq_gemm_tc2_kernel, grid2, dim3(kGemmThreads), smem2, as_stream(stream), p2), "awq_gemm");
}

extern "C" int kuiper_awq_gemm_f32(const float* x, const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales,
                                   float* y, const float* residual, int accumulate, int M, int K, int N, int group,
                                   void* workspace, size_t workspace_bytes, kuiper_stream_t stream) {
    KUIPER_REQUIRE(x != nullptr, "awq_gemm: null tensor pointer");
    return gemm_common(x, nullptr, qweight, qzeros, scales, y, residual, accumulate, M, K, N, group, workspace, workspace_bytes, stream);
}

extern "C" int kuiper_awq_gemm_f16in_f32(const uint16_t* x16, const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales,
                                         float* y, const float* residual, int accumulate, int M, int K, int N, int group,
                                         kuiper_stream_t stream) {
    KUIPER_REQUIRE(x16 != nullptr, "awq_gemm_f16in: null tensor pointer");
    return gemm_common(nullptr, reinterpret_cast<const __half*>(x16), qweight, qzeros, scales, y, residual, accumulate, M, K, N, group,
                       nullptr, 0, stream);
}
