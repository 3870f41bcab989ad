// Causal attention for a prompt chunk: M consecutive token rows of ONE sequence against the bf16 KV cache (which already
// holds the chunk's own rows), tiled so that every K / V tile is loaded once per block of query rows instead of once
// per row.  Fills the same placeholder as the decode kernel (kuiper/include/op/mha.h:1-11 of the reference).
//
// Grid (ceil(M / BR), Nkv): a CTA owns BR = 64 / R consecutive query rows of one kv head, i.e. 64 query vectors
// (row, head) with R = Nq / Nkv heads per kv head; warp w owns vectors 16w .. 16w+15 (vector v = row * R + head).
// Per 64-row cache tile (cp.async into a two-stage ring, 16-byte chunks XOR-swizzled by row so that ldmatrix is
// conflict free):
//   S = Q . K^T   mma.sync.m16n8k16 bf16: A = q (pre-scaled, bf16 high + low parts, kept in registers for the whole
//                 kernel), B = K rows as they lie in the cache (ldmatrix)
//   online softmax in fp32 on the accumulator fragments (causal mask by position)
//   O += P . V    A = probabilities straight from the S fragments (bf16 high + low parts), B = V by ldmatrix.trans
// K and V are exact bf16 operands; q and P keep 16 significant bits through the two-part split, as in the decode
// kernel.  No split over the KV range: a chunk has enough (row block, kv head) pairs to fill the GPU.
#include <cstring>

#include "common.cuh"

namespace kuiper {
namespace {

constexpr int kPD = 128;          // head dimension
constexpr int kPTile = 64;        // cache rows per tile
constexpr int kPWarps = 4;
constexpr int kPTileBytes = kPTile * kPD * 2;   // 16 KB per K or V tile

struct PrefillParams {
    const float* q;        // [M, Nq, 128]
    const uint16_t* kc;    // cache[(slot * Nkv + kvh) * max_seq + pos][128]
    const uint16_t* vc;
    float* out;            // [M, Nq, 128]
    int M, Nq, Nkv, max_seq;
    int pos0;              // position of row 0; row m sits at pos0 + m and sees cache rows [0, pos0 + m]
    int slot;
};

__device__ __forceinline__ uint32_t ps_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void pmma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// (x, y) as bf16 high parts in one register (x in the low half) and what is left of them as bf16 low parts
__device__ __forceinline__ void psplit(float x, float y, uint32_t& hi, uint32_t& lo) {
    const uint32_t xh = float_to_bf16_bits(x), yh = float_to_bf16_bits(y);
    hi = xh | (yh << 16);
    const float xr = x - bf16_bits_to_float(uint16_t(xh)), yr = y - bf16_bits_to_float(uint16_t(yh));
    lo = uint32_t(float_to_bf16_bits(xr)) | (uint32_t(float_to_bf16_bits(yr)) << 16);
}
// byte offset of 16-byte chunk `chunk` (0..15) of tile row `row` (0..63): chunks are XORed with the row's low bits
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) { return uint32_t(row * 256 + ((chunk ^ (row & 7)) << 4)); }

template <int R>
__global__ void __launch_bounds__(kPWarps * 32, 2)
flash_prefill_kernel(const PrefillParams p) {
    constexpr int BR = 64 / R;  // query rows per CTA
    extern __shared__ __align__(128) unsigned char psm[];  // 2 stages x (K tile | V tile)
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int kvh = blockIdx.y;
    const int m0 = blockIdx.x * BR;
    pdl_launch_dependents();
    pdl_wait();  // q and the newest cache rows come from the previous kernel

    // this warp's two fragment rows: vectors v0 = 16 warp + g and v0 + 8; vector v = (row v / R, head v % R)
    const int v0 = 16 * warp + g, v1 = v0 + 8;
    const int r0 = m0 + v0 / R, r1 = m0 + v1 / R;          // token rows
    const int h0 = kvh * R + v0 % R, h1 = kvh * R + v1 % R;  // q heads
    const bool live0 = r0 < p.M, live1 = r1 < p.M;
    const int pos_r0 = p.pos0 + r0, pos_r1 = p.pos0 + r1;    // last visible cache row of each

    // q as A fragments, pre-scaled by 1/sqrt(128): k-step ks covers dimensions 16 ks .. 16 ks + 15
    const float scale = 0.08838834764831845f;
    uint32_t qh[8][4], ql[8][4];
    {
        const float* q0 = p.q + (size_t(live0 ? r0 : 0) * p.Nq + h0) * kPD;
        const float* q1 = p.q + (size_t(live1 ? r1 : 0) * p.Nq + h1) * kPD;
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
            const float2 a = live0 ? __ldcg(reinterpret_cast<const float2*>(q0 + 16 * ks + 2 * t)) : make_float2(0.f, 0.f);
            const float2 b = live1 ? __ldcg(reinterpret_cast<const float2*>(q1 + 16 * ks + 2 * t)) : make_float2(0.f, 0.f);
            const float2 c = live0 ? __ldcg(reinterpret_cast<const float2*>(q0 + 16 * ks + 8 + 2 * t)) : make_float2(0.f, 0.f);
            const float2 d = live1 ? __ldcg(reinterpret_cast<const float2*>(q1 + 16 * ks + 8 + 2 * t)) : make_float2(0.f, 0.f);
            psplit(a.x * scale, a.y * scale, qh[ks][0], ql[ks][0]);
            psplit(b.x * scale, b.y * scale, qh[ks][1], ql[ks][1]);
            psplit(c.x * scale, c.y * scale, qh[ks][2], ql[ks][2]);
            psplit(d.x * scale, d.y * scale, qh[ks][3], ql[ks][3]);
        }
    }

    // cache rows this CTA needs: everything up to the position of its last live row
    const int last_row = min(m0 + BR, p.M) - 1;
    const int kv_end = min(p.pos0 + last_row + 1, p.max_seq);
    const int n_tiles = (kv_end + kPTile - 1) / kPTile;
    const size_t head_off = (size_t(p.slot) * p.Nkv + kvh) * p.max_seq * kPD;
    const uint16_t* kb = p.kc + head_off;
    const uint16_t* vb = p.vc + head_off;
    const uint32_t sm0 = ps_u32(psm);

    // a tile = 64 rows x 16 chunks of 16 bytes for K and for V: 2048 chunks, 16 per thread
    auto load_tile = [&](int tile, int stage) {
        const int row_base = tile * kPTile;
        const uint32_t ks_addr = sm0 + stage * 2 * kPTileBytes, vs_addr = ks_addr + kPTileBytes;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int c = tid + i * 128;           // chunk id 0..1023
            const int row = c >> 4, chunk = c & 15;
            // rows past the end of the cache range are clamped (their scores are masked anyway)
            const int src_row = min(row_base + row, p.max_seq - 1);
            cp_async16(ks_addr + tile_off(row, chunk), kb + size_t(src_row) * kPD + chunk * 8);
            cp_async16(vs_addr + tile_off(row, chunk), vb + size_t(src_row) * kPD + chunk * 8);
        }
        cp_async_commit();
    };

    float oacc[16][4];
#pragma unroll
    for (int n = 0; n < 16; n++) { oacc[n][0] = oacc[n][1] = oacc[n][2] = oacc[n][3] = 0.f; }
    float mx0 = -INFINITY, mx1 = -INFINITY, sum0 = 0.f, sum1 = 0.f;

    if (n_tiles > 0) load_tile(0, 0);
    for (int tile = 0; tile < n_tiles; tile++) {
        const int stage = tile & 1;
        if (tile + 1 < n_tiles) {
            load_tile(tile + 1, stage ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t ks_addr = sm0 + stage * 2 * kPTileBytes, vs_addr = ks_addr + kPTileBytes;
        const int kv0 = tile * kPTile;

        // ---- S = q . K^T for the 64 cache rows of the tile: 8 column tiles of 8 rows
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; j++) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            // ldmatrix.x4: matrices 0..3 = dimensions chunks (2 kk, 2 kk + 1) of k-steps kk, kk+... of cache rows 8j..8j+7
#pragma unroll
            for (int kp = 0; kp < 4; kp++) {  // pairs of k-steps: dimensions 32 kp .. 32 kp + 31 = chunks 4 kp .. 4 kp + 3
                uint32_t b[4];
                const int row = 8 * j + (lane & 7);
                const int chunk = 4 * kp + (lane >> 3);
                ldmatrix_x4(b, ks_addr + tile_off(row, chunk));
                // b[0], b[1]: k-step 2 kp (dims +0..7, +8..15); b[2], b[3]: k-step 2 kp + 1
                pmma_bf16(s[j], qh[2 * kp][0], qh[2 * kp][1], qh[2 * kp][2], qh[2 * kp][3], b[0], b[1]);
                pmma_bf16(s[j], ql[2 * kp][0], ql[2 * kp][1], ql[2 * kp][2], ql[2 * kp][3], b[0], b[1]);
                pmma_bf16(s[j], qh[2 * kp + 1][0], qh[2 * kp + 1][1], qh[2 * kp + 1][2], qh[2 * kp + 1][3], b[2], b[3]);
                pmma_bf16(s[j], ql[2 * kp + 1][0], ql[2 * kp + 1][1], ql[2 * kp + 1][2], ql[2 * kp + 1][3], b[2], b[3]);
            }
        }
        // ---- causal mask + online softmax: fragment entries 0,1 belong to vector v0 (cache rows kv0 + 8j + 2t, +1),
        //      entries 2,3 to vector v1
        float bm0 = -INFINITY, bm1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int c = kv0 + 8 * j + 2 * t;
            s[j][0] = (live0 && c <= pos_r0) ? s[j][0] : -INFINITY;
            s[j][1] = (live0 && c + 1 <= pos_r0) ? s[j][1] : -INFINITY;
            s[j][2] = (live1 && c <= pos_r1) ? s[j][2] : -INFINITY;
            s[j][3] = (live1 && c + 1 <= pos_r1) ? s[j][3] : -INFINITY;
            bm0 = fmaxf(bm0, fmaxf(s[j][0], s[j][1]));
            bm1 = fmaxf(bm1, fmaxf(s[j][2], s[j][3]));
        }
        bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, 1));
        bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, 2));
        bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, 1));
        bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, 2));
        const float nm0 = fmaxf(mx0, bm0), nm1 = fmaxf(mx1, bm1);
        // a vector that has seen no visible row yet keeps max = -inf: no rescaling, its probabilities are all zero
        const float corr0 = (nm0 == -INFINITY || mx0 == -INFINITY) ? (nm0 == -INFINITY ? 1.f : 0.f) : __expf(mx0 - nm0);
        const float corr1 = (nm1 == -INFINITY || mx1 == -INFINITY) ? (nm1 == -INFINITY ? 1.f : 0.f) : __expf(mx1 - nm1);
        mx0 = nm0;
        mx1 = nm1;
        sum0 *= corr0;
        sum1 *= corr1;
#pragma unroll
        for (int n = 0; n < 16; n++) {
            oacc[n][0] *= corr0; oacc[n][1] *= corr0; oacc[n][2] *= corr1; oacc[n][3] *= corr1;
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            s[j][0] = (s[j][0] == -INFINITY) ? 0.f : __expf(s[j][0] - nm0);
            s[j][1] = (s[j][1] == -INFINITY) ? 0.f : __expf(s[j][1] - nm0);
            s[j][2] = (s[j][2] == -INFINITY) ? 0.f : __expf(s[j][2] - nm1);
            s[j][3] = (s[j][3] == -INFINITY) ? 0.f : __expf(s[j][3] - nm1);
            sum0 += s[j][0] + s[j][1];
            sum1 += s[j][2] + s[j][3];
        }
        // ---- O += P . V: k-step kk covers cache rows 16 kk .. 16 kk + 15 of the tile = column tiles 2 kk, 2 kk + 1 of S
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {
            uint32_t ph[4], pl[4];
            psplit(s[2 * kk][0], s[2 * kk][1], ph[0], pl[0]);          // vector v0, rows 2t, 2t+1
            psplit(s[2 * kk][2], s[2 * kk][3], ph[1], pl[1]);          // vector v1
            psplit(s[2 * kk + 1][0], s[2 * kk + 1][1], ph[2], pl[2]);  // vector v0, rows 2t+8, 2t+9
            psplit(s[2 * kk + 1][2], s[2 * kk + 1][3], ph[3], pl[3]);
#pragma unroll
            for (int np = 0; np < 8; np++) {  // pairs of dimension tiles: dimensions 16 np .. 16 np + 15 = chunks 2 np, 2 np + 1
                uint32_t b[4];
                // transposed 8x8 loads: matrix 0 = rows 16kk..+7 x chunk 2np, 1 = rows +8..+15 x chunk 2np,
                // 2 = rows 16kk..+7 x chunk 2np+1, 3 = rows +8..+15 x chunk 2np+1
                const int row = 16 * kk + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int chunk = 2 * np + (lane >> 4);
                ldmatrix_x4_trans(b, vs_addr + tile_off(row, chunk));
                pmma_bf16(oacc[2 * np], ph[0], ph[1], ph[2], ph[3], b[0], b[1]);
                pmma_bf16(oacc[2 * np], pl[0], pl[1], pl[2], pl[3], b[0], b[1]);
                pmma_bf16(oacc[2 * np + 1], ph[0], ph[1], ph[2], ph[3], b[2], b[3]);
                pmma_bf16(oacc[2 * np + 1], pl[0], pl[1], pl[2], pl[3], b[2], b[3]);
            }
        }
        __syncthreads();  // the stage is reloaded two iterations from now by all threads
    }
    // row sums over the four lanes of a quad
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    const float inv0 = sum0 > 0.f ? 1.f / sum0 : 0.f, inv1 = sum1 > 0.f ? 1.f / sum1 : 0.f;
    if (live0) {
        float* o = p.out + (size_t(r0) * p.Nq + h0) * kPD;
#pragma unroll
        for (int n = 0; n < 16; n++) *reinterpret_cast<float2*>(o + 8 * n + 2 * t) = make_float2(oacc[n][0] * inv0, oacc[n][1] * inv0);
    }
    if (live1) {
        float* o = p.out + (size_t(r1) * p.Nq + h1) * kPD;
#pragma unroll
        for (int n = 0; n < 16; n++) *reinterpret_cast<float2*>(o + 8 * n + 2 * t) = make_float2(oacc[n][2] * inv1, oacc[n][3] * inv1);
    }
}

template <int R>
int launch_prefill(const PrefillParams& p, cudaStream_t stream) {
    constexpr int BR = 64 / R;
    auto kern = flash_prefill_kernel<R>;
    const size_t smem = 4 * kPTileBytes;  // two stages of a K and a V tile
    static size_t configured[kMaxDevices] = {};
    if (!ensure_dynamic_smem(kern, smem, configured)) {
        set_error("flash_prefill: cannot reserve %zu bytes of shared memory", smem);
        return KUIPER_INTERNAL_ERROR;
    }
    const dim3 grid((p.M + BR - 1) / BR, p.Nkv, 1);
    return pdl_status(launch_pdl(kern, grid, dim3(kPWarps * 32), smem, stream, p), "flash_prefill");
}

}  // namespace
}  // namespace kuiper

using namespace kuiper;

extern "C" int kuiper_flash_prefill(const float* q, const uint16_t* kcache, const uint16_t* vcache, float* out, int M, int Nq,
                                    int Nkv, int D, int max_seq, int n_slots, int pos0, int slot, kuiper_stream_t stream) {
    KUIPER_REQUIRE(q && kcache && vcache && out, "flash_prefill: null tensor pointer");
    KUIPER_REQUIRE(D == kPD, "flash_prefill: head_dim %d is not supported (128 only)", D);
    KUIPER_REQUIRE(M > 0 && Nq > 0 && Nkv > 0 && max_seq > 0 && n_slots > 0, "flash_prefill: empty shape");
    KUIPER_REQUIRE(Nq % Nkv == 0, "flash_prefill: Nq=%d is not a multiple of Nkv=%d", Nq, Nkv);
    KUIPER_REQUIRE(slot >= 0 && slot < n_slots, "flash_prefill: sequence slot %d out of range", slot);
    KUIPER_REQUIRE(pos0 >= 0 && pos0 + M <= max_seq, "flash_prefill: rows %d..%d exceed max_seq %d", pos0, pos0 + M - 1, max_seq);
    KUIPER_REQUIRE(((reinterpret_cast<uintptr_t>(kcache) | reinterpret_cast<uintptr_t>(vcache) | reinterpret_cast<uintptr_t>(q) |
                     reinterpret_cast<uintptr_t>(out)) & 15) == 0,
                   "flash_prefill: tensors must be 16-byte aligned");
    KUIPER_REQUIRE(Nkv <= 65535, "flash_prefill: grid too large");
    const int R = Nq / Nkv;
    KUIPER_REQUIRE(R == 1 || R == 2 || R == 4 || R == 8, "flash_prefill: group size %d is not supported", R);
    PrefillParams p;
    p.q = q; p.kc = kcache; p.vc = vcache; p.out = out;
    p.M = M; p.Nq = Nq; p.Nkv = Nkv; p.max_seq = max_seq; p.pos0 = pos0; p.slot = slot;
    switch (R) {
        case 1: return launch_prefill<1>(p, as_stream(stream));
        case 2: return launch_prefill<2>(p, as_stream(stream));
        case 4: return launch_prefill<4>(p, as_stream(stream));
        default: return launch_prefill<8>(p, as_stream(stream));
    }
}
