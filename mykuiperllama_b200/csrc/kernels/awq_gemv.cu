// INT4-AWQ dequant-fused GEMV for sm_100a (decode, M = 1..8 token rows).
//
// Fills the reference's empty matmul placeholder (kuiper/include/op/matmul.h:1-11) for
// quantised layers (LayerParam quant fields, kuiper/include/op/layer.h:151-155).
//
// Data movement: the weight is read exactly once, in its native AWQ layout
// int32 [K, N/8].  A warp owns a 512-byte run of one weight row (32 lanes x 16 bytes =
// 1024 logical columns); the 8 warps of a CTA interleave over the rows of one K slice,
// so a CTA streams a dense [KC x 512 B] block with every global load a full 128-bit
// coalesced access.  All loads of a thread (up to 8 x 16 B) are issued before the first
// use, and they are issued before the programmatic-dependent-launch wait, so the weight
// stream of this GEMV overlaps the tail of the kernel that produces x.
//
// Dequant: the AWQ nibble order [0,2,4,6,1,3,5,7] puts logical columns (0,1) (2,3) (4,5)
// (6,7) of a word at nibble pairs (0,4) (1,5) (2,6) (3,7), which is what one LOP3 per
// pair extracts: (w & 0x000f000f) | 0x64006400 is the half2 (1024+q_a, 1024+q_b) and
// (w & 0x00f000f0) | 0x64006400 is (1024+16 q_a, 1024+16 q_b).  Subtracting the same
// pattern of the zero-point word (one HSUB2 / HFMA2 per pair) gives the exact integers
// q - z as half2.  Products with x are accumulated in fp32; the fp16 scale of the
// group is applied once per K slice after the cross-warp reduction.
//
// Split-K: grid = (column tiles, K slices).  Every CTA writes its scaled partial row to
// the workspace; the last CTA to arrive at a column tile (arrival counter) adds the
// slices in index order, so the result does not depend on scheduling.
#include "common.cuh"

namespace kuiper {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kTileCols = 1024;  // logical columns per CTA tile (32 lanes x 32 columns)
constexpr uint32_t kMagic = 0x64006400u;  // half2 (1024, 1024)

enum MathMode {
    kMathMixed = 0,  // x in fp16, fma.rn.f32.f16: exact products, fp32 accumulation
    kMathF32 = 1,    // x in fp32, q-z converted to fp32, FFMA
    kMathHalf2 = 2,  // x in fp16, half2 accumulation per K slice (fast, approximate)
};

struct GemvParams {
    const float* x;      // [M, K]
    const uint4* qw;     // [K, N/32] 16-byte chunks
    const uint4* qz;     // [K/128, N/32]
    const __half* scales;  // [K/128, N]
    float* y;            // [M, N]
    const float* residual;
    float* partial;      // [S, MT, N]
    int* counters;       // [column tiles]
    int K, N, nchunks, S;
};

__device__ __forceinline__ float fma_f16(uint16_t a, uint16_t b, float c) {
    float d;
    asm("fma.rn.f32.f16 %0, %1, %2, %3;" : "=f"(d) : "h"(a), "h"(b), "f"(c));
    return d;
}

struct ZeroConst {
    __half2 lo0, hi0, lo1, hi1;  // (1024+z) pairs and -(64+z) pairs
};

__device__ __forceinline__ __half2 as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ uint32_t as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }

__device__ __forceinline__ ZeroConst make_zero_const(uint32_t zw) {
    ZeroConst z;
    const __half2 neg_sixteenth = __floats2half2_rn(-0.0625f, -0.0625f);
    z.lo0 = as_h2((zw & 0x000f000fu) | kMagic);
    z.hi0 = __hmul2(as_h2((zw & 0x00f000f0u) | kMagic), neg_sixteenth);  // -(64 + z)
    uint32_t z8 = zw >> 8;
    z.lo1 = as_h2((z8 & 0x000f000fu) | kMagic);
    z.hi1 = __hmul2(as_h2((z8 & 0x00f000f0u) | kMagic), neg_sixteenth);
    return z;
}

// exact q - z of one packed word as four half2 pairs, in logical column order
__device__ __forceinline__ void dequant_word(uint32_t w, const ZeroConst& z, __half2 (&d)[4]) {
    const __half2 sixteenth = __floats2half2_rn(0.0625f, 0.0625f);
    uint32_t w8 = w >> 8;
    d[0] = __hsub2(as_h2((w & 0x000f000fu) | kMagic), z.lo0);
    d[1] = __hfma2(as_h2((w & 0x00f000f0u) | kMagic), sixteenth, z.hi0);
    d[2] = __hsub2(as_h2((w8 & 0x000f000fu) | kMagic), z.lo1);
    d[3] = __hfma2(as_h2((w8 & 0x00f000f0u) | kMagic), sixteenth, z.hi1);
}

template <int MODE, int MT>
struct Accum;

template <int MT>
struct Accum<kMathMixed, MT> {
    float acc[MT][32];
    __device__ __forceinline__ void init() {
#pragma unroll
        for (int m = 0; m < MT; m++)
#pragma unroll
            for (int c = 0; c < 32; c++) acc[m][c] = 0.f;
    }
    // xv[m]: activation of row m for this weight row
    __device__ __forceinline__ void row(const uint4& w, const ZeroConst (&z)[4], const float (&xv)[MT]) {
        uint16_t xh[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) xh[m] = __half_as_ushort(__float2half_rn(xv[m]));
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            __half2 d[4];
            dequant_word(ww[j], z[j], d);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint32_t u = as_u32(d[i]);
                uint16_t a = uint16_t(u & 0xffffu), b = uint16_t(u >> 16);
#pragma unroll
                for (int m = 0; m < MT; m++) {
                    acc[m][8 * j + 2 * i] = fma_f16(a, xh[m], acc[m][8 * j + 2 * i]);
                    acc[m][8 * j + 2 * i + 1] = fma_f16(b, xh[m], acc[m][8 * j + 2 * i + 1]);
                }
            }
        }
    }
    __device__ __forceinline__ float get(int m, int c) const { return acc[m][c]; }
};

template <int MT>
struct Accum<kMathF32, MT> {
    float acc[MT][32];
    __device__ __forceinline__ void init() {
#pragma unroll
        for (int m = 0; m < MT; m++)
#pragma unroll
            for (int c = 0; c < 32; c++) acc[m][c] = 0.f;
    }
    __device__ __forceinline__ void row(const uint4& w, const ZeroConst (&z)[4], const float (&xv)[MT]) {
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            __half2 d[4];
            dequant_word(ww[j], z[j], d);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float2 f = __half22float2(d[i]);
#pragma unroll
                for (int m = 0; m < MT; m++) {
                    acc[m][8 * j + 2 * i] = fmaf(f.x, xv[m], acc[m][8 * j + 2 * i]);
                    acc[m][8 * j + 2 * i + 1] = fmaf(f.y, xv[m], acc[m][8 * j + 2 * i + 1]);
                }
            }
        }
    }
    __device__ __forceinline__ float get(int m, int c) const { return acc[m][c]; }
};

template <int MT>
struct Accum<kMathHalf2, MT> {
    __half2 acc[MT][16];
    __device__ __forceinline__ void init() {
#pragma unroll
        for (int m = 0; m < MT; m++)
#pragma unroll
            for (int c = 0; c < 16; c++) acc[m][c] = __floats2half2_rn(0.f, 0.f);
    }
    __device__ __forceinline__ void row(const uint4& w, const ZeroConst (&z)[4], const float (&xv)[MT]) {
        __half2 xh[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) xh[m] = __float2half2_rn(xv[m]);
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            __half2 d[4];
            dequant_word(ww[j], z[j], d);
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int m = 0; m < MT; m++) acc[m][4 * j + i] = __hfma2(d[i], xh[m], acc[m][4 * j + i]);
        }
    }
    __device__ __forceinline__ float get(int m, int c) const {
        return (c & 1) ? __high2float(acc[m][c >> 1]) : __low2float(acc[m][c >> 1]);
    }
};

// ROWS weight rows per thread; the CTA covers KC = ROWS * 8 rows of one quantisation group.
template <int MODE, int MT, int ROWS>
__global__ void __launch_bounds__(kThreads, (MT == 1 ? 2 : 1))
awq_gemv_kernel(const GemvParams p) {
    extern __shared__ float4 red[];  // [kWarps][MT][256] float4, column slots rotated per lane
    __shared__ int s_last;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int chunk = blockIdx.x * 32 + lane;
    const bool active = chunk < p.nchunks;
    const int k0 = blockIdx.y * (ROWS * kWarps);
    const int group = k0 >> 7;
    constexpr int kBatch = ROWS < 8 ? ROWS : 8;

    Accum<MODE, MT> acc;
    acc.init();

    const uint4* wp = p.qw + size_t(k0 + warp) * p.nchunks + (active ? chunk : 0);
    const size_t row_step = size_t(kWarps) * p.nchunks;

    // weights and zero points do not depend on the previous kernel: fetch them first
    uint4 w[kBatch];
#pragma unroll
    for (int r = 0; r < kBatch; r++) w[r] = active ? ld_stream_u4(wp + r * row_step) : make_uint4(0, 0, 0, 0);
    uint4 zq = active ? __ldg(p.qz + size_t(group) * p.nchunks + chunk) : make_uint4(0, 0, 0, 0);

    pdl_launch_dependents();
    pdl_wait();

    ZeroConst z[4] = {make_zero_const(zq.x), make_zero_const(zq.y), make_zero_const(zq.z), make_zero_const(zq.w)};

#pragma unroll
    for (int b = 0; b < ROWS / kBatch; b++) {
        float xv[kBatch][MT];
#pragma unroll
        for (int r = 0; r < kBatch; r++)
#pragma unroll
            for (int m = 0; m < MT; m++) xv[r][m] = __ldcg(p.x + size_t(m) * p.K + k0 + warp + (b * kBatch + r) * kWarps);
#pragma unroll
        for (int r = 0; r < kBatch; r++) {
            acc.row(w[r], z, xv[r]);
            // refill the slot with the same row of the next batch
            if (b + 1 < ROWS / kBatch)
                w[r] = active ? ld_stream_u4(wp + ((b + 1) * kBatch + r) * row_step) : make_uint4(0, 0, 0, 0);
        }
    }

    // cross-warp reduction through shared memory; slot rotation keeps 16-byte stores conflict free
#pragma unroll
    for (int m = 0; m < MT; m++)
#pragma unroll
        for (int i = 0; i < 8; i++)
            red[(warp * MT + m) * 256 + lane * 8 + ((i + lane) & 7)] =
                make_float4(acc.get(m, 4 * i), acc.get(m, 4 * i + 1), acc.get(m, 4 * i + 2), acc.get(m, 4 * i + 3));
    __syncthreads();

    // thread t owns logical float4 t of the tile: lane t/8, slot t%8
    const int t = threadIdx.x;
    const int src = (t >> 3) * 8 + (((t & 7) + (t >> 3)) & 7);
    const int col = blockIdx.x * kTileCols + t * 4;
    const bool col_ok = col < p.N;
    float4 sum[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int wi = 0; wi < kWarps; wi++) {
            float4 v = red[(wi * MT + m) * 256 + src];
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        sum[m] = s;
    }
    if (col_ok) {
        const uint2 sraw = __ldg(reinterpret_cast<const uint2*>(p.scales + size_t(group) * p.N + col));
        const float2 s01 = __half22float2(as_h2(sraw.x)), s23 = __half22float2(as_h2(sraw.y));
#pragma unroll
        for (int m = 0; m < MT; m++) {
            sum[m].x *= s01.x; sum[m].y *= s01.y; sum[m].z *= s23.x; sum[m].w *= s23.y;
        }
    }

    if (p.S > 1) {
        if (col_ok) {
#pragma unroll
            for (int m = 0; m < MT; m++)
                *reinterpret_cast<float4*>(p.partial + (size_t(blockIdx.y) * MT + m) * p.N + col) = sum[m];
        }
        __threadfence();
        __syncthreads();
        if (t == 0) {
            int prev = atomicAdd(p.counters + blockIdx.x, 1);
            s_last = (prev == p.S - 1);
            if (s_last) p.counters[blockIdx.x] = 0;  // leave the counter ready for the next call
        }
        __syncthreads();
        if (!s_last) return;
        __threadfence();
        if (col_ok) {
#pragma unroll
            for (int m = 0; m < MT; m++) {
                float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int ks = 0; ks < p.S; ks++) {
                    float4 v = __ldcg(reinterpret_cast<const float4*>(p.partial + (size_t(ks) * MT + m) * p.N + col));
                    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
                }
                sum[m] = s;
            }
        }
    }
    if (col_ok) {
#pragma unroll
        for (int m = 0; m < MT; m++) {
            float4 s = sum[m];
            if (p.residual) {
                float4 r = __ldcg(reinterpret_cast<const float4*>(p.residual + size_t(m) * p.N + col));
                s.x += r.x; s.y += r.y; s.z += r.z; s.w += r.w;
            }
            *reinterpret_cast<float4*>(p.y + size_t(m) * p.N + col) = s;
        }
    }
}

// Any N % 8 == 0: one thread per packed word column, whole K, one token row.  Slow path
// for shapes the tiled kernel does not take (N not a multiple of 32).
__global__ void awq_gemv_generic_kernel(const float* x, const int32_t* qw, const int32_t* qz, const __half* scales,
                                        float* y, const float* residual, int K, int N) {
    pdl_wait();
    const int NW = N / 8;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= NW) return;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int g = 0; g < K / 128; g++) {
        ZeroConst z = make_zero_const(uint32_t(qz[size_t(g) * NW + j]));
        float part[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int k = g * 128; k < (g + 1) * 128; k++) {
            __half2 d[4];
            dequant_word(uint32_t(qw[size_t(k) * NW + j]), z, d);
            float xv = x[k];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float2 f = __half22float2(d[i]);
                part[2 * i] = fmaf(f.x, xv, part[2 * i]);
                part[2 * i + 1] = fmaf(f.y, xv, part[2 * i + 1]);
            }
        }
#pragma unroll
        for (int c = 0; c < 8; c++) acc[c] = fmaf(part[c], __half2float(scales[size_t(g) * N + 8 * j + c]), acc[c]);
    }
#pragma unroll
    for (int c = 0; c < 8; c++) {
        float v = acc[c];
        if (residual) v += residual[8 * j + c];
        y[8 * j + c] = v;
    }
}

int g_force_rows = 0;  // tuning override: rows per thread (4, 8 or 16); 0 = heuristic
int g_force_math = -1;
int g_force_impl = 0;  // 0: persistent tensor-core kernel where it applies; 2: persistent SIMT kernel; 1: register-staged kernel

int pick_rows(int K, int N) {
    if (g_force_rows == 4 || g_force_rows == 8 || g_force_rows == 16) return g_force_rows;
    const int tiles = (N + kTileCols - 1) / kTileCols;
    // largest K slice that still gives about one and a half CTAs per SM
    for (int rows : {16, 8}) {
        if (tiles * (K / (rows * kWarps)) >= 222) return rows;
    }
    return 4;
}

template <int MODE, int MT, int ROWS>
int launch(const GemvParams& p, cudaStream_t stream) {
    auto kern = awq_gemv_kernel<MODE, MT, ROWS>;
    const size_t smem = size_t(kWarps) * MT * 256 * sizeof(float4);
    static size_t configured[kMaxDevices] = {};  // per instantiation and device
    if (!ensure_dynamic_smem(kern, smem, configured)) {
        set_error("awq_gemv: cannot reserve %zu bytes of shared memory", smem);
        return KUIPER_INTERNAL_ERROR;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((p.N + kTileCols - 1) / kTileCols, p.S, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl_enabled ? 1 : 0;
    cudaError_t err = cudaLaunchKernelEx(&cfg, kern, p);
    if (err != cudaSuccess) {
        set_error("awq_gemv launch failed: %s", cudaGetErrorString(err));
        return KUIPER_INTERNAL_ERROR;
    }
    return KUIPER_OK;
}

template <int MODE, int MT>
int launch_rows(const GemvParams& p, int rows, cudaStream_t stream) {
    switch (rows) {
        case 16: return launch<MODE, MT, 16>(p, stream);
        case 8: return launch<MODE, MT, 8>(p, stream);
        default: return launch<MODE, MT, 4>(p, stream);
    }
}

template <int MT>
int launch_mode(const GemvParams& p, int mode, int rows, cudaStream_t stream) {
    switch (mode) {
        case kMathF32: return launch_rows<kMathF32, MT>(p, rows, stream);
        case kMathHalf2: return launch_rows<kMathHalf2, MT>(p, rows, stream);
        default: return launch_rows<kMathMixed, MT>(p, rows, stream);
    }
}

}  // namespace

// tuning hooks used by the benchmark sweeps
void awq_gemv_tma_set_tuning(const char* key, int value);
void awq_gemv_mma_set_tuning(const char* key, int value);

void awq_gemv_set_tuning(const char* key, int value) {
    if (!strcmp(key, "gemv_rows")) g_force_rows = value;
    if (!strcmp(key, "gemv_math")) g_force_math = value;
    if (!strcmp(key, "gemv_impl")) g_force_impl = value;
    awq_gemv_tma_set_tuning(key, value);
    awq_gemv_mma_set_tuning(key, value);
}

// persistent TMA-fed variant (awq_gemv_tma.cu)
size_t awq_gemv_tma_workspace_bytes(int K, int N);
bool awq_gemv_tma_supported(int K, int N);
int awq_gemv_tma_status();
int awq_gemv_tma_launch(const float* x, const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales, float* y,
                        const float* residual, int rows, int K, int N, void* workspace, bool accumulate,
                        const uint16_t* norm_w, float eps, cudaStream_t stream);

// persistent TMA-fed variant with the dot products on the tensor cores (awq_gemv_mma.cu)
bool awq_gemv_mma_supported(int K, int N);
int awq_gemv_mma_status();
int awq_gemv_mma_max_rows(bool accumulate);
int awq_gemv_mma_launch(const float* x, const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales, float* y,
                        const float* residual, int rows, int K, int N, void* workspace, bool accumulate,
                        const uint16_t* norm_w, float eps, bool swiglu, int* tickets, bool int_operand, cudaStream_t stream);
size_t awq_gemv_group_table_bytes(int n_items);
long long awq_gemv_group_fill(const kuiper_gemv_item* items, int n_items, void* host_table);
int awq_gemv_group_launch(const void* device_table, int n_items, long long units, int* tickets, bool int_operand,
                          cudaStream_t stream);

}  // namespace kuiper

using namespace kuiper;

extern "C" size_t kuiper_awq_gemv_workspace_bytes(int M, int K, int N) {
    if (M <= 0 || K <= 0 || N <= 0) return 0;
    // up to K/32 K slices of two rows each, plus one counter per column tile
    const size_t slices = size_t(K) / 32;
    const size_t partial = slices * 2 * size_t(N) * sizeof(float);
    const size_t counters = size_t((N + kTileCols - 1) / kTileCols) * sizeof(int);
    const size_t legacy = ((counters + 255) / 256) * 256 + partial;
    const size_t tma = awq_gemv_tma_workspace_bytes(K, N);
    return legacy > tma ? legacy : tma;
}

extern "C" int kuiper_awq_gemv_f32(const float* x, const int32_t* qweight, const int32_t* qzeros,
                                   const uint16_t* scales, float* y, const float* residual,
                                   int M, int K, int N, int group, int act_mode,
                                   void* workspace, size_t workspace_bytes, kuiper_stream_t stream) {
    KUIPER_REQUIRE(x && qweight && qzeros && scales && y, "awq_gemv: null tensor pointer");
    KUIPER_REQUIRE(M > 0 && K > 0 && N > 0, "awq_gemv: empty shape M=%d K=%d N=%d", M, K, N);
    KUIPER_REQUIRE(group == 128, "awq_gemv: group size %d is not supported (128 only)", group);
    KUIPER_REQUIRE(K % 128 == 0, "awq_gemv: K=%d is not a multiple of the group size", K);
    KUIPER_REQUIRE(N % 8 == 0, "awq_gemv: N=%d is not a multiple of 8", N);
    KUIPER_REQUIRE(act_mode == KUIPER_ACT_FP16 || act_mode == KUIPER_ACT_FP32 || act_mode == KUIPER_ACT_INT16_BLOCK,
                   "awq_gemv: unknown act_mode %d", act_mode);
    cudaStream_t st = as_stream(stream);

    if (N % 32 != 0) {
        const int NW = N / 8;
        for (int m = 0; m < M; m++) {
            awq_gemv_generic_kernel<<<(NW + 127) / 128, 128, 0, st>>>(
                x + size_t(m) * K, qweight, qzeros, reinterpret_cast<const __half*>(scales), y + size_t(m) * N,
                residual ? residual + size_t(m) * N : nullptr, K, N);
        }
        return launch_status("awq_gemv_generic");
    }

    KUIPER_REQUIRE((reinterpret_cast<uintptr_t>(qweight) & 15) == 0 && (reinterpret_cast<uintptr_t>(qzeros) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(scales) & 15) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(x) & 3) == 0 && (!residual || (reinterpret_cast<uintptr_t>(residual) & 15) == 0),
                   "awq_gemv: tensors must be 16-byte aligned");
    const bool int_operand = act_mode == KUIPER_ACT_INT16_BLOCK && M == 1;  // more rows round to fp16
    KUIPER_REQUIRE(!int_operand || (g_force_impl == 0 && g_force_math < 0 && awq_gemv_mma_supported(K, N)),
                   "awq_gemv: the integer operand needs the tensor-core kernel (N %% 32 == 0, K %% 128 == 0)");
    const bool want_tma = (g_force_impl == 0 || g_force_impl == 2) && g_force_math < 0 && act_mode != KUIPER_ACT_FP32 &&
                          awq_gemv_tma_supported(K, N);
    if (want_tma) {
        const bool mma = g_force_impl == 0 && awq_gemv_mma_supported(K, N);
        KUIPER_REQUIRE(workspace != nullptr && workspace_bytes >= awq_gemv_tma_workspace_bytes(K, N),
                       "awq_gemv: workspace of %zu bytes is too small", workspace_bytes);
        KUIPER_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 15) == 0, "awq_gemv: workspace must be 16-byte aligned");
        for (int m0 = 0; m0 < M;) {
            const int mt = (M - m0 >= 2) ? 2 : 1;
            const float* xm = x + size_t(m0) * K;
            float* ym = y + size_t(m0) * N;
            const float* rm = residual ? residual + size_t(m0) * N : nullptr;
            int rc = mma ? awq_gemv_mma_launch(xm, qweight, qzeros, scales, ym, rm, mt, K, N, workspace, false, nullptr, 0.f, false, nullptr,
                                               int_operand, st)
                         : awq_gemv_tma_launch(xm, qweight, qzeros, scales, ym, rm, mt, K, N, workspace, false, nullptr, 0.f, st);
            if (rc != KUIPER_OK) return rc;
            m0 += mt;
        }
        return KUIPER_OK;
    }

    const int rows = pick_rows(K, N);
    const int S = K / (rows * kWarps);
    const size_t counters_bytes = ((size_t((N + kTileCols - 1) / kTileCols) * sizeof(int) + 255) / 256) * 256;
    if (S > 1) {
        KUIPER_REQUIRE(workspace != nullptr, "awq_gemv: split-K needs a workspace");
        KUIPER_REQUIRE(workspace_bytes >= counters_bytes + size_t(S) * 2 * N * sizeof(float),
                       "awq_gemv: workspace of %zu bytes is too small", workspace_bytes);
        KUIPER_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 15) == 0, "awq_gemv: workspace must be 16-byte aligned");
    }
    KUIPER_REQUIRE((reinterpret_cast<uintptr_t>(qweight) & 15) == 0 && (reinterpret_cast<uintptr_t>(qzeros) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(scales) & 7) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0 &&
                       (!residual || (reinterpret_cast<uintptr_t>(residual) & 15) == 0),
                   "awq_gemv: tensors must be 16-byte aligned");

    int mode = act_mode == KUIPER_ACT_FP32 ? kMathF32 : kMathMixed;
    if (g_force_math >= 0) mode = g_force_math;

    GemvParams p;
    p.qw = reinterpret_cast<const uint4*>(qweight);
    p.qz = reinterpret_cast<const uint4*>(qzeros);
    p.scales = reinterpret_cast<const __half*>(scales);
    p.counters = reinterpret_cast<int*>(workspace);
    p.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + counters_bytes);
    p.K = K;
    p.N = N;
    p.nchunks = N / 32;
    p.S = S;
    for (int m0 = 0; m0 < M;) {
        const int mt = (M - m0 >= 2) ? 2 : 1;
        p.x = x + size_t(m0) * K;
        p.y = y + size_t(m0) * N;
        p.residual = residual ? residual + size_t(m0) * N : nullptr;
        int rc = mt == 2 ? launch_mode<2>(p, mode, rows, st) : launch_mode<1>(p, mode, rows, st);
        if (rc != KUIPER_OK) return rc;
        m0 += mt;
    }
    return KUIPER_OK;
}

static int awq_gemv_accum_common(const float* x, const uint16_t* norm_w, float eps, bool swiglu, const int32_t* qweight,
                                 const int32_t* qzeros, const uint16_t* scales, float* y, int M, int K, int N, int group,
                                 void* tickets, int act_mode, kuiper_stream_t stream) {
    KUIPER_REQUIRE(act_mode == KUIPER_ACT_FP16 || act_mode == KUIPER_ACT_INT16_BLOCK, "awq_gemv_accum: unknown act_mode %d", act_mode);
    KUIPER_REQUIRE(x && qweight && qzeros && scales && y, "awq_gemv_accum: null tensor pointer");
    KUIPER_REQUIRE(M > 0 && K > 0 && N > 0, "awq_gemv_accum: empty shape M=%d K=%d N=%d", M, K, N);
    KUIPER_REQUIRE(group == 128, "awq_gemv_accum: group size %d is not supported (128 only)", group);
    KUIPER_REQUIRE(K % 128 == 0 && N % 32 == 0, "awq_gemv_accum: needs K %% 128 == 0 and N %% 32 == 0 (K=%d N=%d)", K, N);
    KUIPER_REQUIRE(((reinterpret_cast<uintptr_t>(qweight) | reinterpret_cast<uintptr_t>(qzeros) | reinterpret_cast<uintptr_t>(scales) |
                     reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(x)) & 15) == 0,
                   "awq_gemv_accum: tensors must be 16-byte aligned");
    KUIPER_REQUIRE(awq_gemv_tma_supported(K, N), "awq_gemv_accum: tensor-map support is unavailable");
    cudaStream_t st = as_stream(stream);
    const bool mma = g_force_impl != 2 && awq_gemv_mma_supported(K, N);
    KUIPER_REQUIRE(mma || !swiglu, "awq_gemv_accum: the fused SwiGLU needs the tensor-core kernel");
    KUIPER_REQUIRE((reinterpret_cast<uintptr_t>(tickets) & 7) == 0, "awq_gemv_accum: tickets must be 8-byte aligned");
    // (more rows than one launch takes: the row blocks are consecutive launches that may overlap, so they cannot
    // share the counters and are dealt out statically)
    // the integer operand is a one-row kernel: it serves single-row calls, everything else rounds to fp16
    const bool int_operand = act_mode == KUIPER_ACT_INT16_BLOCK && M == 1 && mma;
    const int max_rows = mma ? awq_gemv_mma_max_rows(true) : 2;
    for (int m0 = 0; m0 < M;) {
        const int mt = (M - m0 >= max_rows) ? max_rows : (M - m0);
        const float* xm = x + size_t(m0) * K * (swiglu ? 2 : 1);
        float* ym = y + size_t(m0) * N;
        int rc = mma ? awq_gemv_mma_launch(xm, qweight, qzeros, scales, ym, nullptr, mt, K, N, nullptr, true, norm_w, eps, swiglu,
                                         M <= max_rows ? static_cast<int*>(tickets) : nullptr, int_operand, st)
                     : awq_gemv_tma_launch(xm, qweight, qzeros, scales, ym, nullptr, mt, K, N, nullptr, true, norm_w, eps, st);
        if (rc != KUIPER_OK) return rc;
        m0 += mt;
    }
    return KUIPER_OK;
}

extern "C" int kuiper_awq_gemv_accum_f32(const float* x, const int32_t* qweight, const int32_t* qzeros,
                                         const uint16_t* scales, float* y, int M, int K, int N, int group,
                                         kuiper_stream_t stream) {
    return awq_gemv_accum_common(x, nullptr, 0.f, false, qweight, qzeros, scales, y, M, K, N, group, nullptr, KUIPER_ACT_FP16, stream);
}

extern "C" int kuiper_rmsnorm_awq_gemv_accum_f32(const float* h, const uint16_t* norm_w, float eps, const int32_t* qweight,
                                                 const int32_t* qzeros, const uint16_t* scales, float* y, int M, int K,
                                                 int N, int group, kuiper_stream_t stream) {
    KUIPER_REQUIRE(norm_w != nullptr, "rmsnorm_awq_gemv_accum: null norm weight");
    KUIPER_REQUIRE((reinterpret_cast<uintptr_t>(norm_w) & 15) == 0, "rmsnorm_awq_gemv_accum: norm weight must be 16-byte aligned");
    return awq_gemv_accum_common(h, norm_w, eps, false, qweight, qzeros, scales, y, M, K, N, group, nullptr, KUIPER_ACT_FP16, stream);
}

extern "C" int kuiper_swiglu_awq_gemv_accum_f32(const float* gate_up, const int32_t* qweight, const int32_t* qzeros,
                                                const uint16_t* scales, float* y, int M, int K, int N, int group,
                                                kuiper_stream_t stream) {
    return awq_gemv_accum_common(gate_up, nullptr, 0.f, true, qweight, qzeros, scales, y, M, K, N, group, nullptr, KUIPER_ACT_FP16, stream);
}

#ifdef KUIPER_TRACE
namespace kuiper {
int awq_gemv_trace_read(long long* out, int max_values);
}
extern "C" KUIPER_API int kuiper_gemv_trace_read(int64_t* out, int max_values) {
    KUIPER_REQUIRE(out != nullptr && max_values > 0, "gemv_trace_read: empty destination");
    return kuiper::awq_gemv_trace_read(reinterpret_cast<long long*>(out), max_values);
}
#endif

extern "C" size_t kuiper_awq_gemv_ticket_bytes(void) { return 2 * sizeof(int); }

extern "C" int kuiper_awq_gemv_accum_balanced_f32(const float* x, const uint16_t* norm_w, float eps, int swiglu,
                                                  const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales,
                                                  float* y, int M, int K, int N, int group, int act_mode, void* tickets,
                                                  kuiper_stream_t stream) {
    KUIPER_REQUIRE(!(norm_w && swiglu), "awq_gemv_accum_balanced: the fused norm and the fused SwiGLU exclude each other");
    KUIPER_REQUIRE((reinterpret_cast<uintptr_t>(norm_w) & 15) == 0, "awq_gemv_accum_balanced: norm weight must be 16-byte aligned");
    return awq_gemv_accum_common(x, norm_w, eps, swiglu != 0, qweight, qzeros, scales, y, M, K, N, group, tickets, act_mode, stream);
}

extern "C" size_t kuiper_awq_gemv_group_table_bytes(int n_items) { return awq_gemv_group_table_bytes(n_items); }

extern "C" int kuiper_awq_gemv_group_plan(const kuiper_gemv_item* items, int n_items, int group, void* host_table,
                                          int64_t* units) {
    KUIPER_REQUIRE(items && host_table && units, "awq_gemv_group_plan: null pointer");
    KUIPER_REQUIRE(n_items > 0 && n_items <= 65536, "awq_gemv_group_plan: %d items", n_items);
    KUIPER_REQUIRE(group == 128, "awq_gemv_group_plan: group size %d is not supported (128 only)", group);
    KUIPER_REQUIRE(awq_gemv_mma_supported(128, 32), "awq_gemv_group_plan: tensor-map support is unavailable");
    for (int i = 0; i < n_items; i++) {
        const kuiper_gemv_item& o = items[i];
        KUIPER_REQUIRE(o.x && o.qweight && o.qzeros && o.scales && o.y, "awq_gemv_group_plan: null tensor pointer in item %d", i);
        KUIPER_REQUIRE(o.K > 0 && o.N > 0 && o.K % 128 == 0 && o.N % 32 == 0,
                       "awq_gemv_group_plan: item %d needs K %% 128 == 0 and N %% 32 == 0 (K=%d N=%d)", i, o.K, o.N);
        KUIPER_REQUIRE(((reinterpret_cast<uintptr_t>(o.qweight) | reinterpret_cast<uintptr_t>(o.qzeros) |
                         reinterpret_cast<uintptr_t>(o.scales) | reinterpret_cast<uintptr_t>(o.y) | reinterpret_cast<uintptr_t>(o.x)) & 15) == 0,
                       "awq_gemv_group_plan: tensors of item %d must be 16-byte aligned", i);
    }
    const long long u = awq_gemv_group_fill(items, n_items, host_table);
    if (u <= 0) {
        set_error("awq_gemv_group_plan: tensor map encoding failed or the list is too long");
        return KUIPER_INTERNAL_ERROR;
    }
    *units = u;
    return KUIPER_OK;
}

extern "C" int kuiper_awq_gemv_group_f32(const void* device_table, int n_items, int64_t units, int act_mode, void* tickets,
                                         kuiper_stream_t stream) {
    KUIPER_REQUIRE(act_mode == KUIPER_ACT_FP16 || act_mode == KUIPER_ACT_INT16_BLOCK, "awq_gemv_group: unknown act_mode %d", act_mode);
    KUIPER_REQUIRE(device_table && (reinterpret_cast<uintptr_t>(device_table) & 63) == 0,
                   "awq_gemv_group: the item table must be 64-byte aligned device memory");
    KUIPER_REQUIRE(n_items > 0 && units > 0 && units <= 0x3fffffff, "awq_gemv_group: empty call");
    KUIPER_REQUIRE((reinterpret_cast<uintptr_t>(tickets) & 7) == 0, "awq_gemv_group: tickets must be 8-byte aligned");
    return awq_gemv_group_launch(device_table, n_items, units, static_cast<int*>(tickets), act_mode == KUIPER_ACT_INT16_BLOCK,
                                 as_stream(stream));
}

extern "C" int kuiper_awq_gemv_status(void) {
    int v = awq_gemv_tma_status();
    if (v == 0) v = awq_gemv_mma_status();
    if (v == 0) return KUIPER_OK;
    set_error("awq_gemv: a bounded pipeline wait ran out (code %d)", v);
    return KUIPER_INTERNAL_ERROR;
}
