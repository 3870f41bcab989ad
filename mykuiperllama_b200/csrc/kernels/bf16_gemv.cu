// BF16 GEMV for sm_100a: y[M,N] = x[M,K] . W[N,K]^T, W in bf16 (the lm_head, one row
// per vocabulary entry).  Fills the non-quantised side of the reference's empty matmul
// placeholder (kuiper/include/op/matmul.h:1-11).
//
// A warp owns whole weight rows: 32 lanes x 16 bytes = one 512-byte coalesced run per
// load, four loads in flight per lane, rows strided over all warps of a persistent grid
// (4 CTAs per SM).  x sits in shared memory as fp32 and is read as two float4 per
// 16-byte weight chunk; accumulation is fp32; one shuffle reduction per row.  Calls of three rows or more take the
// tensor-core kernel further down.
#include <cstring>

#include "common.cuh"

namespace kuiper {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

template <int MT>
__device__ __forceinline__ void fma_chunk(const uint4& w, const float* xs, int K, int k, float (&acc)[MT]) {
    const float wf[8] = {bf16_lo(w.x), bf16_hi(w.x), bf16_lo(w.y), bf16_hi(w.y),
                         bf16_lo(w.z), bf16_hi(w.z), bf16_lo(w.w), bf16_hi(w.w)};
#pragma unroll
    for (int m = 0; m < MT; m++) {
        // x is stored split: first halves of every 8-element chunk, then second halves,
        // so that the 16-byte reads of a warp are contiguous (no bank conflicts)
        const float4 a = reinterpret_cast<const float4*>(xs + m * K)[k >> 3];
        const float4 b = reinterpret_cast<const float4*>(xs + m * K)[(K >> 3) + (k >> 3)];
        float s = acc[m];
        s = fmaf(wf[0], a.x, s); s = fmaf(wf[1], a.y, s); s = fmaf(wf[2], a.z, s); s = fmaf(wf[3], a.w, s);
        s = fmaf(wf[4], b.x, s); s = fmaf(wf[5], b.y, s); s = fmaf(wf[6], b.z, s); s = fmaf(wf[7], b.w, s);
        acc[m] = s;
    }
}

template <int MT>
__global__ void __launch_bounds__(kThreads, 4)
bf16_gemv_kernel(const float* x, const uint16_t* __restrict__ W, float* y, int K, int N) {
    extern __shared__ float xs[];  // [MT][K]
    const int lane = threadIdx.x & 31;
    const int warp_global = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    const int warps_total = gridDim.x * (kThreads / 32);
    const int steps = K / 256;  // full 512-byte steps per row

    pdl_launch_dependents();
    pdl_wait();
    for (int i = threadIdx.x; i < MT * K / 4; i += kThreads) {
        const int m = i / (K / 4), f = i - m * (K / 4);
        reinterpret_cast<float4*>(xs + m * K)[(f & 1) * (K >> 3) + (f >> 1)] = __ldcg(reinterpret_cast<const float4*>(x) + i);
    }
    __syncthreads();

    for (int n = warp_global; n < N; n += warps_total) {
        const uint4* row = reinterpret_cast<const uint4*>(W + size_t(n) * K);
        float acc[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) acc[m] = 0.f;
        int s = 0;
        for (; s + kUnroll <= steps; s += kUnroll) {
            uint4 w[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; u++) w[u] = ld_stream_u4(row + (s + u) * 32 + lane);
#pragma unroll
            for (int u = 0; u < kUnroll; u++) fma_chunk<MT>(w[u], xs, K, ((s + u) * 32 + lane) * 8, acc);
        }
        for (; s < steps; s++) {
            uint4 w = ld_stream_u4(row + s * 32 + lane);
            fma_chunk<MT>(w, xs, K, (s * 32 + lane) * 8, acc);
        }
        // tail of K (multiple of 8, shorter than one warp step)
        const int kt = steps * 256 + lane * 8;
        if (kt < K) {
            uint4 w = ld_stream_u4(row + steps * 32 + lane);
            fma_chunk<MT>(w, xs, K, kt, acc);
        }
#pragma unroll
        for (int m = 0; m < MT; m++) {
            float v = warp_sum(acc[m]);
            if (lane == 0) y[size_t(m) * N + n] = v;
        }
    }
}

template <int MT>
int launch(const float* x, const uint16_t* W, float* y, int K, int N, cudaStream_t stream) {
    auto kern = bf16_gemv_kernel<MT>;
    const size_t smem = size_t(MT) * K * sizeof(float);
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    const int rows_per_cta = kThreads / 32;
    int grid = 148 * 4;
    if (grid > (N + rows_per_cta - 1) / rows_per_cta) grid = (N + rows_per_cta - 1) / rows_per_cta;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl_enabled ? 1 : 0;
    cudaError_t err = cudaLaunchKernelEx(&cfg, kern, x, W, y, K, N);
    if (err != cudaSuccess) {
        set_error("bf16_gemv launch failed: %s", cudaGetErrorString(err));
        return KUIPER_INTERNAL_ERROR;
    }
    return KUIPER_OK;
}

// ---------------------------------------------------------------------------------------------
// Three to eight token rows per pass on the tensor cores.  With several rows the SIMT kernel above is bound by its
// shared-memory reads of x (4 rows: 223 us for 151 936 x 2560, twice the time of one row), so decode batches paid a
// weight pass per 2-4 sequences.  Here a warp owns 16 weight rows: they are the A operand of mma.sync.m16n8k16 (bf16,
// straight from global memory: lane (g, tig) loads 16 bytes of rows g and g + 8, which are its fragments for two
// contraction steps - the contraction index is permuted the same way on both operands), the eight columns of B are the
// token rows.  x is split once per CTA into three bf16 planes (x = hi + mid + lo exactly to 24 bits), so the products
// are those of the fp32 operand; accumulation is fp32.  One CTA of 16 warps per SM (the planes take up to 198 KB).
constexpr int kMmaThreads = 512;
constexpr int kMmaRows = 8;     // token rows per pass
constexpr int kMmaUnroll = 4;   // 32-column steps in flight per lane

__device__ __forceinline__ uint32_t bf16_round_bits(float v) {  // round to nearest even, as the reference conversion does
    const uint32_t u = __float_as_uint(v);
    return (u + 0x7fffu + ((u >> 16) & 1u)) >> 16;
}

__global__ void __launch_bounds__(kMmaThreads, 1)
bf16_rows_mma_kernel(const float* x, const uint16_t* __restrict__ W, float* y, int M, int K, int N) {
    extern __shared__ __align__(16) unsigned char planes[];  // [3 planes][8 rows][2 K + 64 bytes]
    const int row_bytes = 2 * K + 64;  // the 64 bytes stagger the rows over the banks (16-byte reads of a quarter warp)
    const int lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
    const int warp_global = blockIdx.x * (kMmaThreads / 32) + (threadIdx.x >> 5);
    const int warps_total = gridDim.x * (kMmaThreads / 32);

    pdl_launch_dependents();
    pdl_wait();
    for (int i = threadIdx.x; i < kMmaRows * (K >> 1); i += kMmaThreads) {
        const int m = i / (K >> 1), k = (i - m * (K >> 1)) * 2;
        float2 v = make_float2(0.f, 0.f);
        if (m < M) v = __ldcg(reinterpret_cast<const float2*>(x + size_t(m) * K + k));
        float r0 = v.x, r1 = v.y;
#pragma unroll
        for (int p = 0; p < 3; p++) {
            const uint32_t b0 = bf16_round_bits(r0), b1 = bf16_round_bits(r1);
            *reinterpret_cast<uint32_t*>(planes + size_t(p * kMmaRows + m) * row_bytes + k * 2) = b0 | (b1 << 16);
            r0 -= __uint_as_float(b0 << 16);  // exact: the part just taken out
            r1 -= __uint_as_float(b1 << 16);
        }
    }
    __syncthreads();

    const unsigned char* xrow = planes + size_t(g) * row_bytes + tig * 16;
    const size_t plane_bytes = size_t(kMmaRows) * row_bytes;
    for (int n0 = warp_global * 16; n0 < N; n0 += warps_total * 16) {
        const int ra = min(n0 + g, N - 1), rb = min(n0 + g + 8, N - 1);  // rows past the end repeat the last one, unused
        const uint16_t* pa = W + size_t(ra) * K + tig * 8;
        const uint16_t* pb = W + size_t(rb) * K + tig * 8;
        // The tensor core adds into its fp32 accumulator by truncation, which over the 768 mma of a 4096-column row
        // drifts to ~1e-5 of the result; so a chain is kept to the six mma of one 32-column step and the steps are
        // summed with ordinary fp32 additions.
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int kk = 0; kk < K; kk += 32 * kMmaUnroll) {
            uint4 wa[kMmaUnroll], wb[kMmaUnroll];
#pragma unroll
            for (int u = 0; u < kMmaUnroll; u++) {
                const bool in = kk + u * 32 < K;
                wa[u] = in ? ld_stream_u4(pa + kk + u * 32) : make_uint4(0, 0, 0, 0);
                wb[u] = in ? ld_stream_u4(pb + kk + u * 32) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < kMmaUnroll; u++) {
                if (kk + u * 32 < K) {
                    float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int p = 2; p >= 0; p--) {  // smallest parts first
                        const uint4 xb = *reinterpret_cast<const uint4*>(xrow + p * plane_bytes + size_t(kk + u * 32) * 2);
                        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                                     : "r"(wa[u].x), "r"(wb[u].x), "r"(wa[u].y), "r"(wb[u].y), "r"(xb.x), "r"(xb.y));
                        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                                     : "r"(wa[u].z), "r"(wb[u].z), "r"(wa[u].w), "r"(wb[u].w), "r"(xb.z), "r"(xb.w));
                    }
                    acc[0] += d[0]; acc[1] += d[1]; acc[2] += d[2]; acc[3] += d[3];
                }
            }
        }
        // accumulator rows g, g + 8 = weight rows; columns 2 tig, 2 tig + 1 = token rows
        const int m0 = 2 * tig, m1 = 2 * tig + 1;
        if (n0 + g < N) {
            if (m0 < M) y[size_t(m0) * N + n0 + g] = acc[0];
            if (m1 < M) y[size_t(m1) * N + n0 + g] = acc[1];
        }
        if (n0 + g + 8 < N) {
            if (m0 < M) y[size_t(m0) * N + n0 + g + 8] = acc[2];
            if (m1 < M) y[size_t(m1) * N + n0 + g + 8] = acc[3];
        }
    }
}

int g_bf16_mma = 1;  // tuning key "bf16_mma": 0 keeps every call on the SIMT kernel

size_t mma_smem_bytes(int K) { return size_t(3 * kMmaRows) * size_t(2 * K + 64); }

int launch_mma_rows(const float* x, const uint16_t* W, float* y, int M, int K, int N, cudaStream_t stream) {
    const size_t smem = mma_smem_bytes(K);
    static size_t configured[kMaxDevices] = {};
    if (!ensure_dynamic_smem(bf16_rows_mma_kernel, smem, configured)) {
        set_error("bf16_gemv: cannot reserve %zu bytes of shared memory", smem);
        return KUIPER_INTERNAL_ERROR;
    }
    int grid = device_sm_count();
    const int groups = (N + 15) / 16, per_cta = kMmaThreads / 32;
    if (grid > (groups + per_cta - 1) / per_cta) grid = (groups + per_cta - 1) / per_cta;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(kMmaThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl_enabled ? 1 : 0;
    cudaError_t err = cudaLaunchKernelEx(&cfg, bf16_rows_mma_kernel, x, W, y, M, K, N);
    if (err != cudaSuccess) {
        set_error("bf16_gemv (tensor-core rows) launch failed: %s", cudaGetErrorString(err));
        return KUIPER_INTERNAL_ERROR;
    }
    return KUIPER_OK;
}

}  // namespace

void bf16_gemv_set_tuning(const char* key, int value) {
    if (!strcmp(key, "bf16_mma")) g_bf16_mma = value;
}

}  // namespace kuiper

using namespace kuiper;

extern "C" int kuiper_bf16_gemv_f32(const float* x, const uint16_t* W, float* y, int M, int K, int N,
                                    kuiper_stream_t stream) {
    KUIPER_REQUIRE(x && W && y, "bf16_gemv: null tensor pointer");
    KUIPER_REQUIRE(M > 0 && K > 0 && N > 0, "bf16_gemv: empty shape M=%d K=%d N=%d", M, K, N);
    KUIPER_REQUIRE(K % 8 == 0, "bf16_gemv: K=%d is not a multiple of 8", K);
    KUIPER_REQUIRE(size_t(K) * 4 * sizeof(float) <= 200 * 1024, "bf16_gemv: K=%d does not fit shared memory", K);
    KUIPER_REQUIRE((reinterpret_cast<uintptr_t>(W) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0,
                   "bf16_gemv: x and W must be 16-byte aligned");
    cudaStream_t st = as_stream(stream);
    // three rows or more: passes of up to eight rows on the tensor cores (K in whole 32-column steps, planes in shared memory)
    if (g_bf16_mma && M >= 3 && K % 32 == 0 && mma_smem_bytes(K) <= 220 * 1024) {
        for (int m0 = 0; m0 < M; m0 += kMmaRows) {
            const int rows = M - m0 < kMmaRows ? M - m0 : kMmaRows;
            const int rc = launch_mma_rows(x + size_t(m0) * K, W, y + size_t(m0) * N, rows, K, N, st);
            if (rc != KUIPER_OK) return rc;
        }
        return KUIPER_OK;
    }
    for (int m0 = 0; m0 < M;) {
        const int left = M - m0;
        int rc;
        const float* xp = x + size_t(m0) * K;
        float* yp = y + size_t(m0) * N;
        if (left >= 4) { rc = launch<4>(xp, W, yp, K, N, st); m0 += 4; }
        else if (left >= 2) { rc = launch<2>(xp, W, yp, K, N, st); m0 += 2; }
        else { rc = launch<1>(xp, W, yp, K, N, st); m0 += 1; }
        if (rc != KUIPER_OK) return rc;
    }
    return KUIPER_OK;
}
