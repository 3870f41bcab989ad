// BF16 GEMV for sm_100a: y[M,N] = x[M,K] . W[N,K]^T, W in bf16 (the lm_head, one row
// per vocabulary entry).  Fills the non-quantised side of the reference's empty matmul
// placeholder (kuiper/include/op/matmul.h:1-11).
//
// A warp owns whole weight rows: 32 lanes x 16 bytes = one 512-byte coalesced run per
// load, four loads in flight per lane, rows strided over all warps of a persistent grid
// (4 CTAs per SM).  x sits in shared memory as fp32 and is read as two float4 per
// 16-byte weight chunk; accumulation is fp32; one shuffle reduction per row.
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

}  // namespace
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
