// Shared helpers of the sm_100a decode kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <utility>

#include "kuiper_b200.h"

namespace kuiper {

// tuning: 0 launches every kernel without the programmatic-dependent-launch attribute
extern int g_pdl_enabled;

// thread-local text behind kuiper_last_error()
void set_error(const char* fmt, ...);

#define KUIPER_REQUIRE(cond, ...)                 \
    do {                                          \
        if (!(cond)) {                            \
            ::kuiper::set_error(__VA_ARGS__);     \
            return KUIPER_INVALID_ARGUMENT;       \
        }                                         \
    } while (0)

// after a launch: map a launch failure onto the InternalError status
inline int launch_status(const char* what) {
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        set_error("%s launch failed: %s", what, cudaGetErrorString(err));
        return KUIPER_INTERNAL_ERROR;
    }
    return KUIPER_OK;
}

// Launch with the programmatic-dependent-launch attribute: the kernel may be scheduled while its
// predecessor in the stream is still running, so it must call pdl_wait() before touching anything
// the predecessor produces (every kernel of this library does, at its top or after a prefetch).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl_enabled ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

inline int pdl_status(cudaError_t err, const char* what) {
    if (err != cudaSuccess) {
        set_error("%s launch failed: %s", what, cudaGetErrorString(err));
        return KUIPER_INTERNAL_ERROR;
    }
    return KUIPER_OK;
}

inline cudaStream_t as_stream(kuiper_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// Per-device facts and one-time settings.  cudaFuncSetAttribute and the SM count belong to a device, not to the
// process, so both are tracked per device ordinal (a process may drive several GPUs).  Races between host threads
// are benign: every writer stores the same value, and setting a function attribute twice is harmless.
constexpr int kMaxDevices = 64;
inline int current_device() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= kMaxDevices) d = 0;
    return d;
}
inline int device_sm_count() {
    static int count[kMaxDevices] = {};
    const int d = current_device();
    if (count[d] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, d) != cudaSuccess || n <= 0) n = 148;
        count[d] = n;
    }
    return count[d];
}
// raises the dynamic shared-memory limit of `kernel` on the current device the first time it is launched there;
// `done` is the caller's per-instantiation table
template <typename Kernel>
inline bool ensure_dynamic_smem(Kernel kernel, size_t bytes, size_t (&done)[kMaxDevices]) {
    const int d = current_device();
    if (done[d] >= bytes && done[d] != 0) return true;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes)) != cudaSuccess) return false;
    done[d] = bytes;
    return true;
}

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float(uint32_t(b) << 16); }
// low / high bf16 of a packed 32-bit word
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ uint16_t float_to_bf16_bits(float f) {
    uint32_t u = __float_as_uint(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return uint16_t(u >> 16);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// streaming 16-byte load that does not allocate in L1 (weights are read exactly once)
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

// Programmatic dependent launch: let the next grid start its prologue, and wait for
// the previous grid's writes before touching anything it produced.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

}  // namespace kuiper
