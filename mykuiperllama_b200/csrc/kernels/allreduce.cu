// One-shot all-reduce (sum, fp32) over peer-mapped buffers for the tensor-parallel decode step.
//
// The row-split projections (O and down) leave a partial row of `hidden` floats on every rank and the step
// needs their sum 72 times per token.  At 16 KB a library all-reduce is pure latency, so each rank instead
// stores its partial row straight into a slot of every peer's exchange buffer (plain stores over NVLink),
// raises a per-source flag there, waits for the flags of all sources in its own buffer and adds the slots in
// rank order (every rank computes the same sum in the same order: bit-identical results on all ranks).
// The reference has no multi-GPU code; this sits behind parallel::Communicator.
//
// Exchange buffer of one rank (kuiper_allreduce_buffer_bytes):
//   data  [2 parities][world][max_count floats]      slot (parity, src) is written by rank src only
//   flags [2 parities][world] uint32, 128 bytes apart  flag (parity, src) = sequence number of the data in the slot
// Two parities: a rank can be one all-reduce ahead of a peer (it has all flags of call k, the peer may still be
// adding the slots of call k), never two (it would need the peer's flag of call k + 1, raised after the peer
// finished call k).
//
// Every wait is bounded by a wall-clock limit; when it runs out the kernel records an error word and returns
// (the result of that call is then void).  No multicast, no library call on peer memory.
#include <cstring>

#include "common.cuh"

namespace kuiper {
namespace {

constexpr int kArMaxWorld = 8;
constexpr int kArThreads = 1024;
constexpr int kFlagStride = 32;  // uint32 per flag: 128 bytes apart

long long g_ar_timeout_ns = 5000000000ll;  // five seconds: ranks may be this far apart after start-up work (graph capture)

struct ArParams {
    float* data;              // [count] partial row in, sum out
    unsigned char* bufs[kArMaxWorld];  // exchange buffer of every rank as mapped in this process
    unsigned int* state;      // [0] sequence number of the last completed call, [1] error word
    long long timeout_ns;
    int count, rank, world, max_count;
};

__device__ __forceinline__ float* ar_slot(unsigned char* buf, int parity, int src, int world, int max_count) {
    return reinterpret_cast<float*>(buf) + (size_t(parity) * world + src) * size_t(max_count);
}
__device__ __forceinline__ unsigned int* ar_flag(unsigned char* buf, int parity, int src, int world, int max_count) {
    unsigned char* flags = buf + size_t(2) * world * size_t(max_count) * sizeof(float);
    return reinterpret_cast<unsigned int*>(flags) + (size_t(parity) * world + src) * kFlagStride;
}
__device__ __forceinline__ long long ar_now() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__global__ void __launch_bounds__(kArThreads, 1) allreduce_oneshot_kernel(const ArParams p) {
    __shared__ int s_ok;
    pdl_launch_dependents();
    pdl_wait();  // the partial row comes from the previous kernel
    const int tid = threadIdx.x;
    const unsigned int seq = p.state[0] + 1u;
    const int parity = int(seq & 1u);
    const int n4 = p.count >> 2;
    if (tid == 0) s_ok = 1;

    // 1. my partial row into my slot of every rank's buffer (my own included)
    const float4* src = reinterpret_cast<const float4*>(p.data);
    for (int r = 0; r < p.world; r++) {
        float4* dst = reinterpret_cast<float4*>(ar_slot(p.bufs[r], parity, p.rank, p.world, p.max_count));
        for (int i = tid; i < n4; i += kArThreads) dst[i] = src[i];
    }
    __threadfence_system();
    __syncthreads();
    if (tid < p.world) {
        // 2. tell rank `tid` that my slot there is complete ...
        unsigned int* f = ar_flag(p.bufs[tid], parity, p.rank, p.world, p.max_count);
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(seq) : "memory");
        // ... and wait until source `tid` has completed its slot in my buffer
        const unsigned int* mine = ar_flag(p.bufs[p.rank], parity, tid, p.world, p.max_count);
        const long long t0 = ar_now();
        unsigned int seen;
        while (true) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
            if (seen == seq) break;
            if (ar_now() - t0 > p.timeout_ns) {
                atomicExch(&p.state[1], 1u + unsigned(tid));  // which source never arrived
                s_ok = 0;
                break;
            }
        }
    }
    __syncthreads();
    if (s_ok) {
        // 3. add the slots in rank order
        float4* out = reinterpret_cast<float4*>(p.data);
        for (int i = tid; i < n4; i += kArThreads) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int r = 0; r < p.world; r++) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(ar_slot(p.bufs[p.rank], parity, r, p.world, p.max_count)) + i);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
            out[i] = acc;
        }
    }
    __syncthreads();
    if (tid == 0) p.state[0] = seq;  // also after a timeout: the next call must not reuse this sequence number
}

}  // namespace

void allreduce_set_tuning(const char* key, int value) {
    if (!strcmp(key, "allreduce_timeout_ms")) g_ar_timeout_ns = (long long)value * 1000000ll;
}

}  // namespace kuiper

using namespace kuiper;

extern "C" size_t kuiper_allreduce_buffer_bytes(int world, int64_t max_count) {
    if (world < 1 || world > kArMaxWorld || max_count <= 0) return 0;
    return size_t(2) * world * size_t(max_count) * sizeof(float) + size_t(2) * world * kFlagStride * sizeof(unsigned int);
}

extern "C" int kuiper_allreduce_oneshot_f32(float* data, int64_t count, int rank, int world, void* const* rank_buffers,
                                            int64_t max_count, uint32_t* state, kuiper_stream_t stream) {
    KUIPER_REQUIRE(data && rank_buffers && state, "allreduce: null pointer");
    KUIPER_REQUIRE(world >= 1 && world <= kArMaxWorld && rank >= 0 && rank < world, "allreduce: bad rank %d of %d", rank, world);
    KUIPER_REQUIRE(count > 0 && count <= max_count && count % 4 == 0 && max_count % 32 == 0 && max_count <= (1 << 26),
                   "allreduce: count %lld does not fit the exchange slots (%lld floats; count a multiple of 4, slots a multiple of 32)", (long long)count,
                   (long long)max_count);
    KUIPER_REQUIRE((reinterpret_cast<uintptr_t>(data) & 15) == 0, "allreduce: data must be 16-byte aligned");
    ArParams p;
    p.data = data;
    for (int r = 0; r < kArMaxWorld; r++) p.bufs[r] = nullptr;
    for (int r = 0; r < world; r++) {
        KUIPER_REQUIRE(rank_buffers[r] != nullptr && (reinterpret_cast<uintptr_t>(rank_buffers[r]) & 127) == 0,
                       "allreduce: exchange buffer of rank %d is null or not 128-byte aligned", r);
        p.bufs[r] = static_cast<unsigned char*>(rank_buffers[r]);
    }
    p.state = state;
    p.timeout_ns = g_ar_timeout_ns;
    p.count = int(count);
    p.rank = rank;
    p.world = world;
    p.max_count = int(max_count);
    return pdl_status(launch_pdl(allreduce_oneshot_kernel, dim3(1), dim3(kArThreads), 0, as_stream(stream), p), "allreduce_oneshot");
}

extern "C" int kuiper_allreduce_status(const uint32_t* state) {
    KUIPER_REQUIRE(state != nullptr, "allreduce: null state");
    uint32_t host[2] = {0, 0};
    if (cudaMemcpy(host, state, sizeof(host), cudaMemcpyDeviceToHost) != cudaSuccess) {
        set_error("allreduce: cannot read the state words");
        return KUIPER_INTERNAL_ERROR;
    }
    if (host[1] == 0) return KUIPER_OK;
    set_error("allreduce: the flag of rank %u did not arrive within the time limit", host[1] - 1);
    return KUIPER_INTERNAL_ERROR;
}
