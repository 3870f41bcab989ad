// Tensor-parallel exchanges for decode rows over peer-mapped buffers: a low-latency all-reduce (sum, fp32) that also
// adds the residual stream, and the all-gather of per-rank (maximum, index) pairs behind the vocabulary-split lm_head.
// The reference has no multi-GPU code; this sits behind parallel::Communicator.
//
// The row-split projections (O and down) leave a partial row of `hidden` floats on every rank and the step needs
// their sum 72 times per token.  At 16 KB the exchange is pure latency, so it is built like a low-latency protocol:
// every value travels as an 8-byte word {value bits, sequence number} written with ONE store straight into a slot of
// every peer's exchange buffer (plain stores over NVLink).  The receiver polls the words themselves - a word whose
// second half equals the call's sequence number is complete, because an aligned 8-byte store is a single transaction -
// so there is no separate flag, no fence and no barrier between sending and receiving: each thread sends its element,
// then waits for the same element from every rank and adds them in rank order (every rank computes the same sum in
// the same order: bit-identical results on all ranks).
//
// Exchange buffer of one rank (kuiper_allreduce_buffer_bytes):
//   sum words   [2 parities][world][max_count] x 8 bytes    slot (parity, src) is written by rank src only
//   argmax words [2 parities][world][kArgmaxRows] x 16 bytes  {max bits, seq} {index, seq}
// Two parities: a rank can be one call ahead of a peer (it has every word of call k, the peer may still be adding
// its words of call k), never two (it would need the peer's words of call k + 1, sent after the peer finished k).
// Sequence numbers live on the device (state words, one per CTA of the sum kernel and one for the argmax kernel), so
// a call is replayable inside a CUDA graph.
//
// Every wait is bounded by a wall-clock limit; when it runs out the kernel records an error word, uses zero for what
// did not arrive and returns (the result of that call is void; the engine reads the word after its next stream
// synchronisation).  No multicast, no library call on peer memory.
#include <cstring>

#include "common.cuh"

namespace kuiper {
namespace {

constexpr int kArMaxWorld = 8;
constexpr int kArThreads = 1024;
constexpr int kArMaxCtas = 64;      // sum kernel: one sequence counter per CTA
constexpr int kArgmaxRows = 16;     // rows of one argmax exchange
constexpr int kStateWords = kArMaxCtas + 2;   // per-CTA sequence numbers, argmax sequence number, error word
constexpr int kStateArgmax = kArMaxCtas, kStateError = kArMaxCtas + 1;

long long g_ar_timeout_ns = 5000000000ll;  // five seconds: ranks may be this far apart after start-up work (graph capture)

struct ArParams {
    const float* partial;     // [count] this rank's partial row
    float* partial_clear;     // same buffer when it is to be zeroed after reading, else null
    const float* residual;    // [count] or null: added first, identical on every rank
    float* out;               // [count]
    unsigned char* bufs[kArMaxWorld];  // exchange buffer of every rank as mapped in this process
    unsigned int* state;
    long long timeout_ns;
    int count, rank, world, max_count;
};

__device__ __forceinline__ long long ar_now() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void st_word(void* p, unsigned int a, unsigned int b) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ uint2 ld_word(const void* p) {
    uint2 v;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
// waits until the word carries sequence number `seq`; false when the time limit ran out
__device__ __forceinline__ bool wait_word(const void* p, unsigned int seq, long long timeout_ns, uint2& v) {
    v = ld_word(p);
    if (v.y == seq) return true;
    const long long t0 = ar_now();
    unsigned int spins = 0;
    while (true) {
        v = ld_word(p);
        if (v.y == seq) return true;
        if ((++spins & 63u) == 0u && ar_now() - t0 > timeout_ns) return false;
    }
}
__device__ __forceinline__ unsigned char* sum_slot(unsigned char* buf, int parity, int src, int world, int max_count) {
    return buf + (size_t(parity) * world + src) * size_t(max_count) * 8;
}
__device__ __forceinline__ unsigned char* argmax_slot(unsigned char* buf, int parity, int src, int world, int max_count) {
    return buf + size_t(2) * world * size_t(max_count) * 8 + (size_t(parity) * world + src) * kArgmaxRows * 16;
}

// out = residual + sum over ranks of partial, element by element; grid = ceil(count / 1024) CTAs
__global__ void __launch_bounds__(kArThreads, 1) allreduce_ll_kernel(const ArParams p) {
    pdl_launch_dependents();
    pdl_wait();  // the partial row comes from the previous kernel
    const int e = blockIdx.x * kArThreads + threadIdx.x;
    const unsigned int seq = __ldcg(p.state + blockIdx.x) + 1u;
    const int parity = int(seq & 1u);
    if (e < p.count) {
        const float v = __ldcg(p.partial + e);
        if (p.partial_clear) p.partial_clear[e] = 0.f;
        // 1. my element into my slot of every rank's buffer (my own included)
#pragma unroll 1
        for (int r = 0; r < p.world; r++)
            st_word(sum_slot(p.bufs[r], parity, p.rank, p.world, p.max_count) + size_t(e) * 8, __float_as_uint(v), seq);
        // 2. the same element from every rank, added in rank order
        float acc = p.residual ? __ldcg(p.residual + e) : 0.f;
        unsigned char* mine = p.bufs[p.rank];
        for (int r = 0; r < p.world; r++) {
            uint2 w;
            if (wait_word(sum_slot(mine, parity, r, p.world, p.max_count) + size_t(e) * 8, seq, p.timeout_ns, w)) {
                acc += __uint_as_float(w.x);
            } else {
                atomicExch(p.state + kStateError, 1u + unsigned(r));  // which source never arrived
            }
        }
        p.out[e] = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0) p.state[blockIdx.x] = seq;  // also after a timeout: the next call must not reuse this number
}

struct ArgmaxParams {
    const float* logits;      // [M, V_local]: this rank's slice of the vocabulary
    int32_t* next;            // [M]
    unsigned char* bufs[kArMaxWorld];
    unsigned int* state;
    long long timeout_ns;
    int M, V_local, rank, world, max_count;
};

// per row: lowest index of the maximum over this rank's slice, then the same over all ranks' (maximum, index) pairs
__global__ void __launch_bounds__(kArThreads, 1) argmax_allgather_kernel(const ArgmaxParams p) {
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ float s_best_val[kArgmaxRows];
    __shared__ int s_best_idx[kArgmaxRows];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int m = 0; m < p.M; m++) {
        const float* row = p.logits + size_t(m) * p.V_local;
        float best = -INFINITY;
        int idx = 0x7fffffff;
        for (int i = tid; i < p.V_local; i += kArThreads) {
            const float v = __ldcg(row + i);
            if (v > best) { best = v; idx = i; }  // ascending i per thread: the first maximum stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
        }
        if (lane == 0) { s_val[warp] = best; s_idx[warp] = idx; }
        __syncthreads();
        if (warp == 0) {
            best = s_val[lane];
            idx = s_idx[lane];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
                if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
            }
            if (lane == 0) {
                s_best_val[m] = best;
                s_best_idx[m] = idx == 0x7fffffff ? 0 : idx;
            }
        }
        __syncthreads();
    }
    const unsigned int seq = __ldcg(p.state + kStateArgmax) + 1u;
    const int parity = int(seq & 1u);
    if (tid < p.M) {
        const int m = tid;
        const unsigned int vbits = __float_as_uint(s_best_val[m]);
        const unsigned int gidx = unsigned(p.rank * p.V_local + s_best_idx[m]);
        for (int r = 0; r < p.world; r++) {
            unsigned char* slot = argmax_slot(p.bufs[r], parity, p.rank, p.world, p.max_count) + size_t(m) * 16;
            st_word(slot, vbits, seq);
            st_word(slot + 8, gidx, seq);
        }
        float best = -INFINITY;
        unsigned int best_idx = 0;
        bool any = false;
        for (int r = 0; r < p.world; r++) {
            const unsigned char* slot = argmax_slot(p.bufs[p.rank], parity, r, p.world, p.max_count) + size_t(m) * 16;
            uint2 a, b;
            if (wait_word(slot, seq, p.timeout_ns, a) && wait_word(slot + 8, seq, p.timeout_ns, b)) {
                const float v = __uint_as_float(a.x);
                // ranks are visited in ascending order and hold ascending index ranges: strict > keeps the lowest index
                if (!any || v > best) { best = v; best_idx = b.x; any = true; }
            } else {
                atomicExch(p.state + kStateError, 1u + unsigned(r));
            }
        }
        p.next[m] = int32_t(best_idx);
    }
    __syncthreads();
    if (tid == 0) p.state[kStateArgmax] = seq;
}

int fill_bufs(unsigned char* (&bufs)[kArMaxWorld], void* const* rank_buffers, int world) {
    for (int r = 0; r < kArMaxWorld; r++) bufs[r] = nullptr;
    for (int r = 0; r < world; r++) {
        KUIPER_REQUIRE(rank_buffers[r] != nullptr && (reinterpret_cast<uintptr_t>(rank_buffers[r]) & 127) == 0,
                       "allreduce: exchange buffer of rank %d is null or not 128-byte aligned", r);
        bufs[r] = static_cast<unsigned char*>(rank_buffers[r]);
    }
    return KUIPER_OK;
}

}  // namespace

void allreduce_set_tuning(const char* key, int value) {
    if (!strcmp(key, "allreduce_timeout_ms")) g_ar_timeout_ns = (long long)value * 1000000ll;
}

}  // namespace kuiper

using namespace kuiper;

extern "C" size_t kuiper_allreduce_buffer_bytes(int world, int64_t max_count) {
    if (world < 1 || world > kArMaxWorld || max_count <= 0) return 0;
    return size_t(2) * world * size_t(max_count) * 8 + size_t(2) * world * kArgmaxRows * 16;
}

extern "C" size_t kuiper_allreduce_state_bytes(void) { return kStateWords * sizeof(unsigned int); }

extern "C" int kuiper_allreduce_sum_f32(const float* partial, const float* residual, float* out, int clear_partial,
                                        int64_t count, int rank, int world, void* const* rank_buffers, int64_t max_count,
                                        uint32_t* state, kuiper_stream_t stream) {
    KUIPER_REQUIRE(partial && out && rank_buffers && state, "allreduce: null pointer");
    KUIPER_REQUIRE(world >= 1 && world <= kArMaxWorld && rank >= 0 && rank < world, "allreduce: bad rank %d of %d", rank, world);
    KUIPER_REQUIRE(count > 0 && count <= max_count && max_count % 16 == 0 && max_count <= int64_t(kArMaxCtas) * kArThreads,
                   "allreduce: count %lld does not fit the exchange slots (%lld floats, at most %d)", (long long)count,
                   (long long)max_count, kArMaxCtas * kArThreads);
    ArParams p;
    p.partial = partial;
    p.partial_clear = clear_partial ? const_cast<float*>(partial) : nullptr;
    p.residual = residual;
    p.out = out;
    int rc = fill_bufs(p.bufs, rank_buffers, world);
    if (rc != KUIPER_OK) return rc;
    p.state = state;
    p.timeout_ns = g_ar_timeout_ns;
    p.count = int(count);
    p.rank = rank;
    p.world = world;
    p.max_count = int(max_count);
    const int ctas = int((count + kArThreads - 1) / kArThreads);
    return pdl_status(launch_pdl(allreduce_ll_kernel, dim3(ctas), dim3(kArThreads), 0, as_stream(stream), p), "allreduce_sum");
}

extern "C" int kuiper_argmax_allgather(const float* logits_local, int32_t* next, int M, int V_local, int rank, int world,
                                       void* const* rank_buffers, int64_t max_count, uint32_t* state, kuiper_stream_t stream) {
    KUIPER_REQUIRE(logits_local && next && rank_buffers && state, "argmax_allgather: null pointer");
    KUIPER_REQUIRE(world >= 1 && world <= kArMaxWorld && rank >= 0 && rank < world, "argmax_allgather: bad rank %d of %d", rank, world);
    KUIPER_REQUIRE(M > 0 && M <= kArgmaxRows && V_local > 0 && int64_t(V_local) * world <= 0x7fffffff,
                   "argmax_allgather: %d rows of %d logits do not fit (at most %d rows)", M, V_local, kArgmaxRows);
    KUIPER_REQUIRE(max_count > 0 && max_count % 16 == 0, "argmax_allgather: bad slot size");
    ArgmaxParams p;
    p.logits = logits_local;
    p.next = next;
    int rc = fill_bufs(p.bufs, rank_buffers, world);
    if (rc != KUIPER_OK) return rc;
    p.state = state;
    p.timeout_ns = g_ar_timeout_ns;
    p.M = M;
    p.V_local = V_local;
    p.rank = rank;
    p.world = world;
    p.max_count = int(max_count);
    return pdl_status(launch_pdl(argmax_allgather_kernel, dim3(1), dim3(kArThreads), 0, as_stream(stream), p), "argmax_allgather");
}

// synchronous: 0 if no bounded wait has run out since the word was last cleared; clear != 0 resets it
extern "C" int kuiper_allreduce_status(uint32_t* state, int clear) {
    KUIPER_REQUIRE(state != nullptr, "allreduce: null state");
    uint32_t word = 0;
    if (cudaMemcpy(&word, state + kStateError, sizeof(word), cudaMemcpyDeviceToHost) != cudaSuccess) {
        set_error("allreduce: cannot read the state words");
        return KUIPER_INTERNAL_ERROR;
    }
    if (word == 0) return KUIPER_OK;
    if (clear) cudaMemset(state + kStateError, 0, sizeof(uint32_t));
    set_error("allreduce: the words of rank %u did not arrive within the time limit", word - 1);
    return KUIPER_INTERNAL_ERROR;
}
