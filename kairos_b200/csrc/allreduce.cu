// One-shot all-reduce over peer memory for the small outputs of row-parallel layers (decode steps).
//
// Tensor parallelism sums the partial outputs of o_proj / down_proj over the ranks.  At decode sizes (a few
// tokens x hidden size, tens of KB) that sum is pure latency: a library all-reduce costs a launch plus several
// protocol hops.  Here every rank holds its partial in a buffer its peers can address (NVLink peer mapping);
// one kernel per rank
//   1. tells every peer "my partial is complete" by storing a sequence number into that peer's signal pad
//      (release, system scope), and waits until all peers' numbers have arrived in its own pad;
//   2. reads its slice of columns from ALL ranks' buffers with plain 16-byte peer loads, sums in fp32 in rank
//      order 0..t-1 (every rank forms the same sum bit for bit) and writes fp16 to its local output.
// Every rank reads everything (t x the data over NVLink), which is the right trade below ~1 MB; above that the
// caller keeps the library's bandwidth-optimal all-reduce.
//
// The partial buffers alternate between two slots from call to call.  A rank writes slot s again only after its
// kernel of the call in between has completed, whose step 1 proves that every peer has started that call and
// therefore finished reading slot s: no second barrier is needed.
//
// Sequence numbers live in device memory (one counter per block, advanced by the kernel itself), so a CUDA graph
// that holds the launch can be replayed: nothing in the arguments changes from call to call.  Every rank must
// issue the same sequence of calls.  The wait is bounded (about a second); on a timeout the block raises the
// device status word, skips the sum and returns, leaving the context usable.
//
// Only plain loads and stores touch peer memory: no TMA, no multicast, no library kernel.
#include "common.cuh"

namespace kairos {

int* device_status_word();    // api.cu

constexpr int kArBlocks = 128;       // most blocks per launch = signal slots per peer (a launch uses 4..128 by size)
constexpr int kArThreads = 256;
constexpr int kArMaxWorld = 8;

struct ArParams {
    const uint4* in[kArMaxWorld];     // every rank's partial (slot of this call), [n / 8] 16-byte words
    uint32_t* signal[kArMaxWorld];    // every rank's signal pad: [world][kArBlocks] sequence numbers
    uint32_t* counter;                // this rank's [kArBlocks] sequence counters
    uint4* out;                       // local output
    long long words;                  // n / 8
    int world, rank;
    int* status;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_peer(const uint4* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

__global__ void __launch_bounds__(kArThreads) oneshot_allreduce_kernel(const ArParams p) {
    chain_release();
    chain_wait();                      // the partial was written by the kernel before this one in the stream
    __shared__ uint32_t s_seq;
    __shared__ int s_ok;
    const int b = blockIdx.x;
    if (threadIdx.x == 0) {
        s_seq = p.counter[b] + 1;
        s_ok = 1;
    }
    __syncthreads();
    const uint32_t seq = s_seq;
    if (threadIdx.x < p.world) {
        const int peer = threadIdx.x;
        // the stores of the producing kernel are ordered before this release by the stream order and the fence
        __threadfence_system();
        st_release_sys(p.signal[peer] + p.rank * kArBlocks + b, seq);
        const uint32_t* mine = p.signal[p.rank] + peer * kArBlocks + b;
        bool ok = false;
        for (int spin = 0; spin < (1 << 21); ++spin) {          // ~1 s with the sleeps below
            if ((int32_t)(ld_acquire_sys(mine) - seq) >= 0) { ok = true; break; }
            if (spin > 64) __nanosleep(spin > 4096 ? 500 : 40);
        }
        if (!ok) s_ok = 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) p.counter[b] = seq;                  // stay in step with the peers even after a timeout
    if (!s_ok) {
        if (threadIdx.x == 0) atomicExch(p.status, KAIROS_ERR_DEVICE);
        return;
    }
    for (long long i = (long long)b * kArThreads + threadIdx.x; i < p.words; i += (long long)gridDim.x * kArThreads) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        uint4 v[kArMaxWorld];
#pragma unroll
        for (int r = 0; r < kArMaxWorld; ++r)
            if (r < p.world) v[r] = ld_peer(p.in[r] + i);       // all loads in flight before the first add
#pragma unroll
        for (int r = 0; r < kArMaxWorld; ++r) {
            if (r < p.world) {
                const __half2* h = reinterpret_cast<const __half2*>(&v[r]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __half22float2(h[j]);
                    acc[2 * j] += f.x;
                    acc[2 * j + 1] += f.y;
                }
            }
        }
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) oh[j] = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
        p.out[i] = o;
    }
}

}  // namespace kairos

extern "C" int kairos_peer_allreduce_signal_bytes(void) {
    return (kairos::kArMaxWorld + 1) * kairos::kArBlocks * (int)sizeof(uint32_t);
}

extern "C" int kairos_peer_allreduce_f16(const void* const* peer_in, void* const* peer_signal, int world, int rank,
                                         void* out, long long n, kairos_stream_t stream) {
    using namespace kairos;
    if (world < 1 || world > kArMaxWorld || rank < 0 || rank >= world || n < 0 || (n % 8) != 0) return KAIROS_ERR_SHAPE;
    if (!peer_in || !peer_signal || !out || ((uintptr_t)out & 15)) return KAIROS_ERR_ALIGN;
    if (n == 0) return KAIROS_OK;
    ArParams p;
    for (int r = 0; r < kArMaxWorld; ++r) {
        p.in[r] = nullptr;
        p.signal[r] = nullptr;
    }
    for (int r = 0; r < world; ++r) {
        if (!peer_in[r] || !peer_signal[r] || ((uintptr_t)peer_in[r] & 15) || ((uintptr_t)peer_signal[r] & 3))
            return KAIROS_ERR_ALIGN;
        p.in[r] = static_cast<const uint4*>(peer_in[r]);
        p.signal[r] = static_cast<uint32_t*>(peer_signal[r]);
    }
    // this rank's counters sit behind the [world][blocks] slots of its own pad
    p.counter = p.signal[rank] + kArMaxWorld * kArBlocks;
    p.out = static_cast<uint4*>(out);
    p.words = n / 8;
    p.world = world;
    p.rank = rank;
    p.status = device_status_word();
    if (!p.status) return KAIROS_ERR_CUDA;
    // one 16-byte word per thread up to 128 blocks: a block's flag exchange runs beside the others', so more
    // blocks cost no latency, while a block that loops pays a peer round trip per iteration.  Every rank passes
    // the same n, so the ranks agree on the blocks that take part (each block keeps its own sequence).
    long long want = (p.words + kArThreads - 1) / kArThreads;
    const int blocks = want < 4 ? 4 : (want > kArBlocks ? kArBlocks : (int)want);
    const cudaError_t e = launch_chained(oneshot_allreduce_kernel, dim3(blocks), dim3(kArThreads), 0,
                                         reinterpret_cast<cudaStream_t>(stream), p);
    if (e != cudaSuccess) return note_cuda_error(e);
    return launch_status();
}
