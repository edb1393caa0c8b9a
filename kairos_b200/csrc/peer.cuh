// Peer-memory building blocks shared by the stand-alone all-reduce (allreduce.cu) and the RMSNorm kernels that
// sum a row-parallel layer's partial outputs while they load them (glue.cu).  Plain loads and stores only.
#pragma once
#include "common.cuh"

namespace kairos {

constexpr int kArBlocks = 128;       // signal slots per peer = most blocks (or tokens) of one call
constexpr int kArThreads = 256;
constexpr int kArMaxWorld = 8;

// What a kernel needs to meet its peers: every rank's partial buffer and signal pad as mapped in this process.
// A signal pad holds [kArMaxWorld][kArBlocks] sequence numbers written by the peers, followed by this rank's own
// [kArBlocks] counters.
struct PeerSet {
    const uint4* in[kArMaxWorld];
    uint32_t* signal[kArMaxWorld];
    uint32_t* counter;
    int world, rank;
    int* status;
};

#ifdef __CUDACC__
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

// Block-wide meeting point, called by every thread of the block after the producer of this rank's partial has
// completed (stream order): tells every peer "slot `slot` of my partial is complete" with the slot's next
// sequence number and waits until all peers said the same.  The sequence lives in device memory, so a replayed
// CUDA graph advances it by itself.  Bounded (about a second): on a timeout the status word is raised and false
// is returned to every thread; the sequence still advances, so later calls stay in step with the peers.
__device__ __forceinline__ bool peer_barrier(const PeerSet& p, int slot) {
    __shared__ uint32_t s_seq;
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
        s_seq = p.counter[slot] + 1;
        s_ok = 1;
    }
    __syncthreads();
    const uint32_t seq = s_seq;
    if (threadIdx.x < p.world) {
        const int peer = threadIdx.x;
        __threadfence_system();
        st_release_sys(p.signal[peer] + p.rank * kArBlocks + slot, seq);
        const uint32_t* mine = p.signal[p.rank] + peer * kArBlocks + slot;
        bool ok = false;
        for (int spin = 0; spin < (1 << 21); ++spin) {          // ~1 s with the sleeps below
            if ((int32_t)(ld_acquire_sys(mine) - seq) >= 0) { ok = true; break; }
            if (spin > 64) __nanosleep(spin > 4096 ? 500 : 40);
        }
        if (!ok) s_ok = 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        p.counter[slot] = seq;
        if (!s_ok) atomicExch(p.status, KAIROS_ERR_DEVICE);
    }
    return s_ok != 0;
}

// fp16(sum over the ranks, in rank order, of the 8 fp16 values at word i of every partial)
__device__ __forceinline__ uint4 peer_sum8(const PeerSet& p, long long i) {
    uint4 v[kArMaxWorld];
#pragma unroll
    for (int r = 0; r < kArMaxWorld; ++r)
        if (r < p.world) v[r] = ld_peer(p.in[r] + i);           // all loads in flight before the first add
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
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
    return o;
}
#endif

// Host side: checks the pointer arrays and fills a PeerSet (status word included).  KAIROS_OK or an error code.
int make_peer_set(PeerSet* ps, const void* const* peer_in, void* const* peer_signal, int world, int rank);

}  // namespace kairos
