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
#include "peer.cuh"

namespace kairos {

int* device_status_word();    // api.cu

struct ArParams {
    PeerSet peers;                    // every rank's partial (slot of this call) and signal pad
    uint4* out;                       // local output
    long long words;                  // n / 8
};

__global__ void __launch_bounds__(kArThreads) oneshot_allreduce_kernel(const ArParams p) {
    chain_release();
    chain_wait();                      // the partial was written by the kernel before this one in the stream
    if (!peer_barrier(p.peers, blockIdx.x)) return;
    for (long long i = (long long)blockIdx.x * kArThreads + threadIdx.x; i < p.words;
         i += (long long)gridDim.x * kArThreads)
        p.out[i] = peer_sum8(p.peers, i);
}

int make_peer_set(PeerSet* ps, const void* const* peer_in, void* const* peer_signal, int world, int rank) {
    if (world < 1 || world > kArMaxWorld || rank < 0 || rank >= world) return KAIROS_ERR_SHAPE;
    if (!peer_in || !peer_signal) return KAIROS_ERR_ALIGN;
    for (int r = 0; r < kArMaxWorld; ++r) {
        ps->in[r] = nullptr;
        ps->signal[r] = nullptr;
    }
    for (int r = 0; r < world; ++r) {
        if (!peer_in[r] || !peer_signal[r] || ((uintptr_t)peer_in[r] & 15) || ((uintptr_t)peer_signal[r] & 3))
            return KAIROS_ERR_ALIGN;
        ps->in[r] = static_cast<const uint4*>(peer_in[r]);
        ps->signal[r] = static_cast<uint32_t*>(peer_signal[r]);
    }
    // this rank's counters sit behind the [ranks][slots] sequence numbers of its own pad
    ps->counter = ps->signal[rank] + kArMaxWorld * kArBlocks;
    ps->world = world;
    ps->rank = rank;
    ps->status = device_status_word();
    return ps->status ? KAIROS_OK : KAIROS_ERR_CUDA;
}

}  // namespace kairos

extern "C" int kairos_peer_allreduce_signal_bytes(void) {
    return (kairos::kArMaxWorld + 1) * kairos::kArBlocks * (int)sizeof(uint32_t);
}

extern "C" int kairos_peer_allreduce_f16(const void* const* peer_in, void* const* peer_signal, int world, int rank,
                                         void* out, long long n, kairos_stream_t stream) {
    using namespace kairos;
    if (n < 0 || (n % 8) != 0) return KAIROS_ERR_SHAPE;
    if (!out || ((uintptr_t)out & 15)) return KAIROS_ERR_ALIGN;
    ArParams p;
    const int rc = make_peer_set(&p.peers, peer_in, peer_signal, world, rank);
    if (rc != KAIROS_OK) return rc;
    if (n == 0) return KAIROS_OK;
    p.out = static_cast<uint4*>(out);
    p.words = n / 8;
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
