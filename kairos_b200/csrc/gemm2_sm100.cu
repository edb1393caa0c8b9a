// Large-M GEMMs on CTA pairs: Y[M,N] = X . W^T with both operands staged by TMA (W8A8 kind::i8 and FP16
// kind::f16), one 256 (tokens) x 256 (weight rows) tile per cluster of two CTAs.
//
// Why pairs: with one CTA per 128 x 256 tile the int8 MMA drains its shared-memory operands (48 KB per
// 128-byte k block) faster than one SM's shared memory can deliver them (tensor pipe 50 % active).  With
// tcgen05.mma.cta_group::2 each CTA stages 128 tokens (its half of the MMA's M = 256) and only HALF of
// the weight tile (32 KB per k block), the pair's tensor cores share the operands, and each CTA keeps
// its 128 x 256 accumulator in its own TMEM.
//
// Tokens sit on the MMA's M here (unlike the one-CTA kernel, where few tokens must go on N): a TMEM lane
// is then a token and the accumulator columns are consecutive n, i.e. consecutive addresses of a row of
// Y, so the epilogue stores 16 bytes per instruction and needs no address arithmetic per element.  The
// epilogue's instruction stream is what this kernel loses to its mainloop (it shares schedulers with the
// TMA- and MMA-issuing threads), so its length matters.
//
// Protocol (no multicast anywhere):
//   * both CTAs issue plain TMA loads into their own shared memory; the loads of both signal the FULL
//     barrier of the leader (rank 0), which its producers armed with the byte count of both CTAs;
//   * the leader's MMA thread issues the pair-wide MMAs and commits twice per stage: once to its own
//     EMPTY barrier, once to the peer's (address mapped into the cluster window), same for the
//     accumulator-ready barriers;
//   * the peer's epilogue warps release the accumulator buffer by remote arrives on the leader's barrier.
// Every mbarrier wait is bounded (status word on timeout); the two cluster-wide barriers at start and end
// are reached by every thread on every path.
#include <cuda.h>
#include <cstdlib>

#include "common.cuh"

namespace kairos {

int make_tmap(CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle);   // tensormap.cu
int device_sm_count();        // gemm_sm100.cu
int* device_status_word();    // api.cu

constexpr int kP2Rows = 128;                       // rows of either operand staged per CTA (256 per pair)
constexpr int kP2Tokens = 256;                     // tokens per tile = weight rows per tile
constexpr int kP2StageBytes = 2 * kP2Rows * 128;   // 128 tokens + 128 weight rows, one 128-byte k block
constexpr int kP2Stages = 6;
constexpr int kP2Threads = 32 * 7;
constexpr int kP2SmemBytes = kP2Stages * kP2StageBytes + 8 * (2 * kP2Stages + 4) + 64 + 1024;

struct Pair2Params {
    int M, N, K;
    int n_tiles, m_tiles, kb_total;
    const __half* s1;
    const __half* sx;
    const __half* bias;
    __half* Y;
    int32_t* acc_dbg;
    int* status;
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t peer_addr(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load of a CTA of a pair: data into this CTA's shared memory, completion on `bar_cluster_addr`
__device__ __forceinline__ void tma_load_3d_pair(void* dst, const void* tmap, uint32_t bar_cluster_addr, int c0, int c1,
                                                 int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, "
        "%5}], [%2];" ::"r"(smem_u32(dst)),
        "l"(tmap), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
                 : "memory");
}
// Tile order: bands of kP2Band token tiles; inside a band the token tile runs fastest, then the weight tile.
// The clusters running at one time then share one band of activations (16 tiles = 4096 tokens, 16 MB of int8
// at K = 4096) and a few weight tiles, and a band's activations stay in L2 while all weight tiles pass; with
// the token tile running fastest over ALL of M, activations beyond the L2 size were re-read per weight tile.
constexpr int kP2Band = 16;
__device__ __forceinline__ void pair_tile_coords(int tile, int m_tiles, int n_tiles, int& m_tile, int& n_tile) {
    const int per_band = kP2Band * n_tiles;
    const int band = tile / per_band;
    const int r = tile - band * per_band;
    const int m0 = band * kP2Band;
    const int width = m_tiles - m0 < kP2Band ? m_tiles - m0 : kP2Band;   // the last band may be narrower
    n_tile = r / width;
    m_tile = m0 + r - n_tile * width;
}

template <bool kInt8>
__device__ __forceinline__ void umma_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
    if constexpr (kInt8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

template <bool kInt8>
__global__ void __launch_bounds__(kP2Threads, 1)
    umma_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                          const Pair2Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kP2Stages * kP2StageBytes);   // used in the leader only
    uint64_t* empty = full + kP2Stages;                                                // one set per CTA
    uint64_t* tmem_full = empty + kP2Stages;                                           // [2], per CTA
    uint64_t* tmem_empty = tmem_full + 2;                                              // [2], leader only
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;
    // pair-wide instruction: M = 256 (128 tokens per CTA), N = 256 weight rows
    constexpr uint32_t kIdesc = (kInt8 ? (2u << 4) | (1u << 7) | (1u << 10) : (1u << 4)) |
                                ((uint32_t)(kP2Tokens >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kP2Stages; ++s) {
            mbar_init(&full[s], 2);              // the leader's two producers (they arm both CTAs' bytes)
            mbar_init(&empty[s], 1);             // one commit of the leader's MMA thread
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], 8);        // four epilogue warps of each CTA
        }
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmap_w);
        tma_prefetch_desc(&tmap_x);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                          // the peer's barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int n_clusters = gridDim.x >> 1, cluster_id = blockIdx.x >> 1;
    const int total_tiles = p.n_tiles * p.m_tiles;

    if (warp == 0 || warp == 6) {
        // ---------------- producers (both CTAs): warp 0 = weights, warp 6 = activations ----------------
        if (lane == 0) {
            const bool is_w = warp == 0;
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = cluster_id; tile < total_tiles && ok; tile += n_clusters) {
                int m_tile, n_tile;
                pair_tile_coords(tile, p.m_tiles, p.n_tiles, m_tile, n_tile);
                const int row0 = is_w ? n_tile * 256 + (int)rank * kP2Rows : m_tile * kP2Tokens + (int)rank * 128;
                for (int kb = 0; kb < p.kb_total; ++kb) {
                    if (!mbar_wait(&empty[s], phase ^ 1, abort_flag)) { ok = false; break; }
                    uint8_t* st = smem + s * kP2StageBytes + (is_w ? kP2Rows * 128 : 0);   // A = tokens, B = weights
                    if (leader) mbar_arrive_expect_tx(&full[s], 2 * kP2Rows * 128);   // this CTA's bytes + the peer's
                    tma_load_3d_pair(st, is_w ? (const void*)&tmap_w : (const void*)&tmap_x,
                                     peer_addr(smem_u32(&full[s]), 0), 0, row0, kb);
                    if (++s == kP2Stages) { s = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader only) ----------------
        if (leader && lane == 0) {
            int s = 0, it = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = cluster_id; tile < total_tiles && ok; tile += n_clusters, ++it) {
                const int b = it & 1;
                if (!mbar_wait(&tmem_empty[b], ((it >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(b * kP2Tokens);
                for (int kb = 0; kb < p.kb_total; ++kb) {
                    if (!mbar_wait(&full[s], phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    uint8_t* st = smem + s * kP2StageBytes;
                    const uint64_t adesc = umma_desc_sw128(smem_u32(st));
                    const uint64_t bdesc = umma_desc_sw128(smem_u32(st + kP2Rows * 128));
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        umma_pair<kInt8>(d_tmem, adesc + 2 * j, bdesc + 2 * j, kIdesc, (kb > 0 || j > 0) ? 1u : 0u);
                    umma_commit_pair(smem_u32(&empty[s]));                    // this CTA's stage is free
                    umma_commit_pair(peer_addr(smem_u32(&empty[s]), 1));      // and the peer's
                    if (++s == kP2Stages) { s = 0; phase ^= 1; }
                }
                if (ok) {
                    umma_commit_pair(smem_u32(&tmem_full[b]));
                    umma_commit_pair(peer_addr(smem_u32(&tmem_full[b]), 1));
                }
            }
        }
    } else {
        // ---------------- epilogue (warps 2..5 of both CTAs) ----------------
        // lane = token, accumulator column = weight row n
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const bool has_bias = p.bias != nullptr;
        const bool vec_ok = (p.N % 8) == 0 && ((uintptr_t)p.Y & 15) == 0 && !has_bias && p.acc_dbg == nullptr;
        int it = 0;
        bool ok = true;
        for (int tile = cluster_id; tile < total_tiles && ok; tile += n_clusters, ++it) {
            int m_tile, n_tile;
            pair_tile_coords(tile, p.m_tiles, p.n_tiles, m_tile, n_tile);
            const int m = m_tile * kP2Tokens + (int)rank * kP2Rows + row;
            const bool m_ok = m < p.M;
            const int n_base = n_tile * 256;
            const int b = it & 1;
            float sxf = 0.f;
            if constexpr (kInt8) sxf = m_ok ? __half2float(__ldg(p.sx + m)) : 0.f;
            // per-column factors of 64 columns, two per lane, handed round by shuffle
            auto load_s1 = [&](int n_first) {
                const int n = n_first + lane;
                return (kInt8 && n < p.N) ? __half2float(__ldg(p.s1 + n)) : 0.f;
            };
            auto load_bias = [&](int n_first) {
                const int n = n_first + lane;
                return (has_bias && n < p.N) ? __ldg(p.bias + n) : __float2half_rn(0.f);
            };
            // 64 accumulator columns of this lane's token: scale, round, (add bias,) store
            auto emit = [&](const uint32_t (&r)[64], int c0, float s1a, float s1b) {
                const int n0 = n_base + c0;
                if (vec_ok && n0 + 64 <= p.N) {
                    // the common case: 16-byte stores of 8 consecutive n, no per-element checks
                    uint4* yp = reinterpret_cast<uint4*>(p.Y + (size_t)m * p.N + n0);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        __half2 h[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int c = 8 * j + 2 * e;
                            float v0, v1;
                            if constexpr (kInt8) {
                                // half(float(acc) * (float(s1[n]) * float(sx[m])))
                                const float f0 = __shfl_sync(0xffffffffu, c < 32 ? s1a : s1b, c & 31);
                                const float f1 = __shfl_sync(0xffffffffu, c + 1 < 32 ? s1a : s1b, (c + 1) & 31);
                                v0 = __fmul_rn((float)(int32_t)r[c], __fmul_rn(f0, sxf));
                                v1 = __fmul_rn((float)(int32_t)r[c + 1], __fmul_rn(f1, sxf));
                            } else {
                                v0 = __uint_as_float(r[c]);
                                v1 = __uint_as_float(r[c + 1]);
                            }
                            h[e] = __floats2half2_rn(v0, v1);
                        }
                        if (m_ok) yp[j] = *reinterpret_cast<const uint4*>(h);
                    }
                    return;
                }
                const __half ba = load_bias(n0), bb = load_bias(n0 + 32);
#pragma unroll
                for (int c = 0; c < 64; ++c) {
                    const int n = n0 + c;
                    const float s1f = kInt8 ? __shfl_sync(0xffffffffu, c < 32 ? s1a : s1b, c & 31) : 0.f;
                    const __half bias_n = __shfl_sync(0xffffffffu, c < 32 ? ba : bb, c & 31);
                    if (!m_ok || n >= p.N) continue;
                    __half y;
                    if constexpr (kInt8) {
                        y = __float2half_rn(__fmul_rn((float)(int32_t)r[c], __fmul_rn(s1f, sxf)));
                        if (p.acc_dbg) p.acc_dbg[(size_t)m * p.N + n] = (int32_t)r[c];
                    } else {
                        y = __float2half_rn(__uint_as_float(r[c]));
                    }
                    if (has_bias) y = __hadd(y, bias_n);
                    p.Y[(size_t)m * p.N + n] = y;
                }
            };
            float s1_a = load_s1(n_base), s1_b = load_s1(n_base + 32);
            if (!mbar_wait(&tmem_full[b], (it >> 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * kP2Tokens);
            // Few, large TMEM loads and a lean store loop.  On M=8192, K=4096, N=14336 (int8), with the weight
            // rows on the lanes, this kernel took 441 us with 16-column loads, 374 us with 64-column loads and
            // 320 us once the common case dropped its per-element checks; the mainloop alone (no epilogue) runs
            // in 280 us, and so does the kernel with the TMEM loads but no arithmetic or stores.  With tokens on
            // the lanes and 16-byte stores it is still 320 us there (M=2048, K=N=4096: 43 -> 34 us): what is
            // left is the output itself, 13 % more traffic through an L2 that the operand loads already fill.
#pragma unroll 1
            for (int c0 = 0; c0 < 256; c0 += 64) {
                const float s0 = s1_a, s1 = s1_b;
                if (c0 + 64 < 256) {
                    s1_a = load_s1(n_base + c0 + 64);
                    s1_b = load_s1(n_base + c0 + 96);
                }
                uint32_t r[64];
                tmem_ld64(taddr + c0, r);
                tmem_ld_wait();
                emit(r, c0, s0, s1);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(peer_addr(smem_u32(&tmem_empty[b]), 0));   // the leader's barrier
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) atomicExch(p.status, KAIROS_ERR_DEVICE);
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    cluster_sync_all();                          // nobody signals a CTA that has already left
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

// Returns KAIROS_OK after launching, or 1 when the problem does not suit CTA pairs (caller falls back to
// the one-CTA kernel).
template <bool kInt8>
int launch_gemm_pair(const void* X, const void* W, const __half* s1, const __half* sx, const __half* bias, void* Y,
                     void* acc_dbg, int M, int N, int K, cudaStream_t stream) {
    const int sms = device_sm_count();
    const int n_tiles = (N + 255) / 256, m_tiles = (M + kP2Tokens - 1) / kP2Tokens;
    // Measured on B200 (W8A8 and FP16, graph-timed): the pair kernel overtakes the one-CTA kernel only once the
    // problem holds about five rounds of 256 x 256 tiles (M = 2048 on the 14336-wide shapes, M = 8192 on
    // 4096 x 4096); below that the one-CTA kernel's smaller tiles fill the SMs better.
    if (M < 512 || n_tiles * m_tiles < 5 * (sms / 2)) return 1;
    const uint64_t es = kInt8 ? 1 : 2, bk = kInt8 ? 128 : 64;
    CUtensorMap tw, tx;
    int rc;
    {
        const uint64_t dims[3] = {bk, (uint64_t)N, (uint64_t)K / bk}, strides[2] = {(uint64_t)K * es, 128};
        const uint32_t box[3] = {(uint32_t)bk, kP2Rows, 1};
        if ((rc = make_tmap(&tw, kInt8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, W, dims,
                            strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) != KAIROS_OK) return rc;
    }
    {
        const uint64_t dims[3] = {bk, (uint64_t)M, (uint64_t)K / bk}, strides[2] = {(uint64_t)K * es, 128};
        const uint32_t box[3] = {(uint32_t)bk, 128, 1};
        if ((rc = make_tmap(&tx, kInt8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, X, dims,
                            strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) != KAIROS_OK) return rc;
    }
    Pair2Params p;
    p.M = M; p.N = N; p.K = K;
    p.n_tiles = n_tiles; p.m_tiles = m_tiles; p.kb_total = K / (int)bk;
    p.s1 = s1; p.sx = sx; p.bias = bias;
    p.Y = static_cast<__half*>(Y);
    p.acc_dbg = static_cast<int32_t*>(acc_dbg);
    p.status = device_status_word();
    if (!p.status) return KAIROS_ERR_CUDA;
    static PerDeviceFlag smem_attr;    // per instantiation
    {
        const int rc = ensure_dynamic_smem(smem_attr, umma_gemm_pair_kernel<kInt8>, kP2SmemBytes);
        if (rc != KAIROS_OK) return rc;
    }
    int clusters = n_tiles * m_tiles;
    if (clusters > sms / 2) clusters = sms / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * clusters));
    cfg.blockDim = dim3(kP2Threads);
    cfg.dynamicSmemBytes = kP2SmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, umma_gemm_pair_kernel<kInt8>, tw, tx, p);
    if (e != cudaSuccess) return note_cuda_error(e);
    return launch_status();
}

template int launch_gemm_pair<true>(const void*, const void*, const __half*, const __half*, const __half*, void*, void*,
                                    int, int, int, cudaStream_t);
template int launch_gemm_pair<false>(const void*, const void*, const __half*, const __half*, const __half*, void*,
                                     void*, int, int, int, cudaStream_t);

}  // namespace kairos
