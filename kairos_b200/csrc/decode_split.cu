// Decode-side W4A16 for small batches (path item a9): Y[M,N] = X[M,K] . dequant(W)^T, 1 <= M <= 32.
//
// The packed weight is the only large traffic and is read exactly once, so the kernel is organised
// around keeping every SM's memory pipe full from the first to the last cycle of a launch:
//   * the work is cut into many small CTAs (four warps; several CTAs resident per SM) instead of one
//     persistent CTA per SM.  A CTA owns 32 weight rows and one slice of K; the K slices of a row tile
//     form a thread-block cluster and meet through distributed shared memory, so small problems
//     (N = 1024 .. 4096) still give every SM several CTAs -- no scratch memory, no atomics, no second
//     launch;
//   * a warp walks its quantization groups (128 k) with the packed bytes going from global memory
//     straight into registers: a lane's two 16-byte loads are 32 consecutive k of weight rows g and
//     g + 8, and a warp-wide load covers whole 128-byte lines.  The loads of the next group are
//     issued before the arithmetic of the current one (register double buffer), and those of the
//     first group before the kernel waits for its predecessor in the stream, so the weight stream of
//     launch i + 1 overlaps the tail of launch i;
//   * the uint4 values go through ONE lop3 per pair into the A fragment of mma.sync.m16n8k16 as
//     fp16 (1024 + q), or (1024 + 16 q) for the odd nibbles, with fp32 accumulation: no subtraction
//     and no scaling per element.  The offsets are undone per group on the accumulators:
//       sum q x = (C_lo - 1024 X_lo) + (C_hi - 1024 X_hi) / 16,
//     where X_lo / X_hi (sums of x over the k of the even / odd nibbles) come from MMAs against an
//     all-ones A fragment; then y += s * (sum q x) + z * (X_lo + X_hi) with the stored fp16 factors.
//
// Reference counterpart: gemv_forward_cuda_new
// (thirdparty/AWQ/kernels/csrc/quantization_new/gemv/gemv_cuda.cu:74-463).
// Algorithmic bytes per call: K*N/2 + 4*(K/128)*N + 2*M*K + 2*M*N.
#include <cuda.h>

#include "common.cuh"

namespace kairos {

int make_tmap(CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle);   // tensormap.cu
int device_sm_count();        // gemm_sm100.cu
int* device_status_word();    // api.cu

constexpr int kDsMaxWarps = 4;
constexpr int kDsMaxCluster = 8;

struct SplitParams {
    const __half* X;
    const uint8_t* qw;
    const __half* scales;
    const __half* zeros;
    const __half* bias;
    __half* Y;
    int M, N, K, G;   // G = K / 128 quantization groups
    int C;            // CTAs per cluster = K slices of a row tile
    int gpc;          // groups per K slice
    int silu;         // 1: the weight rows are gate / up rows in the blocked order (16 gate rows, their 16 up rows,
                      // ...) and Y is [M, N / 2]: Y[m, i] = half(half(silu(gate_i)) * up_i), the epilogue of a gated MLP
    int* status;      // raised when a bounded wait runs out
};

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// word w of a chunk (fixed c) -> e[b] for b = 0..3: b even: half2(1024 + q), b odd: half2(1024 + 16 q)
__device__ __forceinline__ void nibble_pairs4(uint32_t w, uint32_t (&e)[4]) {
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(e[0]) : "r"(w));
    asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xea;" : "=r"(e[1]) : "r"(w));
    const uint32_t w8 = w >> 8;
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(e[2]) : "r"(w8));
    asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xea;" : "=r"(e[3]) : "r"(w8));
}

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of `p` (a shared-memory address of this CTA) in the shared memory of CTA `rank` of the cluster
__device__ __forceinline__ uint32_t cluster_map(const void* p, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

__device__ __forceinline__ uint4 lds16(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float lds_h2f(uint32_t addr) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return __half2float(__ushort_as_half(v));
}

// Shared-memory layout of one pipeline stage of one warp (one quantization group, 128 k); every part is
// one tiled bulk-tensor copy, so a stage costs the issuing lane four instructions:
//   packed weights  [4 RB qweight rows][256 B]
//   activations     [XR tokens][256 B]   (rows beyond M arrive as zeros)
//   factors         scales of the 16 RB rows; 128 bytes further (a bulk-tensor copy lands on a 128-byte
//                   boundary) their scaled zeros
template <int NT, int RB, int XR>   // token tiles of 8, MMA row blocks (16 weight rows) per warp, token rows staged
struct SplitCfg {
    static constexpr int kRows = 16 * RB;                      // weight rows of a CTA (all its warps: they split K)
    static constexpr int kWBytes = 1024 * RB;
    static constexpr int kXBytes = 256 * XR;
    static constexpr int kFBytes = 256;                        // scales at 0, scaled zeros at 128
    static constexpr int kFTx = 64 * RB;                       // bytes the two factor copies bring
    static_assert(32 * RB <= 128, "a factor row slice must fit its 128-byte slot");
    static constexpr int kStageBytes = (kWBytes + kXBytes + kFBytes + 127) / 128 * 128;
    static constexpr int kStages = kStageBytes <= 2560 ? 4 : (kStageBytes <= 5120 ? 3 : 2);
    static constexpr int kOut = kRows * 8 * NT;                // outputs of a row tile
    static constexpr int kRingBytes = kStages * kStageBytes > kOut * 4 ? kStages * kStageBytes : kOut * 4;
    static constexpr int kWarpBytes = kRingBytes + 128;        // + the stage barriers
    // (five resident CTAs per SM cap the four-row-block variants at 96 registers, which spills; four leave 128)
    static constexpr int kMinBlocks = NT == 1 ? (RB == 4 ? 4 : 5) : (NT == 2 ? (RB == 4 ? 2 : 4) : 2);
    static size_t smem_bytes(int warps, int cluster) {
        return 128 + (size_t)warps * kWarpBytes + 16 + (cluster > 1 ? (size_t)cluster * kOut * 4 : 0);
    }
};

template <int NT, int RB, int XR>
__global__ void __launch_bounds__(32 * kDsMaxWarps, SplitCfg<NT, RB, XR>::kMinBlocks)
    decode_split_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                        const __grid_constant__ CUtensorMap tmap_s, const __grid_constant__ CUtensorMap tmap_z,
                        const SplitParams p) {
    using Cfg = SplitCfg<NT, RB, XR>;
    constexpr int kOut = Cfg::kOut;
    constexpr int kStages = Cfg::kStages;
    constexpr int kRows = Cfg::kRows;
    constexpr int kStageBytes = Cfg::kStageBytes;
    extern __shared__ uint8_t ds_smem_raw[];
    uint8_t* ds_smem = reinterpret_cast<uint8_t*>(((uintptr_t)ds_smem_raw + 127) & ~(uintptr_t)127);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, W = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    // per-warp ring of kStages groups (afterwards its first bytes hold the warp's partial sums) + its barriers
    uint8_t* ring = ds_smem + warp * Cfg::kWarpBytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(ring + Cfg::kRingBytes);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(ds_smem + W * Cfg::kWarpBytes);
    float* gather = reinterpret_cast<float*>(ds_smem + W * Cfg::kWarpBytes + 16);   // [C][kOut], used in cluster rank 0
    const uint32_t ring_u32 = smem_u32(ring);

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) mbar_init(&full[s], 2);   // the weight-side and the activation-side arrival
        if (warp == 0) {
            *abort_flag = 0;
            tma_prefetch_desc(&tmap_w);
            tma_prefetch_desc(&tmap_x);
            tma_prefetch_desc(&tmap_s);
            tma_prefetch_desc(&tmap_z);
        }
        fence_mbar_init();
    }
    const bool clustered = p.C > 1;
    const uint32_t crank = clustered ? cluster_rank() : 0u;
    // every CTA of the cluster has arrived here before any of them writes a peer's shared memory below
    if (clustered) cluster_arrive();
    __syncthreads();
    chain_release();

    const int row0 = (blockIdx.x / p.C) * kRows;
    // K slice of the CTA, then a contiguous run of its groups for each warp (long runs of one qweight row)
    const int gs0 = (int)crank * p.gpc;
    const int gs1 = min(p.G, gs0 + p.gpc);
    const int gpw = (gs1 - gs0 + W - 1) / W;
    const int g_first = gs0 + warp * gpw;
    const int n_it = max(0, min(gs1, g_first + gpw) - g_first);

    // stage `s` <- group `grp`: rows and columns beyond the tensors arrive as zeros and count as bytes
    auto issue_weights = [&](int s, int grp) {
        if (elect_one()) {
            uint8_t* st = ring + s * kStageBytes;
            mbar_arrive_expect_tx(&full[s], Cfg::kWBytes + Cfg::kFTx);
            tma_load_2d(st, &tmap_w, &full[s], grp * 256, row0 / 4);                       // bytes of the row, qweight row
            tma_load_2d(st + Cfg::kWBytes + Cfg::kXBytes, &tmap_s, &full[s], row0, grp);   // weight row, group
            tma_load_2d(st + Cfg::kWBytes + Cfg::kXBytes + 128, &tmap_z, &full[s], row0, grp);
        }
    };
    auto issue_x = [&](int s, int grp) {
        if (elect_one()) {
            mbar_arrive_expect_tx(&full[s], Cfg::kXBytes);
            tma_load_2d(ring + s * kStageBytes + Cfg::kWBytes, &tmap_x, &full[s], grp * kGroup, 0);   // k, token
        }
    };

    float acc[RB][NT][4];
#pragma unroll
    for (int rb = 0; rb < RB; ++rb)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[rb][nt][i] = 0.f;

    // ---- prologue: the packed weights of the first groups are requested before this kernel waits for the
    // one before it in the stream (they are constant); the activations only after that wait ----
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s)
        if (s < n_it) issue_weights(s, g_first + s);
    chain_wait();
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s)
        if (s < n_it) issue_x(s, g_first + s);

    // the lane's bytes inside a stage: its 16-byte chunk of weight rows g (+ 8 h + 16 rb), its x, its factors
    const uint32_t w_lane = ring_u32 + (g >> 2) * 256 + (t >> 1) * 128 + ((2 * (g & 3) + (t & 1)) << 4);
    const uint32_t x_lane = ring_u32 + Cfg::kWBytes + g * 256 + 64 * t;
    const uint32_t f_lane = ring_u32 + Cfg::kWBytes + Cfg::kXBytes + 2 * g;

    const uint32_t ones = 0x3c003c00u;      // half2(1, 1)
    const __half2 k16th = __half2half2(__ushort_as_half(0x2c00));   // 1/16
    bool ok = true;
    uint32_t parity = 0;
    // The loop over the warp's groups is unrolled by the ring depth: the stage read (s) and the stage refilled
    // (fs, the one read in the previous iteration) are then compile-time constants, and so are all shared-memory
    // offsets and barrier addresses of an iteration.
#pragma unroll 1
    for (int it0 = 0; it0 < n_it && ok; it0 += kStages, parity ^= 1u) {
#pragma unroll
    for (int s = 0; s < kStages; ++s) {
        const int it = it0 + s;
        if (it >= n_it) break;
        const int fs = (s + kStages - 1) % kStages;
        // refill the slot read in the previous iteration: every lane is done with it
        __syncwarp();
        if (it + kStages - 1 < n_it) {
            // both arrivals and the four copies of the stage from one elected lane
            if (elect_one()) {
                const int grp = g_first + it + kStages - 1;
                uint8_t* st = ring + fs * kStageBytes;
                mbar_arrive_expect_tx(&full[fs], Cfg::kWBytes + Cfg::kFTx);
                mbar_arrive_expect_tx(&full[fs], Cfg::kXBytes);
                tma_load_2d(st, &tmap_w, &full[fs], grp * 256, row0 / 4);
                tma_load_2d(st + Cfg::kWBytes, &tmap_x, &full[fs], grp * kGroup, 0);
                tma_load_2d(st + Cfg::kWBytes + Cfg::kXBytes, &tmap_s, &full[fs], row0, grp);
                tma_load_2d(st + Cfg::kWBytes + Cfg::kXBytes + 128, &tmap_z, &full[fs], row0, grp);
            }
        }
        if (!mbar_wait(&full[s], parity, abort_flag)) { ok = false; break; }
        const uint32_t so = (uint32_t)(s * kStageBytes);

        // The lane's 32 activations of token g (+ 8 nt) as 16 words, word 4 b + c = k 8 b + 2 c (+1).  The
        // words of the odd nibbles (b = 1, 3) are scaled by 1/16 here, because those nibbles enter the MMA
        // as 1024 + 16 q: one accumulator then holds sum q x + 1024 (X_lo + X_hi / 16), X_lo / X_hi being
        // the sums of x over the k of the even / odd nibbles, which MMAs against an all-ones A fragment give.
        uint32_t xw[NT][16];
        float x_sum[NT][2], x_off[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const bool staged = XR >= 8 * (nt + 1) || g + 8 * nt < XR;      // token rows beyond M hold zeros
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const uint4 v = staged ? lds16(x_lane + so + 8 * nt * 256 + 16 * b) : make_uint4(0u, 0u, 0u, 0u);
                xw[nt][4 * b + 0] = v.x; xw[nt][4 * b + 1] = v.y; xw[nt][4 * b + 2] = v.z; xw[nt][4 * b + 3] = v.w;
            }
#pragma unroll
            for (int b = 1; b < 4; b += 2)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const __half2 h = __hmul2(*reinterpret_cast<const __half2*>(&xw[nt][4 * b + c]), k16th);
                    xw[nt][4 * b + c] = *reinterpret_cast<const uint32_t*>(&h);
                }
            float x_lo[4] = {0.f, 0.f, 0.f, 0.f}, x_hi[4] = {0.f, 0.f, 0.f, 0.f};   // X_lo, X_hi / 16
#pragma unroll
            for (int c = 0; c < 4; c += 2) {
                mma16816(x_lo, ones, ones, ones, ones, xw[nt][c], xw[nt][c + 1]);
                mma16816(x_hi, ones, ones, ones, ones, xw[nt][4 + c], xw[nt][4 + c + 1]);
                mma16816(x_lo, ones, ones, ones, ones, xw[nt][8 + c], xw[nt][8 + c + 1]);
                mma16816(x_hi, ones, ones, ones, ones, xw[nt][12 + c], xw[nt][12 + c + 1]);
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {          // tokens 2t, 2t+1
                x_sum[nt][j] = fmaf(16.f, x_hi[j], x_lo[j]);
                x_off[nt][j] = 1024.f * (x_lo[j] + x_hi[j]);
            }
        }
#pragma unroll
        for (int rb = 0; rb < RB; ++rb) {
            const uint4 raw0 = lds16(w_lane + so + 1024 * rb);         // row g of the block
            const uint4 raw1 = lds16(w_lane + so + 1024 * rb + 512);   // row g + 8
            const uint32_t w0[4] = {raw0.x, raw0.y, raw0.z, raw0.w}, w1[4] = {raw1.x, raw1.y, raw1.z, raw1.w};
            // two accumulators per token tile (nibbles b = 0, 1 and b = 2, 3): chains of four dependent MMAs
            // instead of eight
            float cacc[NT][4], cacc2[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) cacc[nt][i] = cacc2[nt][i] = 0.f;
#pragma unroll
            for (int cp = 0; cp < 4; cp += 2) {
                // words cp, cp + 1: nibble b of each half = k 8 b + 2 c (+1); e[b] = half2(1024 + q) (b even) or
                // half2(1024 + 16 q) (b odd).  The MMA of nibble b takes the words' pair as its two k halves, so
                // its B operand is the adjacent register pair (x word 4 b + cp, 4 b + cp + 1).
                uint32_t e00[4], e10[4], e01[4], e11[4];    // [row g / g + 8][word cp / cp + 1]
                nibble_pairs4(w0[cp], e00);
                nibble_pairs4(w1[cp], e10);
                nibble_pairs4(w0[cp + 1], e01);
                nibble_pairs4(w1[cp + 1], e11);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int b = 0; b < 4; ++b)
                        mma16816(b < 2 ? cacc[nt] : cacc2[nt], e00[b], e10[b], e01[b], e11[b], xw[nt][4 * b + cp],
                                 xw[nt][4 * b + cp + 1]);
            }
            float sc[2], zc[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                sc[h] = lds_h2f(f_lane + so + 32 * rb + 16 * h);
                zc[h] = lds_h2f(f_lane + so + 128 + 32 * rb + 16 * h);
            }
            // c[0], c[1]: row g, tokens 2t, 2t+1;  c[2], c[3]: row g + 8, same tokens
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float qx = (cacc[nt][i] + cacc2[nt][i]) - x_off[nt][i & 1];
                    acc[rb][nt][i] = fmaf(sc[i >> 1], qx, acc[rb][nt][i]);
                    acc[rb][nt][i] = fmaf(zc[i >> 1], x_sum[nt][i & 1], acc[rb][nt][i]);
                }
        }
    }
    }
    __syncwarp();

    // ---- the K slices of the CTA's warps meet in shared memory (each warp's slab: start of its ring) ----
    float* slab = reinterpret_cast<float*>(ring);
    if (ok) {
#pragma unroll
        for (int rb = 0; rb < RB; ++rb)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    slab[(8 * nt + 2 * t + (i & 1)) * kRows + 16 * rb + g + 8 * (i >> 1)] = acc[rb][nt][i];
    }
    __syncthreads();
    const bool failed = *abort_flag != 0;
    if (failed && threadIdx.x == 0) {
        atomicExch(p.status, KAIROS_ERR_DEVICE);
        for (int i = 0; i < 64; ++i) __nanosleep(1000);    // let issued copies land before the CTA leaves
    }
    auto cta_sum = [&](int o) {
        float v = 0.f;
        for (int w = 0; w < W; ++w) v += reinterpret_cast<const float*>(ds_smem + w * Cfg::kWarpBytes)[o];
        return v;
    };
    auto store_out = [&](int o, float v) {
        const int tok = o / kRows, n = row0 + o % kRows;
        if (tok >= p.M || n >= p.N || failed) return;
        __half y = __float2half_rn(v);
        if (p.bias) y = __hadd(y, p.bias[n]);
        p.Y[(size_t)tok * p.N + n] = y;
    };
    const int n_out = kRows * min(8 * NT, (p.M + 1) & ~1);   // token columns that exist (pairs)
    // Gated-MLP epilogue: output o2 = (token, channel r of the tile's kRows / 2 inner channels) takes the gate row
    // 32 (r / 16) + r % 16 of the tile and the up row 16 further.  Same arithmetic as the stand-alone kernel: the
    // two linear outputs rounded to fp16 (+ bias), SiLU in fp32 rounded to fp16, fp16 product.
    auto store_gated = [&](int o2, float gv, float uv) {
        const int tok = o2 / (kRows / 2), r = o2 % (kRows / 2);
        const int ng = row0 + 32 * (r >> 4) + (r & 15);
        if (tok >= p.M || ng + 16 >= p.N || failed) return;
        __half gh = __float2half_rn(gv), uh = __float2half_rn(uv);
        if (p.bias) {
            gh = __hadd(gh, p.bias[ng]);
            uh = __hadd(uh, p.bias[ng + 16]);
        }
        const float f = __half2float(gh);
        const __half sl = __float2half_rn(f / (1.f + __expf(-f)));
        p.Y[(size_t)tok * (p.N / 2) + row0 / 2 + r] = __hmul(sl, uh);
    };
    auto gate_index = [&](int o2) {
        const int tok = o2 / (kRows / 2), r = o2 % (kRows / 2);
        return tok * kRows + 32 * (r >> 4) + (r & 15);
    };
    if (!clustered) {
        if (p.silu) {
            for (int o2 = threadIdx.x; o2 < n_out / 2; o2 += blockDim.x) {
                const int og = gate_index(o2);
                store_gated(o2, cta_sum(og), cta_sum(og + 16));
            }
        } else {
            for (int o = threadIdx.x; o < n_out; o += blockDim.x) store_out(o, cta_sum(o));
        }
        return;
    }
    // ---- the K slices of the cluster meet in the shared memory of its first CTA ----
    cluster_wait();                              // completes the arrive at the top: all peers are resident
    const uint32_t dst = cluster_map(gather + crank * kOut, 0);
    for (int o = threadIdx.x; o < n_out; o += blockDim.x) st_cluster_f32(dst + 4u * (uint32_t)o, cta_sum(o));
    cluster_arrive();
    cluster_wait();
    if (crank != 0) return;
    auto cluster_sum = [&](int o) {
        float v = 0.f;
        for (int c = 0; c < p.C; ++c) v += gather[c * kOut + o];
        return v;
    };
    if (p.silu) {
        for (int o2 = threadIdx.x; o2 < n_out / 2; o2 += blockDim.x) {
            const int og = gate_index(o2);
            store_gated(o2, cluster_sum(og), cluster_sum(og + 16));
        }
    } else {
        for (int o = threadIdx.x; o < n_out; o += blockDim.x) store_out(o, cluster_sum(o));
    }
}

// Shape of a launch: warps per CTA and K slices (cluster size) per row tile.  Measured on B200: about ten
// resident warps per SM are needed before the weight stream stops being latency-bound, clusters cost more
// the larger they are (co-scheduling in one GPC, the barrier waits for the slowest CTA, rank 0 sums all
// slices), and a warp with a single group cannot hide anything behind its ring.  So: the smallest power-of-two
// cluster that gives 2.5 CTAs of four warps per SM, eight slices only for problems that would otherwise
// leave SMs empty, and never more slices than leave each warp a group.
struct SplitShape {
    int warps, cluster, gpc;
};
static SplitShape split_shape(int N, int K, int rows) {
    const int G = K / kGroup;
    const int tiles = (N + rows - 1) / rows;
    const int sms = device_sm_count();
    SplitShape s;
    s.warps = kDsMaxWarps;
    s.cluster = 1;
    while (s.cluster < 4 && 2 * tiles * s.cluster < 5 * sms) s.cluster *= 2;
    if (s.cluster == 4 && tiles * 4 < sms) s.cluster = 8;
    // long K (64 groups or more): two slices pay even when the row tiles alone would fill the GPU -- each warp still
    // has a long run, and twice the warps hide more latency (K = 8192, N = 14336, M = 1: 20.5 -> 17.6 us)
    if (s.cluster == 1 && G >= 64 && 2 * tiles <= 7 * sms) s.cluster = 2;
    while (s.cluster > 1 && G < s.cluster * s.warps) s.cluster /= 2;
    if (s.cluster > G) s.cluster = G;
    s.gpc = (G + s.cluster - 1) / s.cluster;
    // no empty K slice: shrink the cluster until the last slice has work
    while (s.cluster > 1 && (s.cluster - 1) * s.gpc >= G) {
        --s.cluster;
        s.gpc = (G + s.cluster - 1) / s.cluster;
    }
    if (s.warps > s.gpc) s.warps = s.gpc;
    return s;
}

template <int NT, int RB, int XR>
static int launch_split(const void* X, const void* qweight, const void* scales, const void* scaled_zeros,
                        const void* bias, void* Y, int M, int N, int K, cudaStream_t stream, int silu) {
    using Cfg = SplitCfg<NT, RB, XR>;
    const SplitShape sh = split_shape(N, K, Cfg::kRows);
    SplitParams p;
    p.X = static_cast<const __half*>(X);
    p.qw = static_cast<const uint8_t*>(qweight);
    p.scales = static_cast<const __half*>(scales);
    p.zeros = static_cast<const __half*>(scaled_zeros);
    p.bias = static_cast<const __half*>(bias);
    p.Y = static_cast<__half*>(Y);
    p.M = M; p.N = N; p.K = K; p.G = K / kGroup;
    p.C = sh.cluster;
    p.gpc = sh.gpc;
    p.silu = silu;
    p.status = device_status_word();
    if (!p.status) return KAIROS_ERR_CUDA;
    CUtensorMap tw, tx, ts, tz;
    int rc;
    {   // qweight int16 [N/4, K] as bytes: a stage takes 256 bytes (one group) of 4 RB rows
        const uint64_t dims[2] = {(uint64_t)K * 2, (uint64_t)N / 4}, strides[1] = {(uint64_t)K * 2};
        const uint32_t box[2] = {256, 4 * RB};
        if ((rc = make_tmap(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, qweight, dims, strides, box,
                            CU_TENSOR_MAP_SWIZZLE_NONE)) != KAIROS_OK) return rc;
    }
    {   // X fp16 [M, K]: one group of XR token rows
        const uint64_t dims[2] = {(uint64_t)K, (uint64_t)M}, strides[1] = {(uint64_t)K * 2};
        const uint32_t box[2] = {kGroup, XR};
        if ((rc = make_tmap(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, X, dims, strides, box,
                            CU_TENSOR_MAP_SWIZZLE_NONE)) != KAIROS_OK) return rc;
    }
    {   // factors fp16 [K/128, N]
        const uint64_t dims[2] = {(uint64_t)N, (uint64_t)K / kGroup}, strides[1] = {(uint64_t)N * 2};
        const uint32_t box[2] = {Cfg::kRows, 1};
        if ((rc = make_tmap(&ts, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, scales, dims, strides, box,
                            CU_TENSOR_MAP_SWIZZLE_NONE)) != KAIROS_OK) return rc;
        if ((rc = make_tmap(&tz, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, scaled_zeros, dims, strides, box,
                            CU_TENSOR_MAP_SWIZZLE_NONE)) != KAIROS_OK) return rc;
    }
    const int tiles = (N + Cfg::kRows - 1) / Cfg::kRows;
    const size_t smem = Cfg::smem_bytes(sh.warps, sh.cluster);
    static PerDeviceFlag smem_attr;    // per instantiation
    rc = ensure_dynamic_smem(smem_attr, decode_split_kernel<NT, RB, XR>,
                             (int)Cfg::smem_bytes(kDsMaxWarps, kDsMaxCluster));
    if (rc != KAIROS_OK) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles * sh.cluster);
    cfg.blockDim = dim3(32 * sh.warps);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (chained_launch_enabled()) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (sh.cluster > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = sh.cluster;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, decode_split_kernel<NT, RB, XR>, tw, tx, ts, tz, p);
    if (e != cudaSuccess) return note_cuda_error(e);
    return launch_status();
}

}  // namespace kairos

namespace kairos {
static int decode_entry(const void* X, const void* qweight, const void* scales, const void* scaled_zeros,
                        const void* bias, void* Y, int M, int N, int K, kairos_stream_t stream, int silu) {
    if (M < 0 || M > 32 || N <= 0 || K <= 0 || (N % 8) != 0 || (K % kGroup) != 0 || (silu && (N % 32) != 0))
        return KAIROS_ERR_SHAPE;
    if (M == 0) return KAIROS_OK;
    if (!X || !qweight || !scales || !scaled_zeros || !Y || ((uintptr_t)X & 15) || ((uintptr_t)qweight & 15) ||
        ((uintptr_t)scales & 15) || ((uintptr_t)scaled_zeros & 15) || ((uintptr_t)Y & 1))
        return KAIROS_ERR_ALIGN;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    // Row blocks per warp: four (64 weight rows share one fetch of the activations) once the activations
    // are a noticeable part of the traffic and the matrix still yields enough row tiles, else two.
    // (measured: M = 4 gains 10-20 % from four row blocks on matrices of 7168 rows or more, loses below)
    const bool rb4 = M <= 8 ? ((M > 4 && N >= 4096) || (M > 2 && N >= 7168)) : (M <= 16 && N >= 2048 && N < 8192);
#define KAIROS_SPLIT(NT, RB, XR) launch_split<NT, RB, XR>(X, qweight, scales, scaled_zeros, bias, Y, M, N, K, st, silu)
    if (M <= 1) return rb4 ? KAIROS_SPLIT(1, 4, 1) : KAIROS_SPLIT(1, 2, 1);
    if (M <= 2) return rb4 ? KAIROS_SPLIT(1, 4, 2) : KAIROS_SPLIT(1, 2, 2);
    if (M <= 4) return rb4 ? KAIROS_SPLIT(1, 4, 4) : KAIROS_SPLIT(1, 2, 4);
    if (M <= 8) return rb4 ? KAIROS_SPLIT(1, 4, 8) : KAIROS_SPLIT(1, 2, 8);
    if (M <= 16) return rb4 ? KAIROS_SPLIT(2, 4, 16) : KAIROS_SPLIT(2, 2, 16);
    return KAIROS_SPLIT(4, 2, 32);
#undef KAIROS_SPLIT
}
}  // namespace kairos

/* Decode-side W4A16 on warp-level tensor-core instructions, 1 <= M <= 32 (N % 8 == 0). */
extern "C" int kairos_w4a16_decode(const void* X, const void* qweight, const void* scales, const void* scaled_zeros,
                                   const void* bias, void* Y, int M, int N, int K, kairos_stream_t stream) {
    return kairos::decode_entry(X, qweight, scales, scaled_zeros, bias, Y, M, N, K, stream, 0);
}

/* The same with the gated-MLP epilogue: N = 2 I stacked gate / up rows in the blocked order, Y_act [M, I]. */
extern "C" int kairos_w4a16_decode_silu(const void* X, const void* qweight, const void* scales, const void* scaled_zeros,
                                        const void* bias, void* Y_act, int M, int N, int K, kairos_stream_t stream) {
    return kairos::decode_entry(X, qweight, scales, scaled_zeros, bias, Y_act, M, N, K, stream, 1);
}
