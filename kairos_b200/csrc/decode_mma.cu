// Decode-side W4A16 for small batches on the legacy warp-level tensor path (path item a9,
// batches the CUDA-core GEMV cannot serve at HBM speed): Y[M,N] = X[M,K] . dequant(W)^T, M <= 16.
//
// Weight streaming is the only large traffic, so the kernel is built around the packed base:
//   * a warp step is one quantization group (128 k) of 64 weight rows = 4 KB of qweight, read as
//     eight 128-bit loads per lane that coalesce into full 128-byte lines;
//   * the uint4 values never leave registers: one lop3 turns a nibble pair into the fp16 pair
//     (1024 + q) -- or (1024 + 16 q) for the odd nibbles -- which goes straight into the A
//     fragment of mma.sync.m16n8k16 (fp32 accumulate).  No subtraction, no scaling per element;
//   * the offsets are undone per group on the accumulators:  sum q x = (C_lo - 1024 X_lo)
//     + (C_hi - 1024 X_hi) / 16, where X_lo / X_hi = sum of x over the k of even / odd nibbles come
//     from one extra MMA against an all-ones A fragment; then y += s * (sum q x) + z * (X_lo + X_hi)
//     with the stored per-group fp16 factors, in fp32;
//   * every lane's 32 k of activations (64 bytes per token) are loaded once per step and reused by
//     the four 16-row blocks of the step.
// K is split over the 8 warps of a CTA (shared-memory reduction) and, for shapes with few row
// blocks, over the CTAs of a thread-block cluster (reduction through distributed shared memory).
// No scratch memory, no atomics, one launch.
//
// Algorithmic bytes per call: K*N/2 + 4*(K/128)*N + 2*M*K + 2*M*N.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace kairos {

constexpr int kDecThreads = 256;
constexpr int kDecWarps = kDecThreads / 32;
constexpr int kDecRows = 64;              // weight rows per CTA (4 blocks of 16)

__device__ __forceinline__ void mma_m16n8k16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// word w of a chunk (fixed c) -> e[b] for b = 0..3: b even: half2(1024 + q), b odd: half2(1024 + 16 q)
__device__ __forceinline__ void nibble_pairs(uint32_t w, uint32_t (&e)[4]) {
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(e[0]) : "r"(w));
    asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xea;" : "=r"(e[1]) : "r"(w));
    const uint32_t w8 = w >> 8;
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(e[2]) : "r"(w8));
    asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xea;" : "=r"(e[3]) : "r"(w8));
}

template <int NT>   // token tiles of 8: 1 (M <= 8) or 2 (M <= 16)
__global__ void __launch_bounds__(kDecThreads, 2) decode_mma_kernel(const __half* __restrict__ X,
                                                                 const uint4* __restrict__ qweight,
                                                                 const __half* __restrict__ scales,
                                                                 const __half* __restrict__ scaled_zeros,
                                                                 const __half* __restrict__ bias,
                                                                 __half* __restrict__ Y, int M, int N, int K,
                                                                 int ksplit) {
    __shared__ float red[kDecWarps][kDecRows][8 * NT];        // per-warp partial outputs
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int row_base = (blockIdx.x / ksplit) * kDecRows;
    const int krank = blockIdx.x % ksplit;                    // this CTA's slice of K (= rank in the cluster)
    const int groups = K / kGroup;
    const int groups_per_cta = (groups + ksplit - 1) / ksplit;
    const int grp_begin = krank * groups_per_cta;
    const int grp_end = min(groups, grp_begin + groups_per_cta);

    float acc[4][NT][4];
#pragma unroll
    for (int rb = 0; rb < 4; ++rb)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[rb][nt][i] = 0.f;

    // rows of this lane: block rb -> rows row_base + 16 rb + g and + 8
    int chunk_off[4][2];       // 16-byte index of (row, k = 0) minus the k part
    bool row_ok[4][2];
#pragma unroll
    for (int rb = 0; rb < 4; ++rb)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = row_base + 16 * rb + g + 8 * h;
            row_ok[rb][h] = row < N;
            chunk_off[rb][h] = (row >> 2) * (K / 8) + 2 * (row & 3);
        }
    const uint32_t ones = 0x3c003c00u;     // half2(1, 1)

    for (int grp = grp_begin + warp; grp < grp_end; grp += kDecWarps) {
        // lane's 32 k of this group: k block 2*grp + (t >> 1), half t & 1
        const int kc = 8 * (2 * grp + (t >> 1)) + (t & 1);              // 16-byte chunk column
        uint4 raw[4][2];
#pragma unroll
        for (int rb = 0; rb < 4; ++rb)
#pragma unroll
            for (int h = 0; h < 2; ++h)
                raw[rb][h] = row_ok[rb][h] ? __ldg(qweight + chunk_off[rb][h] + kc) : make_uint4(0, 0, 0, 0);
        // activations of token g (and g + 8): the same 32 k, 64 bytes
        uint4 xv[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int tok = g + 8 * nt;
            const uint4* xp = reinterpret_cast<const uint4*>(X + (size_t)min(tok, M - 1) * K + kGroup * grp + 32 * t);
#pragma unroll
            for (int b = 0; b < 4; ++b) xv[nt][b] = tok < M ? __ldg(xp + b) : make_uint4(0, 0, 0, 0);
        }
        __half sc[4][2], zc[4][2];
#pragma unroll
        for (int rb = 0; rb < 4; ++rb)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = row_base + 16 * rb + g + 8 * h;
                sc[rb][h] = row_ok[rb][h] ? __ldg(scales + (size_t)grp * N + row) : __float2half_rn(0.f);
                zc[rb][h] = row_ok[rb][h] ? __ldg(scaled_zeros + (size_t)grp * N + row) : __float2half_rn(0.f);
            }

        // X_lo / X_hi of tokens (2t, 2t+1): ones . x over the k of even / odd nibbles
        float xs_lo[NT][4], xs_hi[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int i = 0; i < 4; ++i) xs_lo[nt][i] = xs_hi[nt][i] = 0.f;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const uint32_t* xw = reinterpret_cast<const uint32_t*>(&xv[nt][b]);
                if (b & 1) {
                    mma_m16n8k16(xs_hi[nt], ones, ones, ones, ones, xw[0], xw[1]);
                    mma_m16n8k16(xs_hi[nt], ones, ones, ones, ones, xw[2], xw[3]);
                } else {
                    mma_m16n8k16(xs_lo[nt], ones, ones, ones, ones, xw[0], xw[1]);
                    mma_m16n8k16(xs_lo[nt], ones, ones, ones, ones, xw[2], xw[3]);
                }
            }
        }

#pragma unroll
        for (int rb = 0; rb < 4; ++rb) {
            float c_lo[NT][4], c_hi[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) c_lo[nt][i] = c_hi[nt][i] = 0.f;
            // e0[c][b], e1[c][b]: nibble pairs of the chunk of row g / row g + 8
            uint32_t e0[4][4], e1[4][4];
            nibble_pairs(raw[rb][0].x, e0[0]); nibble_pairs(raw[rb][0].y, e0[1]);
            nibble_pairs(raw[rb][0].z, e0[2]); nibble_pairs(raw[rb][0].w, e0[3]);
            nibble_pairs(raw[rb][1].x, e1[0]); nibble_pairs(raw[rb][1].y, e1[1]);
            nibble_pairs(raw[rb][1].z, e1[2]); nibble_pairs(raw[rb][1].w, e1[3]);
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                // k = 8b + 2c (+d): the four pairs c = 0..3 of nibble b line up with the b-th 16 bytes of x
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const uint32_t* xw = reinterpret_cast<const uint32_t*>(&xv[nt][b]);
                    if (b & 1) {
                        mma_m16n8k16(c_hi[nt], e0[0][b], e1[0][b], e0[1][b], e1[1][b], xw[0], xw[1]);
                        mma_m16n8k16(c_hi[nt], e0[2][b], e1[2][b], e0[3][b], e1[3][b], xw[2], xw[3]);
                    } else {
                        mma_m16n8k16(c_lo[nt], e0[0][b], e1[0][b], e0[1][b], e1[1][b], xw[0], xw[1]);
                        mma_m16n8k16(c_lo[nt], e0[2][b], e1[2][b], e0[3][b], e1[3][b], xw[2], xw[3]);
                    }
                }
            }
            // c[0], c[1]: row g, tokens 2t, 2t+1;  c[2], c[3]: row g + 8, same tokens
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int h = i >> 1;
                    const float xl = xs_lo[nt][i & 1], xh = xs_hi[nt][i & 1];
                    const float qx = (c_lo[nt][i] - 1024.f * xl) + (c_hi[nt][i] - 1024.f * xh) * 0.0625f;
                    acc[rb][nt][i] += __half2float(sc[rb][h]) * qx + __half2float(zc[rb][h]) * (xl + xh);
                }
        }
    }

    // ---- reduce over the warps of the CTA ----
#pragma unroll
    for (int rb = 0; rb < 4; ++rb)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i)
                red[warp][16 * rb + g + 8 * (i >> 1)][8 * nt + 2 * t + (i & 1)] = acc[rb][nt][i];
    __syncthreads();
    float* out = &red[0][0][0];                // [row][token] sums of this CTA, in place of warp 0's slab
    for (int o = threadIdx.x; o < kDecRows * 8 * NT; o += kDecThreads) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) v += (&red[w][0][0])[o];
        __syncwarp();
        out[o] = v;                            // o is owned by this thread in every slab: no hazard
    }
    // ---- reduce over the CTAs of the cluster (K slices), rank 0 writes ----
    if (ksplit > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        if (krank == 0) {
            for (int o = threadIdx.x; o < kDecRows * 8 * NT; o += kDecThreads) {
                float v = out[o];
                for (int r = 1; r < ksplit; ++r) v += cluster.map_shared_rank(out, r)[o];
                out[o] = v;
            }
        }
        cluster.sync();                        // remote shared memory stays valid until it has been read
        if (krank != 0) return;
    }
    __syncthreads();
    // token-major write: consecutive threads -> consecutive rows
    for (int o = threadIdx.x; o < kDecRows * 8 * NT; o += kDecThreads) {
        const int tok = o / kDecRows, r = o % kDecRows;
        const int n = row_base + r;
        if (tok >= M || n >= N) continue;
        __half y = __float2half_rn(out[r * (8 * NT) + tok]);
        if (bias) y = __hadd(y, bias[n]);
        Y[(size_t)tok * N + n] = y;
    }
}

int device_sm_count();   // gemm_sm100.cu

}  // namespace kairos

/* Decode-side W4A16 on warp-level tensor-core instructions, 1 <= M <= 16. */
extern "C" int kairos_w4a16_decode(const void* X, const void* qweight, const void* scales, const void* scaled_zeros,
                                   const void* bias, void* Y, int M, int N, int K, kairos_stream_t stream) {
    using namespace kairos;
    if (M < 0 || M > 16 || N <= 0 || K <= 0 || (N % kInterleave) != 0 || (K % kGroup) != 0) return KAIROS_ERR_SHAPE;
    if (M == 0) return KAIROS_OK;
    if (!X || !qweight || !scales || !scaled_zeros || !Y || ((uintptr_t)X & 15) || ((uintptr_t)qweight & 15) ||
        ((uintptr_t)Y & 1))
        return KAIROS_ERR_ALIGN;
    const int row_blocks = (N + kDecRows - 1) / kDecRows;
    const int groups = K / kGroup;
    // split K over a cluster while the grid is under two CTAs per SM and at least half the warps keep a group
    int ksplit = 1;
    const int sms = device_sm_count();
    while (ksplit < 8 && row_blocks * ksplit < 2 * sms && groups / (ksplit * 2) >= kDecWarps / 2) ksplit *= 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(row_blocks * ksplit));
    cfg.blockDim = dim3(kDecThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)ksplit;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const __half* x = static_cast<const __half*>(X);
    const uint4* qw = static_cast<const uint4*>(qweight);
    const __half* sc = static_cast<const __half*>(scales);
    const __half* sz = static_cast<const __half*>(scaled_zeros);
    const __half* b = static_cast<const __half*>(bias);
    __half* y = static_cast<__half*>(Y);
    cudaError_t e;
    if (M <= 8)
        e = cudaLaunchKernelEx(&cfg, decode_mma_kernel<1>, x, qw, sc, sz, b, y, M, N, K, ksplit);
    else
        e = cudaLaunchKernelEx(&cfg, decode_mma_kernel<2>, x, qw, sc, sz, b, y, M, N, K, ksplit);
    if (e != cudaSuccess) return note_cuda_error(e);
    return launch_status();
}
