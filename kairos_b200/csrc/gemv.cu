// Decode-side W4A16 GEMV (path item a9): Y[M,N] = X[M,K] . dequant(W)^T, small M.
//
// HBM-bound weight streaming on the CUDA cores.  A warp owns 4 interleaved weight rows
// (one qweight row n0) over a K slice and walks it in 256-wide steps: each step is one
// fully coalesced 512-byte burst (32 lanes x 128-bit loads), of which a lane's 16 bytes
// are 32 consecutive k of ONE weight row.  Up to four such loads are in flight per lane
// before the first is consumed.  The uint4 values are expanded in registers
// (lop3 magic-number trick), scaled with the stored fp16 (scale, scaled_zero) exactly as
// the fp16 conversion does, multiplied with X in half2 over the 32-k chunk and
// accumulated across chunks in fp32.  The 8 lanes of a weight row are reduced with
// shuffles, the K slices of a block through shared memory.  No scratch memory, no atomics.
// Up to eight tokens share one pass over the weight; more tokens take further passes (grid.y), so
// beyond M = 8 this kernel is only the fallback for N % 8 == 4, which the warp-MMA decode kernel
// (and the reference's own GEMV, gemv_cuda.cu:277) does not accept.
//
// Algorithmic bytes per call: K*N/2 (weights) + 4*(K/128)*N (factors) + 2*M*K + 2*M*N.
#include "common.cuh"

namespace kairos {

int device_sm_count();   // gemm_sm100.cu

constexpr int kGvThreads = 256;
constexpr int kGvWarps = kGvThreads / 32;
constexpr int kGvUnroll = 4;

template <int MT>
__global__ void __launch_bounds__(kGvThreads) gemv_kernel(const __half* __restrict__ X,
                                                          const uint4* __restrict__ qweight,
                                                          const __half* __restrict__ scales,
                                                          const __half* __restrict__ scaled_zeros,
                                                          const __half* __restrict__ bias, __half* __restrict__ Y,
                                                          int M, int N, int K, int slices, int steps_per_slice) {
    __shared__ float red[kGvWarps][kInterleave][MT];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rows_per_block = kGvWarps / slices;          // qweight rows (n0) per block
    const int n0 = blockIdx.x * rows_per_block + warp / slices;
    const int slice = warp % slices;
    const int m_base = blockIdx.y * MT;
    const int n1 = lane >> 3;
    const int kb_total = K / kKStride;
    const int a = lane & 1;
    const bool row_ok = n0 < N / kInterleave;
    const int n = kInterleave * n0 + n1;

    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;

    if (row_ok) {
        const uint4* wrow = qweight + (size_t)n0 * (K / 8) + 2 * n1 + a;
        const int step0 = slice * steps_per_slice;
        for (int st = 0; st < steps_per_slice; st += kGvUnroll) {
            uint4 raw[kGvUnroll];
            __half s[kGvUnroll], z[kGvUnroll];
            int kk[kGvUnroll];
#pragma unroll
            for (int u = 0; u < kGvUnroll; ++u) {
                const int step = step0 + st + u;
                const int k0 = 4 * step + ((lane & 7) >> 1);
                const bool ok = (st + u < steps_per_slice) && (k0 < kb_total);
                kk[u] = ok ? kKStride * k0 + 32 * a : -1;
                if (ok) {
                    raw[u] = __ldg(wrow + 8 * k0);
                    const int g = kk[u] / kGroup;
                    s[u] = __ldg(scales + (size_t)g * N + n);
                    z[u] = __ldg(scaled_zeros + (size_t)g * N + n);
                }
            }
#pragma unroll
            for (int u = 0; u < kGvUnroll; ++u) {
                if (kk[u] < 0) continue;
                __half2 w[16];
                dequant_chunk32(raw[u], __half2half2(s[u]), __half2half2(z[u]), w);
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const int mm = min(m_base + m, M - 1);
                    const uint4* xp = reinterpret_cast<const uint4*>(X + (size_t)mm * K + kk[u]);
                    __half2 p0 = __float2half2_rn(0.f), p1 = __float2half2_rn(0.f);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint4 xv = __ldg(xp + j);
                        const __half2* x2 = reinterpret_cast<const __half2*>(&xv);
                        p0 = __hfma2(w[4 * j + 0], x2[0], p0);
                        p1 = __hfma2(w[4 * j + 1], x2[1], p1);
                        p0 = __hfma2(w[4 * j + 2], x2[2], p0);
                        p1 = __hfma2(w[4 * j + 3], x2[3], p1);
                    }
                    const float2 f0 = __half22float2(p0), f1 = __half22float2(p1);
                    acc[m] += (f0.x + f0.y) + (f1.x + f1.y);
                }
            }
        }
    }
    // the 8 lanes of one weight row
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], 1);
        acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], 2);
        acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], 4);
    }
    if ((lane & 7) == 0) {
#pragma unroll
        for (int m = 0; m < MT; ++m) red[warp][n1][m] = acc[m];
    }
    __syncthreads();
    // one thread per (row of the block, token)
    const int outs = rows_per_block * kInterleave * MT;
    for (int o = threadIdx.x; o < outs; o += kGvThreads) {
        const int m = o % MT;
        const int r = o / MT;                 // row within the block: 4*r0 + n1
        const int r0 = r / kInterleave, rn1 = r % kInterleave;
        const int nn = (blockIdx.x * rows_per_block + r0) * kInterleave + rn1;
        if (nn >= N || m_base + m >= M) continue;
        float v = 0.f;
        for (int sidx = 0; sidx < slices; ++sidx) v += red[r0 * slices + sidx][rn1][m];
        __half y = __float2half_rn(v);
        if (bias) y = __hadd(y, bias[nn]);
        Y[(size_t)(m_base + m) * N + nn] = y;
    }
}

}  // namespace kairos

extern "C" int kairos_w4a16_gemv(const void* X, const void* qweight, const void* scales, const void* scaled_zeros,
                                 const void* bias, void* Y, int M, int N, int K, kairos_stream_t stream) {
    using namespace kairos;
    if (M < 0 || M > 32 || N <= 0 || K <= 0 || (N % kInterleave) != 0 || (K % kGroup) != 0) return KAIROS_ERR_SHAPE;
    if (M == 0) return KAIROS_OK;
    if (!X || !qweight || !scales || !scaled_zeros || !Y || ((uintptr_t)X & 15) || ((uintptr_t)qweight & 15) ||
        ((uintptr_t)Y & 1))
        return KAIROS_ERR_ALIGN;
    // K slices per qweight row: aim at <= 4 steps (of 256 k) per warp, at most 8 warps per row;
    // use all 8 when the grid would otherwise be under two blocks per SM
    const int steps = (K / kKStride + 3) / 4;
    int slices = 1;
    while (slices < kGvWarps && (steps + slices - 1) / slices > kGvUnroll) slices *= 2;
    const int n_rows = N / kInterleave;
    while (slices < kGvWarps && (n_rows * slices) / kGvWarps < 2 * device_sm_count()) slices *= 2;
    const int steps_per_slice = (steps + slices - 1) / slices;
    const int rows_per_block = kGvWarps / slices;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const __half* x = static_cast<const __half*>(X);
    const uint4* qw = static_cast<const uint4*>(qweight);
    const __half* sc = static_cast<const __half*>(scales);
    const __half* sz = static_cast<const __half*>(scaled_zeros);
    const __half* b = static_cast<const __half*>(bias);
    __half* y = static_cast<__half*>(Y);
    const unsigned gx = (unsigned)((n_rows + rows_per_block - 1) / rows_per_block);
#define KAIROS_GEMV_CASE(MT_)                                                                               \
    gemv_kernel<MT_><<<dim3(gx, (unsigned)((M + MT_ - 1) / MT_)), kGvThreads, 0, st>>>(x, qw, sc, sz, b, y, M, N, K, \
                                                                                    slices, steps_per_slice)
    switch (M) {
        case 1: KAIROS_GEMV_CASE(1); break;
        case 2: KAIROS_GEMV_CASE(2); break;
        case 3: KAIROS_GEMV_CASE(3); break;
        case 4: KAIROS_GEMV_CASE(4); break;
        case 5: KAIROS_GEMV_CASE(5); break;
        case 6: KAIROS_GEMV_CASE(6); break;
        case 7: KAIROS_GEMV_CASE(7); break;
        default: KAIROS_GEMV_CASE(8); break;
    }
#undef KAIROS_GEMV_CASE
    return launch_status();
}
