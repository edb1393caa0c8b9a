// Per-token symmetric int8 activation quantization (path item a6).
//
// One CTA of 256 threads per token.  The token row is read from HBM once (consecutive lanes read
// consecutive 16-byte chunks), kept in registers across the block-wide amax reduction, and written back
// as int8: 2 bytes read + 1 byte written per element, the algorithmic minimum.
//
// Arithmetic, kRefCuda = false: the reference's torch twin quantize_tensor_int8(x,'S',-1)
// (kairos/quantization.py:111-141): fp32 amax clamped at 1e-7, scale = amax/127 by IEEE division,
// q = rint(x/scale) with the IEEE quotient and round-half-even (quant8_chunk forms the quotient by division
// only next to a rounding boundary), sx = fp16(scale).
// kRefCuda = true: the reference's CUDA kernel as its build (nvcc --use_fast_math) compiles it
// (kernels/csrc/kairos_kernel/quant/quant_f16_to_i8.cu:54-77): sx = fp16(amax / 127),
// q = cvt.rni.sat.s8(x * (127 / amax)), both divisions approximate (div.approx.ftz), amax not clamped (an
// all-zero token gives 127/0 = inf, 0 * inf = NaN, which the saturating conversion turns into 0).
#include "common.cuh"

namespace kairos {

constexpr int kAqThreads = 256;

template <int R, bool kRefCuda>   // R = 8-element chunks per thread, upper bound
__global__ void __launch_bounds__(kAqThreads) act_quant_kernel(const __half* __restrict__ X,
                                                               int8_t* __restrict__ Xq,
                                                               __half* __restrict__ sx, int K) {
    chain_release();
    chain_wait();
    const int token = blockIdx.x;
    const int chunks = K >> 3;
    const uint4* row = reinterpret_cast<const uint4*>(X + (size_t)token * K);
    uint4 v[R];
    __half2 hmax = __float2half2_rn(0.f);
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int c = threadIdx.x + r * kAqThreads;
        if (c < chunks) {
            v[r] = __ldcg(row + c);
            const __half2* h = reinterpret_cast<const __half2*>(&v[r]);
#pragma unroll
            for (int i = 0; i < 4; ++i) hmax = __hmax2(hmax, __habs2(h[i]));   // exact: the maximum of fp16 values
        }
    }
    const float2 hm = __half22float2(hmax);
    float amax = fmaxf(hm.x, hm.y);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    __shared__ float warp_max[kAqThreads / 32];
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = warp_max[0];
#pragma unroll
    for (int w = 1; w < kAqThreads / 32; ++w) amax = fmaxf(amax, warp_max[w]);

    uint2* out = reinterpret_cast<uint2*>(Xq + (size_t)token * K);
    if constexpr (kRefCuda) {
        float sc, mult;
        asm("div.approx.ftz.f32 %0, %1, 0f42FE0000;" : "=f"(sc) : "f"(amax));      // amax / 127
        asm("div.approx.ftz.f32 %0, 0f42FE0000, %1;" : "=f"(mult) : "f"(amax));    // 127 / amax
        if (threadIdx.x == 0) sx[token] = __float2half_rn(sc);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int c = threadIdx.x + r * kAqThreads;
            if (c < chunks) {
                const __half2* h = reinterpret_cast<const __half2*>(&v[r]);
                uint32_t b[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __half22float2(h[i]);
                    float p0, p1;
                    asm("mul.ftz.f32 %0, %1, %2;" : "=f"(p0) : "f"(f.x), "f"(mult));
                    asm("mul.ftz.f32 %0, %1, %2;" : "=f"(p1) : "f"(f.y), "f"(mult));
                    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(b[2 * i]) : "f"(p0));
                    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(b[2 * i + 1]) : "f"(p1));
                }
                uint2 o;
                o.x = (b[0] & 0xff) | ((b[1] & 0xff) << 8) | ((b[2] & 0xff) << 16) | (b[3] << 24);
                o.y = (b[4] & 0xff) | ((b[5] & 0xff) << 8) | ((b[6] & 0xff) << 16) | (b[7] << 24);
                out[c] = o;
            }
        }
    } else {
        const float scale = __fdiv_rn(fmaxf(amax, 1e-7f), 127.0f);
        if (threadIdx.x == 0) sx[token] = __float2half_rn(scale);
        const float inv = __frcp_rn(scale);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int c = threadIdx.x + r * kAqThreads;
            if (c < chunks) {
                out[c] = quant8_chunk(v[r], scale, inv);
            }
        }
    }
}

}  // namespace kairos

extern "C" int kairos_act_quant_i8(const void* X, void* Xq, void* sx, int M, int K, kairos_stream_t stream) {
    using namespace kairos;
    if (M < 0 || K <= 0 || (K % 16) != 0) return KAIROS_ERR_SHAPE;
    if (M == 0) return KAIROS_OK;
    if (!X || !Xq || !sx || ((uintptr_t)X & 15) || ((uintptr_t)Xq & 15) || ((uintptr_t)sx & 1))
        return KAIROS_ERR_ALIGN;
    const int per_thread = (K / 8 + kAqThreads - 1) / kAqThreads;
    const __half* x = static_cast<const __half*>(X);
    int8_t* q = static_cast<int8_t*>(Xq);
    __half* s = static_cast<__half*>(sx);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    cudaError_t e;
    const bool ref_cuda = arithmetic_rule() == KAIROS_ARITH_REFERENCE_CUDA;
#define KAIROS_AQ(R)                                                                                         \
    (ref_cuda ? launch_chained(act_quant_kernel<R, true>, dim3(M), dim3(kAqThreads), 0, st, x, q, s, K)     \
              : launch_chained(act_quant_kernel<R, false>, dim3(M), dim3(kAqThreads), 0, st, x, q, s, K))
    if (per_thread <= 1)
        e = KAIROS_AQ(1);
    else if (per_thread <= 2)
        e = KAIROS_AQ(2);
    else if (per_thread <= 4)
        e = KAIROS_AQ(4);
    else if (per_thread <= 8)
        e = KAIROS_AQ(8);
    else if (per_thread <= 16)
        e = KAIROS_AQ(16);
    else
        return KAIROS_ERR_SHAPE;   // K > 32768
#undef KAIROS_AQ
    if (e != cudaSuccess) return note_cuda_error(e);
    return launch_status();
}
