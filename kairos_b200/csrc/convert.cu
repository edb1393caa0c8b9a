// On-the-fly weight conversion from the resident packed-uint4 base (path items a7, a8)
// and the AWQ -> QServe nibble permutation.
//
// Base layout: with n = 4*n0 + n1 and k = 64*k0 + 32*a + 8*b + 2*c + d, nibble b of
// qweight[n0, 64*k0 + 16*n1 + 8*a + 2*c + d] (int16) is q[n,k]
// (thirdparty/AWQ/awq_method.py:3-38).  A 16-byte chunk of a qweight row therefore
// holds 32 consecutive k of ONE weight row.
//
// A warp takes 512 contiguous bytes of a qweight row (4 k-blocks x 4 interleaved rows
// x 2 halves): the reads are one fully coalesced 512-byte burst, and the lanes are
// permuted so that the 8 lanes of one output row write 8 x 32 (int8) or 8 x 64 (fp16)
// contiguous bytes.  Traffic = K*N/2 read + K*N (or 2*K*N) written + the factor tensors:
// the algorithmic minimum, no shared memory.
#include "common.cuh"

namespace kairos {

constexpr int kCvThreads = 256;

// kFma selects the rounding of q*s + sz: false = product rounded, then sum rounded (the reference's torch
// functions); true = one fused multiply-add, as in the reference's CUDA kernels
// (dequant_awq_format/dequant_i4_to_f16.cu:17-35).
template <bool kToInt8, bool kFma>
__global__ void __launch_bounds__(kCvThreads) convert_kernel(const uint4* __restrict__ qweight,
                                                             const __half* __restrict__ scales,
                                                             const __half* __restrict__ scaled_zeros,
                                                             void* __restrict__ out, int N, int K) {
    const int kb_total = K / kKStride;                 // 64-wide k blocks per row
    const int kgroups = (kb_total + 3) >> 2;           // warp tasks per qweight row
    const long long task = (long long)blockIdx.x * (kCvThreads / 32) + (threadIdx.x >> 5);
    const long long n_tasks = (long long)(N / kInterleave) * kgroups;
    if (task >= n_tasks) return;
    const int n0 = (int)(task / kgroups);
    const int kg = (int)(task % kgroups);
    const int lane = threadIdx.x & 31;
    const int n1 = lane >> 3;
    const int k0 = 4 * kg + ((lane & 7) >> 1);
    const int a = lane & 1;
    if (k0 >= kb_total) return;
    const int n = kInterleave * n0 + n1;
    const int k = kKStride * k0 + 32 * a;
    // chunk index within the row, in 16-byte units: (64*k0 + 16*n1 + 8*a) int16 / 8
    const uint4 raw = __ldg(qweight + (size_t)n0 * (K / 8) + 8 * k0 + 2 * n1 + a);
    const int g = k / kGroup;
    const __half2 s = __half2half2(__ldg(scales + (size_t)g * N + n));
    const __half2 z = __half2half2(__ldg(scaled_zeros + (size_t)g * N + n));
    __half2 w[16];
    if constexpr (kFma)
        dequant_chunk32_fma(raw, s, z, w);
    else
        dequant_chunk32(raw, s, z, w);
    if constexpr (kToInt8) {
        // (int8) of an fp16 value truncates toward zero
        // (kernels/csrc/kairos_kernel/dequant_awq_format/dequant_i4_to_i8.cu:143-146)
        uint32_t o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int q0 = __half2int_rz(__low2half(w[2 * j]));
            const int q1 = __half2int_rz(__high2half(w[2 * j]));
            const int q2 = __half2int_rz(__low2half(w[2 * j + 1]));
            const int q3 = __half2int_rz(__high2half(w[2 * j + 1]));
            o[j] = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) |
                   ((uint32_t)(q3 & 0xff) << 24);
        }
        uint4* dst = reinterpret_cast<uint4*>(static_cast<int8_t*>(out) + (size_t)n * K + k);
        dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
    } else {
        uint4* dst = reinterpret_cast<uint4*>(static_cast<__half*>(out) + (size_t)n * K + k);
        const uint32_t* u = reinterpret_cast<const uint32_t*>(w);
#pragma unroll
        for (int j = 0; j < 4; ++j) dst[j] = make_uint4(u[4 * j], u[4 * j + 1], u[4 * j + 2], u[4 * j + 3]);
    }
}

// One thread per 32-bit output word of the QServe layout.  Output byte order is the
// flattening of (n/32, k/32, n%8, (k%16)/4, (k%32)/16, (n%16)/8, k%4) with the low
// nibble from row n (n%32 < 16) and the high nibble from row n+16
// (pack_int_qserve, test/test_trans_layout.py:7-13).
__global__ void __launch_bounds__(256) awq_to_qserve_kernel(const uint16_t* __restrict__ qweight,
                                                            uint32_t* __restrict__ out, int N, int K) {
    const long long word = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long n_words = (long long)N * K / 8;
    if (word >= n_words) return;
    long long f = word;
    const int i2 = (int)(f & 1); f >>= 1;
    const int j1 = (int)(f & 1); f >>= 1;
    const int j2 = (int)(f & 3); f >>= 2;
    const int i3 = (int)(f & 7); f >>= 3;
    const int k32 = (int)(f % (K / 32));
    const int n32 = (int)(f / (K / 32));
    const int kbase = 32 * k32 + 16 * j1 + 4 * j2;     // four consecutive k: j3 = 0..3
    const int k0 = kbase >> 6, a = (kbase >> 5) & 1, b = (kbase >> 3) & 3, c = (kbase >> 1) & 3;   // d = j3 & 1
    uint32_t bytes = 0;
#pragma unroll
    for (int i1 = 0; i1 < 2; ++i1) {
        const int n = 32 * n32 + 16 * i1 + 8 * i2 + i3;
        const uint16_t* src = qweight + (size_t)(n >> 2) * K + 64 * k0 + 16 * (n & 3) + 8 * a + 2 * c;
        const uint2 v = __ldg(reinterpret_cast<const uint2*>(src));      // 4 int16: (c, d), (c, d+1), (c+1, ..)
        const uint32_t h[4] = {v.x & 0xffffu, v.x >> 16, v.y & 0xffffu, v.y >> 16};
#pragma unroll
        for (int j3 = 0; j3 < 4; ++j3) bytes |= ((h[j3] >> (4 * b)) & 0xfu) << (8 * j3 + 4 * i1);
    }
    out[word] = bytes;
}

static int check_base(const void* qweight, const void* s, const void* z, const void* out, int N, int K) {
    if (N <= 0 || K <= 0 || (N % kInterleave) != 0 || (K % kGroup) != 0) return KAIROS_ERR_SHAPE;
    if (!qweight || !s || !z || !out || ((uintptr_t)qweight & 15) || ((uintptr_t)out & 15) ||
        ((uintptr_t)s & 1) || ((uintptr_t)z & 1))
        return KAIROS_ERR_ALIGN;
    return KAIROS_OK;
}

template <bool kToInt8>
static int launch_convert(const void* qweight, const void* s, const void* z, void* out, int N, int K,
                          kairos_stream_t stream) {
    const int rc = check_base(qweight, s, z, out, N, K);
    if (rc != KAIROS_OK) return rc;
    const int kgroups = (K / kKStride + 3) / 4;
    const long long tasks = (long long)(N / kInterleave) * kgroups;
    const int warps = kCvThreads / 32;
    const unsigned grid = (unsigned)((tasks + warps - 1) / warps);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (arithmetic_rule() == KAIROS_ARITH_REFERENCE_CUDA)
        convert_kernel<kToInt8, true><<<grid, kCvThreads, 0, st>>>(
            static_cast<const uint4*>(qweight), static_cast<const __half*>(s), static_cast<const __half*>(z), out, N, K);
    else
        convert_kernel<kToInt8, false><<<grid, kCvThreads, 0, st>>>(
            static_cast<const uint4*>(qweight), static_cast<const __half*>(s), static_cast<const __half*>(z), out, N, K);
    return launch_status();
}

}  // namespace kairos

extern "C" int kairos_w4_to_w8(const void* qweight, const void* scales_to8, const void* scaled_zeros_to8, void* W8,
                               int N, int K, kairos_stream_t stream) {
    return kairos::launch_convert<true>(qweight, scales_to8, scaled_zeros_to8, W8, N, K, stream);
}

extern "C" int kairos_w4_to_f16(const void* qweight, const void* scales, const void* scaled_zeros, void* W16, int N,
                                int K, kairos_stream_t stream) {
    return kairos::launch_convert<false>(qweight, scales, scaled_zeros, W16, N, K, stream);
}

extern "C" int kairos_awq_to_qserve(const void* qweight, void* out, int N, int K, kairos_stream_t stream) {
    if (N <= 0 || K <= 0 || (N % 32) != 0 || (K % 64) != 0) return KAIROS_ERR_SHAPE;
    if (!qweight || !out || ((uintptr_t)qweight & 15) || ((uintptr_t)out & 15)) return KAIROS_ERR_ALIGN;
    const long long words = (long long)N * K / 8;
    const unsigned grid = (unsigned)((words + 255) / 256);
    kairos::awq_to_qserve_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(qweight), static_cast<uint32_t*>(out), N, K);
    return kairos::launch_status();
}
