// Element-wise operators that sit directly before / after the switched linears of a decoder layer,
// each as ONE pass over the activations: RMSNorm, SiLU(gate) * up, and rotary embedding fused with the
// KV-cache write.  The reference vendors (and never calls) rms_norm_general and silu_and_mul
// (thirdparty/AWQ/kernels/csrc/w8a8/layernorm.cu:56-231, act.cu:34-140); in a stock torch / HuggingFace
// decoder these steps are ~40 small kernels per layer and dominate both the decode step and the
// non-GEMM part of prefill.  All are HBM-bound: 2 bytes read + 2 bytes written per element.
#include "common.cuh"
#include "peer.cuh"

namespace kairos {

// Row chunk of the residual stream: x, or (with a pending delta H) x + h in fp16, which is also written
// back to X -- the residual addition of the layer before rides in the norm that follows it.
__device__ __forceinline__ uint4 load_residual(__half* X, const __half* H, size_t row_off, int c) {
    uint4* xp = reinterpret_cast<uint4*>(X + row_off) + c;
    uint4 v = __ldcg(xp);
    if (H) {
        const uint4 h4 = __ldcg(reinterpret_cast<const uint4*>(H + row_off) + c);
        __half2* a = reinterpret_cast<__half2*>(&v);
        const __half2* b = reinterpret_cast<const __half2*>(&h4);
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = __hadd2(a[i], b[i]);
        *xp = v;
    }
    return v;
}

// The same with the pending delta still spread over a tensor-parallel group: the delta is the output of a
// row-parallel linear, every rank holds its partial in peer-addressable memory, and the norm sums the partials in
// rank order (fp32, one rounding to fp16: the bits the stand-alone all-reduce produces) while it loads them.
// The all-reduce then costs no kernel of its own.
__device__ __forceinline__ uint4 load_residual_peer(__half* X, const PeerSet& ps, size_t row_off, int c) {
    uint4* xp = reinterpret_cast<uint4*>(X + row_off) + c;
    uint4 v = __ldcg(xp);
    const uint4 h4 = peer_sum8(ps, (long long)(row_off >> 3) + c);
    __half2* a = reinterpret_cast<__half2*>(&v);
    const __half2* b = reinterpret_cast<const __half2*>(&h4);
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = __hadd2(a[i], b[i]);
    *xp = v;
    return v;
}

// y = half( float(x) * rsqrt(mean(x^2) + eps) * float(w) ), one CTA per token, row kept in registers
template <int R, bool kPeer>
__global__ void __launch_bounds__(256) rms_norm_kernel(__half* X, const __half* __restrict__ H, const PeerSet ps,
                                                       const __half* __restrict__ W, __half* __restrict__ Y, int K,
                                                       float eps) {
    chain_release();
    chain_wait();
    const int token = blockIdx.x;
    if constexpr (kPeer) {
        if (!peer_barrier(ps, token)) return;       // the token's row of every rank's partial is complete
    }
    const int chunks = K >> 3;
    uint4 v[R];
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int c = threadIdx.x + r * 256;
        if (c < chunks) {
            if constexpr (kPeer) v[r] = load_residual_peer(X, ps, (size_t)token * K, c);
            else v[r] = load_residual(X, H, (size_t)token * K, c);
            const __half2* h = reinterpret_cast<const __half2*>(&v[r]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(h[i]);
                ss += f.x * f.x + f.y * f.y;
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    __shared__ float part[8];
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    ss = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) ss += part[w];
    const float inv = rsqrtf(ss / (float)K + eps);
    uint4* out = reinterpret_cast<uint4*>(Y + (size_t)token * K);
    const uint4* wv = reinterpret_cast<const uint4*>(W);
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int c = threadIdx.x + r * 256;
        if (c < chunks) {
            const uint4 wq = __ldg(wv + c);
            const __half2* h = reinterpret_cast<const __half2*>(&v[r]);
            const __half2* g = reinterpret_cast<const __half2*>(&wq);
            uint4 o4;
            __half2* o = reinterpret_cast<__half2*>(&o4);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(h[i]), gw = __half22float2(g[i]);
                o[i] = __floats2half2_rn(f.x * inv * gw.x, f.y * inv * gw.y);
            }
            out[c] = o4;
        }
    }
}

// Where gate and up of inner channel i sit in a row of the stacked activation [2 I]:
//   plain layout    gate at i, up at I + i (the two weights stacked one after the other);
//   blocked layout  16 gate channels, then their 16 up channels, and so on: gate at 32 (i / 16) + i % 16, up 16
//                   further.  A row tile of the decode kernel (32 or 64 weight rows) then holds matching gate and
//                   up rows, so that kernel can apply SiLU(gate) * up in its epilogue (kairos_w4a16_decode_silu).
// In 16-byte chunks of 8 channels: chunk c of the result reads gate chunk gate_chunk(c) and up chunk up_chunk(c).
__device__ __forceinline__ int gate_chunk(int c, int per_row, bool blocked) { return blocked ? 4 * (c >> 1) + (c & 1) : c; }
__device__ __forceinline__ int up_chunk(int c, int per_row, bool blocked) {
    return blocked ? 4 * (c >> 1) + (c & 1) + 2 : per_row + c;
}

// Y[m, i] = half( half(silu(gate)) * up )
__global__ void __launch_bounds__(256) silu_mul_kernel(const __half* __restrict__ GU, __half* __restrict__ Y, int M,
                                                       int I, int blocked) {
    chain_release();
    chain_wait();
    const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;       // one 8-element chunk
    const int per_row = I >> 3;
    if (idx >= (long long)M * per_row) return;
    const int m = (int)(idx / per_row), c = (int)(idx % per_row);
    const uint4* row = reinterpret_cast<const uint4*>(GU + (size_t)m * 2 * I);
    const uint4 g4 = __ldcg(row + gate_chunk(c, per_row, blocked != 0));
    const uint4 u4 = __ldcg(row + up_chunk(c, per_row, blocked != 0));
    const __half2* g = reinterpret_cast<const __half2*>(&g4);
    const __half2* u = reinterpret_cast<const __half2*>(&u4);
    uint4 o4;
    __half2* o = reinterpret_cast<__half2*>(&o4);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(g[i]);
        const __half2 s = __floats2half2_rn(f.x / (1.f + __expf(-f.x)), f.y / (1.f + __expf(-f.y)));
        o[i] = __hmul2(s, u[i]);
    }
    reinterpret_cast<uint4*>(Y + (size_t)m * I)[c] = o4;
}

// Block-wide max of a non-negative value (256 threads), result in every thread.
__device__ __forceinline__ float block_max_256(float v, float* scratch8) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();                       // scratch may still be read from a previous reduction
    if ((threadIdx.x & 31) == 0) scratch8[threadIdx.x >> 5] = v;
    __syncthreads();
    v = scratch8[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) v = fmaxf(v, scratch8[w]);
    return v;
}

// Per-token symmetric int8 quantization of 8 fp16 values held in a uint4, with the arithmetic of
// act_quant_kernel (IEEE division, round-half-even): bit-identical to quantizing the stored fp16 tensor.
__device__ __forceinline__ uint2 quant8(const uint4& v, float scale, float inv) { return quant8_chunk(v, scale, inv); }

__device__ __forceinline__ float absmax8(const uint4& v) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
    return m;
}

// RMSNorm that hands its result to a W8A8 linear in the precision that kernel consumes: the fp16 result is
// formed in registers, quantized per token to int8 (+ fp16 scale) and written ONCE as int8; the fp16 tensor
// is written only when a consumer needs it (Y != null).  Output equals act_quant(rms_norm(X)) bit for bit.
template <int R, bool kPeer>
__global__ void __launch_bounds__(256) rms_norm_quant_kernel(__half* X, const __half* __restrict__ H, const PeerSet ps,
                                                             const __half* __restrict__ W, __half* __restrict__ Y,
                                                             int8_t* __restrict__ Xq, __half* __restrict__ sx, int K,
                                                             float eps) {
    __shared__ float part[8];
    chain_release();
    chain_wait();
    const int token = blockIdx.x;
    if constexpr (kPeer) {
        if (!peer_barrier(ps, token)) return;
    }
    const int chunks = K >> 3;
    uint4 v[R];
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int c = threadIdx.x + r * 256;
        if (c < chunks) {
            if constexpr (kPeer) v[r] = load_residual_peer(X, ps, (size_t)token * K, c);
            else v[r] = load_residual(X, H, (size_t)token * K, c);
            const __half2* h = reinterpret_cast<const __half2*>(&v[r]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(h[i]);
                ss += f.x * f.x + f.y * f.y;
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    ss = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) ss += part[w];
    const float inv = rsqrtf(ss / (float)K + eps);
    const uint4* wv = reinterpret_cast<const uint4*>(W);
    float amax = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int c = threadIdx.x + r * 256;
        if (c < chunks) {
            const uint4 wq = __ldg(wv + c);
            const __half2* h = reinterpret_cast<const __half2*>(&v[r]);
            const __half2* g = reinterpret_cast<const __half2*>(&wq);
            uint4 o4;
            __half2* o = reinterpret_cast<__half2*>(&o4);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(h[i]), gw = __half22float2(g[i]);
                o[i] = __floats2half2_rn(f.x * inv * gw.x, f.y * inv * gw.y);
            }
            v[r] = o4;                                       // the fp16 result replaces the input
            amax = fmaxf(amax, absmax8(o4));
            if (Y) reinterpret_cast<uint4*>(Y + (size_t)token * K)[c] = o4;
        }
    }
    amax = block_max_256(amax, part);
    const float scale = __fdiv_rn(fmaxf(amax, 1e-7f), 127.0f);
    if (threadIdx.x == 0) sx[token] = __float2half_rn(scale);
    const float inv_scale = __frcp_rn(scale);
    uint2* out = reinterpret_cast<uint2*>(Xq + (size_t)token * K);
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int c = threadIdx.x + r * 256;
        if (c < chunks) out[c] = quant8(v[r], scale, inv_scale);
    }
}

// SiLU(gate) * up followed by the same per-token int8 quantization, one CTA per token.
template <int R>
__global__ void __launch_bounds__(256) silu_mul_quant_kernel(const __half* __restrict__ GU, __half* __restrict__ Y,
                                                             int8_t* __restrict__ Xq, __half* __restrict__ sx, int I,
                                                             int blocked) {
    __shared__ float part[8];
    chain_release();
    chain_wait();
    const int token = blockIdx.x;
    const int chunks = I >> 3;
    const uint4* row = reinterpret_cast<const uint4*>(GU + (size_t)token * 2 * I);
    uint4 v[R];
    float amax = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int c = threadIdx.x + r * 256;
        if (c < chunks) {
            const uint4 g4 = __ldcg(row + gate_chunk(c, chunks, blocked != 0));
            const uint4 u4 = __ldcg(row + up_chunk(c, chunks, blocked != 0));
            const __half2* g = reinterpret_cast<const __half2*>(&g4);
            const __half2* u = reinterpret_cast<const __half2*>(&u4);
            uint4 o4;
            __half2* o = reinterpret_cast<__half2*>(&o4);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(g[i]);
                const __half2 sl = __floats2half2_rn(f.x / (1.f + __expf(-f.x)), f.y / (1.f + __expf(-f.y)));
                o[i] = __hmul2(sl, u[i]);
            }
            v[r] = o4;
            amax = fmaxf(amax, absmax8(o4));
            if (Y) reinterpret_cast<uint4*>(Y + (size_t)token * I)[c] = o4;
        }
    }
    amax = block_max_256(amax, part);
    const float scale = __fdiv_rn(fmaxf(amax, 1e-7f), 127.0f);
    if (threadIdx.x == 0) sx[token] = __float2half_rn(scale);
    const float inv_scale = __frcp_rn(scale);
    uint2* out = reinterpret_cast<uint2*>(Xq + (size_t)token * I);
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int c = threadIdx.x + r * 256;
        if (c < chunks) out[c] = quant8(v[r], scale, inv_scale);
    }
}

// Rotary embedding (rotate-half convention) of the q and k heads of a fused QKV activation and the
// KV-cache write, one thread per pair (d, d + D/2) of one head of one token.
//   QKV  [B*S, (H + 2 Hkv) * D]      Q_out [B, H, S, D]      cache K / V [B, Hkv, max_len, D]
// Token (b, s) sits at position pos0 + s, with pos0 = *pos_dev when pos_dev is given (decode step whose
// position lives in device memory so that a CUDA graph can be replayed) and pos0_host otherwise.
__global__ void __launch_bounds__(256) rope_kv_kernel(const __half* __restrict__ QKV, const __half* __restrict__ cosT,
                                                      const __half* __restrict__ sinT, const long long* pos_dev,
                                                      int pos0_host, __half* __restrict__ Q_out,
                                                      __half* __restrict__ Kc, __half* __restrict__ Vc, int B, int S,
                                                      int H, int Hkv, int D, int max_len) {
    chain_release();
    chain_wait();
    const int half_d = D >> 1;
    const int heads = H + 2 * Hkv;
    const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
    const long long total = (long long)B * S * heads * half_d;
    if (idx >= total) return;
    const int d = (int)(idx % half_d);
    long long r = idx / half_d;
    const int head = (int)(r % heads);
    r /= heads;
    const int s = (int)(r % S), b = (int)(r / S);
    const int pos = (pos_dev ? (int)__ldcg(pos_dev) : pos0_host) + s;
    const __half* src = QKV + ((size_t)(b * S + s) * heads + head) * D;
    const __half h1 = __ldcg(src + d), h2 = __ldcg(src + d + half_d);
    const float x1 = __half2float(h1), x2 = __half2float(h2);
    if (head < H + Hkv) {
        const float c = __half2float(cosT[(size_t)pos * half_d + d]), sn = __half2float(sinT[(size_t)pos * half_d + d]);
        const __half y1 = __float2half_rn(x1 * c - x2 * sn), y2 = __float2half_rn(x2 * c + x1 * sn);
        __half* dst = head < H ? Q_out + (((size_t)b * H + head) * S + s) * D
                               : Kc + (((size_t)b * Hkv + (head - H)) * max_len + pos) * D;
        dst[d] = y1;
        dst[d + half_d] = y2;
    } else {
        __half* dst = Vc + (((size_t)b * Hkv + (head - H - Hkv)) * max_len + pos) * D;
        dst[d] = h1;
        dst[d + half_d] = h2;
    }
}

}  // namespace kairos

namespace kairos {
static int run_rms_norm(void* X, const void* H, const void* W, void* Y, int M, int K, float eps, cudaStream_t st,
                        const PeerSet* peers = nullptr) {
    __half* x = static_cast<__half*>(X);
    const __half* h = static_cast<const __half*>(H);
    const __half* w = static_cast<const __half*>(W);
    __half* y = static_cast<__half*>(Y);
    const int per = (K / 8 + 255) / 256;
    PeerSet ps = {};
    if (peers) ps = *peers;
    cudaError_t e;
#define KAIROS_NORM(R)                                                                                             \
    (peers ? launch_chained(rms_norm_kernel<R, true>, dim3(M), dim3(256), 0, st, x, h, ps, w, y, K, eps)           \
           : launch_chained(rms_norm_kernel<R, false>, dim3(M), dim3(256), 0, st, x, h, ps, w, y, K, eps))
    if (per <= 1) e = KAIROS_NORM(1);
    else if (per <= 2) e = KAIROS_NORM(2);
    else if (per <= 4) e = KAIROS_NORM(4);
    else e = KAIROS_NORM(8);
#undef KAIROS_NORM
    if (e != cudaSuccess) return note_cuda_error(e);
    return launch_status();
}

static int run_rms_norm_quant(void* X, const void* H, const void* W, void* Y, void* Xq, void* sx, int M, int K,
                              float eps, cudaStream_t st, const PeerSet* peers = nullptr) {
    __half* x = static_cast<__half*>(X);
    const __half* h = static_cast<const __half*>(H);
    const __half* w = static_cast<const __half*>(W);
    __half* y = static_cast<__half*>(Y);
    int8_t* q = static_cast<int8_t*>(Xq);
    __half* s = static_cast<__half*>(sx);
    const int per = (K / 8 + 255) / 256;
    PeerSet ps = {};
    if (peers) ps = *peers;
    cudaError_t e;
#define KAIROS_NORMQ(R)                                                                                                  \
    (peers ? launch_chained(rms_norm_quant_kernel<R, true>, dim3(M), dim3(256), 0, st, x, h, ps, w, y, q, s, K, eps)     \
           : launch_chained(rms_norm_quant_kernel<R, false>, dim3(M), dim3(256), 0, st, x, h, ps, w, y, q, s, K, eps))
    if (per <= 1) e = KAIROS_NORMQ(1);
    else if (per <= 2) e = KAIROS_NORMQ(2);
    else if (per <= 4) e = KAIROS_NORMQ(4);
    else e = KAIROS_NORMQ(8);
#undef KAIROS_NORMQ
    if (e != cudaSuccess) return note_cuda_error(e);
    return launch_status();
}
}  // namespace kairos

extern "C" int kairos_rms_norm(const void* X, const void* W, void* Y, int M, int K, float eps, kairos_stream_t stream) {
    using namespace kairos;
    if (M < 0 || K <= 0 || (K % 8) != 0 || K > 8 * 256 * 8) return KAIROS_ERR_SHAPE;
    if (M == 0) return KAIROS_OK;
    if (!X || !W || !Y || ((uintptr_t)X & 15) || ((uintptr_t)W & 15) || ((uintptr_t)Y & 15)) return KAIROS_ERR_ALIGN;
    return run_rms_norm(const_cast<void*>(X), nullptr, W, Y, M, K, eps, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int kairos_add_rms_norm(void* X, const void* H, const void* W, void* Y, int M, int K, float eps,
                                   kairos_stream_t stream) {
    using namespace kairos;
    if (M < 0 || K <= 0 || (K % 8) != 0 || K > 8 * 256 * 8) return KAIROS_ERR_SHAPE;
    if (M == 0) return KAIROS_OK;
    if (!X || !H || !W || !Y || ((uintptr_t)X & 15) || ((uintptr_t)H & 15) || ((uintptr_t)W & 15) ||
        ((uintptr_t)Y & 15))
        return KAIROS_ERR_ALIGN;
    return run_rms_norm(X, H, W, Y, M, K, eps, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int kairos_add_rms_norm_peer(void* X, const void* const* peer_in, void* const* peer_signal, int world, int rank,
                                        const void* W, void* Y, int M, int K, float eps, kairos_stream_t stream) {
    using namespace kairos;
    if (M < 0 || M > kArBlocks || K <= 0 || (K % 8) != 0 || K > 8 * 256 * 8) return KAIROS_ERR_SHAPE;
    if (!X || !W || !Y || ((uintptr_t)X & 15) || ((uintptr_t)W & 15) || ((uintptr_t)Y & 15)) return KAIROS_ERR_ALIGN;
    PeerSet ps;
    const int rc = make_peer_set(&ps, peer_in, peer_signal, world, rank);
    if (rc != KAIROS_OK) return rc;
    if (M == 0) return KAIROS_OK;
    return run_rms_norm(X, nullptr, W, Y, M, K, eps, reinterpret_cast<cudaStream_t>(stream), &ps);
}

extern "C" int kairos_rms_norm_quant_peer(void* X, const void* const* peer_in, void* const* peer_signal, int world,
                                          int rank, const void* W, void* Y_or_null, void* Xq, void* sx, int M, int K,
                                          float eps, kairos_stream_t stream) {
    using namespace kairos;
    if (M < 0 || M > kArBlocks || K <= 0 || (K % 16) != 0 || K > 8 * 256 * 8) return KAIROS_ERR_SHAPE;
    if (!X || !W || !Xq || !sx || ((uintptr_t)X & 15) || ((uintptr_t)W & 15) || ((uintptr_t)Xq & 15) ||
        ((uintptr_t)Y_or_null & 15))
        return KAIROS_ERR_ALIGN;
    PeerSet ps;
    const int rc = make_peer_set(&ps, peer_in, peer_signal, world, rank);
    if (rc != KAIROS_OK) return rc;
    if (M == 0) return KAIROS_OK;
    return run_rms_norm_quant(X, nullptr, W, Y_or_null, Xq, sx, M, K, eps, reinterpret_cast<cudaStream_t>(stream), &ps);
}

static int run_silu_mul(const void* GU, void* Y, int M, int I, int blocked, kairos_stream_t stream) {
    using namespace kairos;
    if (M < 0 || I <= 0 || (I % 8) != 0 || (blocked && (I % 16) != 0)) return KAIROS_ERR_SHAPE;
    if (M == 0) return KAIROS_OK;
    if (!GU || !Y || ((uintptr_t)GU & 15) || ((uintptr_t)Y & 15)) return KAIROS_ERR_ALIGN;
    const long long chunks = (long long)M * (I / 8);
    const cudaError_t e = launch_chained(silu_mul_kernel, dim3((unsigned)((chunks + 255) / 256)), dim3(256), 0,
                                         reinterpret_cast<cudaStream_t>(stream), static_cast<const __half*>(GU),
                                         static_cast<__half*>(Y), M, I, blocked);
    if (e != cudaSuccess) return note_cuda_error(e);
    return launch_status();
}

extern "C" int kairos_silu_mul(const void* GU, void* Y, int M, int I, kairos_stream_t stream) {
    return run_silu_mul(GU, Y, M, I, 0, stream);
}
extern "C" int kairos_silu_mul_blocked(const void* GU, void* Y, int M, int I, kairos_stream_t stream) {
    return run_silu_mul(GU, Y, M, I, 1, stream);
}

extern "C" int kairos_rope_kv(const void* QKV, const void* cos_table, const void* sin_table, const void* pos_dev_or_null,
                              int pos0, void* Q_out, void* K_cache, void* V_cache, int B, int S, int H, int Hkv, int D,
                              int max_len, kairos_stream_t stream) {
    using namespace kairos;
    if (B <= 0 || S <= 0 || H <= 0 || Hkv <= 0 || D <= 0 || (D & 1) || max_len <= 0) return KAIROS_ERR_SHAPE;
    if (!pos_dev_or_null && (pos0 < 0 || pos0 + S > max_len)) return KAIROS_ERR_SHAPE;
    if (!QKV || !cos_table || !sin_table || !Q_out || !K_cache || !V_cache) return KAIROS_ERR_ALIGN;
    const long long total = (long long)B * S * (H + 2 * Hkv) * (D / 2);
    const cudaError_t e = launch_chained(
        rope_kv_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
        static_cast<const __half*>(QKV), static_cast<const __half*>(cos_table), static_cast<const __half*>(sin_table),
        static_cast<const long long*>(pos_dev_or_null), pos0, static_cast<__half*>(Q_out),
        static_cast<__half*>(K_cache), static_cast<__half*>(V_cache), B, S, H, Hkv, D, max_len);
    if (e != cudaSuccess) return note_cuda_error(e);
    return launch_status();
}

extern "C" int kairos_rms_norm_quant(void* X, const void* H_or_null, const void* W, void* Y_or_null, void* Xq, void* sx,
                                     int M, int K, float eps, kairos_stream_t stream) {
    using namespace kairos;
    if (M < 0 || K <= 0 || (K % 16) != 0 || K > 8 * 256 * 8) return KAIROS_ERR_SHAPE;
    if (M == 0) return KAIROS_OK;
    if (!X || !W || !Xq || !sx || ((uintptr_t)X & 15) || ((uintptr_t)W & 15) || ((uintptr_t)Xq & 15) ||
        ((uintptr_t)Y_or_null & 15) || ((uintptr_t)H_or_null & 15))
        return KAIROS_ERR_ALIGN;
    return run_rms_norm_quant(X, H_or_null, W, Y_or_null, Xq, sx, M, K, eps, reinterpret_cast<cudaStream_t>(stream));
}

static int run_silu_mul_quant(const void* GU, void* Y_or_null, void* Xq, void* sx, int M, int I, int blocked,
                              kairos_stream_t stream);

extern "C" int kairos_silu_mul_quant(const void* GU, void* Y_or_null, void* Xq, void* sx, int M, int I,
                                     kairos_stream_t stream) {
    return run_silu_mul_quant(GU, Y_or_null, Xq, sx, M, I, 0, stream);
}
extern "C" int kairos_silu_mul_quant_blocked(const void* GU, void* Y_or_null, void* Xq, void* sx, int M, int I,
                                             kairos_stream_t stream) {
    return run_silu_mul_quant(GU, Y_or_null, Xq, sx, M, I, 1, stream);
}

static int run_silu_mul_quant(const void* GU, void* Y_or_null, void* Xq, void* sx, int M, int I, int blocked,
                              kairos_stream_t stream) {
    using namespace kairos;
    if (M < 0 || I <= 0 || (I % 16) != 0 || I > 8 * 256 * 16) return KAIROS_ERR_SHAPE;
    if (M == 0) return KAIROS_OK;
    if (!GU || !Xq || !sx || ((uintptr_t)GU & 15) || ((uintptr_t)Xq & 15) || ((uintptr_t)Y_or_null & 15))
        return KAIROS_ERR_ALIGN;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const __half* gu = static_cast<const __half*>(GU);
    __half* y = static_cast<__half*>(Y_or_null);
    int8_t* q = static_cast<int8_t*>(Xq);
    __half* s = static_cast<__half*>(sx);
    const int per = (I / 8 + 255) / 256;
    cudaError_t e;
    if (per <= 4) e = launch_chained(silu_mul_quant_kernel<4>, dim3(M), dim3(256), 0, st, gu, y, q, s, I, blocked);
    else if (per <= 8) e = launch_chained(silu_mul_quant_kernel<8>, dim3(M), dim3(256), 0, st, gu, y, q, s, I, blocked);
    else e = launch_chained(silu_mul_quant_kernel<16>, dim3(M), dim3(256), 0, st, gu, y, q, s, I, blocked);
    if (e != cudaSuccess) return note_cuda_error(e);
    return launch_status();
}
