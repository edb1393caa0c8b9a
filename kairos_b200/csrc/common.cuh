// Shared device helpers for the sm_100a kernels: status codes, bounded mbarrier
// waits, TMA / tcgen05 PTX wrappers and the uint4 -> fp16 unpack.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/kairos_b200.h"

namespace kairos {

// ---- base-format constants (one resident weight: packed uint4, group 128) ----
constexpr int kGroup = 128;       // K elements sharing one (scale, scaled_zero)
constexpr int kInterleave = 4;    // weight rows interleaved into one int16 row
constexpr int kKStride = 64;      // k extent of one interleave block

inline int padded_groups(int K) { return ((K / kGroup + 7) / 8) * 8; }

#define KAIROS_CUDA_OK(expr)                                   \
    do {                                                       \
        cudaError_t _e = (expr);                               \
        if (_e != cudaSuccess) return kairos::note_cuda_error(_e); \
    } while (0)

int note_cuda_error(cudaError_t e);   // records the message, returns KAIROS_ERR_CUDA
int launch_status();                  // cudaGetLastError() -> status
void set_last_error(const char* msg); // detail text returned by kairos_last_error()
bool chained_launch_enabled();        // false when the environment sets KAIROS_NO_PDL=1
int arithmetic_rule();                // KAIROS_ARITH_TORCH or KAIROS_ARITH_REFERENCE_CUDA (kairos_set_arithmetic)

// Function attributes belong to a device's context, so "already set" is tracked per device: a process that
// drives several GPUs raises the dynamic shared-memory limit of a kernel once on each of them.
struct PerDeviceFlag {
    std::atomic<unsigned char> set[64];
};
template <typename Kernel>
inline int ensure_dynamic_smem(PerDeviceFlag& flag, Kernel kernel, int bytes) {
    int dev = 0;
    const cudaError_t e0 = cudaGetDevice(&dev);
    if (e0 != cudaSuccess) return note_cuda_error(e0);
    if (dev < 0 || dev >= 64) return KAIROS_ERR_ARG;
    if (!flag.set[dev].load(std::memory_order_acquire)) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return note_cuda_error(e);
        flag.set[dev].store(1, std::memory_order_release);
    }
    return KAIROS_OK;
}

// ---------------------------------------------------------------------------
// Programmatic dependent launch.  A kernel launched through launch_chained may become resident while the
// kernel before it in the stream is still running; it must execute chain_wait() before it touches
// anything an earlier kernel wrote (or writes anything an earlier kernel reads).  What it does before
// that -- barrier set-up, descriptor prefetch, streaming of CONSTANT inputs such as the packed weights --
// overlaps the tail of its predecessor.  chain_release() lets the kernel after it start the same way.
// Both instructions are no-ops in a kernel launched the ordinary way.
// ---------------------------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                  Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = chained_launch_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// ---------------------------------------------------------------------------
// rint(x / scale) with the result of IEEE division, without dividing in the common case.  x * (1/scale)
// differs from the correctly rounded quotient by at most 3 * 2^-24 * |q| <= 2.3e-5 for |q| <= 127, so
// both round to the same integer unless the product lies within 1e-4 of a rounding boundary (k + 0.5);
// only then is the quotient formed by IEEE division (a dozen instructions) and rounded half-to-even.
// Non-finite inputs take the division path as well.  `inv` = __frcp_rn(scale), once per token.
// ---------------------------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ int rint_div(float x, float scale, float inv) {
    const float r = __fmul_rn(x, inv);
    const float t = rintf(r);
    if (!(fabsf(r - t) <= 0.4999f)) return __float2int_rn(__fdiv_rn(x, scale));
    return (int)t;
}

// Eight fp16 values -> eight int8 (two words), q = rint(x / scale) as above.  The product is rounded to an
// integer by adding 1.5 * 2^23 (round-to-nearest-even of the fp32 adder); the low byte of the sum's bit
// pattern is then q in two's complement (|q| <= 127), so no float-to-int conversion or masking is needed,
// and one test per chunk sends a chunk with any quotient next to a rounding boundary (or a non-finite
// value) to the exact divisions.
__device__ __forceinline__ uint2 quant8_chunk(const uint4& v, float scale, float inv) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
    const float magic = 12582912.f;
    float x[8];
    uint32_t u[8];
    bool exact = false;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        x[2 * i] = f.x;
        x[2 * i + 1] = f.y;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float r = __fmul_rn(x[i], inv);
        const float s = __fadd_rn(r, magic);
        const float t = __fadd_rn(s, -magic);
        exact |= !(fabsf(__fadd_rn(r, -t)) <= 0.4999f);
        u[i] = __float_as_uint(s);
    }
    if (exact) {
#pragma unroll
        for (int i = 0; i < 8; ++i) u[i] = (uint32_t)__float2int_rn(__fdiv_rn(x[i], scale));
    }
    uint2 out;
    out.x = __byte_perm(__byte_perm(u[0], u[1], 0x0040), __byte_perm(u[2], u[3], 0x0040), 0x5410);
    out.y = __byte_perm(__byte_perm(u[4], u[5], 0x0040), __byte_perm(u[6], u[7], 0x0040), 0x5410);
    return out;
}
#endif

// ---------------------------------------------------------------------------
// uint4 unpack.  A 32-bit word of the base holds, for fixed (row, a, c), the
// eight values k = 32a + 8b + 2c + d (b = nibble index within each 16-bit half,
// d = which half).  unpack8 returns four half2, h[b] = (q[b,d=0], q[b,d=1]),
// i.e. two CONSECUTIVE k for each b.  All results are exact integers 0..15.
// The magic-number idiom (or the nibble into the mantissa of 1024, then subtract, or scale by 1/16 and
// subtract 64) is the one the wire format was designed for; the reference's form of it is
// dequantize_s4_to_fp16x2, thirdparty/AWQ/kernels/csrc/quantization_new/dequantize.cuh:18-80.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void unpack8(uint32_t w, __half2 (&h)[4]) {
    // (w & 0x000f000f) | 0x64006400  ==  half2(1024 + q_lo, 1024 + q_hi)
    uint32_t t0, t1, t2, t3;
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(t0) : "r"(w));
    asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xea;" : "=r"(t1) : "r"(w));
    const uint32_t w8 = w >> 8;
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(t2) : "r"(w8));
    asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xea;" : "=r"(t3) : "r"(w8));
    const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));   // 1024
    const __half2 k64 = __half2half2(__ushort_as_half(0x5400));     // 64
    const __half2 k16th = __half2half2(__ushort_as_half(0x2c00));   // 1/16
    h[0] = __hsub2(*reinterpret_cast<__half2*>(&t0), k1024);
    // (1024 + 16 q) / 16 - 64 = q, exact in one fma
    h[1] = __hfma2(*reinterpret_cast<__half2*>(&t1), k16th, __hneg2(k64));
    h[2] = __hsub2(*reinterpret_cast<__half2*>(&t2), k1024);
    h[3] = __hfma2(*reinterpret_cast<__half2*>(&t3), k16th, __hneg2(k64));
}

// fp16(fp16(q*s) + z): two roundings, matching torch's mul_ then add_ on fp16.
__device__ __forceinline__ __half2 scale_then_shift(__half2 q, __half2 s, __half2 z) {
    // the _rn forms forbid contraction of the pair into one fma
    return __hadd2_rn(__hmul2_rn(q, s), z);
}

// 16-byte chunk (four words c = 0..3) -> 32 consecutive-k fp16 values
// out[kk/2] for kk = 8b + 2c (+d), already scaled.  `out` is 16 half2 in k order.
__device__ __forceinline__ void dequant_chunk32(const uint4& raw, __half2 s, __half2 z, __half2 (&out)[16]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        __half2 h[4];
        unpack8(w[c], h);
#pragma unroll
        for (int b = 0; b < 4; ++b) out[4 * b + c] = scale_then_shift(h[b], s, z);
    }
}

// Same expansion with q*s+z as ONE fused multiply-add (one rounding).  Used where the fp16
// weight only feeds a tolerance-checked GEMM and instruction count matters.
__device__ __forceinline__ void dequant_chunk32_fma(const uint4& raw, __half2 s, __half2 z, __half2 (&out)[16]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        __half2 h[4];
        unpack8(w[c], h);
#pragma unroll
        for (int b = 0; b < 4; ++b) out[4 * b + c] = __hfma2(h[b], s, z);
    }
}

// ---------------------------------------------------------------------------
// shared-memory / mbarrier / TMA / tcgen05 wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Same test, but the hardware may park the thread for up to `ns` nanoseconds (it is woken when the phase
// completes): a waiting warp then does not burn issue slots that working warps need.
__device__ __forceinline__ bool mbar_try_wait_parked(uint64_t* bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false when the limit ran out or another role of this CTA
// already gave up (`*abort_flag` != 0); the caller then leaves its loop and goes to
// the common teardown.  The limit is ~2 s of polling; a healthy pipeline waits
// microseconds.
constexpr long long kWaitCycles = 4000000000LL;
__device__ __forceinline__ bool mbar_wait_limit(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                long long limit_cycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 16; ++i)
            if (mbar_try_wait_parked(bar, parity, 20000u)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > limit_cycles) {
            *abort_flag = 1;
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    return mbar_wait_limit(bar, parity, abort_flag, kWaitCycles);
}

// One lane of the (converged) warp is elected; the others get false.  Unlike a test of the lane index, the
// election tells the compiler that the guarded region runs in exactly one thread of a converged warp, so
// operands of the tensor-core and bulk-copy instructions inside it can stay in the warp-wide (uniform)
// registers those instructions read, instead of being moved there before every instruction.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// 2-D tiled TMA load, completion signalled on an mbarrier of this CTA.  No multicast.
__device__ __forceinline__ void tma_load_2d(void* dst, const void* tmap, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            smem_u32(dst)),
        "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const void* tmap, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
            smem_u32(dst)),
        "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
                 "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// All tcgen05.mma issued so far by this thread arrive (once) on `bar` when they retire.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
template <bool kInt8>
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                     uint32_t accumulate) {
    if constexpr (kInt8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}
// 32 lanes x 16 consecutive 32-bit columns of TMEM -> 16 registers per thread.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns of TMEM -> 32 registers per thread.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
// 32 lanes x 64 consecutive 32-bit columns of TMEM -> 64 registers per thread (one instruction: the
// tensor pipe is interrupted once per 8 KB instead of once per 2 KB).
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t (&r)[64]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// K-major, 128-byte-swizzled operand tile whose rows are 128 bytes and whose 8-row
// groups are 1024 bytes apart: 64-bit shared-memory matrix descriptor.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFF)      // start address / 16
           | (1ull << 16)                              // leading byte offset (unused with swizzle)
           | (64ull << 32)                             // stride byte offset 1024 / 16
           | (1ull << 46)                              // descriptor version (Blackwell)
           | (2ull << 61);                             // layout: SWIZZLE_128B
}

}  // namespace kairos
