// Prefill-side tensor-core GEMMs (path items a10, a11, a12 and kernel id 3):
// one persistent, warp-specialised tcgen05 kernel template.
//
//   D[n, m] (TMEM, 128 lanes x BT columns) += W_tile[128 n, BK] . X_tile[BT m, BK]^T
//
// The WEIGHT rows ride on the UMMA M dimension (always 128) and the TOKENS on the UMMA N
// dimension (BT = 16..256), so a small batch wastes no tensor-core rows and a CTA at
// BT = 256 amortises every expanded weight element over 256 tokens.
//
//   kind::i8  (W8A8):  Xq, W8 int8 via TMA, int32 accumulators, scale epilogue
//   kind::f16 (FP16):  X, W16 fp16 via TMA, fp32 accumulators
//   kind::f16 (W4A16): X via TMA; the packed uint4 tile (4 KB per 128x64 weights) via
//                      TMA, expanded by 8 producer warps into the 128B-swizzled K-major
//                      fp16 operand tile in shared memory
//   kind::f16 (W8A16): same, int8 tile widened to fp16 and multiplied by s1[n]
//
// Warp roles: 0 = TMA producer, 1 = MMA issuer (+TMEM owner), 2..5 = epilogue
// (TMEM -> registers -> global), 6..13 = weight expanders (dequant modes only).
// The accumulator is double-buffered in TMEM so the epilogue of one tile overlaps the
// main loop of the next.  Small problems are split along K: each split writes its
// partial tile to scratch and a second, grid-wide kernel sums the partials in split
// order (deterministic; exact for int32) and runs the epilogue.
//
// Every mbarrier wait is bounded; on a timeout the CTA raises a status word and drains.
#include <cuda.h>

#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace kairos {

enum : int { kModeTma = 0, kModeW4 = 1, kModeW8 = 2 };

constexpr int kTileN = 128;           // weight rows per tile (UMMA M)
constexpr int kRowBytes = 128;        // K extent of one pipeline stage, in bytes of the MMA operand
constexpr int kATileBytes = kTileN * kRowBytes;
constexpr int kNumExpandWarps = 16;
constexpr int kExpandGroups = 4;                                   // k blocks expanded concurrently
constexpr int kExpandGroupWarps = kNumExpandWarps / kExpandGroups;
constexpr int kSmemBudget = 224 * 1024;      // of the 227 KB a CTA may use; barriers and alignment slack come on top

struct GemmParams {
    int M, N, K;
    int n_tiles, m_tiles, splits, kb_per_split, kb_total;
    const __half* scales;        // W4 mode: [G_pad, N]
    const __half* scaled_zeros;  // W4 mode: [G_pad, N]
    const __half* s1;            // [N]: W8 mode operand scale / int8 epilogue scale
    const __half* sx;            // [M]: int8 epilogue scale
    const __half* bias;          // [N] or null
    __half* Y;                   // [M, N]
    int32_t* acc_dbg;            // [M, N] or null (int8 only)
    uint32_t* partials;          // split-K partial tiles [tile][split][BT][128]
    int* status;                 // raised on a bounded wait that ran out
    long long* trace;            // diagnostic: per-k-block clock64 stamps of CTA 0 (null = off)
};

// Pipeline trace (build with -DKAIROS_TRACE): CTA 0 stamps clock64() per k block and role into p.trace.
// Compiled out of the shipped library.
#ifdef KAIROS_TRACE
constexpr int kTraceSlots = 8;     // stamps per k block: see trace_stamp() call sites
constexpr int kTraceBlocks = 64;   // k blocks recorded
__device__ __forceinline__ void trace_stamp(const GemmParams& p, uint32_t i, int slot) {
    if (p.trace && blockIdx.x == 0 && i < kTraceBlocks && (threadIdx.x & 31) == 0) p.trace[i * kTraceSlots + slot] = clock64();
}
#else
__device__ __forceinline__ void trace_stamp(const GemmParams&, uint32_t, int) {}
#endif

template <bool kInt8, int kMode, int BT>
struct GemmCfg {
    // k blocks (128 bytes of K per operand row) moved per pipeline stage.  Issuing a TMA copy costs
    // the issuing thread a few hundred cycles whatever its size, so small token tiles bundle four
    // k blocks into every copy.
    static constexpr int kSub = BT <= 64 ? 4 : (BT == 128 ? 2 : 1);
    static constexpr int kBlockK = kInt8 ? 128 : 64;                  // elements of K per k block
    static constexpr int kXTileBytes = BT * kRowBytes;                // per k block
    static constexpr int kXStageBytes = kSub * kXTileBytes;
    // weight side of a stage
    static constexpr int kFactorGroups = kSub >= 2 ? kSub / 2 : 1;   // W4: quantization groups per stage
    static constexpr int kPackedBytes = kSub * 32 * 128;              // W4: [32 rows][kSub x 128 B]
    static constexpr int kWStageBytes = kMode == kModeW4 ? kPackedBytes + 1024
                                       : kMode == kModeW8 ? kSub * kTileN * 64
                                                          : kSub * kATileBytes;
    static constexpr int kWTxBytes = kMode == kModeW4 ? kPackedBytes + 2 * kFactorGroups * 256 : kWStageBytes;
    static constexpr int kStageBytes = kWStageBytes + kXStageBytes;
    // one expanded-operand slot per expander group: a slot is always refilled by the same group, in order
    static constexpr int kAStages = kMode == kModeTma ? 0 : kExpandGroups;
    static constexpr int kStagesFit = (kSmemBudget - kAStages * kATileBytes) / kStageBytes;
    static constexpr int kStages = kStagesFit > 8 ? 8 : kStagesFit;
    static constexpr int kWarps = (kMode == kModeTma ? 6 : 6 + kNumExpandWarps) + 1;   // + activation producer
    static constexpr int kThreads = 32 * kWarps;
    static constexpr int kTmemCols = 2 * BT < 32 ? 32 : 2 * BT;
    static constexpr int kBarBytes = 8 * (2 * kStages + 2 * (kAStages ? kAStages : 1) + 4) + 64;
    static constexpr int kSmemBytes = kStages * kStageBytes + kAStages * kATileBytes + kBarBytes + 1024;
    static_assert(kStages >= 2, "pipeline too shallow");
    static_assert(kSmemBytes <= 227 * 1024, "exceeds the shared memory a CTA may use");
    static_assert(kWStageBytes % 1024 == 0 && kXTileBytes % 1024 == 0, "operand tiles must stay 1024-byte aligned");
    static_assert(kExpandGroups % kSub == 0, "a stage must hold whole expander rounds");
    // instruction descriptor: D format (bits 4-5), A/B formats (7-9, 10-12), K-major both,
    // N >> 3 at bit 17, M >> 4 at bit 24
    static constexpr uint32_t kIdesc = (kInt8 ? (2u << 4) | (1u << 7) | (1u << 10) : (1u << 4)) |
                                       ((uint32_t)(BT >> 3) << 17) | ((uint32_t)(kTileN >> 4) << 24);
};

// int8 x 4 (one 32-bit word, k order) -> two half2 (exact), times s
__device__ __forceinline__ void widen_s8x4(uint32_t w, __half2 s, __half2& lo, __half2& hi) {
    const uint32_t u = w ^ 0x80808080u;                         // x + 128 as unsigned bytes
    uint32_t p0, p1;
    asm("prmt.b32 %0, %1, %2, 0x5140;" : "=r"(p0) : "r"(u), "r"(0x64646464u));   // (1024 + u0, 1024 + u1)
    asm("prmt.b32 %0, %1, %2, 0x5342;" : "=r"(p1) : "r"(u), "r"(0x64646464u));   // (1024 + u2, 1024 + u3)
    const __half2 k1152 = __half2half2(__ushort_as_half(0x6480));                 // 1152
    lo = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&p0), k1152), s);
    hi = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&p1), k1152), s);
}

// One output element: scale (int8), round to fp16, add bias, store.
//   int8: half(float(acc) * (float(s1[n]) * float(sx[m])))
//         (thirdparty/AWQ/kernels/csrc/w8a8/w8a8_gemm_cuda.cu:896-901)
template <bool kInt8>
__device__ __forceinline__ void store_output(const GemmParams& p, uint32_t v, int m, int n, float s1f, float sxf,
                                             bool has_bias, __half bias_n) {
    __half y;
    if constexpr (kInt8) {
        const float sc = __fmul_rn(s1f, sxf);
        y = __float2half_rn(__fmul_rn((float)(int32_t)v, sc));
        if (p.acc_dbg) p.acc_dbg[(size_t)m * p.N + n] = (int32_t)v;
    } else {
        y = __float2half_rn(__uint_as_float(v));
    }
    if (has_bias) y = __hadd(y, bias_n);
    p.Y[(size_t)m * p.N + n] = y;
}

// Split-K second pass: sums the partial tiles of every output tile in split order and runs the
// epilogue.  One CTA per (tile, token column), one thread per weight row: every load is a coalesced
// 512-byte row of a partial tile, and the loads of a thread (one per split) are independent.
template <bool kInt8>
__global__ void __launch_bounds__(kTileN) splitk_reduce_kernel(const GemmParams p, int bt) {
    chain_release();
    chain_wait();
    const int tile = blockIdx.x / bt, c = blockIdx.x % bt;
    const int m_tile = tile % p.m_tiles, n_tile = tile / p.m_tiles;
    const int n = n_tile * kTileN + threadIdx.x;
    const int m = m_tile * bt + c;
    if (n >= p.N || m >= p.M) return;
    const uint32_t* base = p.partials + ((size_t)tile * p.splits * bt + c) * kTileN + threadIdx.x;
    uint32_t acc = kInt8 ? 0u : __float_as_uint(0.f);
    int sp = 0;
    for (; sp + 4 <= p.splits; sp += 4) {
        uint32_t v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = __ldcg(base + (size_t)(sp + u) * bt * kTileN);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if constexpr (kInt8) acc = (uint32_t)((int32_t)acc + (int32_t)v[u]);
            else acc = __float_as_uint(__fadd_rn(__uint_as_float(acc), __uint_as_float(v[u])));
        }
    }
    for (; sp < p.splits; ++sp) {
        const uint32_t v = __ldcg(base + (size_t)sp * bt * kTileN);
        if constexpr (kInt8) acc = (uint32_t)((int32_t)acc + (int32_t)v);
        else acc = __float_as_uint(__fadd_rn(__uint_as_float(acc), __uint_as_float(v)));
    }
    float s1f = 0.f;
    if constexpr (kInt8) s1f = __half2float(__ldg(p.s1 + n));
    const bool has_bias = p.bias != nullptr;
    const __half bias_n = has_bias ? __ldg(p.bias + n) : __float2half_rn(0.f);
    float sxf = 0.f;
    if constexpr (kInt8) sxf = __half2float(__ldcg(p.sx + m));
    store_output<kInt8>(p, acc, m, n, s1f, sxf, has_bias, bias_n);
}

// The k-block range of a work unit.  Ranges start and end on multiples of the stage bundle; k blocks
// past the end of K are zero-filled by TMA and contribute nothing.
struct UnitRange {
    int tile, m_tile, n_tile, kb0, kb1;
};
__device__ __forceinline__ UnitRange unit_range(const GemmParams& p, int unit) {
    UnitRange u;
    const int split = unit % p.splits;
    u.tile = unit / p.splits;
    u.m_tile = u.tile % p.m_tiles;
    u.n_tile = u.tile / p.m_tiles;
    // the stage bundles of K are dealt out as evenly as whole bundles allow (split i: bundles
    // [i S / s, (i + 1) S / s) of S); kb_per_split holds the bundle size
    const int bundles = p.kb_total / p.kb_per_split;
    u.kb0 = (int)((long long)split * bundles / p.splits) * p.kb_per_split;
    u.kb1 = (int)((long long)(split + 1) * bundles / p.splits) * p.kb_per_split;
    return u;
}

template <bool kInt8, int kMode, int BT>
__global__ void __launch_bounds__(GemmCfg<kInt8, kMode, BT>::kThreads, 1)
    umma_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                     const __grid_constant__ CUtensorMap tmap_s, const __grid_constant__ CUtensorMap tmap_z,
                     const GemmParams p) {
    using Cfg = GemmCfg<kInt8, kMode, BT>;
    constexpr int kStages = Cfg::kStages;
    constexpr int kAStages = Cfg::kAStages;
    constexpr int kSub = Cfg::kSub;
    constexpr bool kExpand = kMode != kModeTma;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* stage_base = smem;
    uint8_t* a_ring = smem + kStages * Cfg::kStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(a_ring + kAStages * kATileBytes);
    uint64_t* full = bars;
    uint64_t* empty = full + kStages;
    uint64_t* a_full = empty + kStages;
    uint64_t* a_empty = a_full + (kAStages ? kAStages : 1);
    uint64_t* tmem_full = a_empty + (kAStages ? kAStages : 1);
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 2);                                   // weight producer + activation producer
            mbar_init(&empty[s], kExpand ? 1 + kSub * kExpandGroupWarps : 1);
        }
        for (int s = 0; s < kAStages; ++s) {
            mbar_init(&a_full[s], kExpandGroupWarps);
            mbar_init(&a_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], 4);
        }
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmap_w);
        tma_prefetch_desc(&tmap_x);
        if constexpr (kMode == kModeW4) {
            tma_prefetch_desc(&tmap_s);
            tma_prefetch_desc(&tmap_z);
        }
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // set-up above may overlap the kernel before this one; its results (activations, converted weights,
    // the shared split-K workspace) are touched only after this point
    chain_release();
    chain_wait();

    const int total_units = p.n_tiles * p.m_tiles * p.splits;

    if (warp == 0) {
        // ------------------------------ weight-side TMA producer -------------------
        // (the whole warp walks the loop, one elected lane issues: see elect_one)
        {
            int s = 0;
            uint32_t phase = 0, ti = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
                const UnitRange u = unit_range(p, unit);
                for (int kb = u.kb0; kb < u.kb1; kb += kSub, ti += kSub) {
                    if (!mbar_wait(&empty[s], phase ^ 1, abort_flag)) { ok = false; break; }
                    uint8_t* st = stage_base + s * Cfg::kStageBytes;
                    if (elect_one()) {
                    mbar_arrive_expect_tx(&full[s], Cfg::kWTxBytes);
                    if constexpr (kMode == kModeW4) {
                        // qweight [N/4, K] int16: 32 rows x (kSub x 64) columns
                        tma_load_2d(st, &tmap_w, &full[s], kb * 64, u.n_tile * (kTileN / kInterleave));
                        // factors [G, N] fp16: this tile's 128 rows, the stage's groups
                        tma_load_2d(st + Cfg::kPackedBytes, &tmap_s, &full[s], u.n_tile * kTileN, kb >> 1);
                        tma_load_2d(st + Cfg::kPackedBytes + Cfg::kFactorGroups * 256, &tmap_z, &full[s],
                                    u.n_tile * kTileN, kb >> 1);
                    } else if constexpr (kMode == kModeW8) {
                        // W8 [N, K] int8: 128 rows x (kSub x 64) bytes
                        tma_load_2d(st, &tmap_w, &full[s], kb * 64, u.n_tile * kTileN);
                    } else {
                        // operand tiles [k block][128 rows][128 B], swizzled
                        tma_load_3d(st, &tmap_w, &full[s], 0, u.n_tile * kTileN, kb);
                    }
                    }
                    __syncwarp();
                    trace_stamp(p, ti, 0);
                    if (++s == kStages) { s = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == Cfg::kWarps - 1) {
        // ------------------------------ activation TMA producer --------------------
        {
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
                const UnitRange u = unit_range(p, unit);
                for (int kb = u.kb0; kb < u.kb1; kb += kSub) {
                    if (!mbar_wait(&empty[s], phase ^ 1, abort_flag)) { ok = false; break; }
                    uint8_t* st = stage_base + s * Cfg::kStageBytes + Cfg::kWStageBytes;
                    if (elect_one()) {
                        mbar_arrive_expect_tx(&full[s], Cfg::kXStageBytes);
                        tma_load_3d(st, &tmap_x, &full[s], 0, u.m_tile * BT, kb);   // [k block][BT rows][128 B]
                    }
                    __syncwarp();
                    if (++s == kStages) { s = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        // (the whole warp walks the loop, one elected lane issues)
        {
            int s = 0, as = 0, it = 0;
            uint32_t phase = 0, aphase = 0, ti = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x, ++it) {
                const UnitRange u = unit_range(p, unit);
                const int b = it & 1;
                if (!mbar_wait(&tmem_empty[b], ((it >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(b * BT);
                for (int kb = u.kb0; kb < u.kb1 && ok; kb += kSub) {
                    if (!mbar_wait(&full[s], phase, abort_flag)) { ok = false; break; }
                    trace_stamp(p, ti, 1);
                    uint8_t* st = stage_base + s * Cfg::kStageBytes;
#pragma unroll
                    for (int sub = 0; sub < kSub; ++sub, ++ti) {
                        if constexpr (kExpand)
                            if (!mbar_wait(&a_full[as], aphase, abort_flag)) { ok = false; break; }
                        trace_stamp(p, ti, 2);
                        tc_fence_after();
                        const uint32_t a_addr =
                            kExpand ? smem_u32(a_ring + as * kATileBytes) : smem_u32(st + sub * kATileBytes);
                        const uint64_t adesc = umma_desc_sw128(a_addr);
                        const uint64_t bdesc =
                            umma_desc_sw128(smem_u32(st + Cfg::kWStageBytes + sub * Cfg::kXTileBytes));
                        if (elect_one()) {
#pragma unroll
                            for (int j = 0; j < 4; ++j)   // 4 x (K = 32 bytes) per 128-byte row; +2 = 32 bytes >> 4
                                umma<kInt8>(d_tmem, adesc + 2 * j, bdesc + 2 * j, Cfg::kIdesc,
                                            (kb + sub > u.kb0 || j > 0) ? 1u : 0u);
                            if constexpr (kExpand) umma_commit(&a_empty[as]);
                        }
                        __syncwarp();
                        if constexpr (kExpand) {
                            if (++as == kAStages) { as = 0; aphase ^= 1; }
                        }
                        trace_stamp(p, ti, 3);
                    }
                    if (ok && elect_one()) umma_commit(&empty[s]);
                    __syncwarp();
                    if (++s == kStages) { s = 0; phase ^= 1; }
                }
                if (ok && elect_one()) umma_commit(&tmem_full[b]);
                __syncwarp();
            }
        }
    } else if (warp < 6) {
        // ------------------------------ epilogue ----------------------------------
        const int q = warp & 3;                    // TMEM lane quarter this warp may read
        const int row = q * 32 + lane;
        int it = 0;
        bool ok = true;
        for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x, ++it) {
            const UnitRange u = unit_range(p, unit);
            const int n = u.n_tile * kTileN + row;
            const bool n_ok = n < p.N;
            const int b = it & 1;
            float s1f = 0.f;
            if constexpr (kInt8) s1f = n_ok ? __half2float(__ldg(p.s1 + n)) : 0.f;
            const bool has_bias = p.bias != nullptr;
            const __half bias_n = (has_bias && n_ok) ? __ldg(p.bias + n) : __float2half_rn(0.f);

            // Token columns are read from TMEM in chunks of kChunk (large loads: the number of loads, not their
            // size, sets the time of the epilogue) and the activation scales of a chunk, one or two per lane,
            // are fetched one chunk ahead and handed round by shuffle.
            // (the dequantizing modes run 23 warps per CTA: their register budget allows 32 columns per load)
            constexpr int kChunk = BT >= 64 ? (kExpand ? 32 : 64) : 16;
            const bool scaled = kInt8 && p.splits == 1;
            auto load_sx = [&](int m_first) {
                const int m = m_first + lane;
                return (scaled && (kChunk > 16 || lane < 16) && m < p.M) ? __half2float(__ldcg(p.sx + m)) : 0.f;
            };
            float sx_a = load_sx(u.m_tile * BT), sx_b = kChunk > 32 ? load_sx(u.m_tile * BT + 32) : 0.f;
            if (!mbar_wait(&tmem_full[b], (it >> 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * BT);
            uint32_t* part = p.partials + ((size_t)unit * BT) * kTileN + row;
#pragma unroll 1
            for (int c0 = 0; c0 < BT; c0 += kChunk) {
                const float s0 = sx_a, s1 = sx_b;
                if (c0 + kChunk < BT) {
                    sx_a = load_sx(u.m_tile * BT + c0 + kChunk);
                    if (kChunk > 32) sx_b = load_sx(u.m_tile * BT + c0 + kChunk + 32);
                }
                uint32_t r[kChunk];
                if constexpr (kChunk == 64) tmem_ld64(taddr + c0, r);
                else if constexpr (kChunk == 32) tmem_ld32(taddr + c0, r);
                else tmem_ld16(taddr + c0, r);
                tmem_ld_wait();
                if (p.splits == 1) {
                    const int m0 = u.m_tile * BT + c0;
                    const bool plain = n_ok && m0 + kChunk <= p.M && !has_bias && p.acc_dbg == nullptr;
                    if (__all_sync(0xffffffffu, plain)) {
                        // the common case (chunk inside the matrix, no bias): no per-element checks
                        __half* yp = p.Y + (size_t)m0 * p.N + n;
#pragma unroll
                        for (int c = 0; c < kChunk; ++c) {
                            if constexpr (kInt8) {
                                const float sxf = __shfl_sync(0xffffffffu, c < 32 ? s0 : s1, c & 31);
                                *yp = __float2half_rn(__fmul_rn((float)(int32_t)r[c], __fmul_rn(s1f, sxf)));
                            } else {
                                *yp = __float2half_rn(__uint_as_float(r[c]));
                            }
                            yp += p.N;
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < kChunk; ++c) {
                            const int m = m0 + c;
                            const float sxf = kInt8 ? __shfl_sync(0xffffffffu, c < 32 ? s0 : s1, c & 31) : 0.f;
                            if (n_ok && m < p.M) store_output<kInt8>(p, r[c], m, n, s1f, sxf, has_bias, bias_n);
                        }
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < kChunk; ++c) part[(size_t)(c0 + c) * kTileN] = r[c];
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[b]);
        }
    } else if constexpr (kExpand) {
        // ------------------------------ weight expanders --------------------------
        // Four groups of two warps; group g expands every fourth k block (four 16-byte chunks per
        // thread), so four k blocks are in flight and the per-block latency chain
        // (wait -> load -> expand -> store -> fence -> arrive) is overlapped instead of serialised.
        const int grp = (warp - 6) / kExpandGroupWarps;
        const int t = threadIdx.x - 192 - grp * (32 * kExpandGroupWarps);     // 0..63
        constexpr int kChunks = 256 / (32 * kExpandGroupWarps);               // chunks per thread: 4
        int n_local[kChunks];
        uint32_t dst_off[kChunks];
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
            const int j = t + 32 * kExpandGroupWarps * c;
            // W4: 16-byte chunk j of a k block's packed [32][128 B] = weight row 4*(j/8) + (j%8)/2,
            //     k half j%2 (32 consecutive k).  W8: [128][64 B] int8, row j/2, half j%2.
            n_local[c] = kMode == kModeW4 ? 4 * (j >> 3) + ((j & 7) >> 1) : (j >> 1);
            dst_off[c] = (uint32_t)((n_local[c] >> 3) * 1024 + (n_local[c] & 7) * 128);
        }
        const int khalf = t & 1;                     // same for all chunks of a thread (stride is even)
        uint32_t i = 0;                              // running k-block count of this CTA
        bool ok = true;
        for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
            const UnitRange u = unit_range(p, unit);
            __half2 s8[kChunks];
            if constexpr (kMode == kModeW8) {
#pragma unroll
                for (int c = 0; c < kChunks; ++c) {
                    const int n = u.n_tile * kTileN + n_local[c];
                    s8[c] = __half2half2(n < p.N ? __ldg(p.s1 + n) : __float2half_rn(0.f));
                }
            }
            for (int kb = u.kb0; kb < u.kb1; ++kb, ++i) {
                const uint32_t stage_no = i / kSub;
                const int sub = (int)(i % kSub);
                const int s = (int)(stage_no % kStages), as = (int)(i % kAStages);
                const uint32_t phase = (stage_no / kStages) & 1u, aphase = (i / kAStages) & 1u;
                // Every group observes every stage fill, in order, also those it does not expand: a
                // parity wait is only valid while the waiter is at most one phase away from the barrier.
                if (!mbar_wait(&full[s], phase, abort_flag)) { ok = false; break; }
                if ((int)(i % kExpandGroups) != grp) continue;
                if (t == 0) trace_stamp(p, i, 4);
                const uint8_t* st = stage_base + s * Cfg::kStageBytes;
                uint4 raw[kChunks], raw_hi[kChunks];
                __half2 sc[kChunks], zc[kChunks];
#pragma unroll
                for (int c = 0; c < kChunks; ++c) {
                    const int j = t + 32 * kExpandGroupWarps * c;
                    if constexpr (kMode == kModeW4) {
                        // packed rows are kSub x 128 bytes long; this k block's 128 bytes start at sub * 128
                        raw[c] = *reinterpret_cast<const uint4*>(st + (j >> 3) * (kSub * 128) + sub * 128 + (j & 7) * 16);
                        // this row's factors of the k block's group, staged by TMA (zero beyond N)
                        const uint8_t* f = st + Cfg::kPackedBytes + (kSub >= 2 ? (sub >> 1) * 256 : 0) + 2 * n_local[c];
                        sc[c] = __half2half2(*reinterpret_cast<const __half*>(f));
                        zc[c] = __half2half2(*reinterpret_cast<const __half*>(f + Cfg::kFactorGroups * 256));
                    } else {
                        const uint8_t* src = st + (j >> 1) * (kSub * 64) + sub * 64 + (j & 1) * 32;
                        raw[c] = *reinterpret_cast<const uint4*>(src);
                        raw_hi[c] = *reinterpret_cast<const uint4*>(src + 16);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);           // packed tile is in registers
                if (t == 0) trace_stamp(p, i, 5);
                if (!mbar_wait(&a_empty[as], aphase ^ 1, abort_flag)) { ok = false; break; }
                if (t == 0) trace_stamp(p, i, 6);
                uint8_t* a_tile = a_ring + as * kATileBytes;
#pragma unroll
                for (int c = 0; c < kChunks; ++c) {
                    __half2 w[16];
                    if constexpr (kMode == kModeW4) {
                        dequant_chunk32_fma(raw[c], sc[c], zc[c], w);
                    } else {
                        widen_s8x4(raw[c].x, s8[c], w[0], w[1]);
                        widen_s8x4(raw[c].y, s8[c], w[2], w[3]);
                        widen_s8x4(raw[c].z, s8[c], w[4], w[5]);
                        widen_s8x4(raw[c].w, s8[c], w[6], w[7]);
                        widen_s8x4(raw_hi[c].x, s8[c], w[8], w[9]);
                        widen_s8x4(raw_hi[c].y, s8[c], w[10], w[11]);
                        widen_s8x4(raw_hi[c].z, s8[c], w[12], w[13]);
                        widen_s8x4(raw_hi[c].w, s8[c], w[14], w[15]);
                    }
                    uint8_t* dst = a_tile + dst_off[c];
                    const int swz = n_local[c] & 7;
                    const uint32_t* uw = reinterpret_cast<const uint32_t*>(w);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        const int chunk = (4 * khalf + q4) ^ swz;   // 128-byte swizzle: 16-byte chunk ^ (row % 8)
                        *reinterpret_cast<uint4*>(dst + 16 * chunk) =
                            make_uint4(uw[4 * q4], uw[4 * q4 + 1], uw[4 * q4 + 2], uw[4 * q4 + 3]);
                    }
                }
                fence_proxy_async_smem();                        // generic-proxy writes -> visible to the MMA
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_full[as]);
                if (t == 0) trace_stamp(p, i, 7);
            }
        }
    }

    // ------------------------------ teardown --------------------------------------
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) atomicExch(p.status, KAIROS_ERR_DEVICE);
        // let copies that were already issued land before the CTA's shared memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// ---------------------------------------------------------------------------------
// W4A16 with the expanded weight operand in TENSOR MEMORY.
//
// In the kernel above the dequantized fp16 tile goes through shared memory: 16 KB written by the expander
// warps and 16 KB read back by the tensor core for every 4 KB of packed weight, on top of the packed tile,
// the activations and their reads.  At 128 bytes per clock the shared memory of an SM is then the bound
// (about 450 cycles per 64-k block at BT = 64, measured with the pipeline trace), far below HBM speed.
// Here the A operand of tcgen05.mma lives in tensor memory instead: an expander thread owns one weight
// row of the tile (TMEM lane = row), dequantizes its 32 k of a k block in registers and stores them with
// tcgen05.st into a ring of 32-column slots; the MMA reads A from that slot and only the activations (B)
// from shared memory.  Shared-memory traffic per k block drops to the packed tile (4 KB in, 4 KB out) and
// the activation tile.
//
//   warp 0      TMA producer: per stage (one quantization group = two k blocks) the packed tile
//               [32 qweight rows][256 B], the group's scales / scaled zeros of the 128 rows, and the
//               activations [2 k blocks][BT tokens][128 B] (128B-swizzled, the tcgen05 B operand)
//   warp 1      MMA issuer, owner of the 512 TMEM columns: D (2 x BT fp32 columns, double-buffered) and
//               the A ring (8 slots x 32 columns: 128 rows x 64 fp16)
//   warps 2-5   epilogue (TMEM -> registers -> Y, or split-K partial tiles)
//   warps 6-21  expanders: four groups of four warps (one per TMEM lane quarter); group g expands k
//               blocks g, g + 4, ...
// ---------------------------------------------------------------------------------
template <int BT>
struct W4Cfg {
    static constexpr int kXTileBytes = BT * kRowBytes;                 // activations of one k block
    static constexpr int kPackedBytes = 32 * 256;                      // [32 qweight rows][two k blocks x 128 B]
    static constexpr int kFactorBytes = 1024;                          // scales at 0, scaled zeros at 256 (128 rows each)
    static constexpr int kStageBytes = 2 * kXTileBytes + kPackedBytes + kFactorBytes;
    static constexpr int kWTxBytes = kPackedBytes + 512;               // packed tile + scales + scaled zeros
    static constexpr int kXTxBytes = 2 * kXTileBytes;
    static constexpr int kStagesFit = kSmemBudget / kStageBytes;
    static constexpr int kStages = kStagesFit > 8 ? 8 : kStagesFit;
    static constexpr int kASlots = 4;                                  // A ring in tensor memory: slots of one stage (64 columns)
    static constexpr int kExpWarps = 16;
    static constexpr int kFirstExpWarp = 8;
    static constexpr int kWarps = kFirstExpWarp + kExpWarps;
    static constexpr int kThreads = 32 * kWarps;
    static constexpr int kTmemCols = 512;
    // Successive MMAs into ONE accumulator tile wait for each other (about 90 cycles apiece at these small N,
    // whatever N is); MMAs into different tiles overlap.  So the K steps of a tile go round-robin to kAcc
    // accumulators, which the epilogue adds.
    static constexpr int kAcc = BT <= 32 ? 4 : (BT <= 64 ? 2 : 1);
    // One issuing thread needs 700-800 cycles per stage (waits, descriptors, eight MMAs, two commits: a chain
    // of dependent instructions in a single thread), more than the expanders or the copies.  With two
    // accumulators or more the stages therefore alternate between TWO issuer warps on different schedulers,
    // each accumulating into its own tiles.
    static constexpr int kIssuers = kAcc >= 2 ? 2 : 1;
    static constexpr int kAccPerIssuer = kAcc / kIssuers;
    static constexpr uint32_t kDCols = kAcc * BT;                      // columns of one (double-buffered) accumulator set
    static constexpr uint32_t kAColBase = 2 * kDCols;                  // the A ring follows the two sets
    static constexpr int kBarBytes = 8 * (2 * kStages + 2 * kASlots + 4) + 64;
    static constexpr int kSmemBytes = kStages * kStageBytes + kBarBytes + 1024;
    static_assert(BT >= 32 && BT <= 128 && BT % 16 == 0, "token tile of the tensor-memory kernel");
    static_assert(2 * kAcc * BT + kASlots * 64 <= 512, "accumulators and the A ring must fit the 512 TMEM columns");
    // an expander warp that only OBSERVES a stage (another group owns it) must never fall two uses of a stage
    // slot behind: the groups are at most kASlots stages apart
    static_assert(kStages > kASlots, "stage ring shorter than the spread of the expander groups");
    static_assert(kSmemBytes <= 227 * 1024, "exceeds the shared memory a CTA may use");
    static constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(BT >> 3) << 17) | ((uint32_t)(kTileN >> 4) << 24);
};

// D[tmem] (+)= A[tmem] . B[smem]^T, kind::f16, one CTA.
__device__ __forceinline__ void umma_f16_a_tmem(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                                uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 16 registers -> 16 consecutive 32-bit columns of the thread's TMEM lane.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <int BT>
__global__ void __launch_bounds__(W4Cfg<BT>::kThreads, 1)
    w4a16_tmem_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                      const __grid_constant__ CUtensorMap tmap_s, const __grid_constant__ CUtensorMap tmap_z,
                      const GemmParams p) {
    using Cfg = W4Cfg<BT>;
    constexpr int kStages = Cfg::kStages;
    constexpr int kASlots = Cfg::kASlots;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* stage_base = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes);
    uint64_t* full = bars;                       // stage filled by TMA
    uint64_t* empty = full + kStages;            // stage released: its 4 expander warps + the MMAs that read its activations
    uint64_t* a_full = empty + kStages;          // A slot written (4 expander warps)
    uint64_t* a_empty = a_full + kASlots;        // A slot read by the MMAs (commit)
    uint64_t* tmem_full = a_empty + kASlots;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 2);                     // the weight-side and the activation-side producer
            mbar_init(&empty[s], 5);
        }
        for (int s = 0; s < kASlots; ++s) {
            mbar_init(&a_full[s], 4);
            mbar_init(&a_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tmem_full[b], Cfg::kIssuers);
            mbar_init(&tmem_empty[b], 4);
        }
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmap_w);
        tma_prefetch_desc(&tmap_x);
        tma_prefetch_desc(&tmap_s);
        tma_prefetch_desc(&tmap_z);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    chain_release();
    chain_wait();

    const int total_units = p.n_tiles * p.m_tiles * p.splits;

    if (warp == 0) {
        // ------------------------------ weight-side TMA producer -------------------
        // (the whole warp walks the loop, one elected lane issues: see elect_one)
        int s = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
            const UnitRange u = unit_range(p, unit);
            for (int kb = u.kb0; kb < u.kb1; kb += 2) {
                if (!mbar_wait(&empty[s], phase ^ 1, abort_flag)) { ok = false; break; }
                uint8_t* wp = stage_base + s * Cfg::kStageBytes + 2 * Cfg::kXTileBytes;
                if (elect_one()) {
                    mbar_arrive_expect_tx(&full[s], Cfg::kWTxBytes);
                    tma_load_2d(wp, &tmap_w, &full[s], kb * 64, u.n_tile * (kTileN / kInterleave));
                    tma_load_2d(wp + Cfg::kPackedBytes, &tmap_s, &full[s], u.n_tile * kTileN, kb >> 1);
                    tma_load_2d(wp + Cfg::kPackedBytes + 256, &tmap_z, &full[s], u.n_tile * kTileN, kb >> 1);
                }
                __syncwarp();
                trace_stamp(p, (uint32_t)(kb - u.kb0), 0);
                if (++s == kStages) { s = 0; phase ^= 1; }
            }
        }
    } else if (warp == 3) {
        // ------------------------------ activation-side TMA producer ---------------
        int s = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
            const UnitRange u = unit_range(p, unit);
            for (int kb = u.kb0; kb < u.kb1; kb += 2) {
                if (!mbar_wait(&empty[s], phase ^ 1, abort_flag)) { ok = false; break; }
                uint8_t* st = stage_base + s * Cfg::kStageBytes;
                if (elect_one()) {
                    mbar_arrive_expect_tx(&full[s], Cfg::kXTxBytes);
                    tma_load_3d(st, &tmap_x, &full[s], 0, u.m_tile * BT, kb);               // [2 k blocks][BT][128 B]
                }
                __syncwarp();
                if (++s == kStages) { s = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1 || warp == 2) {
        // ------------------------------ MMA issuers -------------------------------
        // The whole warp walks the loop (every lane sees the same barriers and counters); one elected lane issues.
        // Issuer `mi` takes the stages mi, mi + kIssuers, ... of the CTA's running stage count: with an even
        // number of stage and A slots it meets every use of the slots it touches, so its parity waits stay valid.
        const int mi = warp - 1;
        if (mi < Cfg::kIssuers) {
            static_assert(Cfg::kIssuers == 1 || (kStages % 2 == 0 && kASlots % 2 == 0), "issuers need even rings");
            uint32_t i = 0;                              // running stage count of this CTA
            int it = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x, ++it) {
                const UnitRange u = unit_range(p, unit);
                const int b = it & 1;
                if (!mbar_wait(&tmem_empty[b], ((it >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)b * Cfg::kDCols + (uint32_t)(mi * Cfg::kAccPerIssuer * BT);
                bool first = true;                       // this issuer's accumulators hold nothing of the tile yet
                for (int kb = u.kb0; kb < u.kb1 && ok; kb += 2, ++i) {
                    if ((int)(i % Cfg::kIssuers) != mi) continue;
                    const int s = (int)(i % kStages), as = (int)(i % kASlots);
                    const uint32_t phase = (i / kStages) & 1u, aphase = (i / kASlots) & 1u;
                    if (!mbar_wait(&full[s], phase, abort_flag)) { ok = false; break; }
                    trace_stamp(p, (uint32_t)(kb - u.kb0), 1);
                    const uint8_t* st = stage_base + s * Cfg::kStageBytes;
                    if (!mbar_wait(&a_full[as], aphase, abort_flag)) { ok = false; break; }
                    trace_stamp(p, (uint32_t)(kb - u.kb0), 2);
                    tc_fence_after();
                    const uint32_t a_tmem = tmem_base + Cfg::kAColBase + (uint32_t)(as * 64);
                    const uint64_t bdesc0 = umma_desc_sw128(smem_u32(st));
                    const uint64_t bdesc1 = umma_desc_sw128(smem_u32(st + Cfg::kXTileBytes));
                    if (elect_one()) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)   // K = 16 per instruction: 8 TMEM columns of A, 32 bytes of a B row
                            umma_f16_a_tmem(d_tmem + (uint32_t)((j % Cfg::kAccPerIssuer) * BT), a_tmem + 8 * j,
                                            (j < 4 ? bdesc0 : bdesc1) + 2 * (j & 3), Cfg::kIdesc,
                                            (!first || j >= Cfg::kAccPerIssuer) ? 1u : 0u);
                        umma_commit(&a_empty[as]);
                        umma_commit(&empty[s]);
                    }
                    __syncwarp();
                    first = false;
                    trace_stamp(p, (uint32_t)(kb - u.kb0), 3);
                }
                if (ok) {
                    // an issuer without a stage in this unit (a unit of one stage) has nothing to commit; the
                    // epilogue leaves its accumulators out
                    if (elect_one()) {
                        if (first) mbar_arrive(&tmem_full[b]);
                        else umma_commit(&tmem_full[b]);
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp >= 4 && warp < 8) {
        // ------------------------------ epilogue ----------------------------------
        const int q = warp & 3;                    // TMEM lane quarter this warp may read
        const int row = q * 32 + lane;
        int it = 0;
        uint32_t i0 = 0;                           // running stage count at the start of the unit
        bool ok = true;
        for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x, ++it) {
            const UnitRange u = unit_range(p, unit);
            const int n = u.n_tile * kTileN + row;
            const bool n_ok = n < p.N;
            const int b = it & 1;
            const bool has_bias = p.bias != nullptr;
            const __half bias_n = (has_bias && n_ok) ? __ldg(p.bias + n) : __float2half_rn(0.f);
            // which issuers had a stage of this unit (stage i goes to issuer i % kIssuers)
            const int unit_stages = (u.kb1 - u.kb0) / 2;
            bool issued[Cfg::kIssuers];
#pragma unroll
            for (int mi = 0; mi < Cfg::kIssuers; ++mi)
                issued[mi] = unit_stages >= Cfg::kIssuers || (unit_stages > 0 && (int)(i0 % Cfg::kIssuers) == mi);
            i0 += (uint32_t)unit_stages;
            if (!mbar_wait(&tmem_full[b], (it >> 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)b * Cfg::kDCols;
            uint32_t* part = p.partials + ((size_t)unit * BT) * kTileN + row;
#pragma unroll 1
            for (int c0 = 0; c0 < BT; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(taddr + c0, r);
                tmem_ld_wait();
                if (!issued[0]) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) r[c] = 0u;
                }
#pragma unroll
                for (int a = 1; a < Cfg::kAcc; ++a) {       // the other accumulators of the set
                    if (!issued[a / Cfg::kAccPerIssuer]) continue;
                    uint32_t r2[32];
                    tmem_ld32(taddr + a * BT + c0, r2);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) + __uint_as_float(r2[c]));
                }
                if (p.splits == 1) {
                    const int m0 = u.m_tile * BT + c0;
                    if (n_ok) {
                        __half* yp = p.Y + (size_t)m0 * p.N + n;
#pragma unroll
                        for (int c = 0; c < 32; ++c) {
                            if (m0 + c < p.M) {
                                __half y = __float2half_rn(__uint_as_float(r[c]));
                                if (has_bias) y = __hadd(y, bias_n);
                                yp[(size_t)c * p.N] = y;
                            }
                        }
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) part[(size_t)(c0 + c) * kTileN] = r[c];
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[b]);
        }
    } else if (warp >= Cfg::kFirstExpWarp) {
        // ------------------------------ weight expanders --------------------------
        // Thread = weight row of the tile (TMEM lane): 32 (warp % 4) + lane.  Its 64 k of a k block are 32 packed
        // bytes: qweight row r >> 2, the k block's 128-byte line, 16-byte units 2 (r & 3) and 2 (r & 3) + 1
        // (k 0..31 and 32..63 of the block).
        const int grp = (warp - Cfg::kFirstExpWarp) >> 2;
        const int row = 32 * (warp & 3) + lane;
        const uint32_t w_off = (uint32_t)(2 * Cfg::kXTileBytes + (row >> 2) * 256 + ((row & 3) << 5));
        const uint32_t f_off = (uint32_t)(2 * Cfg::kXTileBytes + Cfg::kPackedBytes + 2 * row);
        const uint32_t lane_base = tmem_base + ((uint32_t)(32 * (warp & 3)) << 16) + Cfg::kAColBase;
        uint32_t i = 0;                              // running stage count of this CTA
        bool ok = true;
        for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
            const UnitRange u = unit_range(p, unit);
            for (int kb = u.kb0; kb < u.kb1; kb += 2, ++i) {
                const int s = (int)(i % kStages), as = (int)(i % kASlots);
                const uint32_t phase = (i / kStages) & 1u, aphase = (i / kASlots) & 1u;
                // every warp observes every stage fill, in order (a parity wait is only valid one phase away)
                if (!mbar_wait(&full[s], phase, abort_flag)) { ok = false; break; }
                if ((int)(i & 3u) != grp) continue;
                if ((warp & 3) == 0 && lane == 0) trace_stamp(p, (uint32_t)(kb - u.kb0), 4);
                const uint8_t* st = stage_base + s * Cfg::kStageBytes;
                uint4 raw[4];                                    // k 0..31, 32..63 of the first block, then of the second
                raw[0] = *reinterpret_cast<const uint4*>(st + w_off);
                raw[1] = *reinterpret_cast<const uint4*>(st + w_off + 16);
                raw[2] = *reinterpret_cast<const uint4*>(st + w_off + 128);
                raw[3] = *reinterpret_cast<const uint4*>(st + w_off + 144);
                const __half2 sc = __half2half2(*reinterpret_cast<const __half*>(st + f_off));
                const __half2 zc = __half2half2(*reinterpret_cast<const __half*>(st + f_off + 256));
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);           // packed bytes and factors are in registers
                if ((warp & 3) == 0 && lane == 0) trace_stamp(p, (uint32_t)(kb - u.kb0), 5);
                if (!mbar_wait(&a_empty[as], aphase ^ 1, abort_flag)) { ok = false; break; }
                if ((warp & 3) == 0 && lane == 0) trace_stamp(p, (uint32_t)(kb - u.kb0), 6);
                tc_fence_after();
                const uint32_t a_tmem = lane_base + (uint32_t)(as * 64);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    __half2 w[16];
                    dequant_chunk32_fma(raw[c], sc, zc, w);      // 32 k, pairs in k order
                    tmem_st16(a_tmem + 16 * c, *reinterpret_cast<const uint32_t(*)[16]>(w));
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_full[as]);
                if ((warp & 3) == 0 && lane == 0) trace_stamp(p, (uint32_t)(kb - u.kb0), 7);
            }
        }
    }

    // ------------------------------ teardown --------------------------------------
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) atomicExch(p.status, KAIROS_ERR_DEVICE);
        for (int i = 0; i < 64; ++i) __nanosleep(1000);   // let copies that were already issued land
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------
int make_tmap(CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle);   // tensormap.cu

// 2-D row-major tensor [rows, cols] of `elem_bytes` elements; box = box_cols x box_rows, no swizzle.
static int make_tmap_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t rows,
                        uint64_t cols, uint32_t box_cols, uint32_t box_rows) {
    const uint64_t dims[2] = {cols, rows};
    const uint64_t strides[1] = {cols * (uint64_t)elem_bytes};
    const uint32_t box[2] = {box_cols, box_rows};
    return make_tmap(map, dt, 2, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
}

// Row-major operand [rows, K] seen as k blocks of 128 bytes: dims {128 B of K, rows, K / block};
// one copy brings `box_kb` consecutive k blocks of `box_rows` rows, each landing as a 128B-swizzled
// K-major tile [box_rows][128 B] (the layout tcgen05.mma reads), tiles back to back.
static int make_tmap_kblocks(CUtensorMap* map, const void* base, bool int8, uint64_t rows, uint64_t K,
                             uint32_t box_rows, uint32_t box_kb) {
    const uint64_t es = int8 ? 1 : 2, bk = int8 ? 128 : 64;
    const uint64_t dims[3] = {bk, rows, K / bk};
    const uint64_t strides[2] = {K * es, 128};
    const uint32_t box[3] = {(uint32_t)bk, box_rows, box_kb};
    return make_tmap(map, int8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, base, dims,
                     strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

int device_sm_count() {
    static int sms[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!sms[dev]) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        sms[dev] = v;
    }
    return sms[dev];
}

int* device_status_word();   // api.cu: host-mapped word the kernels raise on a timed-out wait

static long long* g_trace = nullptr;   // diagnostic buffer of kTraceBlocks * kTraceSlots stamps, or null


static int token_tile(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256; }

static int stage_bundle(int bt) { return bt <= 64 ? 4 : (bt == 128 ? 2 : 1); }   // GemmCfg::kSub

struct Plan {
    int bt, n_tiles, m_tiles, splits, kb_per_split, kb_total;
    size_t partial_bytes;
};

// Split-K plan, old rule (dequantizing modes, token tiles up to 64, the tensor-memory W4A16 kernel).  When a
// problem has fewer output tiles than the device has SMs, a tile's K range is cut into runs of whole stage
// bundles, one CTA each, and a second pass sums the partial tiles.  Measured on B200: with a tile for three
// SMs in four or more, the second pass and the partial traffic cost more than the idle SMs, so only problems
// with fewer tiles than SMs are split.  The partial tiles (tiles * splits * BT * 128 * 4 bytes) must fit
// `max_partial_bytes` (the caller's scratch, if bounded).
// `w4_tmem` selects the geometry of the W4A16 kernel that keeps the expanded operand in tensor memory:
// token tiles of 32..128 and stages of one quantization group.
static Plan plan_geometry(int M, int N, int K, bool int8, int bt, int sub) {
    Plan pl;
    pl.bt = bt;
    pl.n_tiles = (N + kTileN - 1) / kTileN;
    pl.m_tiles = (M + bt - 1) / bt;
    const int stages_total = (K / (int8 ? 128 : 64) + sub - 1) / sub;   // k blocks past K are zero-filled
    pl.kb_total = stages_total * sub;
    pl.kb_per_split = sub;                                              // bundle size (see unit_range)
    pl.splits = 1;
    pl.partial_bytes = 0;
    return pl;
}

// Plan of the TMA-fed modes (W8A8, FP16) beyond 64 tokens: token tile and K split chosen together by a cost
// model fitted to graph-timed runs on B200 (K = 4096 and 14336, N = 1024..14336, M = 128..2048):
//   * a CTA needs c(BT) microseconds per 128-byte k block (0.34 / 0.375 / 0.53 for int8 at BT = 64 / 128 / 256:
//     the 16 KB weight block, not the MMA, sets the pace of small token tiles), so one round of tiles takes
//     kb * c and smaller token tiles pay when they fill SMs that larger ones leave idle;
//   * all CTAs together draw their operands from L2 at about 11.5 TB/s, which bounds many small tiles;
//   * a K split costs about 6 us (second launch, drained pipeline) plus its partial-tile traffic, so it pays
//     only for very few tiles or long K (it made M = 256..512 on 4096 x 4096 1.5x SLOWER than unsplit tiles).
static Plan make_plan_tma(int M, int N, int K, bool int8, size_t max_partial_bytes) {
    const int sms = device_sm_count();
    const double es = int8 ? 1.0 : 2.0;
    Plan best;
    double best_cost = 1e30;
    for (int bt = 256; bt >= 64; bt >>= 1) {
        if (bt > token_tile(M)) continue;
        const int sub = stage_bundle(bt);
        Plan pl = plan_geometry(M, N, K, int8, bt, sub);
        const int tiles = pl.n_tiles * pl.m_tiles, stages_total = pl.kb_total / sub;
        const double c = (bt == 64 ? 0.34 : bt == 128 ? 0.375 : 0.53) * (int8 ? 1.0 : 0.77);
        const double t_bw = (double)tiles * (kTileN + bt) * K * es / 11.5e6;
        const size_t tile_bytes = (size_t)bt * kTileN * 4;
        const int min_stages = 4 / sub > 0 ? 4 / sub : 1;                 // at least 4 k blocks per run
        int max_s = tiles < sms ? sms / tiles : 1;
        if (max_s > stages_total / min_stages) max_s = stages_total / min_stages > 0 ? stages_total / min_stages : 1;
        for (int sp = 1; sp <= max_s; ++sp) {
            if (sp > 1 && (size_t)tiles * sp * tile_bytes > max_partial_bytes) break;
            const int rounds = (tiles * sp + sms - 1) / sms;
            const double t_lat = rounds * ((double)pl.kb_total / sp) * c;
            double cost = t_lat > t_bw ? t_lat : t_bw;
            if (sp > 1) cost += 6.0 + (double)tiles * sp * tile_bytes / 2.0e6;
            if (cost < best_cost - 1e-9) {
                best_cost = cost;
                best = pl;
                best.splits = sp;
                best.partial_bytes = sp > 1 ? (size_t)tiles * sp * tile_bytes : 0;
            }
        }
    }
    return best;
}

static Plan make_plan(int M, int N, int K, bool int8, size_t max_partial_bytes = ~(size_t)0, bool w4_tmem = false,
                      bool tma_fed = false) {
    if (tma_fed && M > 64) return make_plan_tma(M, N, K, int8, max_partial_bytes);
    int bt = token_tile(M);
    if (w4_tmem) bt = bt < 32 ? 32 : (bt > 128 ? 128 : bt);
    const int sub = w4_tmem ? 2 : stage_bundle(bt);
    Plan pl = plan_geometry(M, N, K, int8, bt, sub);
    const int stages_total = pl.kb_total / sub;
    const int tiles = pl.n_tiles * pl.m_tiles;
    const int sms = device_sm_count();
    const size_t tile_bytes = (size_t)pl.bt * kTileN * 4;
    int splits = 1;
    if (tiles < sms) {
        splits = sms / tiles;
        const int min_stages = 4 / sub > 0 ? 4 / sub : 1;                 // at least 4 k blocks per run
        const int max_by_k = stages_total / min_stages > 0 ? stages_total / min_stages : 1;
        if (splits > max_by_k) splits = max_by_k;
        while (splits > 1 && (size_t)tiles * splits * tile_bytes > max_partial_bytes) --splits;
        if (splits < 1) splits = 1;
    }
    pl.splits = splits;
    pl.partial_bytes = pl.splits > 1 ? (size_t)tiles * pl.splits * tile_bytes : 0;
    return pl;
}

size_t gemm_workspace_bytes(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    const Plan a = make_plan(M, N, K, false, ~(size_t)0, false, true), b = make_plan(M, N, K, true, ~(size_t)0, false, true),
               c = make_plan(M, N, K, false, ~(size_t)0, M <= 128), d = make_plan(M, N, K, false);
    size_t need = a.partial_bytes > b.partial_bytes ? a.partial_bytes : b.partial_bytes;
    if (c.partial_bytes > need) need = c.partial_bytes;
    return need > d.partial_bytes ? need : d.partial_bytes;
}

struct GemmArgs {
    const void* X;       // [M,K] fp16 or int8
    const void* W;       // mode-dependent weight operand
    const __half *scales, *scaled_zeros, *s1, *sx, *bias;
    void* Y;
    void* acc_dbg;
    int M, N, K;
    void* workspace;
    size_t workspace_bytes;
    cudaStream_t stream;
    int* status = nullptr;   // device word for timed-out waits; null = the per-device host-mapped word
    size_t plan_cap = 0;     // upper bound of the split-K scratch the plan may use; 0 = the default bound
};

template <bool kInt8, int kMode, int BT>
static int launch_one(const GemmArgs& a, const Plan& pl) {
    using Cfg = GemmCfg<kInt8, kMode, BT>;
    CUtensorMap tw, tx, ts, tz;
    int rc;
    if constexpr (kMode == kModeW4) {
        rc = make_tmap_2d(&tw, a.W, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, (uint64_t)a.N / kInterleave, (uint64_t)a.K,
                          64 * Cfg::kSub, 32);
        if (rc != KAIROS_OK) return rc;
        // factor tensors [K/128 used rows, N] fp16: 128-wide row slices, the stage's groups
        rc = make_tmap_2d(&ts, a.scales, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (uint64_t)a.K / kGroup, (uint64_t)a.N,
                          kTileN, Cfg::kFactorGroups);
        if (rc != KAIROS_OK) return rc;
        rc = make_tmap_2d(&tz, a.scaled_zeros, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (uint64_t)a.K / kGroup,
                          (uint64_t)a.N, kTileN, Cfg::kFactorGroups);
    } else if constexpr (kMode == kModeW8) {
        rc = make_tmap_2d(&tw, a.W, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)a.N, (uint64_t)a.K, 64 * Cfg::kSub,
                          kTileN);
    } else {
        rc = make_tmap_kblocks(&tw, a.W, kInt8, (uint64_t)a.N, (uint64_t)a.K, kTileN, Cfg::kSub);
    }
    if (rc != KAIROS_OK) return rc;
    rc = make_tmap_kblocks(&tx, a.X, kInt8, (uint64_t)a.M, (uint64_t)a.K, BT, Cfg::kSub);
    if (rc != KAIROS_OK) return rc;
    if constexpr (kMode != kModeW4) {
        ts = tx;   // unused by the kernel in these modes
        tz = tx;
    }

    GemmParams p;
    p.M = a.M; p.N = a.N; p.K = a.K;
    p.n_tiles = pl.n_tiles; p.m_tiles = pl.m_tiles; p.splits = pl.splits;
    p.kb_per_split = pl.kb_per_split; p.kb_total = pl.kb_total;
    p.scales = a.scales; p.scaled_zeros = a.scaled_zeros; p.s1 = a.s1; p.sx = a.sx; p.bias = a.bias;
    p.Y = static_cast<__half*>(a.Y);
    p.acc_dbg = static_cast<int32_t*>(a.acc_dbg);
    p.partials = static_cast<uint32_t*>(a.workspace);
    p.status = a.status ? a.status : device_status_word();
    p.trace = g_trace;
    if (!p.status) return KAIROS_ERR_CUDA;

    static PerDeviceFlag smem_attr;    // per instantiation
    if ((rc = ensure_dynamic_smem(smem_attr, umma_gemm_kernel<kInt8, kMode, BT>, Cfg::kSmemBytes)) != KAIROS_OK) return rc;
    const int units = pl.n_tiles * pl.m_tiles * pl.splits;
    const int sms = device_sm_count();
    const int grid = units < sms ? units : sms;
    cudaError_t e = launch_chained(umma_gemm_kernel<kInt8, kMode, BT>, dim3(grid), dim3(Cfg::kThreads), Cfg::kSmemBytes,
                                   a.stream, tw, tx, ts, tz, p);
    if (e != cudaSuccess) return note_cuda_error(e);
    if (pl.splits > 1) {
        const int rc2 = launch_status();
        if (rc2 != KAIROS_OK) return rc2;
        e = launch_chained(splitk_reduce_kernel<kInt8>, dim3(pl.n_tiles * pl.m_tiles * BT), dim3(kTileN), 0, a.stream, p,
                           (int)BT);
        if (e != cudaSuccess) return note_cuda_error(e);
    }
    return launch_status();
}

template <int BT>
static int launch_w4_tmem(const GemmArgs& a, const Plan& pl) {
    using Cfg = W4Cfg<BT>;
    CUtensorMap tw, tx, ts, tz;
    int rc;
    // qweight int16 [N/4, K]: 32 rows x 128 elements (two k blocks of the tile's 128 weight rows)
    if ((rc = make_tmap_2d(&tw, a.W, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, (uint64_t)a.N / kInterleave, (uint64_t)a.K, 128,
                           32)) != KAIROS_OK) return rc;
    // factors fp16 [K/128, N]: the tile's 128 rows of one group
    if ((rc = make_tmap_2d(&ts, a.scales, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (uint64_t)a.K / kGroup, (uint64_t)a.N,
                           kTileN, 1)) != KAIROS_OK) return rc;
    if ((rc = make_tmap_2d(&tz, a.scaled_zeros, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (uint64_t)a.K / kGroup,
                           (uint64_t)a.N, kTileN, 1)) != KAIROS_OK) return rc;
    if ((rc = make_tmap_kblocks(&tx, a.X, false, (uint64_t)a.M, (uint64_t)a.K, BT, 2)) != KAIROS_OK) return rc;

    GemmParams p;
    p.M = a.M; p.N = a.N; p.K = a.K;
    p.n_tiles = pl.n_tiles; p.m_tiles = pl.m_tiles; p.splits = pl.splits;
    p.kb_per_split = pl.kb_per_split; p.kb_total = pl.kb_total;
    p.scales = a.scales; p.scaled_zeros = a.scaled_zeros; p.s1 = nullptr; p.sx = nullptr; p.bias = a.bias;
    p.Y = static_cast<__half*>(a.Y);
    p.acc_dbg = nullptr;
    p.partials = static_cast<uint32_t*>(a.workspace);
    p.status = a.status ? a.status : device_status_word();
    p.trace = g_trace;
    if (!p.status) return KAIROS_ERR_CUDA;
    static PerDeviceFlag smem_attr;    // per instantiation
    if ((rc = ensure_dynamic_smem(smem_attr, w4a16_tmem_kernel<BT>, Cfg::kSmemBytes)) != KAIROS_OK) return rc;
    const int units = pl.n_tiles * pl.m_tiles * pl.splits;
    const int sms = device_sm_count();
    const int grid = units < sms ? units : sms;
    cudaError_t e = launch_chained(w4a16_tmem_kernel<BT>, dim3(grid), dim3(Cfg::kThreads), Cfg::kSmemBytes, a.stream, tw,
                                   tx, ts, tz, p);
    if (e != cudaSuccess) return note_cuda_error(e);
    if (pl.splits > 1) {
        const int rc2 = launch_status();
        if (rc2 != KAIROS_OK) return rc2;
        e = launch_chained(splitk_reduce_kernel<false>, dim3(pl.n_tiles * pl.m_tiles * BT), dim3(kTileN), 0, a.stream, p,
                           (int)BT);
        if (e != cudaSuccess) return note_cuda_error(e);
    }
    return launch_status();
}

template <bool kInt8>
int launch_gemm_pair(const void* X, const void* W, const __half* s1, const __half* sx, const __half* bias, void* Y,
                     void* acc_dbg, int M, int N, int K, cudaStream_t stream);   // gemm2_sm100.cu

static bool pairs_enabled() {
    static const bool on = [] {
        const char* v = getenv("KAIROS_NO_PAIR");
        return !(v && v[0] == '1');
    }();
    return on;
}

template <bool kInt8, int kMode>
int launch_gemm(const GemmArgs& a) {
    if (a.M < 0 || a.N <= 0 || a.K <= 0 || (a.K % kGroup) != 0 || (a.N % kInterleave) != 0) return KAIROS_ERR_SHAPE;
    if (a.M == 0) return KAIROS_OK;
    if (!a.X || !a.W || !a.Y || ((uintptr_t)a.X & 15) || ((uintptr_t)a.W & 15) || ((uintptr_t)a.Y & 1))
        return KAIROS_ERR_ALIGN;
    if (kMode == kModeW4 && (a.N % 8) != 0) return KAIROS_ERR_SHAPE;   // factor rows must be 16-byte multiples
    if constexpr (kMode == kModeTma) {
        // large problems run on CTA pairs (256 x 256 tiles); 1 = not suitable, use the one-CTA kernel
        if (pairs_enabled()) {
            const int rc = launch_gemm_pair<kInt8>(a.X, a.W, a.s1, a.sx, a.bias, a.Y, a.acc_dbg, a.M, a.N, a.K, a.stream);
            if (rc != 1) return rc;
        }
    }
    // W4A16: up to 128 tokens the kernel that keeps the expanded operand in tensor memory (its token tiles stop
    // at 128); beyond, the shared-memory expander kernel with 256-token tiles
    const bool w4_tmem = kMode == kModeW4 && a.M <= 128;
    const Plan pl = make_plan(a.M, a.N, a.K, kInt8, a.plan_cap ? a.plan_cap : ~(size_t)0, w4_tmem, kMode == kModeTma);
    if (pl.partial_bytes > 0 && (!a.workspace || ((uintptr_t)a.workspace & 15) || a.workspace_bytes < pl.partial_bytes))
        return KAIROS_ERR_WORKSPACE;
    if constexpr (kMode == kModeW4) {
        if (w4_tmem) {
            switch (pl.bt) {
                case 32: return launch_w4_tmem<32>(a, pl);
                case 64: return launch_w4_tmem<64>(a, pl);
                default: return launch_w4_tmem<128>(a, pl);
            }
        }
    }
    switch (pl.bt) {
        case 16: return launch_one<kInt8, kMode, 16>(a, pl);
        case 32: return launch_one<kInt8, kMode, 32>(a, pl);
        case 64: return launch_one<kInt8, kMode, 64>(a, pl);
        case 128: return launch_one<kInt8, kMode, 128>(a, pl);
        default: return launch_one<kInt8, kMode, 256>(a, pl);
    }
}

template int launch_gemm<true, kModeTma>(const GemmArgs&);
template int launch_gemm<false, kModeTma>(const GemmArgs&);
template int launch_gemm<false, kModeW4>(const GemmArgs&);
template int launch_gemm<false, kModeW8>(const GemmArgs&);

}  // namespace kairos

using kairos::GemmArgs;

#ifdef KAIROS_TRACE
/* Diagnostic build only: when given a device buffer of 64 x 8 int64, CTA 0 of every tensor-core GEMM launched
 * afterwards stamps clock64() per k block: [0] TMA issued, [1] MMA saw the stage, [2] MMA saw the
 * expanded operand, [3] MMA committed, [4..7] expander: saw the stage / loaded / got its slot /
 * published.  Null switches it off. */
extern "C" void kairos_debug_trace(void* device_buffer) { kairos::g_trace = static_cast<long long*>(device_buffer); }
#endif

extern "C" size_t kairos_gemm_workspace_bytes(int M, int N, int K) { return kairos::gemm_workspace_bytes(M, N, K); }

extern "C" int kairos_gemm_plan_query(int M, int N, int K, int int8, int* token_tile, int* k_runs, int* tiles) {
    if (M <= 0 || N <= 0 || K <= 0 || (K % 128) != 0 || !token_tile || !k_runs || !tiles) return KAIROS_ERR_ARG;
    const kairos::Plan pl = kairos::make_plan(M, N, K, int8 != 0, ~(size_t)0, false, true);
    *token_tile = pl.bt;
    *k_runs = pl.splits;
    *tiles = pl.n_tiles * pl.m_tiles;
    return KAIROS_OK;
}

extern "C" int kairos_w4a16_gemm(const void* X, const void* qweight, const void* scales, const void* scaled_zeros,
                                 const void* bias, void* Y, int M, int N, int K, void* workspace,
                                 size_t workspace_bytes, kairos_stream_t stream) {
    if (!scales || !scaled_zeros) return KAIROS_ERR_ALIGN;
    GemmArgs a{X, qweight, static_cast<const __half*>(scales), static_cast<const __half*>(scaled_zeros), nullptr,
               nullptr, static_cast<const __half*>(bias), Y, nullptr, M, N, K, workspace, workspace_bytes,
               reinterpret_cast<cudaStream_t>(stream)};
    return kairos::launch_gemm<false, kairos::kModeW4>(a);
}

extern "C" int kairos_w8a16_gemm(const void* X, const void* W8, const void* scales_1, const void* bias, void* Y, int M,
                                 int N, int K, void* workspace, size_t workspace_bytes, kairos_stream_t stream) {
    if (!scales_1) return KAIROS_ERR_ALIGN;
    GemmArgs a{X, W8, nullptr, nullptr, static_cast<const __half*>(scales_1), nullptr,
               static_cast<const __half*>(bias), Y, nullptr, M, N, K, workspace, workspace_bytes,
               reinterpret_cast<cudaStream_t>(stream)};
    return kairos::launch_gemm<false, kairos::kModeW8>(a);
}

extern "C" int kairos_w8a8_gemm(const void* Xq, const void* W8, const void* scales_1, const void* sx, const void* bias,
                                void* Y, void* acc_i32, int M, int N, int K, void* workspace, size_t workspace_bytes,
                                kairos_stream_t stream) {
    if (!scales_1 || !sx) return KAIROS_ERR_ALIGN;
    GemmArgs a{Xq, W8, nullptr, nullptr, static_cast<const __half*>(scales_1), static_cast<const __half*>(sx),
               static_cast<const __half*>(bias), Y, acc_i32, M, N, K, workspace, workspace_bytes,
               reinterpret_cast<cudaStream_t>(stream)};
    return kairos::launch_gemm<true, kairos::kModeTma>(a);
}

extern "C" int kairos_f16_gemm(const void* X, const void* W16, const void* bias, void* Y, int M, int N, int K,
                               void* workspace, size_t workspace_bytes, kairos_stream_t stream) {
    GemmArgs a{X, W16, nullptr, nullptr, nullptr, nullptr, static_cast<const __half*>(bias), Y, nullptr, M, N, K,
               workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream)};
    return kairos::launch_gemm<false, kairos::kModeTma>(a);
}

// ---------------------------------------------------------------------------------
// Allocation-free variant of the W4A16 tensor-core GEMM.
//
// Some hosts of this library may not allocate device memory at call time at all: an inference
// server that hands the whole GPU to its own arena at start-up and forbids later cudaMalloc, or a
// real-time loop whose latency budget has no room for an allocator call.  For those callers the
// split-K scratch of the GEMM lives in a fixed array inside the library image instead of a caller- or
// context-owned buffer.  The first call on a device resolves the array's address and sets kernel
// attributes; make it outside any stream capture.
//
// The array is device memory that every GPU which loads the library keeps until the process ends.
// Its name is only meaningful to device code; the host asks the runtime for its device address once
// per device (with that device current) and hands that address to the kernels like any workspace.
// ---------------------------------------------------------------------------------
#define KAIROS_NOALLOC_SCRATCH_BYTES (5u << 20)

static __device__ __align__(256) unsigned char g_noalloc_scratch[KAIROS_NOALLOC_SCRATCH_BYTES];
static __device__ int g_noalloc_status;   // raised by a bounded wait that ran out (starts at zero)

namespace kairos {
struct NoAllocSlot {
    void* scratch = nullptr;
    int* status = nullptr;
};
static NoAllocSlot g_noalloc_slots[64];
static std::mutex g_noalloc_mu;

// Device address of the built-in scratch on the CURRENT device, resolved on first use.
static int noalloc_slot(NoAllocSlot* out) {
    int dev = 0;
    KAIROS_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return KAIROS_ERR_ARG;
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    NoAllocSlot& slot = g_noalloc_slots[dev];
    if (!slot.scratch) {
        void* scratch = nullptr;
        void* status = nullptr;
        KAIROS_CUDA_OK(cudaGetSymbolAddress(&scratch, g_noalloc_scratch));
        KAIROS_CUDA_OK(cudaGetSymbolAddress(&status, g_noalloc_status));
        slot.status = static_cast<int*>(status);
        slot.scratch = scratch;
    }
    *out = slot;
    return KAIROS_OK;
}

// Status word of the allocation-free entry on the current device: KAIROS_ERR_DEVICE after one of its
// launches gave up on a bounded wait, else 0 (also when the entry was never used on this device).
// Plain copies from and to the symbol's address: nothing is allocated.  Synchronises the device.
int noalloc_status(int clear) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return KAIROS_OK;
    int* word = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_noalloc_mu);
        word = g_noalloc_slots[dev].status;
    }
    if (!word) return KAIROS_OK;
    int v = 0;
    KAIROS_CUDA_OK(cudaMemcpy(&v, word, sizeof(int), cudaMemcpyDeviceToHost));
    if (clear && v != 0) {
        const int zero = 0;
        KAIROS_CUDA_OK(cudaMemcpy(word, &zero, sizeof(int), cudaMemcpyHostToDevice));
    }
    return v;
}
}  // namespace kairos

extern "C" int kairos_w4a16_gemm_noalloc(const void* X, const void* qweight, const void* scales,
                                         const void* scaled_zeros, const void* bias, void* Y, int M, int N, int K,
                                         kairos_stream_t stream) {
    using namespace kairos;
    if (!scales || !scaled_zeros) return KAIROS_ERR_ALIGN;
    if (M < 0 || N <= 0 || K <= 0 || (K % kGroup) != 0 || (N % 8) != 0) return KAIROS_ERR_SHAPE;
    if (M == 0) return KAIROS_OK;
    // The plan of the regular entry point when its scratch fits the built-in array; for M <= 64 otherwise a
    // plan with fewer K runs that does fit; larger problems are rejected.
    size_t need = make_plan(M, N, K, false, ~(size_t)0, M <= 128).partial_bytes;
    if (need > KAIROS_NOALLOC_SCRATCH_BYTES && M <= 64)
        need = make_plan(M, N, K, false, KAIROS_NOALLOC_SCRATCH_BYTES, true).partial_bytes;
    if (need > KAIROS_NOALLOC_SCRATCH_BYTES) {
        set_last_error("kairos_w4a16_gemm_noalloc: this (M, N, K) needs more split-K scratch than the 5 MiB built "
                       "into the library; use kairos_w4a16_gemm with a caller-owned workspace");
        return KAIROS_ERR_WORKSPACE;
    }
    NoAllocSlot slot;
    const int rc = noalloc_slot(&slot);
    if (rc != KAIROS_OK) return rc;
    GemmArgs a{X, qweight, static_cast<const __half*>(scales), static_cast<const __half*>(scaled_zeros), nullptr,
               nullptr, static_cast<const __half*>(bias), Y, nullptr, M, N, K, slot.scratch,
               (size_t)KAIROS_NOALLOC_SCRATCH_BYTES, reinterpret_cast<cudaStream_t>(stream), slot.status,
               (size_t)KAIROS_NOALLOC_SCRATCH_BYTES};
    return launch_gemm<false, kModeW4>(a);
}
