// Decode-side W4A16 for small batches (path item a9): Y[M,N] = X[M,K] . dequant(W)^T, 1 <= M <= 16.
//
// Weight streaming is the only large traffic, so the kernel is a persistent TMA pipeline around
// the packed base with the arithmetic kept off the critical path:
//   * one CTA per SM walks 32-row units of the weight over the full K.  Two producer warps bring
//     1024-k panels into a shared-memory ring with bulk tensor copies -- 16 KB of qweight, the panel's
//     activations and its (scale, scaled-zero) tiles per stage -- several stages ahead of use, so the
//     bytes in flight do not depend on registers or occupancy;
//   * consumer warps each own one of a panel's eight quantization groups (both 16-row blocks of the
//     unit, so a lane's activations are read once); for M <= 8 two sets of eight warps take alternate
//     panels.  The uint4 values go from shared memory through ONE lop3 per pair into the A
//     fragment of mma.sync.m16n8k16 as fp16 (1024 + q) -- or (1024 + 16 q) for the odd nibbles --
//     with fp32 accumulation: no subtraction, no scaling per element;
//   * the offsets are undone per group on the accumulators:  sum q x = (C_lo - 1024 X_lo)
//     + (C_hi - 1024 X_hi) / 16, where X_lo / X_hi (sums of x over the k of the even / odd nibbles)
//     come from MMAs against an all-ones A fragment; then y += s * (sum q x) + z * (X_lo + X_hi)
//     with the stored per-group fp16 factors, in fp32;
//   * the K slices of a unit (one per consumer warp) meet in shared memory at its end.
// No scratch memory, no atomics, one launch.  Every wait is bounded (status word on timeout).
// Launched with programmatic stream serialization: the weight pipeline fills while the kernel before
// this one in the stream is still draining.
//
// Algorithmic bytes per call: K*N/2 + 4*(K/128)*N + 2*M*K + 2*M*N.
#include <cuda.h>

#include "common.cuh"

namespace kairos {

int make_tmap(CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle);   // tensormap.cu
int device_sm_count();        // gemm_sm100.cu
int* device_status_word();    // api.cu

constexpr int kDecRows = 32;                 // weight rows per unit (two MMA row blocks)
constexpr int kDecPanelK = 1024;             // k per pipeline stage (eight groups)
constexpr int kDecGroups = kDecPanelK / kGroup;
constexpr int kDecSetWarps = 8;              // consumer warps per set: one per quantization group of a panel
constexpr int kDecWBytes = (kDecRows / kInterleave) * kDecPanelK * 2;   // 16 KB: [8 qweight rows][2048 B]
constexpr int kDecFBytes = kDecGroups * kDecRows * 2;                    // 512 B: [8 groups][32 rows] fp16

template <int NT>
struct DecCfg {
    static constexpr int kXRows = 8 * NT;
    static constexpr int kXBytes = kXRows * kDecPanelK * 2;              // [tokens][16 k blocks][128 B], 128B-swizzled
    static constexpr int kStageBytes = kDecWBytes + kXBytes + 2 * kDecFBytes;
    static constexpr int kStages = NT == 1 ? 5 : 3;
    // consumer sets take alternate panels: more warps per scheduler hide the unpack -> MMA -> scale chain
    static constexpr int kSets = NT == 1 ? 2 : 1;
    static constexpr int kConsumers = kSets * kDecSetWarps;
    static constexpr int kThreads = 32 * (kConsumers + 2);               // + weight and activation producers
    static constexpr int kRedFloats = kConsumers * kDecRows * 8 * NT;    // per-warp partials of one unit
    static constexpr int kSmemBytes = kStages * kStageBytes + 2 * kRedFloats * 4 + 8 * (2 * kStages + 2) + 64 + 1024;
    static_assert(kSmemBytes <= 227 * 1024, "exceeds the shared memory a CTA may use");
    static_assert(kStageBytes % 1024 == 0, "stages must keep the swizzle alignment");
};

struct DecParams {
    const __half* bias;
    __half* Y;
    int M, N, K;
    int units;      // 32-row units
    int panels;     // 1024-k panels per unit
    int* status;
    int x_bytes;    // bytes one activation copy brings: token rows of the box x 2048
};

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
__global__ void __launch_bounds__(DecCfg<NT>::kThreads, 1)
    decode_mma_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                      const __grid_constant__ CUtensorMap tmap_s, const __grid_constant__ CUtensorMap tmap_z,
                      const DecParams p) {
    using Cfg = DecCfg<NT>;
    constexpr int kStages = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* stage_base = smem;
    float* red = reinterpret_cast<float*>(smem + kStages * Cfg::kStageBytes);
    uint64_t* full = reinterpret_cast<uint64_t*>(red + 2 * Cfg::kRedFloats);
    uint64_t* empty = full + kStages;
    uint64_t* unit_bar = empty + kStages;          // [2]: the partial sums of a unit are in `red`
    volatile int* abort_flag = reinterpret_cast<volatile int*>(unit_bar + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 2);                       // the two producers
            mbar_init(&empty[s], kDecSetWarps);            // the set that consumed the panel
        }
        mbar_init(&unit_bar[0], Cfg::kConsumers);
        mbar_init(&unit_bar[1], Cfg::kConsumers);
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmap_w);
        tma_prefetch_desc(&tmap_x);
        tma_prefetch_desc(&tmap_s);
        tma_prefetch_desc(&tmap_z);
    }
    __syncthreads();
    // The kernel after this one may set up now.  This kernel itself streams the packed weights and
    // their factors (constant inputs) straight away; only the activation producer waits for the
    // kernel before it, and every output is ordered after the activations it is computed from.
    chain_release();

    if (warp == Cfg::kConsumers) {
        // ---------------- producer: packed weights + scales ----------------
        if (lane == 0) {
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < p.units && ok; unit += gridDim.x) {
                for (int pn = 0; pn < p.panels; ++pn) {
                    if (!mbar_wait(&empty[s], phase ^ 1, abort_flag)) { ok = false; break; }
                    uint8_t* st = stage_base + s * Cfg::kStageBytes;
                    mbar_arrive_expect_tx(&full[s], kDecWBytes + kDecFBytes);
                    // qweight as 64-bit elements [N/4, K/4]: 8 rows of 256 elements (1024 k): eight 2 KB lines
                    tma_load_2d(st, &tmap_w, &full[s], pn * 256, unit * (kDecRows / kInterleave));
                    tma_load_2d(st + kDecWBytes + Cfg::kXBytes, &tmap_s, &full[s], unit * kDecRows, pn * kDecGroups);
                    if (++s == kStages) { s = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == Cfg::kConsumers + 1) {
        // ---------------- producer: activations + scaled zeros ----------------
        if (lane == 0) {
            chain_wait();
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < p.units && ok; unit += gridDim.x) {
                for (int pn = 0; pn < p.panels; ++pn) {
                    if (!mbar_wait(&empty[s], phase ^ 1, abort_flag)) { ok = false; break; }
                    uint8_t* st = stage_base + s * Cfg::kStageBytes;
                    mbar_arrive_expect_tx(&full[s], p.x_bytes + kDecFBytes);
                    // X as [M][K/64][64 halves]: 16 lines of 128 bytes for every token row of the box
                    tma_load_3d(st + kDecWBytes, &tmap_x, &full[s], 0, pn * (kDecPanelK / 64), 0);
                    tma_load_2d(st + kDecWBytes + Cfg::kXBytes + kDecFBytes, &tmap_z, &full[s], unit * kDecRows,
                                pn * kDecGroups);
                    if (++s == kStages) { s = 0; phase ^= 1; }
                }
            }
        }
    } else {
        // ---------------- consumers ----------------
        // warp w owns quantization group w % 8 of the panels of its set, for both 16-row blocks of the unit
        const int g = lane >> 2, t = lane & 3;
        const int grp = warp % kDecSetWarps;
        const int set = warp / kDecSetWarps;
        const uint32_t ones = 0x3c003c00u;           // half2(1, 1)
        // packed chunk of (row r, this group): qweight row r >> 2 (2048 bytes per panel), k block
        // k0 = 2 grp + (t >> 1), 16-byte unit 2 (r & 3) + (t & 1) of its 128-byte line
        const int k0 = 2 * grp + (t >> 1);
        uint32_t w_off[2][2];
#pragma unroll
        for (int rb = 0; rb < 2; ++rb)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int r = 16 * rb + g + 8 * h;
                w_off[rb][h] = (uint32_t)((r >> 2) * (kDecPanelK * 2) + k0 * 128 + ((2 * (r & 3) + (t & 1)) << 4));
            }
        // activations of token g (+ 8 nt): the half (t & 1) of the 128-byte line of k block k0; the 16-byte
        // units of a line are XOR-swizzled by k0 & 7 (128-byte swizzle of the tensor map)
        uint32_t x_off[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int b = 0; b < 4; ++b)
                x_off[nt][b] = (uint32_t)(kDecWBytes + (g + 8 * nt) * (kDecPanelK * 2) + k0 * 128 +
                                          (((4 * (t & 1) + b) ^ (k0 & 7)) << 4));
        int s = 0, it = 0;
        uint32_t phase = 0, panel_no = 0;
        bool ok = true;
        for (int unit = blockIdx.x; unit < p.units && ok; unit += gridDim.x, ++it) {
            float acc[2][NT][4];
#pragma unroll
            for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[rb][nt][i] = 0.f;

            for (int pn = 0; pn < p.panels && ok; ++pn) {
                // every warp observes every stage fill in order (a parity wait is only valid one phase
                // away from the barrier); the other set's panels are skipped after the wait
                if (!mbar_wait(&full[s], phase, abort_flag)) { ok = false; break; }
                const uint8_t* st = stage_base + s * Cfg::kStageBytes;
                const int s_now = s;
                if (++s == kStages) { s = 0; phase ^= 1; }
                if (Cfg::kSets > 1 && ((panel_no++ % Cfg::kSets) != (uint32_t)set)) continue;
                // activations (only the lanes whose token exists touch shared memory) and their sums over
                // the k of the even / odd nibbles, by MMAs against an all-ones A fragment
                uint4 xv[NT][4];
                float x_lo[NT][4], x_hi[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const bool tok_ok = g + 8 * nt < p.M;
#pragma unroll
                    for (int b = 0; b < 4; ++b)
                        xv[nt][b] = tok_ok ? *reinterpret_cast<const uint4*>(st + x_off[nt][b]) : make_uint4(0, 0, 0, 0);
#pragma unroll
                    for (int i = 0; i < 4; ++i) x_lo[nt][i] = x_hi[nt][i] = 0.f;
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        const uint32_t* xw = reinterpret_cast<const uint32_t*>(&xv[nt][b]);
                        if (b & 1) {
                            mma_m16n8k16(x_hi[nt], ones, ones, ones, ones, xw[0], xw[1]);
                            mma_m16n8k16(x_hi[nt], ones, ones, ones, ones, xw[2], xw[3]);
                        } else {
                            mma_m16n8k16(x_lo[nt], ones, ones, ones, ones, xw[0], xw[1]);
                            mma_m16n8k16(x_lo[nt], ones, ones, ones, ones, xw[2], xw[3]);
                        }
                    }
                    // tokens 2t, 2t+1: x_sum = X_lo + X_hi and the offset 1024 (X_lo + X_hi / 16) to remove
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const float xl = x_lo[nt][j], xh = x_hi[nt][j];
                        x_lo[nt][j] = xl + xh;                        // reused as x_sum
                        x_hi[nt][j] = 1024.f * xl + 64.f * xh;        // reused as the offset
                    }
                }
                const __half* fs = reinterpret_cast<const __half*>(st + kDecWBytes + Cfg::kXBytes) + grp * kDecRows;
                const __half* fz = fs + kDecGroups * kDecRows;
#pragma unroll
                for (int rb = 0; rb < 2; ++rb) {
                    const uint4 raw0 = *reinterpret_cast<const uint4*>(st + w_off[rb][0]);
                    const uint4 raw1 = *reinterpret_cast<const uint4*>(st + w_off[rb][1]);
                    const float sc0 = __half2float(fs[16 * rb + g]), sc1 = __half2float(fs[16 * rb + g + 8]);
                    const float zc0 = __half2float(fz[16 * rb + g]), zc1 = __half2float(fz[16 * rb + g + 8]);
                    uint32_t e0[4][4], e1[4][4];          // [c][b] nibble pairs of row g / row g + 8
                    nibble_pairs(raw0.x, e0[0]); nibble_pairs(raw0.y, e0[1]);
                    nibble_pairs(raw0.z, e0[2]); nibble_pairs(raw0.w, e0[3]);
                    nibble_pairs(raw1.x, e1[0]); nibble_pairs(raw1.y, e1[1]);
                    nibble_pairs(raw1.z, e1[2]); nibble_pairs(raw1.w, e1[3]);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        float c_lo[4] = {0.f, 0.f, 0.f, 0.f}, c_hi[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int b = 0; b < 4; ++b) {
                            // k = 8b + 2c (+d): the pairs c = 0..3 of nibble b line up with the b-th 16 bytes of x
                            const uint32_t* xw = reinterpret_cast<const uint32_t*>(&xv[nt][b]);
                            if (b & 1) {
                                mma_m16n8k16(c_hi, e0[0][b], e1[0][b], e0[1][b], e1[1][b], xw[0], xw[1]);
                                mma_m16n8k16(c_hi, e0[2][b], e1[2][b], e0[3][b], e1[3][b], xw[2], xw[3]);
                            } else {
                                mma_m16n8k16(c_lo, e0[0][b], e1[0][b], e0[1][b], e1[1][b], xw[0], xw[1]);
                                mma_m16n8k16(c_lo, e0[2][b], e1[2][b], e0[3][b], e1[3][b], xw[2], xw[3]);
                            }
                        }
                        // c[0], c[1]: row g, tokens 2t, 2t+1;  c[2], c[3]: row g + 8, same tokens
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float qx = fmaf(c_hi[i], 0.0625f, c_lo[i]) - x_hi[nt][i & 1];
                            acc[rb][nt][i] = fmaf(i < 2 ? sc0 : sc1, qx, acc[rb][nt][i]);
                            acc[rb][nt][i] = fmaf(i < 2 ? zc0 : zc1, x_lo[nt][i & 1], acc[rb][nt][i]);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s_now]);
            }
            if (!ok) break;
            // ---- the K slices (one per warp) meet in shared memory ----
            float* buf = red + (it & 1) * Cfg::kRedFloats;
            float* slab = buf + warp * (kDecRows * 8 * NT);
#pragma unroll
            for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        slab[(16 * rb + g + 8 * (i >> 1)) * (8 * NT) + 8 * nt + 2 * t + (i & 1)] = acc[rb][nt][i];
            __syncwarp();
            if (lane == 0) mbar_arrive(&unit_bar[it & 1]);
            if (!mbar_wait(&unit_bar[it & 1], (it >> 1) & 1, abort_flag)) { ok = false; break; }
            // 32 rows x 8 NT tokens, one output per thread (consecutive threads -> consecutive rows)
            for (int o = threadIdx.x; o < kDecRows * 8 * NT; o += 32 * Cfg::kConsumers) {
                const int tok = o / kDecRows, r = o % kDecRows;
                const int n = unit * kDecRows + r;
                if (tok >= p.M || n >= p.N) continue;
                float v = 0.f;
#pragma unroll
                for (int sl = 0; sl < Cfg::kConsumers; ++sl) v += buf[sl * (kDecRows * 8 * NT) + r * (8 * NT) + tok];
                __half y = __float2half_rn(v);
                if (p.bias) y = __hadd(y, p.bias[n]);
                p.Y[(size_t)tok * p.N + n] = y;
            }
        }
    }
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) atomicExch(p.status, KAIROS_ERR_DEVICE);
        for (int i = 0; i < 64; ++i) __nanosleep(1000);    // let issued copies land before the CTA leaves
    }
}

template <int NT>
static int launch_decode(const void* X, const void* qweight, const void* scales, const void* scaled_zeros,
                         const void* bias, void* Y, int M, int N, int K, cudaStream_t stream) {
    using Cfg = DecCfg<NT>;
    CUtensorMap tw, tx, ts, tz;
    int rc;
    {   // qweight int16 [N/4, K] viewed as 64-bit elements [N/4, K/4]: long lines keep the copy engine efficient
        const uint64_t dims[2] = {(uint64_t)K / 4, (uint64_t)N / 4}, strides[1] = {(uint64_t)K * 2};
        const uint32_t box[2] = {256, kDecRows / kInterleave};
        if ((rc = make_tmap(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, qweight, dims, strides, box,
                            CU_TENSOR_MAP_SWIZZLE_NONE)) != KAIROS_OK) return rc;
    }
    // only the token rows that exist are copied (power of two >= M)
    int x_rows = 1;
    while (x_rows < M) x_rows *= 2;
    {   // X fp16 [M, K] viewed as [M][K/64][64]: 128-byte lines, 128-byte swizzle
        const uint64_t dims[3] = {64, (uint64_t)K / 64, (uint64_t)M}, strides[2] = {128, (uint64_t)K * 2};
        const uint32_t box[3] = {64, kDecPanelK / 64, (uint32_t)x_rows};
        if ((rc = make_tmap(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, X, dims, strides, box,
                            CU_TENSOR_MAP_SWIZZLE_128B)) != KAIROS_OK) return rc;
    }
    {   // factors fp16 [K/128, N]
        const uint64_t dims[2] = {(uint64_t)N, (uint64_t)K / kGroup}, strides[1] = {(uint64_t)N * 2};
        const uint32_t box[2] = {kDecRows, kDecGroups};
        if ((rc = make_tmap(&ts, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, scales, dims, strides, box,
                            CU_TENSOR_MAP_SWIZZLE_NONE)) != KAIROS_OK) return rc;
        if ((rc = make_tmap(&tz, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, scaled_zeros, dims, strides, box,
                            CU_TENSOR_MAP_SWIZZLE_NONE)) != KAIROS_OK) return rc;
    }
    DecParams p;
    p.bias = static_cast<const __half*>(bias);
    p.Y = static_cast<__half*>(Y);
    p.M = M; p.N = N; p.K = K;
    p.units = (N + kDecRows - 1) / kDecRows;
    p.panels = (K + kDecPanelK - 1) / kDecPanelK;
    p.status = device_status_word();
    p.x_bytes = x_rows * kDecPanelK * 2;
    if (!p.status) return KAIROS_ERR_CUDA;
    static bool attr_set = false;
    if (!attr_set) {
        KAIROS_CUDA_OK(cudaFuncSetAttribute(decode_mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            Cfg::kSmemBytes));
        attr_set = true;
    }
    const int sms = device_sm_count();
    const int grid = p.units < sms ? p.units : sms;
    const cudaError_t e = launch_chained(decode_mma_kernel<NT>, dim3(grid), dim3(Cfg::kThreads), Cfg::kSmemBytes, stream,
                                         tw, tx, ts, tz, p);
    if (e != cudaSuccess) return note_cuda_error(e);
    return launch_status();
}

}  // namespace kairos

/* Decode-side W4A16 on warp-level tensor-core instructions, 1 <= M <= 16 (N % 8 == 0). */
extern "C" int kairos_w4a16_decode(const void* X, const void* qweight, const void* scales, const void* scaled_zeros,
                                   const void* bias, void* Y, int M, int N, int K, kairos_stream_t stream) {
    using namespace kairos;
    if (M < 0 || M > 16 || N <= 0 || K <= 0 || (N % 8) != 0 || (K % kGroup) != 0) return KAIROS_ERR_SHAPE;
    if (M == 0) return KAIROS_OK;
    if (!X || !qweight || !scales || !scaled_zeros || !Y || ((uintptr_t)X & 15) || ((uintptr_t)qweight & 15) ||
        ((uintptr_t)scales & 15) || ((uintptr_t)scaled_zeros & 15) || ((uintptr_t)Y & 1))
        return KAIROS_ERR_ALIGN;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (M <= 8) return launch_decode<1>(X, qweight, scales, scaled_zeros, bias, Y, M, N, K, st);
    return launch_decode<2>(X, qweight, scales, scaled_zeros, bias, Y, M, N, K, st);
}
