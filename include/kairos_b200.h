/* C ABI of the B200 switched quantized-linear library (libkairos_b200.so).
 *
 * Every entry point replaces one native function of xiezx23/Kairos's hot path;
 * the reference file:line is cited beside each declaration.  Conventions:
 *   - all tensor pointers are DEVICE pointers owned by the caller, 16-byte aligned,
 *     dense row-major; the library never frees them;
 *   - work is enqueued on `stream` and is stream-ordered, no hidden synchronisation;
 *   - return value 0 = success, negative = KAIROS_ERR_* (nothing throws, nothing
 *     traps on the device); kairos_status_str() explains a code, and
 *     kairos_last_error() returns the detail message of the last failure on the
 *     calling thread;
 *   - the resident weight format is the reference's: `qweight` int16 [N/4, K]
 *     (AWQ 4-row interleave, 8 nibbles per 32-bit word), factor tensors fp16
 *     group-major [G_pad, N] with G_pad = ceil(K/128/8)*8, `scaled_zero = -(scale*zero)`;
 *   - shape rules: N % 4 == 0, K % 128 == 0, M >= 0 (M == 0 is a no-op).
 */
#ifndef KAIROS_B200_H
#define KAIROS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* kairos_stream_t; /* == cudaStream_t */

enum {
    KAIROS_OK = 0,
    KAIROS_ERR_SHAPE = -1,     /* dimension rule violated */
    KAIROS_ERR_ALIGN = -2,     /* pointer not 16-byte aligned / null */
    KAIROS_ERR_CUDA = -3,      /* a CUDA runtime/driver call failed */
    KAIROS_ERR_WORKSPACE = -4, /* caller-provided or reserved workspace too small */
    KAIROS_ERR_CACHE = -5,     /* conversion cache cannot hold the converted weight */
    KAIROS_ERR_COMP = -6,      /* unknown / unsupported kernel id */
    KAIROS_ERR_DEVICE = -7,    /* a kernel reported a bounded wait that ran out */
    KAIROS_ERR_ARG = -8        /* bad handle or argument */
};

/* kernel ids: COMP_TYPE_NAME of kairos/dynamic_linear.py:8-9 */
enum {
    KAIROS_COMP_W4A16_GEMM = 0,
    KAIROS_COMP_W4A16_GEMV = 1,
    KAIROS_COMP_W8A8 = 2,
    KAIROS_COMP_W8A16_GEMM = 3,
    KAIROS_COMP_FP16 = 5
};

int kairos_abi_version(void);
const char* kairos_status_str(int status);
const char* kairos_last_error(void);
/* Status words the kernels raise when one of their bounded waits runs out (current device), including the
 * word of kairos_w4a16_gemm_noalloc.  Read it after synchronising (the call itself synchronises the device
 * once that entry has been used); clear != 0 resets it.  KAIROS_OK or KAIROS_ERR_DEVICE. */
int kairos_device_status(int clear);
/* Self-test of that mechanism (no counterpart in the reference): launches one CTA that waits, through the
 * routine all pipeline kernels use, on a barrier nothing completes; the wait gives up after about a
 * millisecond, raises the status word and the kernel returns.  After synchronising,
 * kairos_device_status() reports KAIROS_ERR_DEVICE and the device remains usable. */
int kairos_selftest_bounded_wait(kairos_stream_t stream);

/* ---- arithmetic rule of the three bit-exact stages ----------------------------------------
 * The reference states activation quantization and the two weight conversions twice, and the two
 * statements round differently:
 *   KAIROS_ARITH_TORCH (default)  its torch functions (kairos/quantization.py:111-141,
 *       thirdparty/AWQ/awq_method.py:105-116): scale = amax/127 and x/scale by IEEE division,
 *       fp16(fp16(q*s) + sz) with two roundings;
 *   KAIROS_ARITH_REFERENCE_CUDA   its CUDA kernels as nvcc --use_fast_math builds them
 *       (kernels/setup.py:22): sx = fp16(amax / 127) and Xq = cvt.rni.sat.s8(x * (127 / amax)) with
 *       approximate division and no clamp of amax (quant/quant_f16_to_i8.cu:54-77), and
 *       fp16(q*s + sz) as ONE fused multiply-add (dequant_awq_format/dequant_i4_to_f16.cu:17-35,
 *       dequant_i4_to_i8.cu:14-35,143-146).  Under this rule the three stages, and with them the
 *       whole W8A8 path, return the bits the reference's own extension returns on the same GPU.
 * The rule is process-wide, is read when a kernel is launched, and is part of the conversion cache's key.
 * kairos_set_arithmetic returns the previous rule, or KAIROS_ERR_ARG.  The environment variable
 * KAIROS_ARITHMETIC=reference_cuda selects the second rule at load time. */
enum { KAIROS_ARITH_TORCH = 0, KAIROS_ARITH_REFERENCE_CUDA = 1 };
int kairos_set_arithmetic(int rule);
int kairos_get_arithmetic(void);

/* ---- primitive kernels -------------------------------------------------- */

/* Per-token symmetric int8 activation quantization: amax over K in fp32,
 * scale = max(amax,1e-7)/127 (IEEE division), Xq = rint(x/scale), sx = fp16(scale).
 * Replaces quant_fp16_to_int8 (kernels/csrc/kairos_kernel/quant/quant_f16_to_i8.cu:88-103)
 * with the arithmetic of its torch twin quantize_tensor_int8 (kairos/quantization.py:111-141), or, under
 * KAIROS_ARITH_REFERENCE_CUDA, with the arithmetic of that kernel itself. */
int kairos_act_quant_i8(const void* X_f16, void* Xq_i8, void* sx_f16, int M, int K, kairos_stream_t stream);

/* uint4 base -> row-major int8 [N,K]: trunc(fp16(fp16(q*s)+sz)) with the *_to8 factors.
 * Replaces dequant_interleaved_int4_to_int8
 * (kernels/csrc/kairos_kernel/dequant_awq_format/dequant_i4_to_i8.cu:151-181). */
int kairos_w4_to_w8(const void* qweight, const void* scales_to8, const void* scaled_zeros_to8, void* W8, int N,
                    int K, kairos_stream_t stream);

/* uint4 base -> row-major fp16 [N,K]: fp16(fp16(q*s)+sz).
 * Replaces dequant_interleaved_int4_to_fp16
 * (kernels/csrc/kairos_kernel/dequant_awq_format/dequant_i4_to_f16.cu:156-186). */
int kairos_w4_to_f16(const void* qweight, const void* scales, const void* scaled_zeros, void* W16, int N, int K,
                     kairos_stream_t stream);

/* AWQ interleaved int16 [N/4,K] -> QServe W4A8 byte layout int8 [N,K/2] (N % 32 == 0, K % 64 == 0).
 * Replaces trans_layout_c16_to_c8_awq
 * (kernels/csrc/kairos_kernel/trans_layout/trans_layout_marlin_c16_to_c8.cu:113-204). */
int kairos_awq_to_qserve(const void* qweight, void* out_i8, int N, int K, kairos_stream_t stream);

/* Y[M,N] = X[M,K] . dequant(W)^T (+bias), CUDA-core weight-streaming kernel, 1 <= M <= 32; eight tokens
 * share one pass over the weight, so M > 8 reads it ceil(M/8) times: it is the fallback for N % 8 == 4.
 * Replaces gemv_forward_cuda_new
 * (thirdparty/AWQ/kernels/csrc/quantization_new/gemv/gemv_cuda.cu:245-463). */
int kairos_w4a16_gemv(const void* X_f16, const void* qweight, const void* scales, const void* scaled_zeros,
                      const void* bias_f16_or_null, void* Y_f16, int M, int N, int K, kairos_stream_t stream);

/* Same product for 1 <= M <= 32 (N % 8 == 0) on warp-level tensor-core instructions: the packed weight is
 * read once, by many small CTAs whose K slices meet through distributed shared memory (no scratch, one
 * launch); the uint4 values go straight into the MMA and the per-group factors are applied to the
 * accumulators.  Same reference counterpart (gemv_cuda.cu:245-463, template cases Batch = 1..16; the
 * reference runs batch 17..32 through the same template). */
int kairos_w4a16_decode(const void* X_f16, const void* qweight, const void* scales, const void* scaled_zeros,
                        const void* bias_f16_or_null, void* Y_f16, int M, int N, int K, kairos_stream_t stream);
/* The same kernel with the epilogue of a gated MLP (no counterpart in the reference, whose model code leaves
 * SiLU(gate) * up to torch): the N = 2 I weight rows are the gate and up projections stacked in the BLOCKED order
 * (16 gate rows, their 16 up rows, the next 16 gate rows, ...; N % 32 == 0), so a row tile of the kernel holds
 * matching rows, and Y_act [M, I] = half(half(silu(gate)) * up) is written instead of the [M, 2 I] activation:
 * bit-identical to kairos_w4a16_decode followed by kairos_silu_mul_blocked, one kernel and one round trip less. */
int kairos_w4a16_decode_silu(const void* X_f16, const void* qweight, const void* scales, const void* scaled_zeros,
                             const void* bias_or_null, void* Y_act_f16, int M, int N, int K, kairos_stream_t stream);

/* Kernel id 1 as the switched linear runs it: the decode kernel when N % 8 == 0, else the CUDA-core
 * kernel; 1 <= M <= 32.  This is the drop-in for gemv_forward_cuda_new. */
int kairos_w4a16_small_batch(const void* X_f16, const void* qweight, const void* scales, const void* scaled_zeros,
                             const void* bias_f16_or_null, void* Y_f16, int M, int N, int K, kairos_stream_t stream);

/* Bytes of scratch the tensor-core GEMMs need for (M,N,K): the split-K partial tiles (0 when
 * the problem is not split; then `workspace` may be null).  Contents need no initialisation.
 * Calls that share a workspace must be ordered (same stream). */
size_t kairos_gemm_workspace_bytes(int M, int N, int K);
/* Diagnostic: the tiling the one-CTA tensor-core GEMM would use for W8A8 (int8 != 0) or FP16 operands of this
 * shape on the current device: tokens per tile (16..256; weight rows per tile are always 128), the number of K
 * runs a tile is split into (1 = no split-K scratch needed) and the number of output tiles.  Nothing is launched. */
int kairos_gemm_plan_query(int M, int N, int K, int int8, int* token_tile, int* k_runs, int* tiles);

/* Y = X . dequant(W)^T (+bias): tcgen05 f16 MMA, uint4 dequantized in shared memory (N % 8 == 0).
 * Replaces gemm_forward_cuda_new
 * (thirdparty/AWQ/kernels/csrc/quantization_new/gemm/gemm_cuda.cu:1126-1236). */
int kairos_w4a16_gemm(const void* X_f16, const void* qweight, const void* scales, const void* scaled_zeros,
                      const void* bias_f16_or_null, void* Y_f16, int M, int N, int K, void* workspace,
                      size_t workspace_bytes, kairos_stream_t stream);

/* The same W4A16 GEMM for callers that must not allocate device memory (no counterpart in the
 * reference): the split-K scratch is a 5 MiB array built into the library image, so there is no
 * workspace argument and the call runs no cudaMalloc/cudaFree of any kind.  Limits and rules:
 *   - (M, N, K) whose split-K scratch exceeds 5 MiB are rejected with KAIROS_ERR_WORKSPACE
 *     (every M <= 64 fits; larger M fits when kairos_gemm_workspace_bytes(M,N,K) <= 5 MiB);
 *   - the first call on a device resolves the array's device address and sets kernel attributes;
 *     make that first call outside any stream capture;
 *   - all calls on a device share the one array: calls that may overlap on the GPU (different
 *     streams without ordering) race on it.  Nothing in it has to start at zero: every partial
 *     tile is written in full before it is read. */
int kairos_w4a16_gemm_noalloc(const void* X_f16, const void* qweight, const void* scales,
                              const void* scaled_zeros, const void* bias_f16_or_null, void* Y_f16, int M, int N,
                              int K, kairos_stream_t stream);

/* Y = X . (fp16(W8)*s1)^T (+bias): tcgen05 f16 MMA, int8 weight widened in shared memory.
 * Kernel id 3 of kairos/dynamic_linear.py:8-9 (declared there, no kernel in the reference). */
int kairos_w8a16_gemm(const void* X_f16, const void* W8, const void* scales_1, const void* bias_f16_or_null,
                      void* Y_f16, int M, int N, int K, void* workspace, size_t workspace_bytes,
                      kairos_stream_t stream);

/* Y = half(float(Xq.W8^T) * (s1[n]*sx[m])) (+bias): tcgen05 kind::i8, int32 accumulators in TMEM.
 * acc_i32_or_null, when given, receives the raw int32 accumulators [M,N].
 * Replaces w8a8_gemm_forward_cuda (thirdparty/AWQ/kernels/csrc/w8a8/w8a8_gemm_cuda.cu:909-955). */
int kairos_w8a8_gemm(const void* Xq_i8, const void* W8, const void* scales_1, const void* sx_f16,
                     const void* bias_f16_or_null, void* Y_f16, void* acc_i32_or_null, int M, int N, int K,
                     void* workspace, size_t workspace_bytes, kairos_stream_t stream);

/* Y = X . W16^T (+bias), fp32 accumulation.  Replaces the cuBLAS call `input @ tmp_weight.T`
 * (kairos/dynamic_linear.py:163). */
int kairos_f16_gemm(const void* X_f16, const void* W16, const void* bias_f16_or_null, void* Y_f16, int M, int N,
                    int K, void* workspace, size_t workspace_bytes, kairos_stream_t stream);

/* ---- element-wise operators around the linears of a decoder layer (one pass each) ----------------
 * These operators, the decode-side kernel, the activation quantization and the single-CTA GEMM are launched
 * with programmatic stream serialization: each may become resident while the kernel before it in the stream
 * drains, sets up (and, in the decode-side kernel, starts streaming the packed weights -- which must
 * therefore not be written by the kernel directly before it) and only then waits for that kernel's
 * results.  KAIROS_NO_PDL=1 in the environment restores ordinary launches.
 * Counterparts the reference vendors but never calls: rms_norm_general
 * (thirdparty/AWQ/kernels/csrc/w8a8/layernorm.cu:56-231) and silu_and_mul
 * (thirdparty/AWQ/kernels/csrc/w8a8/act.cu:34-140); in its runs these steps are HuggingFace torch code. */
/* Y[m,:] = half(float(X[m,:]) * rsqrt(mean(X[m,:]^2) + eps) * float(W)); K % 8 == 0, K <= 16384 */
int kairos_rms_norm(const void* X_f16, const void* W_f16, void* Y_f16, int M, int K, float eps,
                    kairos_stream_t stream);
/* The residual addition of the layer before, carried by the norm that follows it: X <- half(X + H) in place,
 * then Y = rms_norm(X).  One pass instead of an element-wise add plus a norm. */
int kairos_add_rms_norm(void* X_f16_inout, const void* H_f16, const void* W_f16, void* Y_f16, int M, int K, float eps,
                        kairos_stream_t stream);
/* Y[m,i] = silu(GU[m,i]) * GU[m,I+i] for the fused gate|up activation GU [M, 2I]; I % 8 == 0 */
int kairos_silu_mul(const void* GU_f16, void* Y_f16, int M, int I, kairos_stream_t stream);
/* kairos_silu_mul / kairos_silu_mul_quant for a [M, 2 I] activation in the blocked order (gate of inner channel i at
 * column 32 (i / 16) + i % 16, up 16 columns further; I % 16 == 0): what a gate|up linear with blocked weight rows
 * produces when it does not run the fused decode kernel. */
int kairos_silu_mul_blocked(const void* GU_f16, void* Y_f16, int M, int I, kairos_stream_t stream);
int kairos_silu_mul_quant_blocked(const void* GU_f16, void* Y_or_null, void* Xq_i8, void* sx_f16, int M, int I,
                                  kairos_stream_t stream);
/* The same two operators emitting the precision a following W8A8 linear consumes: per-token int8 Xq + fp16
 * scale sx, bit-identical to kairos_act_quant_i8 applied to the fp16 result; the fp16 tensor itself is
 * written only when Y is given.  With H given, X <- X + H first (as in kairos_add_rms_norm).
 * K % 16 == 0, K <= 16384; I % 16 == 0, I <= 32768. */
int kairos_rms_norm_quant(void* X_f16, const void* H_f16_or_null, const void* W_f16, void* Y_f16_or_null, void* Xq_i8,
                          void* sx_f16, int M, int K, float eps, kairos_stream_t stream);
int kairos_silu_mul_quant(const void* GU_f16, void* Y_f16_or_null, void* Xq_i8, void* sx_f16, int M, int I,
                          kairos_stream_t stream);

/* Rotary embedding (rotate-half) of the q and k heads of a fused QKV activation [B*S, (H+2Hkv)*D] plus the
 * KV-cache write: Q_out [B,H,S,D], caches [B,Hkv,max_len,D]; token (b,s) is at position pos0 + s where
 * pos0 = *pos_dev (int64 in device memory, for graph-replayed decode steps) or the host value. */
int kairos_rope_kv(const void* QKV_f16, const void* cos_table, const void* sin_table, const void* pos_dev_or_null,
                   int pos0, void* Q_out, void* K_cache, void* V_cache, int B, int S, int H, int Hkv, int D,
                   int max_len, kairos_stream_t stream);

/* ---- interval LUT: M -> kernel id  (kernels/csrc/kairos_kernel/lut/lut.h:8-43) ---- */
typedef struct kairos_lut kairos_lut;
kairos_lut* kairos_lut_create(void);
void kairos_lut_destroy(kairos_lut* t);
int kairos_lut_record(kairos_lut* t, int r, int comp_type); /* lut.h:35-38 */
int kairos_lut_get(kairos_lut* t, int m);                   /* lut.h:22-33; KAIROS_ERR_ARG when empty */
void kairos_lut_shrink_to_fit(kairos_lut* t);               /* lut.h:40-43 */
int kairos_lut_size(const kairos_lut* t);

/* ---- tensor parallelism: all-reduce of small row-parallel outputs over peer memory ----------
 * No counterpart in the reference (single GPU, kairos/main.py:19-23).  Sums, over the `world` ranks of a
 * tensor-parallel group, fp16 vectors of n elements (n % 8 == 0) that each rank holds in memory its peers
 * can address (an NVLink peer mapping made by the host, e.g. CUDA IPC or virtual-memory handles):
 * out[i] = fp16(sum over r = 0..world-1, in rank order, of float(peer_in[r][i])), identical on every rank.
 * peer_in[r] / peer_signal[r] are HOST arrays of `world` device pointers: rank r's partial and rank r's
 * signal pad as mapped in THIS process.  A signal pad is kairos_peer_allreduce_signal_bytes() bytes, zeroed
 * once before first use (on every rank, before any rank's first call).  Every rank must issue the same
 * sequence of calls, one process per GPU, and consecutive calls must alternate between two partial buffers
 * (a call's barrier proves the peers have finished reading the buffer of the call before the previous one).
 * Meant for up to ~1 MB; every rank reads every partial.  The wait for the peers is bounded (about a
 * second): on a timeout the kernel raises the device status word (kairos_device_status) and returns without
 * writing `out`.  Plain peer loads and stores only: no multicast, no TMA, no library kernel on peer memory. */
int kairos_peer_allreduce_signal_bytes(void);
int kairos_peer_allreduce_f16(const void* const* peer_in, void* const* peer_signal, int world, int rank, void* out,
                              long long n, kairos_stream_t stream);
/* The same sum folded into its consumer: kairos_add_rms_norm / kairos_rms_norm_quant whose pending delta is the
 * output [M, K] of a row-parallel linear still spread over the group (M <= 128 tokens, one signal slot per
 * token).  X += fp16(sum of the partials in rank order) in place, then the norm: the bits of
 * kairos_peer_allreduce_f16 followed by kairos_add_rms_norm / kairos_rms_norm_quant, without the kernel and the
 * round trip in between.  Counts as one call in the sequence every rank must issue alike. */
int kairos_add_rms_norm_peer(void* X, const void* const* peer_in, void* const* peer_signal, int world, int rank,
                             const void* W, void* Y, int M, int K, float eps, kairos_stream_t stream);
int kairos_rms_norm_quant_peer(void* X, const void* const* peer_in, void* const* peer_signal, int world, int rank,
                               const void* W, void* Y_or_null, void* Xq, void* sx, int M, int K, float eps,
                               kairos_stream_t stream);

/* ---- context: bounded conversion cache + workspaces (one per device) -------------
 * The reference converts the whole weight on every call into a fresh torch.empty
 * (kairos/dynamic_linear.py:145-147,159-161); the context keeps converted weights in
 * an LRU cache of at most `cache_bytes` (0 = convert into a single reusable slot on
 * every call, i.e. the reference's behaviour; SIZE_MAX = keep everything, which is
 * the all-formats-resident SwitchLinear of kairos/switch_linear.py:127-131). */
typedef struct kairos_ctx kairos_ctx;
kairos_ctx* kairos_ctx_create(size_t cache_bytes);
void kairos_ctx_destroy(kairos_ctx* ctx);
/* Pre-size the activation / split-K workspaces for calls up to (max_M, max_N, max_K);
 * without it they grow on demand (a growth synchronises the device once). */
int kairos_ctx_reserve(kairos_ctx* ctx, int max_M, int max_N, int max_K);
/* cache statistics: hits, misses (= conversions run), evictions, bytes in use */
int kairos_ctx_stats(const kairos_ctx* ctx, uint64_t* hits, uint64_t* misses, uint64_t* evictions,
                     uint64_t* bytes_in_use);
void kairos_ctx_clear_cache(kairos_ctx* ctx);

/* ---- one switched linear layer -------------------------------------------- */
typedef struct kairos_layer kairos_layer;
/* Registers the resident tensors of one layer (DynamicLinear.from_module output,
 * kairos/dynamic_linear.py:85-115).  Pointers must stay valid for the layer's life. */
kairos_layer* kairos_layer_create(kairos_ctx* ctx, int N, int K, const void* qweight, const void* scales,
                                  const void* scaled_zeros, const void* scales_to8,
                                  const void* scaled_zeros_to8, const void* scales_1,
                                  const void* bias_f16_or_null);
void kairos_layer_destroy(kairos_layer* layer);

/* DynamicLinear._forward (kairos/dynamic_linear.py:131-172): run kernel `comp_type` on
 * X[M,K] -> Y[M,N].  Activation quantization runs only for W8A8; weight conversion only
 * for ids 2, 3, 5 and only on a cache miss. */
int kairos_switched_linear(kairos_layer* layer, const void* X_f16, void* Y_f16, int M, int comp_type,
                           kairos_stream_t stream);
/* Kernel id 2 for activations that arrive already quantized (by the operators above): conversion on a
 * cache miss, then the W8A8 GEMM; no activation pass. */
int kairos_switched_linear_q8(kairos_layer* layer, const void* Xq_i8, const void* sx_f16, void* Y_f16, int M,
                              kairos_stream_t stream);
/* Convert ahead of use (e.g. on a side stream, one layer ahead): fills the cache entry the
 * given kernel id needs and returns; a later kairos_switched_linear on any stream waits for it. */
int kairos_layer_prefetch(kairos_layer* layer, int comp_type, kairos_stream_t stream);
/* Same call with HOST buffers (pinned for the copies to be asynchronous).  X_host must hold its data when the
 * call is made: the input copy runs on a stream of the context, so that it overlaps the previous call's
 * compute and output copy, and is NOT ordered after earlier work on `stream`.  Y_host is complete once
 * `stream` is synchronized.  Not for use inside a stream capture. */
int kairos_switched_linear_host(kairos_layer* layer, const void* X_host, void* Y_host, int M, int comp_type,
                                kairos_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* KAIROS_B200_H */
