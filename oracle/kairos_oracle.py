"""CPU oracle for the switched quantized-linear path (TEST INFRASTRUCTURE ONLY).

This file restates, in numpy, the torch quantize / pack / dequantize arithmetic
that xiezx23/Kairos uses for its ``DynamicLinear`` path.  It is the checker for
the CUDA kernels: only the test-suite, the smoke entry point and the CPU-baseline
leg of the benchmark may import it.  The shipped package never does.

Parity status: PINNED against outputs of the reference's own Python functions,
generated in a container that holds the reference sources and committed as
``tests/golden/*.npz`` / ``tests/golden/config0_digests.json`` (generator:
``tests/golden/make_golden.py``); the ``*_cuda`` functions, which restate the
reference's CUDA kernels where those round differently from its torch functions,
are pinned against outputs of the reference's own extension run on a B200
(``tests/golden/ref_cuda_*.npz``, generator ``tests/golden/make_golden_cuda.py``).  The reference's own tests pin only the
AWQ->QServe nibble permutation (``test/test_trans_layout.py:46-52``) and the
pack/unpack round trip (``test/depacking.py``); both are restated here too.

Every function cites the reference file:line it follows.  fp16 arithmetic is
done with numpy ``float16`` operands, which rounds once after every operation
exactly as torch's CPU half kernels do (compute in fp32, round to fp16; for two
fp16 operands the fp32 intermediate never causes a double-rounding error).
"""
from __future__ import annotations

import numpy as np

GROUP = 128          # quantization group along K            (kairos/dynamic_linear.py:88)
INTERLEAVE = 4       # rows interleaved per packed int16 row (thirdparty/AWQ/awq_method.py:5)
KSTRIDE = 64         # k-block of the interleave             (thirdparty/AWQ/awq_method.py:5)

# kernel-id enum                                   (kairos/dynamic_linear.py:8-9,
#                                                   kairos/dynamic_linear_v2.py:11-13)
COMP_TYPE_NAME = {'w4a16_gemm': 0, 'w4a16_gemv': 1, 'w8a8': 2, 'w8a16_gemm': 3,
                  'w8a16_gemv': 4, 'fp16': 5, 'w4a16_marlin': 6, 'w4a8_qserve': 7}


# --------------------------------------------------------------------------
# offline weight preparation  (kairos/dynamic_linear.py:85-115)
# --------------------------------------------------------------------------
def quantize_int8_per_row(x):
    """Symmetric per-row int8 quantization.

    Follows ``quantize_tensor_int8(x, 'S', -1)`` (kairos/quantization.py:111-141):
    fp32 maths, ``amax.clamp(min=1e-7)/127``, IEEE division, round half to even,
    scale returned as fp16.  Used both for weights (per output channel) and for
    activations (per token).
    """
    x32 = np.asarray(x).astype(np.float32).reshape(-1, np.asarray(x).shape[-1])
    amax = np.maximum(np.abs(x32).max(axis=1, keepdims=True), np.float32(1e-7))
    scale = (amax / np.float32(127)).astype(np.float32)
    q = np.rint(x32 / scale)
    return q.astype(np.int8).reshape(np.asarray(x).shape), scale.astype(np.float16)


def quantize_uint4_groups(w8, group=GROUP):
    """Asymmetric uint4 quantization of the int8 weight, one (scale, zero) per
    ``group`` consecutive K elements; the zero point is NOT rounded to an integer.

    Follows ``kairos_quantize_tensor_int4`` (kairos/dynamic_linear.py:11-37).
    Returns q4 [N,K] uint8, scale_f [N,G] fp16, zero_f [N,G] fp16.
    """
    n, k = w8.shape
    assert k % group == 0
    x = w8.astype(np.float32).reshape(-1, group)
    mx = x.max(axis=1, keepdims=True)
    mn = x.min(axis=1, keepdims=True)
    scale = (np.maximum(mx - mn, np.float32(1e-5)) / np.float32(15)).astype(np.float32)
    zero = (-(mn / scale)).astype(np.float32)
    q = np.clip(np.rint((x / scale).astype(np.float32) + zero), 0, 15)
    return (q.reshape(n, k).astype(np.uint8),
            scale.astype(np.float16).reshape(n, -1),
            zero.astype(np.float16).reshape(n, -1))


def padded_groups(k, group=GROUP):
    """Row count of the group-major factor tensors: K/group rounded up to a
    multiple of 8 (``calculate_zeros_width`` * pack_num, awq_method.py:40-54,60-64)."""
    g = k // group
    return ((g + 7) // 8) * 8


def factor_layout(scales, zeros, group=GROUP):
    """[N,G] fp16 scale / zero  ->  group-major, zero-padded [G_pad, N] fp16 pair
    (scale, scaled_zero) with ``scaled_zero = -(scale * zero)`` evaluated in fp32.

    Follows ``trans_qfactor_layout_awq(..., method='kairos')`` (awq_method.py:56-75).
    """
    n, g = scales.shape
    gp = padded_groups(g * group, group)
    qs = np.zeros((n, gp), np.float16)
    qs[:, :g] = scales.astype(np.float16)
    sz = np.zeros((n, gp), np.float16)
    sz[:, :g] = (-(qs[:, :g].astype(np.float32) * zeros.astype(np.float32))).astype(np.float16)
    return np.ascontiguousarray(qs.T), np.ascontiguousarray(sz.T)


def pack_awq(q4):
    """uint4 [N,K] -> interleaved int16 [N/4, K].

    Follows ``pack_int_awq`` (awq_method.py:3-38) in the compact form of
    ``test/test_trans_layout.py:15-22``.  Element map: with n = 4*n0 + n1 and
    k = 64*k0 + 32*a + 8*b + 2*c + d, nibble b of
    ``out[n0, 64*k0 + 16*n1 + 8*a + 2*c + d]`` holds q4[n, k].
    """
    n, k = q4.shape
    assert n % INTERLEAVE == 0 and k % KSTRIDE == 0
    p = q4.astype(np.uint16).reshape(n // 4, 4, k // 64, 2, 4, 4, 2).transpose(0, 2, 1, 3, 5, 6, 4)
    packed = p[..., 0] | (p[..., 1] << 4) | (p[..., 2] << 8) | (p[..., 3] << 12)
    return np.ascontiguousarray(packed.reshape(n // 4, k)).view(np.int16)


def unpack_awq(qweight):
    """Inverse of :func:`pack_awq` (test/depacking.py:22-38)."""
    n4, k = qweight.shape
    u = qweight.view(np.uint16)
    nib = np.stack([(u >> s) & 0xF for s in (0, 4, 8, 12)], axis=-1)
    nib = nib.reshape(n4, k // 64, 4, 2, 4, 2, 4).transpose(0, 2, 1, 3, 6, 4, 5)
    return np.ascontiguousarray(nib.reshape(n4 * 4, k)).astype(np.uint8)


def pack_qserve(q4):
    """uint4 [N,K] -> QServe W4A8 byte layout [N, K/2] (test/test_trans_layout.py:7-13)."""
    n, k = q4.shape
    p = q4.astype(np.int8).reshape(n // 32, 2, 2, 8, k // 32, 2, 4, 4).transpose(0, 4, 3, 6, 5, 2, 7, 1)
    packed = ((p[..., 1].astype(np.int16) << 4) + p[..., 0]).astype(np.int8)
    return np.ascontiguousarray(packed.reshape(n, k // 2))


def awq_to_qserve(qweight, n, k):
    """AWQ interleaved int16 [N/4,K] -> QServe int8 [N,K/2]: the permutation the
    reference's ``trans_layout_c16_to_c8_awq`` kernel performs and its only
    bit-exact test checks (test/test_trans_layout.py:24-35,46-52)."""
    return pack_qserve(unpack_awq(qweight.reshape(n // 4, k)))


def from_module(weight_f16):
    """fp16 weight [N,K] -> the resident tensor set of a ``DynamicLinear``.

    Follows ``DynamicLinear.from_module`` (kairos/dynamic_linear.py:85-115).
    """
    w16 = np.asarray(weight_f16, dtype=np.float16)
    n, k = w16.shape
    w8, s1 = quantize_int8_per_row(w16)                          # :97-99
    q4, s2, z2 = quantize_uint4_groups(w8, GROUP)                # :101-103
    scales_to8, scaled_zeros_to8 = factor_layout(s2, z2)         # :104-105
    s_f = (s2 * s1.reshape(n, 1)).astype(np.float16)             # :107 (fp16 product)
    scales, scaled_zeros = factor_layout(s_f, z2)                # :109-110
    return {
        'qweight': pack_awq(q4),                                 # :108
        'scales': scales, 'scaled_zeros': scaled_zeros,
        'scales_to8': scales_to8, 'scaled_zeros_to8': scaled_zeros_to8,
        'scales_1': s1.reshape(-1),                              # :100
        'w8_direct': w8, 'q4': q4,
    }


# --------------------------------------------------------------------------
# on-the-fly conversion  (a7, a8)
# --------------------------------------------------------------------------
def _expand_groups(f, n, k, group=GROUP):
    """[G_pad,N] group-major factor -> [N,K] (each factor repeated over its group)."""
    g = k // group
    return np.repeat(np.ascontiguousarray(f[:g].T), group, axis=1)


def dequant_w16(qweight, scales, scaled_zeros):
    """uint4 base -> fp16 weight [N,K]:  fp16(fp16(q*s) + sz).

    Follows ``dequantize_tensor_awq`` (awq_method.py:105-116: ``mul_`` then
    ``add_`` on fp16 tensors, i.e. two roundings) with the stored factors; this
    is the torch twin of ``dequant_interleaved_int4_to_fp16``
    (kernels/csrc/kairos_kernel/dequant_awq_format/dequant_i4_to_f16.cu:40-186).
    """
    q = unpack_awq(qweight)
    n, k = q.shape
    prod = (q.astype(np.float16) * _expand_groups(scales, n, k)).astype(np.float16)
    return (prod + _expand_groups(scaled_zeros, n, k)).astype(np.float16)


def dequant_w8(qweight, scales_to8, scaled_zeros_to8):
    """uint4 base -> int8 weight [N,K]: truncate-toward-zero of the fp16 value
    ``fp16(fp16(q*s2) + sz2)``.

    Arithmetic rule: product rounded, then sum rounded (torch semantics), then
    ``(int8_t)__half`` = round-toward-zero as in
    kernels/csrc/kairos_kernel/dequant_awq_format/dequant_i4_to_i8.cu:143-146.
    """
    v = dequant_w16(qweight, scales_to8, scaled_zeros_to8).astype(np.float32)
    return np.trunc(v).astype(np.int8)


# --------------------------------------------------------------------------
# the same three stages as the reference's CUDA kernels compute them
# --------------------------------------------------------------------------
def dequant_w16_cuda(qweight, scales, scaled_zeros):
    """uint4 base -> fp16 weight with ONE rounding: fp16(q*s + sz), the ``__hfma2`` of
    kernels/csrc/kairos_kernel/dequant_awq_format/dequant_i4_to_f16.cu:17-35.  q*s + sz is exact in
    fp64 (4 + 11 significant bits times 11, exponents within fp16's range), and numpy converts fp64 to
    fp16 with a single correct rounding.  Pinned by ``tests/golden/ref_cuda_*.npz``, outputs of the
    reference's own extension built for sm_100a and run on a B200."""
    q = unpack_awq(qweight)
    n, k = q.shape
    exact = (q.astype(np.float64) * _expand_groups(scales, n, k).astype(np.float64)
             + _expand_groups(scaled_zeros, n, k).astype(np.float64))
    return exact.astype(np.float16)


def dequant_w8_cuda(qweight, scales_to8, scaled_zeros_to8):
    """``(int8_t)`` (truncation toward zero) of the single-rounded fp16 value
    (dequant_awq_format/dequant_i4_to_i8.cu:14-35,143-146)."""
    return np.trunc(dequant_w16_cuda(qweight, scales_to8, scaled_zeros_to8).astype(np.float32)).astype(np.int8)


def act_quant_cuda(x_f16):
    """Activation quantization as quant_kernel computes it (quant/quant_f16_to_i8.cu:54-77):
    ``sx = fp16(amax / 127)``, ``q = sat_s8(rint(x * (127 / amax)))``, no clamp of amax.

    The kernel is built with --use_fast_math, so both divisions are the GPU's approximate division, whose
    last bit no CPU restatement can promise.  This function divides exactly (IEEE) and also returns a mask
    of the elements that sit close enough to a rounding boundary for a 2-ulp error of ``127 / amax`` to move
    them, and of the tokens whose scale lies next to an fp16 rounding boundary; everywhere else the result is
    the kernel's.  The bit-level pin of those is the comparison with the reference's own extension on the GPU
    and the committed fixtures it produced.  Returns (q int8 [M,K], sx fp16 [M], unsure_q bool [M,K],
    unsure_sx bool [M])."""
    x32 = np.asarray(x_f16).astype(np.float32)
    amax = np.abs(x32).max(axis=1, keepdims=True)
    with np.errstate(divide='ignore', invalid='ignore'):
        mult = (np.float32(127) / amax).astype(np.float32)
        prod = (x32 * mult).astype(np.float32)
        sc = (amax / np.float32(127)).astype(np.float32)
    q = np.clip(np.rint(np.nan_to_num(prod, nan=0.0, posinf=127.0, neginf=-128.0)), -128, 127).astype(np.int8)
    frac = np.abs(prod - np.floor(prod) - np.float32(0.5))
    unsure_q = ~(frac > np.abs(prod) * np.float32(4e-7) + np.float32(1e-30))
    sx = sc.astype(np.float16).reshape(-1)
    lo = (sc * np.float32(1 - 3e-7)).astype(np.float16).reshape(-1)
    hi = (sc * np.float32(1 + 3e-7)).astype(np.float16).reshape(-1)
    return q, sx, unsure_q, (lo != hi)


def y_w8a8_cuda(xq, sx, w8, scales_1):
    """The W8A8 GEMM alone on given int8 operands: ``half(float(acc) * (float(s1[n]) * float(sx[m])))``
    (thirdparty/AWQ/kernels/csrc/w8a8/w8a8_gemm_cuda.cu:896-901)."""
    sc = scales_1.astype(np.float32)[None, :] * sx.astype(np.float32)[:, None]
    return (acc_int32(xq, w8).astype(np.float32) * sc).astype(np.float16)


# --------------------------------------------------------------------------
# activation quantization (a6) and the GEMMs (a9-a12)
# --------------------------------------------------------------------------
def act_quant(x_f16):
    """Per-token symmetric int8: returns (Xq int8 [M,K], sx fp16 [M]).
    Follows ``quantize_tensor_int8(x,'S',-1)`` (kairos/quantization.py:111-141),
    the torch twin of kernels/csrc/kairos_kernel/quant/quant_f16_to_i8.cu:46-103."""
    q, s = quantize_int8_per_row(x_f16)
    return q, s.reshape(-1)


def fake_quant_int8(x_f16):
    """``simu_quantize_tensor(x, 8, 'S')`` (kairos/quantization.py:165-205)."""
    x32 = np.asarray(x_f16).astype(np.float32)
    amax = np.abs(x32).max(axis=1, keepdims=True)
    scale = np.maximum(amax / np.float32(127), np.float32(1e-7)).astype(np.float32)
    q = np.clip(np.rint(x32 / scale), -128, 127)
    return (q * scale.astype(np.float16).astype(np.float32)).astype(np.float16)


def matmul_f16(x_f16, w_f16, bias=None):
    """fp32-accumulated ``X @ W.T`` rounded to fp16 (kairos/dynamic_linear.py:163)."""
    y = x_f16.astype(np.float32) @ w_f16.astype(np.float32).T
    y = y.astype(np.float16)
    if bias is not None:
        y = (y + bias.astype(np.float16)).astype(np.float16)     # dynamic_linear.py:165-166
    return y


def acc_int32(xq, w8):
    """Exact int32 accumulators ``Xq @ W8.T``.  Evaluated in fp64, which is exact
    here (|acc| <= 128*128*K < 2**53)."""
    return np.rint(xq.astype(np.float64) @ w8.astype(np.float64).T).astype(np.int32)


def y_w4a16(x_f16, res, bias=None):
    """Kernel ids 0, 1 and 5: dequantize to fp16, fp32-accumulated matmul."""
    return matmul_f16(x_f16, dequant_w16(res['qweight'], res['scales'], res['scaled_zeros']), bias)


def y_w8a8(x_f16, res, bias=None):
    """Kernel id 2.  Epilogue ``half(float(acc) * (float(s1[n]) * float(sx[m])))``
    follows thirdparty/AWQ/kernels/csrc/w8a8/w8a8_gemm_cuda.cu:896-901."""
    xq, sx = act_quant(x_f16)
    w8 = dequant_w8(res['qweight'], res['scales_to8'], res['scaled_zeros_to8'])
    acc = acc_int32(xq, w8)
    sc = res['scales_1'].astype(np.float32)[None, :] * sx.astype(np.float32)[:, None]
    y = (acc.astype(np.float32) * sc).astype(np.float16)
    if bias is not None:
        y = (y + bias.astype(np.float16)).astype(np.float16)
    return y


def w16_from_w8(res):
    """fp16 weight of the W8A16 kernel (id 3): ``fp16(W8) * s1`` rounded to fp16."""
    w8 = dequant_w8(res['qweight'], res['scales_to8'], res['scaled_zeros_to8'])
    return (w8.astype(np.float16) * res['scales_1'].reshape(-1, 1)).astype(np.float16)


def y_w8a16(x_f16, res, bias=None):
    """Kernel id 3 (declared, never wired, in kairos/dynamic_linear.py:8-9)."""
    return matmul_f16(x_f16, w16_from_w8(res), bias)


def forward(x_f16, res, comp_type, bias=None):
    """``DynamicLinear._forward`` (kairos/dynamic_linear.py:131-172) on the CPU."""
    if comp_type in (0, 1, 5):
        return y_w4a16(x_f16, res, bias)
    if comp_type == 2:
        return y_w8a8(x_f16, res, bias)
    if comp_type == 3:
        return y_w8a16(x_f16, res, bias)
    raise ValueError(f'unknown comp_type {comp_type}')


def within_tolerance(y, y_ref, rtol=1e-2, atol=1e-2):
    """fp16 acceptance rule: |y - ref| <= rtol*|ref| + atol*RMS(ref)."""
    y = np.asarray(y, np.float32)
    r = np.asarray(y_ref, np.float32)
    rms = float(np.sqrt(np.mean(r.astype(np.float64) ** 2))) if r.size else 0.0
    bad = np.abs(y - r) > rtol * np.abs(r) + atol * rms
    return int(bad.sum()), rms


# --------------------------------------------------------------------------
# interval LUT (a4)
# --------------------------------------------------------------------------
class LUT:
    """Interval table M -> kernel id with a one-entry memo.

    Follows the C++ class kernels/csrc/kairos_kernel/lut/lut.h:8-43:
    ``record(r, id)`` appends boundary r+1; ``get(m)`` returns the last id when
    m >= last boundary, else the id of the interval found by upper_bound.
    (The Python twin kairos/perf_profiler.py:24-51 gives the same answers for m >= 1.)
    """

    def __init__(self):
        self.seg = [0]
        self.ids = []
        self.pre_ask, self.pre_res = -1, None

    def record(self, r, comp_type):
        self.seg.append(int(r) + 1)
        self.ids.append(int(comp_type))

    def get(self, m):
        if m == self.pre_ask:
            return self.pre_res
        self.pre_ask = m
        if m >= self.seg[-1]:
            self.pre_res = self.ids[-1]
        else:
            import bisect
            self.pre_res = self.ids[bisect.bisect_right(self.seg, m) - 1]
        return self.pre_res

    def shrink_to_fit(self):
        pass


# --------------------------------------------------------------------------
# seeded workload generator shared by the tests, the smoke run and the bench
# --------------------------------------------------------------------------
def make_case(m, k, n, seed=0, outlier_frac=0.01, outlier_gain=20.0, w_std=0.02):
    """Seeded synthetic (X, W) with the benchmark's value distributions:
    X ~ N(0,1) fp16 with ``ceil(outlier_frac*K)`` seeded input channels scaled by
    ``outlier_gain``; W ~ N(0, w_std) fp16.  Stands in for real activations and
    checkpoints (the reference itself benchmarks on ``torch.randn`` inputs,
    kairos/perf_profiler.py:116)."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((m, k), dtype=np.float32)
    n_out = int(np.ceil(outlier_frac * k))
    cols = rng.permutation(k)[:n_out]
    x[:, cols] *= np.float32(outlier_gain)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(w_std)
    return x.astype(np.float16), w.astype(np.float16)
