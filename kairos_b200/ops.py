"""The native-operator surface of the reference, re-implemented on the B200 C ABI.

Function names and argument order follow the two extension modules the reference's
``DynamicLinear`` calls -- ``kairos_cuda_accel`` (kernels/csrc/pybind.cpp:16-24) and
``awq_backend`` (thirdparty/AWQ/kernels/csrc/pybind.cpp:17-26) -- so a call site can switch
by changing the import.  All tensors must be contiguous CUDA tensors; work is enqueued on
torch's current stream (the reference's GEMV/GEMM launch on the legacy default stream).
"""
from __future__ import annotations

import torch

from ._lib import check, lib
from .runtime import gemm_workspace

_current_device = torch._C._cuda_getDevice
_raw_stream = torch._C._cuda_getCurrentRawStream


class _AlreadyCurrent:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_ALREADY_CURRENT = _AlreadyCurrent()


def _on(device):
    """Device guard for a launch: free when `device` is the current one (one process per GPU), a real
    ``torch.cuda.device`` switch otherwise.  A call costs microseconds of host time, which is what the
    smallest kernels take on the device, so the wrappers avoid work that is not needed."""
    return _ALREADY_CURRENT if device.index == _current_device() else torch.cuda.device(device)


def stream_ptr():
    """torch's current stream on the current device, as the integer the C ABI takes."""
    return _raw_stream(_current_device())


def _chk(t, dtype, name):
    if not (t.is_cuda and t.is_contiguous() and t.dtype == dtype):
        raise ValueError(f'{name}: expected a contiguous CUDA tensor of {dtype}, got {t.dtype} on {t.device}')
    return t.data_ptr()


# ---- kairos_cuda_accel ------------------------------------------------------
def quant_fp16_to_int8(out, input, scale):
    """out[int8 ..,K], scale[fp16 tokens] <- per-token symmetric quantization of input."""
    k = input.shape[-1]
    m = input.numel() // k
    with _on(input.device):
        check(lib.kairos_act_quant_i8(_chk(input, torch.float16, 'input'), _chk(out, torch.int8, 'out'),
                                      _chk(scale, torch.float16, 'scale'), m, k, stream_ptr()), 'quant_fp16_to_int8')


def dequant_interleaved_int4_to_int8(output, input, scale, scaled_zero, group_size=128):
    assert group_size == 128
    n, k = output.shape
    with _on(output.device):
        check(lib.kairos_w4_to_w8(_chk(input, torch.int16, 'input'), _chk(scale, torch.float16, 'scale'),
                                  _chk(scaled_zero, torch.float16, 'scaled_zero'), _chk(output, torch.int8, 'output'),
                                  n, k, stream_ptr()), 'dequant_interleaved_int4_to_int8')


def dequant_interleaved_int4_to_fp16(output, input, scale, scaled_zero, group_size=128):
    assert group_size == 128
    n, k = output.shape
    with _on(output.device):
        check(lib.kairos_w4_to_f16(_chk(input, torch.int16, 'input'), _chk(scale, torch.float16, 'scale'),
                                   _chk(scaled_zero, torch.float16, 'scaled_zero'),
                                   _chk(output, torch.float16, 'output'), n, k, stream_ptr()),
              'dequant_interleaved_int4_to_fp16')


def trans_layout_c16_to_c8_awq(qweight, n, k):
    """AWQ interleaved int16 [N/4,K] -> QServe int8 [N,K/2]."""
    out = torch.empty((n, k // 2), dtype=torch.int8, device=qweight.device)
    with _on(qweight.device):
        check(lib.kairos_awq_to_qserve(_chk(qweight, torch.int16, 'qweight'), out.data_ptr(), n, k, stream_ptr()),
              'trans_layout_c16_to_c8_awq')
    return out


# ---- awq_backend ------------------------------------------------------------
def _bias_ptr(bias):
    return None if bias is None else _chk(bias, torch.float16, 'bias')


def gemv_forward_cuda_new(in_feats, kernel, scaling_factors, zeros, m, n, k, group_size=128, bias=None):
    """Kernel id 1 as the switched linear runs it (CUDA-core streamer or warp-MMA decode kernel)."""
    assert group_size == 128
    x = in_feats.reshape(-1, k)
    out = torch.empty((m, n), dtype=torch.float16, device=x.device)
    with _on(x.device):
        check(lib.kairos_w4a16_small_batch(_chk(x, torch.float16, 'in_feats'), _chk(kernel, torch.int16, 'kernel'),
                                           _chk(scaling_factors, torch.float16, 'scaling_factors'),
                                           _chk(zeros, torch.float16, 'zeros'), _bias_ptr(bias), out.data_ptr(), m,
                                           n, k, stream_ptr()), 'gemv_forward_cuda_new')
    return out


def gemv_cuda_core(in_feats, kernel, scaling_factors, zeros, m, n, k, bias=None):
    """The CUDA-core weight-streaming GEMV alone, 1 <= m <= 32."""
    x = in_feats.reshape(-1, k)
    out = torch.empty((m, n), dtype=torch.float16, device=x.device)
    with _on(x.device):
        check(lib.kairos_w4a16_gemv(_chk(x, torch.float16, 'in_feats'), _chk(kernel, torch.int16, 'kernel'),
                                    _chk(scaling_factors, torch.float16, 'scaling_factors'),
                                    _chk(zeros, torch.float16, 'zeros'), _bias_ptr(bias), out.data_ptr(), m, n, k,
                                    stream_ptr()), 'gemv_forward_cuda_new')
    return out


def decode_forward(in_feats, kernel, scaling_factors, zeros, m, n, k, bias=None):
    """W4A16 for 1 <= m <= 32 on the warp-level tensor-core decode kernel."""
    x = in_feats.reshape(-1, k)
    out = torch.empty((m, n), dtype=torch.float16, device=x.device)
    with _on(x.device):
        check(lib.kairos_w4a16_decode(_chk(x, torch.float16, 'in_feats'), _chk(kernel, torch.int16, 'kernel'),
                                      _chk(scaling_factors, torch.float16, 'scaling_factors'),
                                      _chk(zeros, torch.float16, 'zeros'), _bias_ptr(bias), out.data_ptr(), m, n, k,
                                      stream_ptr()), 'decode_forward')
    return out


def decode_silu_forward(in_feats, kernel, scaling_factors, zeros, m, n, k, bias=None):
    """Gate|up linear (n = 2 I weight rows in the blocked order) with SiLU(gate) * up applied in the decode kernel's
    epilogue, 1 <= m <= 32: returns [m, I]."""
    x = in_feats.reshape(-1, k)
    out = torch.empty((m, n // 2), dtype=torch.float16, device=x.device)
    with _on(x.device):
        check(lib.kairos_w4a16_decode_silu(_chk(x, torch.float16, 'in_feats'), _chk(kernel, torch.int16, 'kernel'),
                                           _chk(scaling_factors, torch.float16, 'scaling_factors'),
                                           _chk(zeros, torch.float16, 'zeros'), _bias_ptr(bias), out.data_ptr(), m, n, k,
                                           stream_ptr()), 'decode_silu_forward')
    return out


def gemm_forward_cuda_new(in_feats, kernel, scaling_factors, zeros, bias=None):
    k = in_feats.shape[-1]
    x = in_feats.reshape(-1, k)
    m, n = x.shape[0], kernel.shape[0] * 4
    out = torch.empty((m, n), dtype=torch.float16, device=x.device)
    with _on(x.device):
        ws = gemm_workspace(x.device, m, n, k)
        check(lib.kairos_w4a16_gemm(_chk(x, torch.float16, 'in_feats'), _chk(kernel, torch.int16, 'kernel'),
                                    _chk(scaling_factors, torch.float16, 'scaling_factors'),
                                    _chk(zeros, torch.float16, 'zeros'), _bias_ptr(bias), out.data_ptr(), m, n, k,
                                    ws.data_ptr(), ws.numel(), stream_ptr()), 'gemm_forward_cuda_new')
    return out


def w8a8_gemm_forward_cuda(in_feats, kernel, wscales, ascales, out_feats, bias=None, acc_out=None):
    m, k = in_feats.shape
    n = kernel.shape[0]
    with _on(in_feats.device):
        ws = gemm_workspace(in_feats.device, m, n, k)
        check(lib.kairos_w8a8_gemm(_chk(in_feats, torch.int8, 'in_feats'), _chk(kernel, torch.int8, 'kernel'),
                                   _chk(wscales, torch.float16, 'wscales'), _chk(ascales, torch.float16, 'ascales'),
                                   _bias_ptr(bias), _chk(out_feats, torch.float16, 'out_feats'),
                                   None if acc_out is None else _chk(acc_out, torch.int32, 'acc_out'), m, n, k,
                                   ws.data_ptr(), ws.numel(), stream_ptr()), 'w8a8_gemm_forward_cuda')
    return out_feats


# ---- kernels the reference reaches through torch / declares without a kernel ----
def f16_gemm(x, w16, bias=None):
    """``input @ weight.T`` with fp32 accumulation (kairos/dynamic_linear.py:163)."""
    m, k = x.shape
    n = w16.shape[0]
    out = torch.empty((m, n), dtype=torch.float16, device=x.device)
    with _on(x.device):
        ws = gemm_workspace(x.device, m, n, k)
        check(lib.kairos_f16_gemm(_chk(x, torch.float16, 'x'), _chk(w16, torch.float16, 'w16'), _bias_ptr(bias),
                                  out.data_ptr(), m, n, k, ws.data_ptr(), ws.numel(), stream_ptr()), 'f16_gemm')
    return out


def w8a16_gemm(x, w8, wscales, bias=None):
    """Kernel id 3: fp16 activations times the int8 weight widened to fp16 * s1."""
    m, k = x.shape
    n = w8.shape[0]
    out = torch.empty((m, n), dtype=torch.float16, device=x.device)
    with _on(x.device):
        ws = gemm_workspace(x.device, m, n, k)
        check(lib.kairos_w8a16_gemm(_chk(x, torch.float16, 'x'), _chk(w8, torch.int8, 'w8'),
                                    _chk(wscales, torch.float16, 'wscales'), _bias_ptr(bias), out.data_ptr(), m, n, k,
                                    ws.data_ptr(), ws.numel(), stream_ptr()), 'w8a16_gemm')
    return out


# ---- element-wise operators around the linears ------------------------------------------------
def rms_norm(x, weight, eps, residual_delta=None):
    """RMSNorm over the last dimension.  With `residual_delta`, x <- x + residual_delta IN PLACE first (the
    residual addition of the preceding block, carried by this pass)."""
    k = x.shape[-1]
    m = x.numel() // k
    y = torch.empty_like(x)
    with _on(x.device):
        if hasattr(residual_delta, 'peer_args'):
            # the delta is still spread over a tensor-parallel group (tp.PendingPeerSum): summed while loaded
            peer_in, peer_sig, world, rank = residual_delta.peer_args()
            check(lib.kairos_add_rms_norm_peer(_chk(x, torch.float16, 'x'), peer_in, peer_sig, world, rank,
                                               _chk(weight, torch.float16, 'weight'), y.data_ptr(), m, k, float(eps),
                                               stream_ptr()), 'add_rms_norm_peer')
        elif residual_delta is None:
            check(lib.kairos_rms_norm(_chk(x, torch.float16, 'x'), _chk(weight, torch.float16, 'weight'), y.data_ptr(),
                                      m, k, float(eps), stream_ptr()), 'rms_norm')
        else:
            check(lib.kairos_add_rms_norm(_chk(x, torch.float16, 'x'), _chk(residual_delta, torch.float16, 'delta'),
                                          _chk(weight, torch.float16, 'weight'), y.data_ptr(), m, k, float(eps),
                                          stream_ptr()), 'add_rms_norm')
    return y


def silu_mul(gate_up, blocked=False):
    """silu(gate) * up for the fused activation [..., 2I] -> [..., I]; `blocked`: gate and up channels alternate
    in blocks of 16 (see the header) instead of lying one after the other."""
    i2 = gate_up.shape[-1]
    m = gate_up.numel() // i2
    out = torch.empty(gate_up.shape[:-1] + (i2 // 2,), dtype=torch.float16, device=gate_up.device)
    fn = lib.kairos_silu_mul_blocked if blocked else lib.kairos_silu_mul
    with _on(gate_up.device):
        check(fn(_chk(gate_up, torch.float16, 'gate_up'), out.data_ptr(), m, i2 // 2, stream_ptr()), 'silu_mul')
    return out


def rope_kv(qkv, cos, sin, q_out, k_cache, v_cache, b, s, h, hkv, d, pos_dev=None, pos0=0):
    """Rotary embedding of q / k and the KV-cache write for a fused QKV activation (see the header)."""
    with _on(qkv.device):
        check(lib.kairos_rope_kv(_chk(qkv, torch.float16, 'qkv'), _chk(cos, torch.float16, 'cos'),
                                 _chk(sin, torch.float16, 'sin'), None if pos_dev is None else pos_dev.data_ptr(),
                                 int(pos0), _chk(q_out, torch.float16, 'q_out'), _chk(k_cache, torch.float16, 'k_cache'),
                                 _chk(v_cache, torch.float16, 'v_cache'), b, s, h, hkv, d, k_cache.shape[2],
                                 stream_ptr()), 'rope_kv')
    return q_out


def rms_norm_quant(x, weight, eps, want_f16=False, residual_delta=None):
    """RMSNorm emitting per-token int8 + fp16 scales (what a W8A8 linear consumes); also the fp16 result
    when `want_f16`; with `residual_delta`, x <- x + residual_delta in place first.
    Returns (xq, sx, y_or_None)."""
    k = x.shape[-1]
    m = x.numel() // k
    xq = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    sx = torch.empty((m,), dtype=torch.float16, device=x.device)
    y = torch.empty_like(x) if want_f16 else None
    if hasattr(residual_delta, 'peer_args'):
        peer_in, peer_sig, world, rank = residual_delta.peer_args()
        with _on(x.device):
            check(lib.kairos_rms_norm_quant_peer(_chk(x, torch.float16, 'x'), peer_in, peer_sig, world, rank,
                                                 _chk(weight, torch.float16, 'weight'), None if y is None else y.data_ptr(),
                                                 xq.data_ptr(), sx.data_ptr(), m, k, float(eps), stream_ptr()),
                  'rms_norm_quant_peer')
        return xq, sx, y
    with _on(x.device):
        check(lib.kairos_rms_norm_quant(_chk(x, torch.float16, 'x'),
                                        None if residual_delta is None else _chk(residual_delta, torch.float16, 'delta'),
                                        _chk(weight, torch.float16, 'weight'), None if y is None else y.data_ptr(), xq.data_ptr(), sx.data_ptr(), m, k,
                                        float(eps), stream_ptr()), 'rms_norm_quant')
    return xq, sx, y


def silu_mul_quant(gate_up, want_f16=False, blocked=False):
    """silu(gate) * up emitting per-token int8 + fp16 scales.  Returns (xq, sx, y_or_None)."""
    i2 = gate_up.shape[-1]
    m = gate_up.numel() // i2
    shape = gate_up.shape[:-1] + (i2 // 2,)
    xq = torch.empty(shape, dtype=torch.int8, device=gate_up.device)
    sx = torch.empty((m,), dtype=torch.float16, device=gate_up.device)
    y = torch.empty(shape, dtype=torch.float16, device=gate_up.device) if want_f16 else None
    fn = lib.kairos_silu_mul_quant_blocked if blocked else lib.kairos_silu_mul_quant
    with _on(gate_up.device):
        check(fn(_chk(gate_up, torch.float16, 'gate_up'), None if y is None else y.data_ptr(), xq.data_ptr(),
                 sx.data_ptr(), m, i2 // 2, stream_ptr()), 'silu_mul_quant')
    return xq, sx, y
