"""``DynamicLinear``: the switched quantized linear layer on the B200 C ABI.

Same module surface as kairos/dynamic_linear.py:39-172 of the reference -- constructor,
``from_module``, ``forward`` (3-D input), ``_forward(x, m, comp_type)``, class attribute
``prof``, instance attributes ``shape``/``pre_m``/``comp_type`` -- so it drops into the
reference's ``quantize_model`` flow.  Only a packed uint4 (group 128) weight is resident; per
call the interval LUT picks a kernel id for M = batch*seq and ONE C call runs it:
activation quantization only for W8A8, weight conversion only for ids 2/3/5 and only on a
miss of the context's bounded conversion cache.
"""
from __future__ import annotations

import torch

from ._lib import KairosError, check, lib
from .awq_format import pack_int_awq, trans_qfactor_layout_awq
from .quantization import kairos_quantize_tensor_int4, quantize_tensor_int8
from .runtime import default_context

# kernel ids (kairos/dynamic_linear.py:8-9; v2 ids 6/7 of dynamic_linear_v2.py:11-13 are
# recognised in LUT files but have no kernel here)
COMP_TYPE_NAME = {'w4a16_gemm': 0, 'w4a16_gemv': 1, 'w8a8': 2,
                  'w8a16_gemm': 3, 'w8a16_gemv': 4, 'fp16': 5,
                  'w4a16_marlin': 6, 'w4a8_qserve': 7}
COMP_TYPE_ID = {v: k for k, v in COMP_TYPE_NAME.items()}
SUPPORTED_COMP_TYPES = (0, 1, 2, 3, 5)

_switched_linear = lib.kairos_switched_linear
_raw_stream = torch._C._cuda_getCurrentRawStream     # current stream of a device index as an integer

_RESIDENT = ('qweight', 'scales', 'scaled_zeros', 'scales_to8', 'scaled_zeros_to8', 'scales_1')


class DynamicLinear(torch.nn.Module):
    """Quantization strategy Ws4WcXAcY: the weight is stored FP16 -> INT8 -> UINT4 once;
    weight and activation compute precisions are selected per call."""

    prof = None          # shared Profiler: get_comp_type((N, K), m) -> kernel id
    context = None       # optional runtime.Context override shared by all instances

    @torch.no_grad()
    def __init__(self, in_features, out_features, bias, device, group_size):
        super().__init__()
        assert group_size == 128, 'the resident format is uint4 with groups of 128'
        self.enable_accel = False
        self.return_dtype = torch.float16
        self.in_features = in_features
        self.out_features = out_features
        self.group_size = group_size
        n, k = out_features, in_features
        gp = ((k // 128 + 7) // 8) * 8
        f16 = dict(device=device, dtype=torch.float16)
        # registered as buffers so state_dict()/.to() see them (the reference keeps plain attributes)
        self.register_buffer('qweight', torch.empty((n // 4, k), device=device, dtype=torch.int16))
        for name in ('scales', 'scaled_zeros', 'scales_to8', 'scaled_zeros_to8'):
            self.register_buffer(name, torch.empty((gp, n), **f16))
        self.register_buffer('scales_1', torch.empty((n,), **f16))
        if bias:
            self.register_buffer('bias', torch.empty((n,), **f16))
        else:
            self.bias = None
        self.shape = (out_features, in_features)
        self.pre_m = 0
        self.pre_comp_type = ''
        self.comp_type = COMP_TYPE_NAME['w4a16_gemm']
        self._handle = None
        self._handle_key = None
        self._ctx = None

    def init(self):
        """Hook kept for quantized models loaded from a checkpoint: drops the native handle
        so that it is rebuilt on the loaded buffers."""
        self._release()

    @classmethod
    @torch.no_grad()
    def from_module(cls, linear, device, return_dtype=torch.float16, init_only=False, name=''):
        """fp16 ``nn.Linear`` -> switched linear (kairos/dynamic_linear.py:85-115)."""
        q_linear = cls(linear.in_features, linear.out_features, linear.bias is not None, device, group_size=128)
        if init_only:
            return q_linear
        weight = linear.weight.data.to(torch.float16)
        n, k = weight.shape
        # step 1: fp16 -> int8 per output channel
        weight_i8, cfg1 = quantize_tensor_int8(weight, max_int=127)
        scale_1 = cfg1['scale']
        # step 2: int8 -> uint4 per group of 128
        weight_i4, cfg2 = kairos_quantize_tensor_int4(weight_i8, group_size=128)
        scale_2_f, zero_2_f = cfg2['scale_f'], cfg2['zero_pt_f']
        scales_to8, scaled_zeros_to8 = trans_qfactor_layout_awq(
            scale_2_f.reshape(n, -1), zero_2_f.reshape(n, -1), 128, method='kairos')
        # step 3: factors that take uint4 straight to fp16
        scale_f = scale_2_f.view(n, -1) * scale_1
        scales, scaled_zeros = trans_qfactor_layout_awq(
            scale_f.reshape(n, -1), zero_2_f.reshape(n, -1), 128, method='kairos')
        q_linear.qweight.copy_(pack_int_awq(weight_i4))
        q_linear.scales.copy_(scales)
        q_linear.scaled_zeros.copy_(scaled_zeros)
        q_linear.scales_to8.copy_(scales_to8)
        q_linear.scaled_zeros_to8.copy_(scaled_zeros_to8)
        q_linear.scales_1.copy_(scale_1.view(-1))
        if linear.bias is not None:
            q_linear.bias.copy_(linear.bias.data.half())
        return q_linear

    # ---- native handle ----------------------------------------------------
    def _cache_context(self):
        return type(self).context or default_context(self.qweight.device)

    def _release(self):
        if self._handle:
            lib.kairos_layer_destroy(self._handle)
        self._handle = None
        self._handle_key = None

    def _native(self):
        key = (self.qweight.data_ptr(), self.scales.data_ptr())
        if self._handle is None or self._handle_key != key:
            self._release()
            if not self.qweight.is_cuda:
                raise KairosError('DynamicLinear runs on a CUDA device only; there is no CPU path')
            self._ctx = self._cache_context()
            ptrs = [getattr(self, n).data_ptr() for n in _RESIDENT]
            with torch.cuda.device(self.qweight.device):
                self._handle = lib.kairos_layer_create(
                    self._ctx.handle, self.out_features, self.in_features, *ptrs,
                    None if self.bias is None else self.bias.data_ptr())
            if not self._handle:
                raise KairosError('kairos_layer_create: ' + lib.kairos_last_error().decode())
            self._handle_key = key
        return self._handle

    def __del__(self):
        try:
            self._release()
        except Exception:
            pass

    def _apply(self, fn, *args, **kwargs):
        # .to() / .cuda() / .half() may move the buffers: the native handle holds raw pointers
        self._release()
        return super()._apply(fn, *args, **kwargs)

    # ---- forward ----------------------------------------------------------
    # forward / _forward / forward_q8 pass raw pointers to the library and build no autograd graph; they carry
    # no torch.no_grad() wrapper because entering one costs about as much host time as the launch itself
    def forward(self, input: torch.Tensor, out=None) -> torch.Tensor:
        """`out`, when given, is a contiguous fp16 [tokens, N] tensor the result is written into (for example a
        buffer that peers of a tensor-parallel group can read); the return value is a view of it."""
        shape = input.shape
        m = input.numel() // shape[-1]
        if m != self.pre_m:
            self.pre_m = m
            self.comp_type = type(self).prof.get_comp_type(self.shape, m)
        return self._forward(input, m, self.comp_type, out).view(shape[0], shape[1], -1)

    def _forward(self, input: torch.Tensor, batch_token_len, comp_type, out=None) -> torch.Tensor:
        """Run kernel `comp_type` on input [M, K] (or [..., K]) and return [M, N] (written into `out`, a
        contiguous fp16 [M, N] tensor, when given)."""
        x = input if input.dim() == 2 else input.reshape(-1, self.in_features)
        if x.dtype != torch.float16:
            x = x.to(torch.float16)
        if not x.is_contiguous():
            x = x.contiguous()
        m = x.shape[0]
        if out is None:
            out = x.new_empty((m, self.out_features))      # the cheapest allocation call torch offers from Python
        elif out.shape != (m, self.out_features) or out.dtype != torch.float16 or not out.is_contiguous():
            raise ValueError('out must be a contiguous fp16 [M, N] tensor')
        rc = _switched_linear(self._handle or self._native(), x.data_ptr(), out.data_ptr(), m, comp_type,
                              _raw_stream(x.device.index))
        if rc:
            check(rc, f'DynamicLinear._forward(comp_type={comp_type}, m={m}, shape={self.shape})')
        return out

    def wants_int8(self, m):
        """True when the LUT sends M = m to the W8A8 kernel: the operator before this layer can then emit
        int8 activations directly (``ops.rms_norm_quant`` / ``ops.silu_mul_quant``) and call
        :meth:`forward_q8`, instead of writing fp16 for a separate quantization pass."""
        if m != self.pre_m:
            self.pre_m = m
            self.comp_type = type(self).prof.get_comp_type(self.shape, m)
        return self.comp_type == COMP_TYPE_NAME['w8a8']

    def forward_q8(self, xq, sx, out=None):
        """W8A8 on activations that are already quantized: xq int8 [..., K], sx fp16 [tokens] -> [..., N]
        (written into `out`, a contiguous fp16 tensor of that many elements, when given)."""
        m = xq.numel() // self.in_features
        if out is None:
            out = torch.empty(xq.shape[:-1] + (self.out_features,), dtype=torch.float16, device=xq.device)
        elif out.numel() != m * self.out_features or out.dtype != torch.float16 or not out.is_contiguous():
            raise ValueError('out must be a contiguous fp16 tensor of tokens x N elements')
        else:
            out = out.view(xq.shape[:-1] + (self.out_features,))
        rc = lib.kairos_switched_linear_q8(self._handle or self._native(), xq.data_ptr(), sx.data_ptr(), out.data_ptr(),
                                           m, _raw_stream(xq.device.index))
        if rc:
            check(rc, f'DynamicLinear.forward_q8(m={m}, shape={self.shape})')
        return out

    @torch.no_grad()
    def prefetch(self, comp_type, stream=None):
        """Convert the weight the kernel id needs ahead of time (e.g. on a side stream)."""
        st = torch.cuda.current_stream(self.qweight.device) if stream is None else stream
        check(lib.kairos_layer_prefetch(self._native(), int(comp_type), st.cuda_stream), 'prefetch')

    # helpers of dynamic_linear_v2.py:214-224, used to time the conversion alone
    @torch.no_grad()
    def _trans_weight_to_8(self):
        from . import ops
        w = torch.empty(self.shape, dtype=torch.int8, device=self.qweight.device)
        ops.dequant_interleaved_int4_to_int8(w, self.qweight, self.scales_to8, self.scaled_zeros_to8, 128)
        return w

    @torch.no_grad()
    def _trans_weight_to_16(self):
        from . import ops
        w = torch.empty(self.shape, dtype=torch.float16, device=self.qweight.device)
        ops.dequant_interleaved_int4_to_fp16(w, self.qweight, self.scales, self.scaled_zeros, 128)
        return w

    def extra_repr(self) -> str:
        return f'in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}'
