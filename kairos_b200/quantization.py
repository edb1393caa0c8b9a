"""Offline weight quantization of the switched linear (host side, torch, any device).

Every division has a TENSOR divisor: torch's CUDA kernels turn division by a Python scalar
into multiplication by its reciprocal, which is not the IEEE quotient the CPU path (and the
reference's fixtures) use; with tensor divisors both devices give identical bits.

Two-level scheme of the reference: fp16 -> per-output-channel symmetric int8 ->
asymmetric uint4 per group of 128 int8 values with a non-integer zero point.
"""
from __future__ import annotations

import torch


@torch.no_grad()
def quantize_tensor_int8(x, q_type='S', group_size=-1, return_dtype=torch.float16, max_int=-1):
    """Per-row (group_size -1) or per-tensor (-2) int8 quantization; same contract and
    arithmetic as kairos/quantization.py:111-141 (fp32 maths, IEEE division, round-half-even)."""
    assert q_type in ('A', 'S'), 'Illegal quantification config.'
    shape = x.shape
    if group_size == -1:
        x = x.reshape(-1, shape[-1])
    elif group_size == -2:
        x = x.reshape(1, -1)
    x = x.to(torch.float32)
    if q_type == 'A':
        if max_int == -1:
            max_int = 255
        mx = x.amax(dim=1, keepdim=True)
        mn = x.amin(dim=1, keepdim=True)
        scale = (mx - mn).clamp(min=1e-7) / x.new_tensor(float(max_int))
        zero_pt = -(mn / scale)
        q = (x / scale + zero_pt).round().to(torch.uint8)
    else:
        if max_int == -1:
            max_int = 127
        scale = x.abs().amax(dim=1, keepdim=True).clamp(min=1e-7) / x.new_tensor(float(max_int))
        zero_pt = torch.tensor([0])
        q = (x / scale).round().to(torch.int8)
    return q.reshape(shape), {'q_type': q_type, 'scale': scale.to(return_dtype),
                              'zero_pt': zero_pt.to(return_dtype)}


@torch.no_grad()
def kairos_quantize_tensor_int4(x, group_size=-1):
    """int8 weight -> uint4 with fp16 (scale, non-integer zero) per group
    (kairos/dynamic_linear.py:11-37)."""
    shape = x.shape
    if group_size < 0:
        x = x.reshape(-1, shape[-1])
    else:
        assert shape[-1] % group_size == 0
        x = x.reshape(-1, group_size)
    x = x.to(torch.float32)
    mx = x.amax(dim=1, keepdim=True)
    mn = x.amin(dim=1, keepdim=True)
    scale_f = (mx - mn).clamp(min=1e-5) / x.new_tensor(15.0)
    zero_pt_f = -(mn / scale_f)
    q = (x / scale_f + zero_pt_f).round().clamp(0, 15)
    return q.reshape(shape).to(torch.int8), {
        'scale_f': scale_f.to(torch.float16), 'scale_i': torch.floor(scale_f).to(torch.int8),
        'zero_pt_f': zero_pt_f.to(torch.float16), 'zero_pt_i': torch.round(zero_pt_f).to(torch.int8),
        'group_size': group_size}
