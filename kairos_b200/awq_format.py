"""Wire format of the single resident weight: packed uint4 with 4-row interleave, plus the
group-major factor tensors.  Host-side (torch) preparation code; runs on any device.

Same function names and results as thirdparty/AWQ/awq_method.py of the reference.
"""
from __future__ import annotations

import torch


@torch.no_grad()
def pack_int_awq(unpacked_qweight, interleave=4, kstride=64):
    """uint4 values [N,K] -> int16 [N/4, K]  (thirdparty/AWQ/awq_method.py:3-38).

    With n = 4*n0 + n1 and k = 64*k0 + 32*a + 8*b + 2*c + d, nibble b of
    out[n0, 64*k0 + 16*n1 + 8*a + 2*c + d] is q[n, k]: every 32-bit word carries two
    consecutive k in each nibble pair (ready for the lop3 unpack), and four weight rows
    share a 128-byte line per 64 k."""
    assert interleave == 4 and kstride == 64
    n, k = unpacked_qweight.shape
    q = unpacked_qweight.to(torch.int32).reshape(n // 4, 4, k // 64, 2, 4, 4, 2)
    #                                             n0   n1  k0      a  b  c  d
    q = q.permute(0, 2, 1, 3, 5, 6, 4)          # n0 k0 n1 a c d | b
    packed = q[..., 0] | (q[..., 1] << 4) | (q[..., 2] << 8) | (q[..., 3] << 12)
    return packed.reshape(n // 4, k).to(torch.int16).contiguous()


@torch.no_grad()
def unpack_int_awq(packed_qweight):
    """Inverse of pack_int_awq (test/depacking.py:22-38 of the reference)."""
    n4, k = packed_qweight.shape
    u = packed_qweight.to(torch.int32) & 0xFFFF
    nib = torch.stack([(u >> s) & 0xF for s in (0, 4, 8, 12)], dim=-1)
    nib = nib.reshape(n4, k // 64, 4, 2, 4, 2, 4).permute(0, 2, 1, 3, 6, 4, 5)
    return nib.reshape(n4 * 4, k).contiguous()


def calculate_zeros_width(in_features, group_size=128, pack_num=8):
    """Rows of the factor tensors / pack_num (thirdparty/AWQ/awq_method.py:40-54)."""
    if group_size >= 128:
        mult = 1
    elif group_size == 64:
        mult = 2
    elif group_size == 32:
        mult = 4
    else:
        raise NotImplementedError
    base = (in_features // group_size + pack_num - 1) // pack_num
    return (base + mult - 1) // mult * mult


@torch.no_grad()
def trans_qfactor_layout_awq(scales, zeros, group_size, method='AWQ'):
    """[N,G] (scale, zero) -> group-major fp16 [G_pad, N] (scale, -(scale*zero)), zero padded
    (thirdparty/AWQ/awq_method.py:56-75)."""
    n, g = scales.shape
    gp = calculate_zeros_width(g * group_size, group_size) * 8
    qscales = torch.zeros((n, gp), dtype=torch.float16, device=scales.device)
    qscales[:, :g] = scales
    if method == 'AWQ':
        zeros = zeros.to(torch.int32)
    scaled_zeros = torch.zeros_like(qscales)
    scaled_zeros[:, :g] = -(qscales[:, :g] * zeros.to(torch.float32)).to(torch.float16)
    return qscales.t().contiguous(), scaled_zeros.t().contiguous()
