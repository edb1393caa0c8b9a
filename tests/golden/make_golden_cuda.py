#!/usr/bin/env python
"""Writes tests/golden/ref_cuda_*.npz: outputs of the REFERENCE'S OWN CUDA extension on seeded inputs.

    python tests/golden/make_golden_cuda.py <dir holding the built reference extensions> <output dir>

Needs a GPU and the reference's two extension modules (kairos_cuda_accel, awq_backend) built unmodified
for the GPU at hand (baseline/build_ref_kernels.sh builds them from a reference source tree).  The inputs
come from the oracle's seeded generators, so the fixtures can be regenerated anywhere the extensions run.
The fixtures pin the rounding of the reference's CUDA kernels where it differs from its torch functions:
one fused multiply-add in the weight conversions, approximate division in activation quantization.

  ref_cuda_case.npz     N=64, K=512, M=16: qweight and factors, x, and what the extension returns for
                        W4->F16, W4->W8, activation quantization and the W8A8 GEMM chained as
                        DynamicLinear._forward chains them (kairos/dynamic_linear.py:143-155)
  ref_cuda_scales.npz   sx for every positive finite fp16 value as a token's amax (31743 tokens)
  ref_cuda_ties.npz     256 tokens whose elements sit on and beside the rounding boundaries of x * (127/amax)
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, '..', '..', 'oracle'))
import kairos_oracle as oracle  # noqa: E402


def tie_inputs():
    """256 tokens of 512 elements: for token t with amax a_t, the fp16 values nearest to (j + 0.5) * a_t / 127
    and their fp16 neighbours, j = 0..126, both signs; the first element is a_t itself."""
    rng = np.random.default_rng(11)
    bits = rng.integers(0x0400, 0x7bff, size=256).astype(np.uint16)       # normal positive fp16 values
    amax = bits.view(np.float16).astype(np.float64)
    x = np.zeros((256, 512), np.float16)
    for t in range(256):
        vals = [amax[t]]
        for j in range(127):
            c = np.float16((j + 0.5) * amax[t] / 127.0)
            for nb in (np.nextafter(c, np.float16(0)), c, np.nextafter(c, np.float16(np.inf))):
                if abs(float(nb)) <= amax[t]:
                    vals.append(float(nb))
        vals = np.array(vals[:512], np.float64)
        sign = np.where(rng.random(vals.size) < 0.5, -1.0, 1.0)
        sign[0] = 1.0
        x[t, :vals.size] = (vals * sign).astype(np.float16)
    return x


def main():
    ext_dir, out_dir = sys.argv[1], sys.argv[2]
    sys.path.insert(0, ext_dir)
    import awq_backend
    import kairos_cuda_accel
    dev = 'cuda:0'
    os.makedirs(out_dir, exist_ok=True)

    # ---- one small layer through every stage ----
    m, k, n = 16, 512, 64
    x, w = oracle.make_case(m, k, n, seed=5)
    res = oracle.from_module(w)
    t = {name: torch.from_numpy(np.ascontiguousarray(res[name])).to(dev)
         for name in ('qweight', 'scales', 'scaled_zeros', 'scales_to8', 'scaled_zeros_to8', 'scales_1')}
    xd = torch.from_numpy(x).to(dev)
    w16 = torch.empty((n, k), dtype=torch.float16, device=dev)
    kairos_cuda_accel.dequant_interleaved_int4_to_fp16(w16, t['qweight'], t['scales'], t['scaled_zeros'], 128)
    w8 = torch.empty((n, k), dtype=torch.int8, device=dev)
    kairos_cuda_accel.dequant_interleaved_int4_to_int8(w8, t['qweight'], t['scales_to8'], t['scaled_zeros_to8'], 128)
    xq = torch.empty_like(xd, dtype=torch.int8)
    sx = torch.empty(m, device=dev, dtype=torch.float16)
    kairos_cuda_accel.quant_fp16_to_int8(xq, xd, sx)
    y = torch.empty((m, n), device=dev, dtype=torch.float16)
    awq_backend.w8a8_gemm_forward_cuda(xq, w8, t['scales_1'].view(-1), sx, y)
    torch.cuda.synchronize()
    np.savez_compressed(os.path.join(out_dir, 'ref_cuda_case.npz'), x=x,
                        **{name: np.ascontiguousarray(res[name]) for name in t},
                        w16=w16.cpu().numpy(), w8=w8.cpu().numpy(), xq=xq.cpu().numpy(), sx=sx.cpu().numpy(),
                        y_w8a8=y.cpu().numpy())

    # ---- the scale of every possible amax ----
    bits = np.arange(1, 0x7c00, dtype=np.uint16)
    rows = np.zeros((bits.size, 128), np.float16)     # 128 columns: the reference's block is then four full warps
    rows[:, 3] = bits.view(np.float16)
    rd = torch.from_numpy(rows).to(dev)
    q = torch.empty_like(rd, dtype=torch.int8)
    s = torch.empty(bits.size, device=dev, dtype=torch.float16)
    kairos_cuda_accel.quant_fp16_to_int8(q, rd, s)
    torch.cuda.synchronize()
    np.savez_compressed(os.path.join(out_dir, 'ref_cuda_scales.npz'), amax_bits=bits,
                        sx_bits=s.cpu().numpy().view(np.uint16), q_of_amax=q.cpu().numpy()[:, 3].copy())

    # ---- elements on and beside the rounding boundaries ----
    xt = tie_inputs()
    td = torch.from_numpy(xt).to(dev)
    q = torch.empty_like(td, dtype=torch.int8)
    s = torch.empty(xt.shape[0], device=dev, dtype=torch.float16)
    kairos_cuda_accel.quant_fp16_to_int8(q, td, s)
    torch.cuda.synchronize()
    np.savez_compressed(os.path.join(out_dir, 'ref_cuda_ties.npz'), x=xt, xq=q.cpu().numpy(), sx=s.cpu().numpy())
    print('wrote', sorted(os.listdir(out_dir)), 'on', torch.cuda.get_device_name(0))


if __name__ == '__main__':
    main()
