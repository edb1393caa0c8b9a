"""Time ONE kernel of the switched linear on seeded synthetic data: the single-kernel companion of bench.py.

    python -m kairos_b200.bench_kernel --kernel w8a8 --m 8192 --k 4096 --n 14336 --iters 3

Use it to compare a kernel before and after a change, or as the small fixed workload of a profiler capture
(one kernel, a few launches, a few hundred MB on the device).

Kernels: decode (kernel id 1), gemv (CUDA-core streamer), w4a16_gemm, w8a16_gemm, w8a8, fp16, act_quant,
to_w8, to_f16.  Prints the mean device time per launch (CUDA events over `iters` launches after
`warmup`), which is NOT a benchmark figure when the process runs under a profiler.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import ops
from .dynamic_linear import DynamicLinear
from .synthetic import make_case


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--kernel', required=True)
    ap.add_argument('--m', type=int, default=16)
    ap.add_argument('--k', type=int, default=4096)
    ap.add_argument('--n', type=int, default=4096)
    ap.add_argument('--iters', type=int, default=3)
    ap.add_argument('--warmup', type=int, default=2)
    a = ap.parse_args()
    torch.cuda.set_device(0)
    x_np, w_np = make_case(a.m, a.k, a.n, seed=0)
    lin = torch.nn.Linear(a.k, a.n, bias=False, dtype=torch.float16)
    lin.weight.data = torch.from_numpy(w_np)
    L = DynamicLinear.from_module(lin.cuda(), 'cuda')
    x = torch.from_numpy(x_np).cuda()
    m, k, n = a.m, a.k, a.n
    if a.kernel == 'decode':
        fn = lambda: ops.decode_forward(x, L.qweight, L.scales, L.scaled_zeros, m, n, k)
    elif a.kernel == 'gemv':
        fn = lambda: ops.gemv_cuda_core(x, L.qweight, L.scales, L.scaled_zeros, m, n, k)
    elif a.kernel == 'w4a16_gemm':
        fn = lambda: ops.gemm_forward_cuda_new(x, L.qweight, L.scales, L.scaled_zeros)
    elif a.kernel in ('w8a8', 'w8a16_gemm', 'to_w8'):
        w8 = torch.empty((n, k), dtype=torch.int8, device='cuda')
        conv = lambda: ops.dequant_interleaved_int4_to_int8(w8, L.qweight, L.scales_to8, L.scaled_zeros_to8, 128)
        conv()
        if a.kernel == 'to_w8':
            fn = conv
        elif a.kernel == 'w8a16_gemm':
            fn = lambda: ops.w8a16_gemm(x, w8, L.scales_1)
        else:
            xq = torch.empty((m, k), dtype=torch.int8, device='cuda')
            sx = torch.empty((m,), dtype=torch.float16, device='cuda')
            ops.quant_fp16_to_int8(xq, x, sx)
            y = torch.empty((m, n), dtype=torch.float16, device='cuda')
            fn = lambda: ops.w8a8_gemm_forward_cuda(xq, w8, L.scales_1, sx, y)
    elif a.kernel in ('fp16', 'to_f16'):
        w16 = torch.empty((n, k), dtype=torch.float16, device='cuda')
        conv = lambda: ops.dequant_interleaved_int4_to_fp16(w16, L.qweight, L.scales, L.scaled_zeros, 128)
        conv()
        fn = conv if a.kernel == 'to_f16' else (lambda: ops.f16_gemm(x, w16))
    elif a.kernel == 'act_quant':
        xq = torch.empty((m, k), dtype=torch.int8, device='cuda')
        sx = torch.empty((m,), dtype=torch.float16, device='cuda')
        fn = lambda: ops.quant_fp16_to_int8(xq, x, sx)
    else:
        raise SystemExit(f'unknown kernel {a.kernel}')
    for _ in range(a.warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(a.iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    print(json.dumps({'kernel': a.kernel, 'M': m, 'K': k, 'N': n, 'us_per_launch': 1e3 * s.elapsed_time(e) / a.iters}))


if __name__ == '__main__':
    main()
