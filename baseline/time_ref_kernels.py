#!/usr/bin/env python
"""Same-box GPU baseline: the reference's own CUDA kernels, rebuilt unmodified for sm_100a by
baseline/build_ref_kernels.sh, timed beside this library's kernels on the points of the benchmark sweep.

    python baseline/time_ref_kernels.py > ref_kernels.jsonl

Protocol: the reference's `timer` (utils/perf_eval.py:21-34): CUDA events around n back-to-back eager calls
after warm-up, one set of weights (so small weights may sit in L2, for both arms alike).  Each arm runs the
complete candidate as DynamicLinear._forward does (kairos/dynamic_linear.py:131-172): W8A8 = weight
conversion + activation quantization + GEMM (the reference converts on every call; this library is timed
both that way, 'cold', and with the converted weight cached, 'warm').

Two configurations of the reference are NOT run, on purpose:
  * gemm_forward_cuda_new with M <= 32: its split-K variant waits, without a bound, on semaphores taken from
    uninitialised memory (thirdparty/AWQ/kernels/csrc/quantization_new/gemm/gemm_cuda.cu:28,548-557);
  * gemv_forward_cuda_new with M = 31, 32: the dispatch instantiates batch 29 / 30 there
    (quantization_new/gemv/gemv_cuda.cu:443-452), so the last rows are garbage.
Before timing, each reference kernel's result is compared with this library's kernel of the same id
(|a-b| <= 2e-2|b| + 2e-2 RMS; the library runs its default arithmetic rule, which follows the reference's
torch functions, so W8A8 differs from the reference's CUDA kernels wherever a converted weight or a
quantized activation rounds the other way), both are compared with an fp32 product over the dequantized
weight (max error / RMS), and the W8A8 path is run once more under the 'reference_cuda' rule, where it must
equal the reference bit for bit.
"""
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, 'baseline', '_ref'))

SHAPES_KN = [(4096, 4096), (4096, 1024), (4096, 14336), (14336, 4096)]
M_LIST = [1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192]


def timed(fn, n, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(n):
        fn()
    e.record()
    torch.cuda.synchronize()
    return 1e3 * s.elapsed_time(e) / n       # microseconds


def close(a, b):
    a, b = a.float(), b.float()
    rms = b.pow(2).mean().sqrt()
    return bool(((a - b).abs() <= 2e-2 * b.abs() + 2e-2 * rms).all())


def main():
    try:
        import awq_backend
        import kairos_cuda_accel
    except ImportError as exc:
        print(json.dumps({'unavailable': f'reference extensions not built ({exc}); run baseline/build_ref_kernels.sh'}))
        return
    import kairos_b200 as kb
    from kairos_b200 import ops, runtime
    from kairos_b200.synthetic import make_case
    torch.cuda.set_device(0)
    dev = 'cuda:0'
    warm_ctx = runtime.Context(dev, cache_bytes=None)
    cold_ctx = runtime.Context(dev, cache_bytes=0)
    for (k, n) in SHAPES_KN:
        x_np, w_np = make_case(max(M_LIST), k, n, seed=0)
        lin = torch.nn.Linear(k, n, bias=False, dtype=torch.float16)
        lin.weight.data = torch.from_numpy(w_np)
        from kairos_b200.perf_profiler import _clone_layer
        layer = kb.DynamicLinear.from_module(lin.to(dev), dev)
        layer._cache_context = lambda: warm_ctx
        cold = _clone_layer(layer, cold_ctx)
        warm_ctx.reserve(max(M_LIST), n, k)
        cold_ctx.reserve(max(M_LIST), n, k)
        x_all = torch.from_numpy(x_np).to(dev)
        w16_gold = torch.empty((n, k), dtype=torch.float16, device=dev)
        ops.dequant_interleaved_int4_to_fp16(w16_gold, layer.qweight, layer.scales, layer.scaled_zeros, 128)
        for m in M_LIST:
            x = x_all[:m].contiguous()
            reps, warm = (200, 20) if m <= 512 else (30, 5)
            row = {'K': k, 'N': n, 'M': m}

            # ---- the reference's kernels, called as its DynamicLinear._forward calls them ----
            def ref_w8a8():
                w8 = torch.empty((n, k), dtype=torch.int8, device=dev)
                kairos_cuda_accel.dequant_interleaved_int4_to_int8(w8, layer.qweight, layer.scales_to8,
                                                                   layer.scaled_zeros_to8, 128)
                xq = torch.empty_like(x, dtype=torch.int8)
                sx = torch.empty(m, device=dev, dtype=torch.float16)
                kairos_cuda_accel.quant_fp16_to_int8(xq, x, sx)
                out = torch.empty((m, n), device=dev, dtype=torch.float16)
                awq_backend.w8a8_gemm_forward_cuda(xq, w8, layer.scales_1, sx, out)
                return out

            def ref_fp16():
                w16 = torch.empty((n, k), dtype=torch.float16, device=dev)
                kairos_cuda_accel.dequant_interleaved_int4_to_fp16(w16, layer.qweight, layer.scales, layer.scaled_zeros, 128)
                return x @ w16.T

            cands = {'w8a8': ref_w8a8, 'fp16': ref_fp16}
            if m <= 16:
                cands['w4a16_gemv'] = lambda: awq_backend.gemv_forward_cuda_new(
                    x, layer.qweight, layer.scales, layer.scaled_zeros, m, n, k, 128)
            if m > 32:
                cands['w4a16_gemm'] = lambda: awq_backend.gemm_forward_cuda_new(
                    x, layer.qweight, layer.scales, layer.scaled_zeros)
            # error of both arms against an fp32 product with the dequantized weight, in units of the output RMS,
            # and agreement of each reference kernel with this library's kernel of the same id
            gold = x.float() @ w16_gold.float().T
            rms = gold.pow(2).mean().sqrt()
            ref_us, agree, ref_err, ours_err = {}, {}, {}, {}
            for name, fn in cands.items():
                y_ref = fn().reshape(m, n)
                y_ours = layer._forward(x, m, kb.COMP_TYPE_NAME[name])
                agree[name] = close(y_ref, y_ours)
                if name == 'w8a8':
                    # under the arithmetic rule that follows the reference's CUDA kernels the path is bit-identical
                    with runtime.arithmetic('reference_cuda'):
                        y_rule = cold._forward(x, m, kb.COMP_TYPE_NAME[name])
                    row['w8a8_bit_identical_under_reference_cuda_rule'] = bool(
                        torch.equal(y_rule.view(torch.int16), y_ref.view(torch.int16)))
                ref_err[name] = round(float((y_ref.float() - gold).abs().max() / rms), 4)
                ours_err[name] = round(float((y_ours.float() - gold).abs().max() / rms), 4)
                ref_us[name] = round(timed(fn, reps, warm), 2)
            # the conversions and the activation quantization alone
            w8 = torch.empty((n, k), dtype=torch.int8, device=dev)
            w16 = torch.empty((n, k), dtype=torch.float16, device=dev)
            xq = torch.empty_like(x, dtype=torch.int8)
            sx = torch.empty(m, device=dev, dtype=torch.float16)
            if m == M_LIST[0]:
                row['ref_to_w8_us'] = round(timed(lambda: kairos_cuda_accel.dequant_interleaved_int4_to_int8(
                    w8, layer.qweight, layer.scales_to8, layer.scaled_zeros_to8, 128), 50, 5), 2)
                row['ref_to_f16_us'] = round(timed(lambda: kairos_cuda_accel.dequant_interleaved_int4_to_fp16(
                    w16, layer.qweight, layer.scales, layer.scaled_zeros, 128), 50, 5), 2)
                row['ours_to_w8_us'] = round(timed(lambda: ops.dequant_interleaved_int4_to_int8(
                    w8, layer.qweight, layer.scales_to8, layer.scaled_zeros_to8, 128), 50, 5), 2)
                row['ours_to_f16_us'] = round(timed(lambda: ops.dequant_interleaved_int4_to_fp16(
                    w16, layer.qweight, layer.scales, layer.scaled_zeros, 128), 50, 5), 2)
            row['ref_act_quant_us'] = round(timed(lambda: kairos_cuda_accel.quant_fp16_to_int8(xq, x, sx), reps, warm), 2)
            row['ours_act_quant_us'] = round(timed(lambda: ops.quant_fp16_to_int8(xq, x, sx), reps, warm), 2)

            # ---- this library: the same candidates, converting on every call (cold) and from the cache (warm) ----
            ours_cold, ours_warm = {}, {}
            for name in ('w4a16_gemv', 'w4a16_gemm', 'w8a8', 'fp16'):
                if name == 'w4a16_gemv' and m > 32:
                    continue
                cid = kb.COMP_TYPE_NAME[name]
                ours_warm[name] = round(timed(lambda: layer._forward(x, m, cid), reps, warm), 2)
                ours_cold[name] = round(timed(lambda: cold._forward(x, m, cid), reps, warm), 2)
            row.update({'ref_us': ref_us, 'ref_matches_ours': agree, 'ref_err': ref_err, 'ours_err': ours_err, 'ours_cold_us': ours_cold, 'ours_warm_us': ours_warm,
                        'ref_best_us': min(ref_us.values()), 'ours_cold_best_us': min(ours_cold.values()),
                        'ours_warm_best_us': min(ours_warm.values())})
            print(json.dumps(row), flush=True)
        layer._release()
        cold._release()
    torch.cuda.synchronize()
    print(json.dumps({'device_status': runtime.device_status()}))


if __name__ == '__main__':
    main()
