"""Generate the golden fixtures from the REFERENCE's own Python functions.

Run once, in a container that holds the reference sources:

    TORCH_COMPILE_DISABLE=1 python tests/golden/make_golden.py /path/to/reference

It imports ``kairos.dynamic_linear`` / ``kairos.quantization`` /
``thirdparty.AWQ.awq_method`` from that tree (with empty stand-ins for the CUDA
extension modules, which are only touched by the GPU forward) and writes

  * ``small_*.npz``           full tensors of small cases (inputs + every
                              intermediate of the path), and
  * ``config0_digests.json``  SHA-256 digests + sampled values of the full-size
                              M=16, K=N=4096 case (too large to commit whole),
  * ``lut_known_answers.json`` answers of the reference's C++ LUT class, compiled
                              from its header, for the shipped Llama tables,
  * ``dequant_fn_n64_k384.npz`` output of the reference's own ``dequantize_tensor_awq``
                              (thirdparty/AWQ/awq_method.py:105-116) on the per-(row, group)
                              factors its ``from_module`` derives.

The fixtures travel with the repository; the reference tree does not.
"""
import hashlib
import json
import os
import subprocess
import sys
import tempfile
import types

import numpy as np

os.environ.setdefault('TORCH_COMPILE_DISABLE', '1')
import torch  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle.kairos_oracle import make_case  # noqa: E402  (input generator only)


def import_reference(ref_root):
    sys.path.insert(0, ref_root)
    for name in ('awq_backend', 'kairos_cuda_accel'):
        sys.modules[name] = types.ModuleType(name)
    colorama = types.ModuleType('colorama')

    class _Any:
        def __getattr__(self, _):
            return ''
    colorama.Fore = colorama.Style = colorama.Back = _Any()
    colorama.init = lambda *a, **k: None
    sys.modules['colorama'] = colorama
    import kairos.dynamic_linear as dl
    import kairos.quantization as qz
    import thirdparty.AWQ.awq_method as awq
    return dl, qz, awq


def ref_unpack_awq(packed):
    """test/depacking.py:22-38 of the reference, verbatim semantics via torch ops."""
    n_out, k = packed.shape
    nib = torch.stack([(packed >> s) & 0xF for s in (0, 4, 8, 12)], dim=-1)
    nib = nib.reshape(n_out, k // 64, 4, 2, 4, 2, 4).permute(0, 2, 1, 3, 6, 4, 5)
    return nib.reshape(n_out * 4, k)


def ref_pack_qserve(q):
    """test/test_trans_layout.py:7-13 of the reference."""
    n, k = q.shape
    p = (q.reshape(n // 32, 2, 2, 8, k // 32, 2, 4, 4).permute(0, 4, 3, 6, 5, 2, 7, 1).contiguous())
    p = p.to(torch.int8)
    p = (p[..., 1] << 4) + p[..., 0]
    return p.reshape(n, k // 2)


def run_reference(dl, qz, awq, x16, w16, bias=None):
    n, k = w16.shape
    lin = torch.nn.Linear(k, n, bias=bias is not None, dtype=torch.float16)
    lin.weight.data = torch.from_numpy(w16.copy())
    if bias is not None:
        lin.bias.data = torch.from_numpy(bias.copy())
    ql = dl.DynamicLinear.from_module(lin, 'cpu')
    x = torch.from_numpy(x16.copy())
    q4 = ref_unpack_awq(ql.qweight.to(torch.int32) & 0xFFFF)
    g = k // 128

    def expand(f):
        return f[:g].T.contiguous().repeat_interleave(128, dim=1)

    # W4 -> fp16: q*s then +sz, each rounded to fp16 (awq_method.py:105-116 mul_/add_)
    w16_deq = q4.to(torch.float16).mul_(expand(ql.scales)).add_(expand(ql.scaled_zeros))
    # W4 -> int8: same arithmetic with the *_to8 factors, then truncation (dequant_i4_to_i8.cu:143)
    w8 = q4.to(torch.float16).mul_(expand(ql.scales_to8)).add_(expand(ql.scaled_zeros_to8)).to(torch.int8)
    xq, cfg = qz.quantize_tensor_int8(x, 'S', -1)
    sx = cfg['scale'].view(-1)
    acc = (xq.to(torch.int64) @ w8.to(torch.int64).T).to(torch.int32)
    y_w4a16 = (x.float() @ w16_deq.float().T).half()
    y_w8a8 = (acc.float() * (ql.scales_1.float()[None, :] * sx.float()[:, None])).half()
    w16_from8 = w8.half() * ql.scales_1.view(-1, 1)
    y_w8a16 = (x.float() @ w16_from8.float().T).half()
    if bias is not None:
        b = torch.from_numpy(bias.copy())
        y_w4a16 = y_w4a16 + b
        y_w8a8 = y_w8a8 + b
        y_w8a16 = y_w8a16 + b
    out = {
        'X': x16, 'W': w16,
        'qweight': ql.qweight.numpy(), 'scales': ql.scales.numpy(),
        'scaled_zeros': ql.scaled_zeros.numpy(), 'scales_to8': ql.scales_to8.numpy(),
        'scaled_zeros_to8': ql.scaled_zeros_to8.numpy(), 'scales_1': ql.scales_1.numpy(),
        'Q4': q4.to(torch.uint8).numpy(), 'W16': w16_deq.numpy(), 'W8': w8.numpy(),
        'Xq': xq.numpy(), 'sx': sx.numpy(), 'acc_i32': acc.numpy(),
        'Y_w4a16': y_w4a16.numpy(), 'Y_w8a8': y_w8a8.numpy(), 'Y_w8a16': y_w8a16.numpy(),
        'fake_quant_X': qz.simu_quantize_tensor(x, 8, 'S').numpy(),
        'qserve': ref_pack_qserve(q4.to(torch.int32)).numpy(),
    }
    if bias is not None:
        out['bias'] = bias
    return out


def dequant_fn_fixture(dl, qz, awq, w16):
    """W16 as the reference's dequantize_tensor_awq computes it.  The factors are re-derived with the
    reference's own functions in the order of DynamicLinear.from_module (kairos/dynamic_linear.py:95-110):
    int8 per row, uint4 per group of 128, scale_f = scale_2 * scale_1."""
    w = torch.from_numpy(w16.copy())
    n, k = w.shape
    w8, cfg1 = qz.quantize_tensor_int8(w, max_int=127)
    w4, cfg2 = dl.kairos_quantize_tensor_int4(w8, group_size=128)
    scale_f = cfg2['scale_f'].view(n, -1) * cfg1['scale']
    zero_f = cfg2['zero_pt_f'].view(n, -1)
    w16_fn = awq.dequantize_tensor_awq(w4.clone().reshape(n, k), scale_f.reshape(n, -1), zero_f.reshape(n, -1), 128)
    return {'W': w16, 'Q4': w4.reshape(n, k).to(torch.uint8).numpy(), 'scale_f': scale_f.numpy(),
            'zero_f': zero_f.to(torch.float16).numpy(), 'W16_fn': w16_fn.reshape(n, k).numpy()}


def digest(a):
    a = np.ascontiguousarray(a)
    return hashlib.sha256(a.tobytes()).hexdigest()


def lut_known_answers(ref_root):
    """Compile the reference's header-only LUT class and query it."""
    src = r'''
#include "lut.h"
#include <cstdio>
#include <cstdlib>
int main(int argc, char** argv) {
  LUT t; int i = 1; int nrec = atoi(argv[i++]);
  for (int r = 0; r < nrec; ++r) { int a = atoi(argv[i++]); int b = atoi(argv[i++]); t.record(a, b); }
  for (; i < argc; ++i) printf("%d ", t.get(atoi(argv[i])));
  return 0; }
'''
    inc = os.path.join(ref_root, 'kernels/csrc/kairos_kernel/lut')
    with tempfile.TemporaryDirectory() as d:
        with open(os.path.join(d, 'q.cpp'), 'w') as f:
            f.write(src)
        exe = os.path.join(d, 'q')
        subprocess.check_call(['g++', '-std=c++17', '-O1', '-I', inc, os.path.join(d, 'q.cpp'), '-o', exe])
        names = {'w4a16_gemm': 0, 'w4a16_gemv': 1, 'w8a8': 2, 'w8a16_gemm': 3, 'w8a16_gemv': 4, 'fp16': 5,
                 'w4a16_marlin': 6, 'w4a8_qserve': 7}
        out = []
        for prof in ('prof_llama', 'prof_qwen'):
            tables = json.load(open(os.path.join(ref_root, prof, 'seg_perf_list.pt')))
            for ti, table in enumerate(tables):
                recs = [(int(t[0]), names[t[1]]) for t in table]
                qs = sorted(set([0, 1, 2, 3] + [r + d for r, _ in recs for d in (-1, 0, 1, 2)] + [100000]))
                qs = [q for q in qs if q >= 0]
                # ask twice in a row as well, to exercise the memo
                qs = qs + qs[::-1] + [qs[0], qs[0]]
                args = [str(len(recs))] + [str(v) for r in recs for v in r] + [str(q) for q in qs]
                ans = subprocess.check_output([exe] + args).decode().split()
                out.append({'profile': prof, 'table': ti, 'records': recs, 'queries': qs,
                            'answers': [int(a) for a in ans]})
        return out


def main():
    if len(sys.argv) < 2 or not os.path.isdir(sys.argv[1]):
        raise SystemExit('usage: make_golden.py <root of the reference source tree> [dequant_fn]')
    ref_root = sys.argv[1]
    dl, qz, awq = import_reference(ref_root)

    # the reference's dequantize_tensor_awq itself (one fixture; the small_* cases restate its mul_/add_)
    _, w16 = make_case(1, 384, 64, seed=11)
    fx = dequant_fn_fixture(dl, qz, awq, w16)
    full = run_reference(dl, qz, awq, make_case(1, 384, 64, seed=11)[0], w16)
    assert np.array_equal(fx['W16_fn'].view(np.uint16), full['W16'].view(np.uint16)), \
        'dequantize_tensor_awq and the restated mul_/add_ disagree'
    assert np.array_equal(fx['Q4'], full['Q4'])
    np.savez_compressed(os.path.join(HERE, 'dequant_fn_n64_k384.npz'), **fx)
    print('wrote dequant_fn fixture')
    if len(sys.argv) > 2 and sys.argv[2] == 'dequant_fn':
        return

    small = [  # (tag, M, K, N, seed, bias)
        ('n64_k256_m5', 5, 256, 64, 1, False),
        ('n128_k512_m16', 16, 512, 128, 2, False),
        ('n96_k1152_m33_bias', 33, 1152, 96, 3, True),   # G=9 -> G_pad=16, ragged M, bias
        ('n256_k128_m1', 1, 128, 256, 4, False),
    ]
    for tag, m, k, n, seed, has_bias in small:
        x16, w16 = make_case(m, k, n, seed=seed)
        bias = None
        if has_bias:
            bias = (np.random.default_rng(seed + 100).standard_normal(n) * 0.1).astype(np.float16)
        r = run_reference(dl, qz, awq, x16, w16, bias)
        np.savez_compressed(os.path.join(HERE, f'small_{tag}.npz'), **r)
        print('wrote', tag)

    # an all-zero token row and an all-zero weight row exercise the clamp() paths.
    # (A constant NON-zero weight group is left out on purpose: the reference then
    # produces an infinite zero point and casts inf to int8, which is undefined.)
    x16, w16 = make_case(4, 256, 32, seed=7)
    x16[2, :] = 0
    w16[5, :] = 0
    r = run_reference(dl, qz, awq, x16, w16)
    np.savez_compressed(os.path.join(HERE, 'small_degenerate.npz'), **r)

    # config 0: M=16, K=N=4096, seed 0 -> digests and samples only
    x16, w16 = make_case(16, 4096, 4096, seed=0)
    r = run_reference(dl, qz, awq, x16, w16)
    rng = np.random.default_rng(123)
    dg = {'M': 16, 'K': 4096, 'N': 4096, 'seed': 0, 'sha256': {}, 'samples': {}}
    for key, val in r.items():
        dg['sha256'][key] = digest(val)
        flat = np.ascontiguousarray(val).reshape(-1)
        idx = rng.integers(0, flat.size, size=16)
        dg['samples'][key] = {'idx': idx.tolist(), 'val': [float(v) for v in flat[idx]]}
    with open(os.path.join(HERE, 'config0_digests.json'), 'w') as f:
        json.dump(dg, f, indent=1)
    print('wrote config0 digests')

    with open(os.path.join(HERE, 'lut_known_answers.json'), 'w') as f:
        json.dump(lut_known_answers(ref_root), f)
    print('wrote LUT known answers')


if __name__ == '__main__':
    main()
