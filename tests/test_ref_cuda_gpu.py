"""Arithmetic rule 'reference_cuda': activation quantization, both weight conversions and the whole W8A8
path must return the bits the reference's own CUDA extension returns.

Two checkers: the committed fixtures that extension produced (tests/golden/ref_cuda_*.npz), and, when the
built extension itself is present next to the repository's baseline scripts (baseline/_ref, made by
baseline/build_ref_kernels.sh), the extension run live on the same GPU on full-size inputs."""
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import kairos_oracle as ko  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, 'golden')
REF_EXT = os.path.join(HERE, '..', 'baseline', '_ref')
NAMES = ('qweight', 'scales', 'scaled_zeros', 'scales_to8', 'scaled_zeros_to8', 'scales_1')


@pytest.fixture(scope='module')
def kb():
    import kairos_b200
    from kairos_b200 import ops, runtime
    assert torch.cuda.is_available()
    with runtime.arithmetic('reference_cuda'):
        yield kairos_b200, ops, runtime
        torch.cuda.synchronize()
    assert runtime.get_arithmetic() == 'torch'
    assert runtime.device_status() == 0


@pytest.fixture(scope='module')
def ref_ext():
    if not os.path.isdir(REF_EXT):
        pytest.skip('the reference extension is not built here (baseline/build_ref_kernels.sh)')
    sys.path.insert(0, REF_EXT)
    try:
        import awq_backend
        import kairos_cuda_accel
    except ImportError as exc:
        pytest.skip(f'the reference extension does not load: {exc}')
    return kairos_cuda_accel, awq_backend


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def golden(name):
    path = os.path.join(GOLDEN, name)
    if not os.path.exists(path):
        pytest.skip(f'{name} not generated yet')
    return np.load(path)


def ours_quant(ops, x):
    xq = torch.empty_like(x, dtype=torch.int8)
    sx = torch.empty(x.shape[0], device=x.device, dtype=torch.float16)
    ops.quant_fp16_to_int8(xq, x, sx)
    return xq, sx


def same_bits(a, b):
    if a.dtype == torch.float16:
        a, b = a.view(torch.int16), b.view(torch.int16)
    return bool(torch.equal(a, b))


# ---------------------------------------------------------------- committed fixtures
def test_fixture_case_every_stage(kb):
    kairos_b200, ops, _ = kb
    g = golden('ref_cuda_case.npz')
    t = {k: dev(g[k]) for k in NAMES}
    n, k = g['w8'].shape
    w16 = torch.empty((n, k), dtype=torch.float16, device='cuda')
    ops.dequant_interleaved_int4_to_fp16(w16, t['qweight'], t['scales'], t['scaled_zeros'], 128)
    assert np.array_equal(w16.cpu().numpy().view(np.uint16), g['w16'].view(np.uint16))
    w8 = torch.empty((n, k), dtype=torch.int8, device='cuda')
    ops.dequant_interleaved_int4_to_int8(w8, t['qweight'], t['scales_to8'], t['scaled_zeros_to8'], 128)
    assert np.array_equal(w8.cpu().numpy(), g['w8'])
    xq, sx = ours_quant(ops, dev(g['x']))
    assert np.array_equal(xq.cpu().numpy(), g['xq'])
    assert np.array_equal(sx.cpu().numpy().view(np.uint16), g['sx'].view(np.uint16))
    # the whole path, through the layer object: kernel id 2 of DynamicLinear._forward
    x, w = ko.make_case(16, 512, 64, seed=5)
    lin = torch.nn.Linear(512, 64, bias=False, dtype=torch.float16)
    lin.weight.data = torch.from_numpy(w.copy())
    layer = kairos_b200.DynamicLinear.from_module(lin.cuda(), 'cuda')
    y = layer._forward(dev(x), 16, 2)
    assert np.array_equal(y.cpu().numpy().view(np.uint16), g['y_w8a8'].view(np.uint16))


def test_fixture_every_scale_and_the_rounding_boundaries(kb):
    _, ops, _ = kb
    g = golden('ref_cuda_scales.npz')
    rows = np.zeros((g['amax_bits'].size, 16), np.float16)
    rows[:, 3] = g['amax_bits'].view(np.float16)
    xq, sx = ours_quant(ops, dev(rows))
    assert np.array_equal(sx.cpu().numpy().view(np.uint16), g['sx_bits'])
    assert np.array_equal(xq.cpu().numpy()[:, 3], g['q_of_amax'])
    t = golden('ref_cuda_ties.npz')
    xq, sx = ours_quant(ops, dev(t['x']))
    assert np.array_equal(xq.cpu().numpy(), t['xq'])
    assert np.array_equal(sx.cpu().numpy().view(np.uint16), t['sx'].view(np.uint16))


def test_rule_is_part_of_the_cache_key(kb):
    """A layer converted under one rule is converted again, not served from the cache, under the other."""
    kairos_b200, ops, runtime = kb
    x, w = ko.make_case(8, 512, 256, seed=9)
    res = ko.from_module(w)
    lin = torch.nn.Linear(512, 256, bias=False, dtype=torch.float16)
    lin.weight.data = torch.from_numpy(w.copy())
    layer = kairos_b200.DynamicLinear.from_module(lin.cuda(), 'cuda')
    xd = dev(x)
    xq, sx, _, _ = ko.act_quant_cuda(x)
    w8 = ko.dequant_w8_cuda(res['qweight'], res['scales_to8'], res['scaled_zeros_to8'])
    y_cuda = layer._forward(xd, 8, 2).cpu().numpy()
    assert np.array_equal(y_cuda.view(np.uint16), ko.y_w8a8_cuda(xq, sx, w8, res['scales_1'].reshape(-1)).view(np.uint16))
    with runtime.arithmetic('torch'):
        y_torch = layer._forward(xd, 8, 2).cpu().numpy()
        assert np.array_equal(y_torch.view(np.uint16), ko.y_w8a8(x, res).view(np.uint16))
    y_again = layer._forward(xd, 8, 2).cpu().numpy()
    assert np.array_equal(y_again.view(np.uint16), y_cuda.view(np.uint16))
    assert not np.array_equal(y_torch.view(np.uint16), y_cuda.view(np.uint16))


# ---------------------------------------------------------------- the extension itself, live
@pytest.mark.parametrize('k,n', [(4096, 4096), (4096, 1024), (14336, 4096), (4096, 14336)])
def test_live_conversions(kb, ref_ext, k, n):
    _, ops, _ = kb
    accel, _ = ref_ext
    _, w = ko.make_case(1, k, n, seed=k + n)
    res = ko.from_module(w)
    t = {key: dev(res[key]) for key in NAMES}
    for dtype, fn_ref, fn_ours, s, z in (
            (torch.float16, accel.dequant_interleaved_int4_to_fp16, ops.dequant_interleaved_int4_to_fp16, 'scales', 'scaled_zeros'),
            (torch.int8, accel.dequant_interleaved_int4_to_int8, ops.dequant_interleaved_int4_to_int8, 'scales_to8', 'scaled_zeros_to8')):
        a = torch.empty((n, k), dtype=dtype, device='cuda')
        b = torch.empty_like(a)
        fn_ref(a, t['qweight'], t[s], t[z], 128)
        fn_ours(b, t['qweight'], t[s], t[z], 128)
        assert same_bits(a, b), (dtype, k, n)


def test_live_activation_quantization_every_amax(kb, ref_ext):
    """One token per positive finite fp16 amax (31743 tokens of 1024 elements drawn inside [-amax, amax])."""
    _, ops, _ = kb
    accel, _ = ref_ext
    g = torch.Generator(device='cuda').manual_seed(1)
    bits = torch.arange(1, 0x7c00, dtype=torch.int16, device='cuda')
    amax = bits.view(torch.float16)
    x = ((torch.rand((bits.numel(), 1024), device='cuda', generator=g) * 2 - 1) * amax.float()[:, None]).half()
    x = torch.minimum(torch.maximum(x, -amax[:, None]), amax[:, None])
    x[:, 7] = amax
    a = torch.empty_like(x, dtype=torch.int8)
    sa = torch.empty(x.shape[0], device='cuda', dtype=torch.float16)
    accel.quant_fp16_to_int8(a, x, sa)
    b, sb = ours_quant(ops, x)
    assert same_bits(sa, sb)
    assert same_bits(a, b)


@pytest.mark.parametrize('m,k,n', [(1, 4096, 4096), (64, 4096, 1024), (300, 14336, 4096), (2048, 4096, 14336)])
def test_live_w8a8_path(kb, ref_ext, m, k, n):
    """Kernel id 2 end to end: the reference's three kernels chained as its DynamicLinear._forward chains
    them (kairos/dynamic_linear.py:143-155) against this library's layer object."""
    kairos_b200, _, _ = kb
    accel, awq = ref_ext
    x, w = ko.make_case(m, k, n, seed=m)
    lin = torch.nn.Linear(k, n, bias=False, dtype=torch.float16)
    lin.weight.data = torch.from_numpy(w.copy())
    layer = kairos_b200.DynamicLinear.from_module(lin.cuda(), 'cuda')
    xd = dev(x)
    w8 = torch.empty((n, k), dtype=torch.int8, device='cuda')
    accel.dequant_interleaved_int4_to_int8(w8, layer.qweight, layer.scales_to8, layer.scaled_zeros_to8, 128)
    xq = torch.empty_like(xd, dtype=torch.int8)
    sx = torch.empty(m, device='cuda', dtype=torch.float16)
    accel.quant_fp16_to_int8(xq, xd, sx)
    y_ref = torch.empty((m, n), device='cuda', dtype=torch.float16)
    awq.w8a8_gemm_forward_cuda(xq, w8, layer.scales_1, sx, y_ref)
    y = layer._forward(xd, m, 2)
    assert same_bits(y_ref, y)
