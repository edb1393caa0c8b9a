"""Oracle restatements of the reference's CUDA rounding against outputs of the reference's own extension
(tests/golden/ref_cuda_*.npz, written on a B200 by tests/golden/make_golden_cuda.py)."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, '..', 'oracle'))
import kairos_oracle as oracle  # noqa: E402

GOLDEN = os.path.join(HERE, 'golden')


def _load(name):
    path = os.path.join(GOLDEN, name)
    if not os.path.exists(path):
        pytest.skip(f'{name} not generated yet')
    return np.load(path)


def test_inputs_are_the_seeded_case():
    g = _load('ref_cuda_case.npz')
    x, w = oracle.make_case(16, 512, 64, seed=5)
    res = oracle.from_module(w)
    assert np.array_equal(g['x'].view(np.uint16), x.view(np.uint16))
    for name in ('qweight', 'scales', 'scaled_zeros', 'scales_to8', 'scaled_zeros_to8', 'scales_1'):
        assert np.array_equal(np.ascontiguousarray(res[name]).view(np.uint8), g[name].view(np.uint8)), name


def test_conversions_single_rounding():
    g = _load('ref_cuda_case.npz')
    w16 = oracle.dequant_w16_cuda(g['qweight'], g['scales'], g['scaled_zeros'])
    assert np.array_equal(w16.view(np.uint16), g['w16'].view(np.uint16))
    w8 = oracle.dequant_w8_cuda(g['qweight'], g['scales_to8'], g['scaled_zeros_to8'])
    assert np.array_equal(w8, g['w8'])
    # and the torch rule really is a different function on these inputs
    assert not np.array_equal(oracle.dequant_w8(g['qweight'], g['scales_to8'], g['scaled_zeros_to8']), g['w8'])


def test_activation_quantization_outside_the_boundary_cases():
    for name in ('ref_cuda_case.npz', 'ref_cuda_ties.npz'):
        g = _load(name)
        q, sx, unsure_q, unsure_sx = oracle.act_quant_cuda(g['x'])
        ok = ~unsure_q
        assert np.array_equal(q[ok], g['xq'][ok]), name
        assert np.array_equal(sx.view(np.uint16)[~unsure_sx], g['sx'].view(np.uint16)[~unsure_sx]), name
        assert ok.mean() > 0.3


def test_every_scale():
    g = _load('ref_cuda_scales.npz')
    amax = g['amax_bits'].view(np.float16)
    rows = np.zeros((amax.size, 16), np.float16)
    rows[:, 3] = amax
    _, sx, _, unsure = oracle.act_quant_cuda(rows)
    assert np.array_equal(sx.view(np.uint16)[~unsure], g['sx_bits'][~unsure])
    assert unsure.mean() < 0.01
    assert np.all(g['q_of_amax'] == 127)


def test_w8a8_gemm_epilogue():
    g = _load('ref_cuda_case.npz')
    y = oracle.y_w8a8_cuda(g['xq'], g['sx'], g['w8'], g['scales_1'].reshape(-1))
    assert np.array_equal(y.view(np.uint16), g['y_w8a8'].view(np.uint16))
