"""The numpy oracle against fixtures produced by the reference's own Python
functions (tests/golden/make_golden.py).  Integer tensors and fp16 bit patterns
must match exactly; fp16 GEMM outputs within the stated tolerance (the matmul's
fp32 summation order is the only freedom)."""
import glob
import hashlib
import json
import os

import numpy as np
import pytest

from oracle import kairos_oracle as ko

SMALL = sorted(glob.glob(os.path.join(os.path.dirname(__file__), 'golden', 'small_*.npz')))


def bits(a):
    return np.ascontiguousarray(a).view(np.uint16) if a.dtype == np.float16 else a


@pytest.mark.parametrize('path', SMALL, ids=[os.path.basename(p)[6:-4] for p in SMALL])
def test_oracle_matches_reference_small(path):
    g = dict(np.load(path))
    res = ko.from_module(g['W'])
    for key in ('qweight', 'scales', 'scaled_zeros', 'scales_to8', 'scaled_zeros_to8', 'scales_1'):
        assert np.array_equal(bits(res[key]), bits(g[key])), key
    assert np.array_equal(ko.unpack_awq(g['qweight']), g['Q4'])
    assert np.array_equal(ko.pack_awq(g['Q4']), g['qweight'])
    assert np.array_equal(bits(ko.dequant_w16(g['qweight'], g['scales'], g['scaled_zeros'])), bits(g['W16']))
    assert np.array_equal(ko.dequant_w8(g['qweight'], g['scales_to8'], g['scaled_zeros_to8']), g['W8'])
    xq, sx = ko.act_quant(g['X'])
    assert np.array_equal(xq, g['Xq'])
    assert np.array_equal(bits(sx), bits(g['sx']))
    assert np.array_equal(ko.acc_int32(xq, g['W8']), g['acc_i32'])
    assert np.array_equal(bits(ko.fake_quant_int8(g['X'])), bits(g['fake_quant_X']))
    assert np.array_equal(ko.awq_to_qserve(g['qweight'], *g['W'].shape), g['qserve'])
    bias = g.get('bias')
    for name, fn in (('Y_w4a16', ko.y_w4a16), ('Y_w8a8', ko.y_w8a8), ('Y_w8a16', ko.y_w8a16)):
        bad, _ = ko.within_tolerance(fn(g['X'], res, bias), g[name])
        assert bad == 0, name
    # the W8A8 epilogue has no summation freedom: bit-exact
    assert np.array_equal(bits(ko.y_w8a8(g['X'], res, bias)), bits(g['Y_w8a8']))


def test_oracle_dequant_matches_reference_function():
    """W16 as produced by the reference's own dequantize_tensor_awq
    (thirdparty/AWQ/awq_method.py:105-116), called by the fixture generator."""
    g = dict(np.load(os.path.join(os.path.dirname(__file__), 'golden', 'dequant_fn_n64_k384.npz')))
    res = ko.from_module(g['W'])
    assert np.array_equal(res['q4'], g['Q4'])
    w16 = ko.dequant_w16(res['qweight'], res['scales'], res['scaled_zeros'])
    assert np.array_equal(bits(w16), bits(g['W16_fn']))
    # the per-(row, group) factors the function was given are the ones the resident tensors hold
    n, k = g['W'].shape
    assert np.array_equal(bits(res['scales'][:k // 128].T), bits(g['scale_f']))


def test_oracle_matches_reference_config0():
    """M=16, K=N=4096, seed 0: digests of every tensor on the path."""
    dg = json.load(open(os.path.join(os.path.dirname(__file__), 'golden', 'config0_digests.json')))
    x, w = ko.make_case(dg['M'], dg['K'], dg['N'], seed=dg['seed'])
    res = ko.from_module(w)
    xq, sx = ko.act_quant(x)
    w8 = ko.dequant_w8(res['qweight'], res['scales_to8'], res['scaled_zeros_to8'])
    got = {
        'X': x, 'W': w, 'qweight': res['qweight'], 'scales': res['scales'],
        'scaled_zeros': res['scaled_zeros'], 'scales_to8': res['scales_to8'],
        'scaled_zeros_to8': res['scaled_zeros_to8'], 'scales_1': res['scales_1'],
        'Q4': res['q4'], 'W16': ko.dequant_w16(res['qweight'], res['scales'], res['scaled_zeros']),
        'W8': w8, 'Xq': xq, 'sx': sx, 'acc_i32': ko.acc_int32(xq, w8),
        'Y_w8a8': ko.y_w8a8(x, res), 'qserve': ko.awq_to_qserve(res['qweight'], dg['N'], dg['K']),
    }
    for key, val in got.items():
        h = hashlib.sha256(np.ascontiguousarray(val).tobytes()).hexdigest()
        assert h == dg['sha256'][key], key
    for name, fn in (('Y_w4a16', ko.y_w4a16), ('Y_w8a16', ko.y_w8a16)):
        y = fn(x, res).reshape(-1).astype(np.float32)
        s = dg['samples'][name]
        ref = np.array(s['val'], np.float32)
        rms = float(np.sqrt(np.mean(y.astype(np.float64) ** 2)))
        assert np.all(np.abs(y[s['idx']] - ref) <= 1e-2 * np.abs(ref) + 1e-2 * rms), name


def test_lut_known_answers():
    """Answers of the reference's C++ LUT class on the shipped Llama/Qwen tables."""
    cases = json.load(open(os.path.join(os.path.dirname(__file__), 'golden', 'lut_known_answers.json')))
    assert cases
    for c in cases:
        t = ko.LUT()
        for r, cid in c['records']:
            t.record(r, cid)
        assert [t.get(q) for q in c['queries']] == c['answers'], (c['profile'], c['table'])


def test_pack_round_trip_and_element_map():
    rng = np.random.default_rng(0)
    q = rng.integers(0, 16, size=(64, 256), dtype=np.uint8)
    p = ko.pack_awq(q)
    assert np.array_equal(ko.unpack_awq(p), q)
    u = p.view(np.uint16)
    for _ in range(200):
        n, k = int(rng.integers(64)), int(rng.integers(256))
        n0, n1 = divmod(n, 4)
        k0, r = divmod(k, 64)
        a, r = divmod(r, 32)
        b, r = divmod(r, 8)
        c, d = divmod(r, 2)
        assert (int(u[n0, 64 * k0 + 16 * n1 + 8 * a + 2 * c + d]) >> (4 * b)) & 0xF == q[n, k]
