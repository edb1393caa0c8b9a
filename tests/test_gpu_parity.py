"""GPU parity: every kernel of the switched-linear path, called through the C ABI, against the
CPU oracle on the same seeded inputs.  Integer stages (activation quantization, both weight
conversions, the nibble permutation, the W8A8 int32 accumulators and its fp16 epilogue) must be
bit-exact; fp16 GEMM/GEMV outputs must satisfy |y - ref| <= 1e-2*|ref| + 1e-2*RMS(ref)."""
import glob
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import kairos_oracle as ko  # noqa: E402

RTOL = ATOL = 1e-2
GOLDEN = os.path.join(os.path.dirname(__file__), 'golden')
SMALL = sorted(glob.glob(os.path.join(GOLDEN, 'small_*.npz')))


@pytest.fixture(scope='module')
def kb():
    import kairos_b200
    from kairos_b200 import ops, runtime
    assert torch.cuda.is_available()
    yield kairos_b200, ops, runtime
    torch.cuda.synchronize()
    assert runtime.device_status() == 0, 'a kernel reported a bounded wait that ran out'


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint16) if a.dtype == np.float16 else a


def assert_close(y, ref, what):
    bad, rms = ko.within_tolerance(y, ref, RTOL, ATOL)
    err = float(np.abs(np.asarray(y, np.float32) - np.asarray(ref, np.float32)).max())
    assert bad == 0, f'{what}: {bad} of {ref.size} outside tolerance (max abs err {err:.4g}, rms {rms:.4g})'


_case_cache = {}


def case(m, k, n, seed=0):
    key = (m, k, n, seed)
    if key not in _case_cache:
        x, w = ko.make_case(m, k, n, seed=seed)
        _case_cache[key] = (x, w, ko.from_module(w))
    return _case_cache[key]


def resident(res):
    return {k: dev(res[k]) for k in ('qweight', 'scales', 'scaled_zeros', 'scales_to8', 'scaled_zeros_to8', 'scales_1')}


# ------------------------------------------------------------------ a6
@pytest.mark.parametrize('m,k', [(1, 128), (5, 256), (16, 4096), (33, 1152), (7, 14336), (3, 28672), (300, 512)])
def test_act_quant_bit_exact(kb, m, k):
    _, ops, _ = kb
    x, _ = ko.make_case(m, k, 4, seed=m + k)
    if m > 2:
        x[1, :] = 0                      # all-zero token: scale clamps at 1e-7/127
        x[2, :] = np.float16(65504.0)    # largest fp16
    xd = dev(x)
    q = torch.empty((m, k), dtype=torch.int8, device='cuda')
    s = torch.empty((m,), dtype=torch.float16, device='cuda')
    ops.quant_fp16_to_int8(q, xd, s)
    q_ref, s_ref = ko.act_quant(x)
    assert np.array_equal(q.cpu().numpy(), q_ref)
    assert np.array_equal(bits(s.cpu().numpy()), bits(s_ref))


def test_act_quant_rounding_boundaries(kb):
    """Quotients on and next to the k + 0.5 rounding boundaries: rows whose scale is a power of two put
    every half-integer quotient exactly on a tie (round half to even); rows with other scales put
    quotients within a few ulp of a boundary, where only the correctly rounded IEEE quotient decides."""
    _, ops, _ = kb
    k = 512
    rows = []
    for amax in (127.0, 254.0, 63.5, 508.0):                 # scale 1, 2, 0.5, 4: x / scale = j + 0.5 exactly
        sc = amax / 127.0
        r = (np.arange(k, dtype=np.float32) % 250 - 125 + 0.5) * sc
        r[0] = amax
        rows.append(r)
    rng = np.random.default_rng(3)
    for amax in (100.0, 3.1, 777.0, 0.013, 41.7, 1999.0):    # near-boundary quotients under awkward scales
        sc = np.float32(np.float16(amax)) / np.float32(127.0)
        j = rng.integers(-126, 126, k).astype(np.float32) + 0.5
        r = (j * sc).astype(np.float16).astype(np.float32)   # fp16 rounding scatters them around the boundary
        r[0] = np.float16(amax)
        rows.append(r)
    x = np.stack(rows).astype(np.float16)
    m = x.shape[0]
    q = torch.empty((m, k), dtype=torch.int8, device='cuda')
    s = torch.empty((m,), dtype=torch.float16, device='cuda')
    ops.quant_fp16_to_int8(q, dev(x), s)
    q_ref, s_ref = ko.act_quant(x)
    assert np.array_equal(bits(s.cpu().numpy()), bits(s_ref))
    assert np.array_equal(q.cpu().numpy(), q_ref)


# ------------------------------------------------------------------ a7, a8, permute
@pytest.mark.parametrize('path', SMALL, ids=[os.path.basename(p)[6:-4] for p in SMALL])
def test_conversions_match_reference_fixtures(kb, path):
    _, ops, _ = kb
    g = dict(np.load(path))
    n, k = g['W'].shape
    w8 = torch.empty((n, k), dtype=torch.int8, device='cuda')
    ops.dequant_interleaved_int4_to_int8(w8, dev(g['qweight']), dev(g['scales_to8']), dev(g['scaled_zeros_to8']), 128)
    assert np.array_equal(w8.cpu().numpy(), g['W8'])
    w16 = torch.empty((n, k), dtype=torch.float16, device='cuda')
    ops.dequant_interleaved_int4_to_fp16(w16, dev(g['qweight']), dev(g['scales']), dev(g['scaled_zeros']), 128)
    assert np.array_equal(bits(w16.cpu().numpy()), bits(g['W16']))
    if n % 32 == 0:
        qs = ops.trans_layout_c16_to_c8_awq(dev(g['qweight']), n, k)
        assert np.array_equal(qs.cpu().numpy(), g['qserve'])
    # activation quantization against the reference fixture as well
    m = g['X'].shape[0]
    q = torch.empty((m, k), dtype=torch.int8, device='cuda')
    s = torch.empty((m,), dtype=torch.float16, device='cuda')
    ops.quant_fp16_to_int8(q, dev(g['X']), s)
    assert np.array_equal(q.cpu().numpy(), g['Xq'])
    assert np.array_equal(bits(s.cpu().numpy()), bits(g['sx']))


@pytest.mark.parametrize('k,n', [(4096, 4096), (4096, 1024), (14336, 4096), (3584, 512), (1152, 96)])
def test_conversions_bit_exact_full_shapes(kb, k, n):
    _, ops, _ = kb
    _, _, res = case(4, k, n, seed=k + n)
    r = resident(res)
    w8 = torch.empty((n, k), dtype=torch.int8, device='cuda')
    ops.dequant_interleaved_int4_to_int8(w8, r['qweight'], r['scales_to8'], r['scaled_zeros_to8'], 128)
    assert np.array_equal(w8.cpu().numpy(), ko.dequant_w8(res['qweight'], res['scales_to8'], res['scaled_zeros_to8']))
    w16 = torch.empty((n, k), dtype=torch.float16, device='cuda')
    ops.dequant_interleaved_int4_to_fp16(w16, r['qweight'], r['scales'], r['scaled_zeros'], 128)
    assert np.array_equal(bits(w16.cpu().numpy()),
                          bits(ko.dequant_w16(res['qweight'], res['scales'], res['scaled_zeros'])))
    if n % 32 == 0:
        qs = ops.trans_layout_c16_to_c8_awq(r['qweight'], n, k)
        assert np.array_equal(qs.cpu().numpy(), ko.awq_to_qserve(res['qweight'], n, k))


# ------------------------------------------------------------------ a9 GEMV
@pytest.mark.parametrize('m,k,n', [(1, 128, 256), (1, 4096, 4096), (2, 4096, 1024), (3, 1152, 96), (4, 14336, 4096),
                                   (5, 256, 64), (8, 4096, 4096), (13, 512, 128), (16, 4096, 4096),
                                   (32, 3584, 512)])
def test_gemv(kb, m, k, n):
    _, ops, _ = kb
    x, _, res = case(m, k, n, seed=m)
    r = resident(res)
    y = ops.gemv_cuda_core(dev(x), r['qweight'], r['scales'], r['scaled_zeros'], m, n, k)
    assert_close(y.cpu().numpy(), ko.y_w4a16(x, res), f'gemv m={m} k={k} n={n}')
    y = ops.gemv_forward_cuda_new(dev(x), r['qweight'], r['scales'], r['scaled_zeros'], m, n, k, 128)
    assert_close(y.cpu().numpy(), ko.y_w4a16(x, res), f'small-batch entry m={m} k={k} n={n}')


@pytest.mark.parametrize('m,k,n', [(1, 128, 256), (1, 4096, 4096), (2, 4096, 1024), (3, 1152, 96), (4, 14336, 4096),
                                   (5, 256, 64), (8, 4096, 14336), (9, 512, 128), (13, 3584, 512),
                                   (16, 4096, 4096), (16, 18944, 3584),
                                   # 17..32 tokens (four token tiles), one row block of a tile missing (N % 32 = 8, 24),
                                   # every cluster size (1, 2, 4, 8 K slices) and both rows-per-warp variants
                                   (17, 1024, 520), (24, 4096, 1024), (32, 4096, 4096), (32, 3584, 512), (31, 128, 40),
                                   (6, 4096, 4104), (7, 2048, 8200), (12, 4096, 2072), (1, 28672, 8192), (2, 8192, 28672),
                                   (8, 384, 1032), (3, 128, 8),
                                   # long K with row tiles enough for the GPU: two K slices all the same; four row blocks at M = 3, 4
                                   (1, 8192, 11872), (4, 8192, 7168), (3, 4096, 14336), (2, 4096, 14336), (1, 256, 14344)])
def test_decode_mma(kb, m, k, n):
    _, ops, _ = kb
    x, _, res = case(m, k, n, seed=m)
    r = resident(res)
    y = ops.decode_forward(dev(x), r['qweight'], r['scales'], r['scaled_zeros'], m, n, k)
    assert_close(y.cpu().numpy(), ko.y_w4a16(x, res), f'decode m={m} k={k} n={n}')


@pytest.mark.parametrize('m,k,n', [(2, 4096, 6144), (1, 14336, 256), (12, 2048, 40), (27, 4096, 1024)])
def test_decode_mma_launches_in_a_row_and_graph_replays(kb, m, k, n):
    """Launches in a row (each may start while its predecessor drains) and replays of a captured pair of
    launches all give the oracle's result."""
    import torch
    _, ops, _ = kb
    x, _, res = case(m, k, n, seed=7 * m)
    r = resident(res)
    want = ko.y_w4a16(x, res)
    xd = dev(x)
    for i in range(4):
        y = ops.decode_forward(xd, r['qweight'], r['scales'], r['scaled_zeros'], m, n, k)
        assert_close(y.cpu().numpy(), want, f'decode launch {i} m={m} k={k} n={n}')
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ops.decode_forward(xd, r['qweight'], r['scales'], r['scaled_zeros'], m, n, k)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        y1 = ops.decode_forward(xd, r['qweight'], r['scales'], r['scaled_zeros'], m, n, k)
        y2 = ops.decode_forward(xd, r['qweight'], r['scales'], r['scaled_zeros'], m, n, k)
    for i in range(3):
        y1.zero_(); y2.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert_close(y1.cpu().numpy(), want, f'replay {i} first m={m} k={k} n={n}')
        assert torch.equal(y1, y2)


def test_decode_mma_bias_vs_reference_fixture(kb):
    _, ops, _ = kb
    g = dict(np.load(os.path.join(GOLDEN, 'small_n96_k1152_m33_bias.npz')))
    x = g['X'][:11]
    y = ops.decode_forward(dev(x), dev(g['qweight']), dev(g['scales']), dev(g['scaled_zeros']), 11, 96, 1152,
                           bias=dev(g['bias']))
    assert_close(y.cpu().numpy(), g['Y_w4a16'][:11], 'decode + bias vs reference fixture')


def test_gemv_bias_and_fixture(kb):
    _, ops, _ = kb
    g = dict(np.load(os.path.join(GOLDEN, 'small_n96_k1152_m33_bias.npz')))
    x = g['X'][:7]
    y = ops.gemv_cuda_core(dev(x), dev(g['qweight']), dev(g['scales']), dev(g['scaled_zeros']), 7, 96, 1152,
                           bias=dev(g['bias']))
    assert_close(y.cpu().numpy(), g['Y_w4a16'][:7], 'gemv + bias vs reference fixture')


# ------------------------------------------------------------------ a11 W8A8
GEMM_SHAPES = [(1, 128, 256), (5, 256, 64), (16, 512, 128), (33, 1152, 96), (16, 4096, 4096), (64, 4096, 1024),
               (100, 4096, 4096), (128, 14336, 4096), (257, 3584, 512), (512, 4096, 4096), (1000, 4096, 1024),
               # ragged in M and N, several token tiles; token tiles of 128 and 64 chosen by the plan's cost model
               (777, 1024, 9480), (300, 512, 2000), (600, 640, 2000),
               # CTA-pair kernel (about five rounds of 256 x 256 tiles or more), ragged in M and N
               (2600, 512, 9480)]


# N % 8 != 0 takes the scalar stores: (1280, 512, 4100) in the one-CTA kernel, (6000, 256, 4100) in the CTA-pair kernel
@pytest.mark.parametrize('m,k,n', GEMM_SHAPES + [(1280, 512, 4100), (6000, 256, 4100)])
def test_w8a8_gemm_bit_exact(kb, m, k, n):
    _, ops, _ = kb
    x, _, res = case(m, k, n, seed=m)
    xq, sx = ko.act_quant(x)
    w8 = ko.dequant_w8(res['qweight'], res['scales_to8'], res['scaled_zeros_to8'])
    y = torch.empty((m, n), dtype=torch.float16, device='cuda')
    acc = torch.empty((m, n), dtype=torch.int32, device='cuda')
    ops.w8a8_gemm_forward_cuda(dev(xq), dev(w8), dev(res['scales_1']), dev(sx), y, acc_out=acc)
    acc_ref = ko.acc_int32(xq, w8)
    assert np.array_equal(acc.cpu().numpy(), acc_ref), 'int32 accumulators'
    sc = res['scales_1'].astype(np.float32)[None, :] * sx.astype(np.float32)[:, None]
    y_ref = (acc_ref.astype(np.float32) * sc).astype(np.float16)
    assert np.array_equal(bits(y.cpu().numpy()), bits(y_ref)), 'scaled fp16 output'


# The code path a production call takes: no accumulator dump, so the CTA-pair kernel runs its 16-byte-store
# epilogue (shuffled activation scales, packed fp16 conversion) and the one-CTA kernel its check-free loop.
@pytest.mark.parametrize('m,k,n', [(777, 1024, 9480), (1280, 512, 4100), (1024, 4096, 4096), (300, 512, 1024),
                                   (512, 4096, 4096), (1000, 4096, 1024), (300, 512, 2000), (600, 640, 2004),
                                   (2600, 512, 9480), (6000, 256, 4100)])
def test_w8a8_gemm_production_epilogue_bit_exact(kb, m, k, n):
    _, ops, _ = kb
    x, _, res = case(m, k, n, seed=m)
    xq, sx = ko.act_quant(x)
    w8 = ko.dequant_w8(res['qweight'], res['scales_to8'], res['scaled_zeros_to8'])
    y = torch.empty((m, n), dtype=torch.float16, device='cuda')
    ops.w8a8_gemm_forward_cuda(dev(xq), dev(w8), dev(res['scales_1']), dev(sx), y)
    acc_ref = ko.acc_int32(xq, w8)
    sc = res['scales_1'].astype(np.float32)[None, :] * sx.astype(np.float32)[:, None]
    y_ref = (acc_ref.astype(np.float32) * sc).astype(np.float16)
    assert np.array_equal(bits(y.cpu().numpy()), bits(y_ref)), 'scaled fp16 output without the accumulator dump'


# ------------------------------------------------------------------ a10, a12, id 3
@pytest.mark.parametrize('m,k,n', GEMM_SHAPES)
def test_f16_gemms(kb, m, k, n):
    _, ops, _ = kb
    x, _, res = case(m, k, n, seed=m)
    r = resident(res)
    xd = dev(x)
    y_ref = ko.y_w4a16(x, res)
    y = ops.gemm_forward_cuda_new(xd, r['qweight'], r['scales'], r['scaled_zeros'])
    assert_close(y.cpu().numpy(), y_ref, 'w4a16 gemm')
    w16 = dev(ko.dequant_w16(res['qweight'], res['scales'], res['scaled_zeros']))
    assert_close(ops.f16_gemm(xd, w16).cpu().numpy(), y_ref, 'fp16 gemm')
    w8 = dev(ko.dequant_w8(res['qweight'], res['scales_to8'], res['scaled_zeros_to8']))
    assert_close(ops.w8a16_gemm(xd, w8, r['scales_1']).cpu().numpy(), ko.y_w8a16(x, res), 'w8a16 gemm')


def test_gemm_bias_vs_reference_fixture(kb):
    _, ops, _ = kb
    g = dict(np.load(os.path.join(GOLDEN, 'small_n96_k1152_m33_bias.npz')))
    b = dev(g['bias'])
    xd = dev(g['X'])
    y = ops.gemm_forward_cuda_new(xd, dev(g['qweight']), dev(g['scales']), dev(g['scaled_zeros']), bias=b)
    assert_close(y.cpu().numpy(), g['Y_w4a16'], 'w4a16 gemm + bias')
    y8 = torch.empty((33, 96), dtype=torch.float16, device='cuda')
    ops.w8a8_gemm_forward_cuda(dev(g['Xq']), dev(g['W8']), dev(g['scales_1']), dev(g['sx']), y8, bias=b)
    assert np.array_equal(bits(y8.cpu().numpy()), bits(g['Y_w8a8']))
    assert_close(ops.w8a16_gemm(xd, dev(g['W8']), dev(g['scales_1']), bias=b).cpu().numpy(), g['Y_w8a16'], 'w8a16')


# ------------------------------------------------------------------ full benchmark sizes: sampled columns
@pytest.mark.parametrize('m,k,n', [(8192, 4096, 4096), (4096, 4096, 14336), (2048, 14336, 4096)])
def test_full_size_sampled_columns(kb, m, k, n):
    """At the benchmark's sizes the oracle is evaluated on a seeded sample of output channels
    (all tokens), which keeps it to seconds; W8A8 stays bit-exact on the sample."""
    _, ops, _ = kb
    x, _, res = case(m, k, n, seed=11)
    r = resident(res)
    xd = dev(x)
    cols = np.sort(np.random.default_rng(5).choice(n, size=48, replace=False))
    w16 = ko.dequant_w16(res['qweight'], res['scales'], res['scaled_zeros'])
    w8 = ko.dequant_w8(res['qweight'], res['scales_to8'], res['scaled_zeros_to8'])
    y_ref = ko.matmul_f16(x, w16[cols])
    y = ops.gemm_forward_cuda_new(xd, r['qweight'], r['scales'], r['scaled_zeros'])
    assert_close(y.cpu().numpy()[:, cols], y_ref, 'w4a16 gemm full size')
    assert_close(ops.f16_gemm(xd, dev(w16)).cpu().numpy()[:, cols], y_ref, 'fp16 gemm full size')
    xq, sx = ko.act_quant(x)
    q = torch.empty((m, k), dtype=torch.int8, device='cuda')
    s = torch.empty((m,), dtype=torch.float16, device='cuda')
    ops.quant_fp16_to_int8(q, xd, s)
    assert np.array_equal(q.cpu().numpy(), xq)
    y8 = torch.empty((m, n), dtype=torch.float16, device='cuda')
    acc = torch.empty((m, n), dtype=torch.int32, device='cuda')
    ops.w8a8_gemm_forward_cuda(q, dev(w8), r['scales_1'], s, y8, acc_out=acc)
    acc_ref = ko.acc_int32(xq, w8[cols])
    assert np.array_equal(acc.cpu().numpy()[:, cols], acc_ref)
    sc = res['scales_1'].astype(np.float32)[None, cols] * sx.astype(np.float32)[:, None]
    y8_ref = (acc_ref.astype(np.float32) * sc).astype(np.float16)
    assert np.array_equal(bits(y8.cpu().numpy()[:, cols]), bits(y8_ref))
    # the same product as a production call runs it (no accumulator dump: the vectorised store loop)
    y8p = torch.empty((m, n), dtype=torch.float16, device='cuda')
    ops.w8a8_gemm_forward_cuda(q, dev(w8), r['scales_1'], s, y8p)
    assert np.array_equal(bits(y8p.cpu().numpy()[:, cols]), bits(y8_ref))
    assert torch.equal(y8p, y8)


# ------------------------------------------------------------------ module level
@pytest.mark.parametrize('path', SMALL, ids=[os.path.basename(p)[6:-4] for p in SMALL])
def test_from_module_on_gpu_matches_reference(kb, path):
    """Weight preparation run with CUDA tensors gives the reference's CPU bits."""
    kairos_b200, _, _ = kb
    g = dict(np.load(path))
    layer = _layer(kairos_b200, g['W'], g.get('bias'))
    for key in ('qweight', 'scales', 'scaled_zeros', 'scales_to8', 'scaled_zeros_to8', 'scales_1'):
        assert np.array_equal(bits(getattr(layer, key).cpu().numpy()), bits(g[key])), key


def _layer(kairos_b200, w, bias=None, cls=None):
    n, k = w.shape
    lin = torch.nn.Linear(k, n, bias=bias is not None, dtype=torch.float16)
    lin.weight.data = torch.from_numpy(w.copy())
    if bias is not None:
        lin.bias.data = torch.from_numpy(bias.copy())
    return (cls or kairos_b200.DynamicLinear).from_module(lin.cuda(), 'cuda')


def test_dynamic_linear_config0_all_kernels(kb):
    """M=16, K=N=4096, seed 0: every kernel id through DynamicLinear._forward."""
    kairos_b200, _, _ = kb
    x, w, res = case(16, 4096, 4096, seed=0)
    layer = _layer(kairos_b200, w)
    for key in ('qweight', 'scales', 'scaled_zeros', 'scales_to8', 'scaled_zeros_to8', 'scales_1'):
        assert np.array_equal(bits(getattr(layer, key).cpu().numpy()), bits(res[key])), key
    xd = dev(x)
    for cid, ref in ((0, ko.y_w4a16), (1, ko.y_w4a16), (5, ko.y_w4a16), (3, ko.y_w8a16)):
        assert_close(layer._forward(xd, 16, cid).cpu().numpy(), ref(x, res), f'comp {cid}')
    assert np.array_equal(bits(layer._forward(xd, 16, 2).cpu().numpy()), bits(ko.y_w8a8(x, res)))
    with pytest.raises(kairos_b200.KairosError):
        layer._forward(xd, 16, 4)
    with pytest.raises(kairos_b200.KairosError):
        layer._forward(dev(np.zeros((40, 4096), np.float16)), 40, 1)   # GEMV serves M <= 32 only


def test_forward_switches_by_lut_and_caches(kb):
    kairos_b200, _, runtime = kb
    from kairos_b200.runtime import Context
    x, w, res = case(48, 512, 128, seed=21)
    bias = (np.random.default_rng(1).standard_normal(128) * 0.1).astype(np.float16)
    layer = _layer(kairos_b200, w, bias)
    ctx = Context('cuda', cache_bytes=1 << 20)
    kairos_b200.DynamicLinear.context = ctx
    try:
        prof = kairos_b200.Profiler([(128, 512)])
        prof.load_table({(128, 512): [(4, 'w4a16_gemv'), (16, 'w4a16_gemm'), (32, 'w8a8'), (40, 'w8a16_gemm'),
                                      (30720, 'fp16')]})
        kairos_b200.DynamicLinear.prof = prof
        for m, cid in ((1, 1), (4, 1), (5, 0), (16, 0), (17, 2), (32, 2), (33, 3), (41, 5), (48, 5)):
            xm = x[:m]
            y = layer(dev(xm).reshape(1, m, 512))
            assert y.shape == (1, m, 128) and layer.comp_type == cid and layer.pre_m == m
            ref = ko.forward(xm, res, cid, bias)
            if cid == 2:
                assert np.array_equal(bits(y.cpu().numpy()[0]), bits(ref))
            else:
                assert_close(y.cpu().numpy()[0], ref, f'forward m={m} comp={cid}')
        st = ctx.stats()
        # W8 converted once (ids 2 and 3 share it), W16 once; later calls hit
        assert st['misses'] == 2 and st['hits'] >= 2 and st['bytes_in_use'] == 128 * 512 * 3
        y = layer(dev(x[:6]).reshape(2, 3, 512))          # batch x seq flattening
        assert y.shape == (2, 3, 128)
        assert_close(y.cpu().numpy().reshape(6, 128), ko.forward(x[:6], res, 0, bias), 'batched forward')
    finally:
        kairos_b200.DynamicLinear.context = None
        kairos_b200.DynamicLinear.prof = None


def test_cache_eviction_and_uncached_mode(kb):
    kairos_b200, _, _ = kb
    from kairos_b200.runtime import Context
    layers, cases = [], []
    for i in range(3):
        x, w, res = case(24, 256, 64, seed=30 + i)
        layers.append(_layer(kairos_b200, w))
        cases.append((x, res))
    for cache_bytes, want_evict in ((2 * 64 * 256, True), (0, False)):
        ctx = Context('cuda', cache_bytes=cache_bytes)     # room for two int8 copies / none
        kairos_b200.DynamicLinear.context = ctx
        try:
            for layer in layers:
                layer._release()
            for _ in range(2):
                for layer, (x, res) in zip(layers, cases):
                    y = layer._forward(dev(x), 24, 2)
                    assert np.array_equal(bits(y.cpu().numpy()), bits(ko.y_w8a8(x, res)))
            st = ctx.stats()
            assert st['misses'] == 6 and st['hits'] == 0      # cyclic access defeats LRU; never stale
            assert (st['evictions'] > 0) == want_evict
            assert st['bytes_in_use'] <= cache_bytes
        finally:
            for layer in layers:
                layer._release()
            kairos_b200.DynamicLinear.context = None


def test_switch_linear_is_all_resident(kb):
    kairos_b200, _, _ = kb
    x, w, res = case(20, 256, 64, seed=40)
    layer = _layer(kairos_b200, w, cls=kairos_b200.SwitchLinear)
    ctx = layer._ctx
    before = ctx.stats()
    assert before['misses'] >= 2
    for cid in (2, 5, 3, 0, 1):
        y = layer._forward(dev(x), 20, cid).cpu().numpy()
        ref = ko.forward(x, res, cid)
        if cid == 2:
            assert np.array_equal(bits(y), bits(ref))
        else:
            assert_close(y, ref, f'SwitchLinear comp {cid}')
    assert ctx.stats()['misses'] == before['misses']           # no conversion at call time


def test_host_buffer_entry_point(kb):
    kairos_b200, _, _ = kb
    from kairos_b200._lib import check, lib
    x, w, res = case(16, 512, 128, seed=50)
    layer = _layer(kairos_b200, w)
    xh = torch.from_numpy(x.copy()).pin_memory()
    yh = torch.empty((16, 128), dtype=torch.float16).pin_memory()
    st = torch.cuda.current_stream().cuda_stream
    for cid in (0, 2):
        check(lib.kairos_switched_linear_host(layer._native(), xh.data_ptr(), yh.data_ptr(), 16, cid, st), 'host')
        torch.cuda.synchronize()
        ref = ko.forward(x, res, cid)
        if cid == 2:
            assert np.array_equal(bits(yh.numpy()), bits(ref))
        else:
            assert_close(yh.numpy(), ref, 'host entry')


def test_host_buffer_entry_point_calls_in_flight(kb):
    """Twelve calls in a row with different inputs, sizes and output buffers and one synchronization at the
    end: the input copy of a call overlaps the call before it, and every output is its own input's result."""
    kairos_b200, _, _ = kb
    from kairos_b200._lib import check, lib
    _, w, res = case(1, 1024, 256, seed=70)
    layer = _layer(kairos_b200, w)
    st = torch.cuda.current_stream().cuda_stream
    calls = []
    for i in range(12):
        m = (64, 512, 16, 300)[i % 4]
        x, _ = ko.make_case(m, 1024, 4, seed=100 + i)
        xh = torch.from_numpy(x.copy()).pin_memory()
        yh = torch.zeros((m, 256), dtype=torch.float16).pin_memory()
        calls.append((x, xh, yh))
        check(lib.kairos_switched_linear_host(layer._native(), xh.data_ptr(), yh.data_ptr(), m, 2, st), 'host')
    torch.cuda.synchronize()
    for x, _, yh in calls:
        assert np.array_equal(bits(yh.numpy()), bits(ko.forward(x, res, 2)))


def test_side_stream_prefetch(kb):
    kairos_b200, _, _ = kb
    x, w, res = case(64, 512, 128, seed=60)
    layer = _layer(kairos_b200, w)
    side = torch.cuda.Stream()
    layer.prefetch(2, stream=side)
    y = layer._forward(dev(x), 64, 2)
    assert np.array_equal(bits(y.cpu().numpy()), bits(ko.y_w8a8(x, res)))


def test_w8a8_linearity_property_full_size(kb):
    """Size-independent check at a benchmark shape: int32 accumulators are additive in the
    activations, acc(Xa + Xb) == acc(Xa) + acc(Xb), exactly."""
    _, ops, _ = kb
    m, k, n = 1024, 4096, 4096
    g = torch.Generator(device='cuda').manual_seed(3)
    xa = torch.randint(-60, 60, (m, k), dtype=torch.int8, device='cuda', generator=g)
    xb = torch.randint(-60, 60, (m, k), dtype=torch.int8, device='cuda', generator=g)
    w8 = torch.randint(-127, 128, (n, k), dtype=torch.int8, device='cuda', generator=g)
    ones_n = torch.ones(n, dtype=torch.float16, device='cuda')
    ones_m = torch.ones(m, dtype=torch.float16, device='cuda')
    y = torch.empty((m, n), dtype=torch.float16, device='cuda')
    accs = []
    for xx in (xa, xb, xa + xb):
        acc = torch.empty((m, n), dtype=torch.int32, device='cuda')
        ops.w8a8_gemm_forward_cuda(xx.contiguous(), w8, ones_n, ones_m, y, acc_out=acc)
        accs.append(acc)
    assert torch.equal(accs[0] + accs[1], accs[2])
    # and one exact spot check of a row against an integer dot product on the host
    row = (xa[7].cpu().to(torch.int64)[None, :] * w8.cpu().to(torch.int64)).sum(dim=1)
    assert torch.equal(accs[0][7].cpu().to(torch.int64), row)
