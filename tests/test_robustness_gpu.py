"""GPU tests of the parts around the kernels: the bounded device-side wait, the conversion cache under
CUDA-graph capture, and the on-device profiler."""
import os
import tempfile

import numpy as np
import pytest
import torch

from oracle import kairos_oracle as ko

pytestmark = pytest.mark.gpu


def _layer(kb, m, k, n, seed, ctx=None):
    x, w = ko.make_case(m, k, n, seed=seed)
    lin = torch.nn.Linear(k, n, bias=False, dtype=torch.float16)
    lin.weight.data = torch.from_numpy(w.copy())
    layer = kb.DynamicLinear.from_module(lin.cuda(), 'cuda')
    if ctx is not None:
        layer._release()
        layer._cache_context = lambda: ctx
    return layer, torch.from_numpy(x).cuda(), x, ko.from_module(w)


def test_bounded_wait_runs_out_and_reports():
    """A wait on a barrier that nothing completes ends by itself, raises the status word, and leaves the
    device usable: the next kernel runs and is correct."""
    import kairos_b200 as kb
    from kairos_b200 import runtime
    from kairos_b200._lib import lib
    torch.cuda.synchronize()
    assert runtime.device_status(clear=True) == 0
    assert lib.kairos_selftest_bounded_wait(torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert runtime.device_status(clear=False) == -7          # KAIROS_ERR_DEVICE, still set
    assert runtime.device_status(clear=True) == -7
    assert runtime.device_status(clear=True) == 0            # cleared
    layer, xd, x, res = _layer(kb, 8, 512, 256, seed=3)
    y = layer._forward(xd, 8, 1).cpu().numpy()
    bad, _ = ko.within_tolerance(y, ko.forward(x, res, 1))
    assert bad == 0
    torch.cuda.synchronize()
    assert runtime.device_status() == 0


def test_cache_miss_during_capture_fails_loudly_and_hits_are_pinned():
    """Inside a stream capture the conversion cache may neither allocate nor evict: a miss is an error,
    and an entry whose address a graph holds is never recycled for another layer."""
    import kairos_b200 as kb
    from kairos_b200 import runtime
    from kairos_b200._lib import KairosError
    k, n, m = 512, 256, 64
    ctx = runtime.Context('cuda', cache_bytes=int(1.5 * n * k))       # room for ONE int8 weight
    ctx.reserve(m, n, k)
    a, xd, x, res_a = _layer(kb, m, k, n, seed=5, ctx=ctx)
    b, _, _, res_b = _layer(kb, m, k, n, seed=6, ctx=ctx)
    ref_a = ko.forward(x, res_a, 2)
    ref_b = ko.forward(x, res_b, 2)
    side = torch.cuda.Stream()
    # 1. a miss while capturing: loud failure, capture abandoned, context still usable
    g = torch.cuda.CUDAGraph()
    with pytest.raises(Exception):
        with torch.cuda.graph(g, stream=side):
            a._forward(xd, m, 2)
    torch.cuda.synchronize()
    # 2. convert eagerly on the stream that will capture, then capture: the hit is captured and pinned
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ya = a._forward(xd, m, 2)
    torch.cuda.synchronize()
    assert np.array_equal(ya.cpu().numpy().view(np.uint16), ref_a.view(np.uint16))
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        y_graph = a._forward(xd, m, 2)
    # 3. the other layer cannot evict the pinned entry: it is served from the transient slot
    yb = b._forward(xd, m, 2)
    assert np.array_equal(yb.cpu().numpy().view(np.uint16), ref_b.view(np.uint16))
    st = ctx.stats()
    assert st['evictions'] == 0
    # 4. the replay still computes with layer a's weights
    y_graph.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert np.array_equal(y_graph.cpu().numpy().view(np.uint16), ref_a.view(np.uint16))
    assert runtime.device_status() == 0
    del g
    a._release(); b._release()
    ctx.close()


def test_workspace_growth_during_capture_is_refused():
    import kairos_b200 as kb
    from kairos_b200 import runtime
    ctx = runtime.Context('cuda', cache_bytes=None)
    layer, xd, x, res = _layer(kb, 64, 4096, 512, seed=7, ctx=ctx)     # 4 weight tiles: the GEMM splits K
    side = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with pytest.raises(Exception):
        with torch.cuda.graph(g, stream=side):
            layer._forward(xd, 64, 0)          # split-K scratch was never reserved
    torch.cuda.synchronize()
    ctx.reserve(64, 512, 4096)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        y = layer._forward(xd, 64, 0)
    g.replay()
    torch.cuda.synchronize()
    bad, _ = ko.within_tolerance(y.cpu().numpy(), ko.forward(x, res, 0))
    assert bad == 0
    del g
    layer._release()
    ctx.close()


def test_profiler_picks_argmin_and_round_trips():
    """Profiler.profiling() on one small shape: every interval's winner is the fastest candidate of its
    grid points, save() -> load() reproduces get_comp_type on the whole grid, and a cold cache (conversion
    on every call) is never faster than a warm one for the kernels that convert."""
    from kairos_b200.dynamic_linear import COMP_TYPE_NAME
    from kairos_b200.perf_profiler import Profiler
    shape = (1024, 2048)                       # (N, K)
    grid = [1, 8, 32, 64, 256, 1024]
    warm = Profiler([shape], m_grid=grid, n=40, warmup=8, cache='warm')
    warm.profiling()
    table = warm.timings[shape]
    assert sorted(table) == grid
    for m in grid:
        best = min(table[m], key=table[m].get)
        assert warm.get_comp_type(shape, m) == COMP_TYPE_NAME[best], (m, table[m])
        assert ('w4a16_gemv' in table[m]) == (m <= 32)
    with tempfile.TemporaryDirectory() as d:
        warm.save(d)
        again = Profiler([shape], m_grid=grid)
        again.load(d)
        for m in range(1, 1100):
            assert again.get_comp_type(shape, m) == warm.get_comp_type(shape, m)
    cold = Profiler([shape], m_grid=[64, 1024], n=40, warmup=8, cache='cold')
    cold.profiling()
    for m in (64, 1024):
        for name in ('w8a8', 'w8a16_gemm', 'fp16'):
            assert cold.timings[shape][m][name] >= 0.9 * table[m][name], (m, name)
        # kernels on the packed base pay no conversion: same time within noise
        assert cold.timings[shape][m]['w4a16_gemm'] <= 1.5 * table[m]['w4a16_gemm'] + 0.005
