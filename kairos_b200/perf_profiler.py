"""Offline profiler and per-shape interval LUT (M -> kernel id).

Mirrors kairos/perf_profiler.py:24-165 of the reference: ``Profiler(shape_list)``,
``profiling()``, ``save()/load()`` of ``<path>/seg_perf_list.pt`` (JSON), ``get_comp_type``,
``record_best_comp``, attributes ``seg_perf_list`` and ``lut``.  The LUT itself is the native
C++ table of the shared library (reference: kernels/csrc/kairos_kernel/lut/lut.h).

Timing is on-device (CUDA events around a CUDA graph of ``_forward`` calls that rotate over copies
of the layer, after warm-up) and INCLUDES activation quantization and weight conversion.
With ``cache='cold'`` (default) every timed call converts the weight again, which is what a
layer sees when the model's converted weights do not fit the bounded cache; ``cache='warm'``
times the steady state of a layer whose converted weight stays cached.
"""
from __future__ import annotations

import json
import os

import torch

from ._lib import KairosError, lib
from .dynamic_linear import COMP_TYPE_ID, COMP_TYPE_NAME, SUPPORTED_COMP_TYPES, DynamicLinear

# M grid of the reference (kairos/perf_profiler.py:88-90)
DEFAULT_M_GRID = ([1, 2, 4, 8, 16, 24, 32, 48, 64, 128, 256, 512]
                  + list(range(1024, 1024 * 8, 1024)) + list(range(1024 * 8, 1024 * 32, 2048)))
DEFAULT_CANDIDATES = ['fp16', 'w4a16_gemm', 'w4a16_gemv', 'w8a8', 'w8a16_gemm']
# a LUT written by the reference may name kernels that have no implementation here;
# they are served by the closest member of this portfolio
SUBSTITUTE = {'w4a16_marlin': 'w4a16_gemm', 'w4a8_qserve': 'w8a8', 'w8a16_gemv': 'w4a16_gemv'}


class LUT:
    """Interval table: ids[i] serves m in (r[i-1], r[i]], the last id everything above.
    Thin wrapper over the native kairos_lut (semantics of lut.h:22-38, memo included)."""

    def __init__(self):
        self._h = lib.kairos_lut_create()
        self._get = lib.kairos_lut_get
        self.records = []

    def get(self, m):
        r = self._get(self._h, m)
        if r < 0:
            raise KairosError('LUT.get on an empty table')
        return r

    def record(self, r, comp_type_id):
        lib.kairos_lut_record(self._h, int(r), int(comp_type_id))
        self.records.append((int(r), int(comp_type_id)))

    def shrink_to_fit(self):
        lib.kairos_lut_shrink_to_fit(self._h)

    def __len__(self):
        return lib.kairos_lut_size(self._h)

    def __del__(self):
        try:
            lib.kairos_lut_destroy(self._h)
        except Exception:
            pass


def resolve_comp_name(name):
    """Kernel name of a LUT file -> id of a kernel this library runs."""
    name = SUBSTITUTE.get(name, name)
    cid = COMP_TYPE_NAME[name]
    if cid not in SUPPORTED_COMP_TYPES:
        raise KairosError(f'no kernel for "{name}"')
    return cid


class Profiler:
    def __init__(self, shape_list, m_grid=None, candidates=None, n=200, warmup=20, cache='cold',
                 linear_cls=DynamicLinear):
        self.shape_list = [tuple(s) for s in shape_list]
        self.seg_perf_list = []
        self.lut = {shape: LUT() for shape in self.shape_list}
        self.m_grid = list(m_grid) if m_grid is not None else list(DEFAULT_M_GRID)
        self.candidates = list(candidates) if candidates is not None else list(DEFAULT_CANDIDATES)
        self.n, self.warmup, self.cache = n, warmup, cache
        self.linear_cls = linear_cls
        self.timings = {}       # shape -> {m: {name: ms}}

    def record_best_comp(self, shape, r, comp_type):
        self.lut[tuple(shape)].record(r, resolve_comp_name(comp_type))

    def profiling(self, device='cuda'):
        for shape in self.shape_list:
            seg, table = test_perf(str(shape), shape[1], shape[0], False, m_grid=self.m_grid,
                                   candidates=self.candidates, n=self.n, warmup=self.warmup, cache=self.cache,
                                   device=device, linear_cls=self.linear_cls)
            for t in seg:
                self.record_best_comp(shape, t[0], t[1])
            self.seg_perf_list.append(seg)
            self.timings[shape] = table

    def get_comp_type(self, shape, m):
        return self.lut[shape].get(m)

    def save(self, path='./prof/'):
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, 'seg_perf_list.pt'), 'w') as f:
            f.write(json.dumps(self.seg_perf_list))

    def load(self, path='./prof/'):
        with open(os.path.join(path, 'seg_perf_list.pt')) as f:
            self.seg_perf_list = json.load(f)
        self.lut = {shape: LUT() for shape in self.shape_list}
        for shape, seg in zip(self.shape_list, self.seg_perf_list):
            for t in seg:
                self.record_best_comp(shape, t[0], t[1])

    def load_table(self, tables):
        """Install interval tables given as {shape: [(m_right, name), ...]}."""
        self.seg_perf_list = []
        self.lut = {shape: LUT() for shape in self.shape_list}
        for shape in self.shape_list:
            seg = [[int(r), name, 0.0] for r, name in tables[shape]]
            for t in seg:
                self.record_best_comp(shape, t[0], t[1])
            self.seg_perf_list.append(seg)


def collapse_segments(perf_list):
    """[(m, best, gain)] per grid point -> one entry per run of equal winners, keyed by the
    run's last m (kairos/perf_profiler.py:150-156)."""
    seg = []
    pre = perf_list[0]
    for t in perf_list:
        if t[1] != pre[1]:
            seg.append(pre)
        pre = t
    seg.append(pre)
    return [list(t) for t in seg]


@torch.no_grad()
def time_forward(layers, x, m, comp_id, n, warmup):
    """Mean milliseconds of one ``_forward``.  The calls go round-robin over `layers` (copies of one
    layer in distinct memory, so that the weights stream from HBM as they do inside a model rather than
    sit in L2), are captured into one CUDA graph and the graph is replayed between two events: device
    time without host launch gaps.  Falls back to an eager loop (utils/perf_eval.py:21-34 of the
    reference) if capture is not possible."""
    stream = torch.cuda.Stream()
    rounds = max(1, n // len(layers))
    with torch.cuda.stream(stream):
        for _ in range(max(1, warmup // len(layers)) + 1):
            for layer in layers:
                layer._forward(x, m, comp_id)
    torch.cuda.synchronize()
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for layer in layers:
                layer._forward(x, m, comp_id)
        graph.replay()
        torch.cuda.synchronize()
        start.record()
        for _ in range(rounds):
            graph.replay()
        end.record()
    except Exception:
        torch.cuda.synchronize()
        start.record()
        for _ in range(rounds):
            for layer in layers:
                layer._forward(x, m, comp_id)
        end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / (rounds * len(layers))


def _clone_layer(layer, ctx):
    """A copy of `layer` whose resident tensors live in fresh memory, bound to context `ctx`."""
    twin = type(layer)(layer.in_features, layer.out_features, layer.bias is not None, layer.qweight.device, 128)
    for name in ('qweight', 'scales', 'scaled_zeros', 'scales_to8', 'scaled_zeros_to8', 'scales_1'):
        getattr(twin, name).copy_(getattr(layer, name))
    if layer.bias is not None:
        twin.bias.copy_(layer.bias)
    twin._cache_context = lambda: ctx
    return twin


@torch.no_grad()
def test_perf(proj_name, K, N, bias, m_grid=None, candidates=None, n=200, warmup=20, cache='cold',
              device='cuda', linear_cls=DynamicLinear, verbose=False):
    """Time every candidate kernel at every M of the grid for one (N, K) shape and return
    (interval list, {m: {name: ms}})  (kairos/perf_profiler.py:83-165)."""
    m_grid = list(m_grid) if m_grid is not None else list(DEFAULT_M_GRID)
    candidates = list(candidates) if candidates is not None else list(DEFAULT_CANDIDATES)
    lin = torch.nn.Linear(K, N, bias=bias, dtype=torch.float16, device=device)
    layer = linear_cls.from_module(lin, device)
    del lin
    from .runtime import Context
    layer._release()
    # cold: a zero-byte cache converts into one reusable slot on every call (no allocator traffic);
    # warm: a private unbounded cache keeps the converted weight after the first call
    own_ctx = Context(layer.qweight.device, cache_bytes=0 if cache == 'cold' else None)
    own_ctx.reserve(max(m_grid), N, K)
    layer._cache_context = lambda: own_ctx
    # enough copies of the layer that a round over them touches more packed weight than twice the L2
    l2 = torch.cuda.get_device_properties(layer.qweight.device).L2_cache_size
    copies = max(2, min(64, int(2.5 * l2 / (K * N // 2)) + 1))
    layers = [layer] + [_clone_layer(layer, own_ctx) for _ in range(copies - 1)]
    table, perf_list = {}, []
    for m in m_grid:
        x = torch.randn((m, K), dtype=torch.float16, device=device)
        best_t, best, orig_t = 1e30, '', 1e30
        table[m] = {}
        for name in candidates:
            if m > 32 and 'gemv' in name:
                continue
            # one NVTX range per timed candidate (the reference marks its experiments the same way,
            # test/test_asyn_trans.py:151,171): a timeline tool shows which kernels belong to which candidate
            torch.cuda.nvtx.range_push(f'{proj_name} {name} m={m}')
            try:
                t = time_forward(layers, x, m, COMP_TYPE_NAME[name], n, warmup)
            finally:
                torch.cuda.nvtx.range_pop()
            table[m][name] = t
            if t < best_t:
                best_t, best = t, name
            if 'w4' in name and t < orig_t:
                orig_t = t
        perf_list.append((m, best, (orig_t - best_t) * 100 / orig_t))
        if verbose:
            print(f'{proj_name} m={m:6d} ' + ' '.join(f'{k}={v * 1e3:8.1f}us' for k, v in table[m].items()))
    for lyr in layers:
        lyr._release()
    return collapse_segments(perf_list), table
