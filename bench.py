#!/usr/bin/env python
"""Benchmark of the switched quantized-linear path on B200.

Workload (N=1): the Llama-3-8B linear-shape sweep -- (K,N) in {(4096,4096), (4096,1024),
(4096,14336), (14336,4096)} x M in {1,2,...,8192} -- on seeded synthetic tensors with the
benchmark's value distributions (X ~ N(0,1) with 1% of channels x20, W ~ N(0,0.02) stored as
uint4 g128).  A "step" is one pass over all 56 (shape, M) points through ``DynamicLinear.forward``
with the interval LUT that the on-device profiler built just before (conversion and activation
quantization included).  ``value`` = total 2*M*K*N of a pass / device time of the pass.

With --gpus N > 1 (under torchrun) the same sweep runs tensor-parallel: k/v and gate/up are
column-split, the (4096,4096) and down projections are row-split and followed by an NCCL
all-reduce; total work is fixed ("strong" scaling, also the label at N = 1).

``python bench.py --impl reference`` times the reference's CPU path (the numpy port under
oracle/, since the reference's torch code cannot travel to the GPU box) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES_KN = [(4096, 4096), (4096, 1024), (4096, 14336), (14336, 4096)]       # (K, N)
# the projection each shape stands for under tensor parallelism (o and down are row-parallel)
SHAPE_ROLE = {(4096, 4096): 'o_proj', (4096, 1024): 'k_proj', (4096, 14336): 'gate_proj', (14336, 4096): 'down_proj'}
M_LIST = [1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192]
METRIC = 'switched-linear TFLOPS over the Llama-3-8B shape x M sweep'


def algorithmic_bytes(m, k, n):
    """Bytes one call must move: uint4 base + one (scale, scaled-zero) pair per group + X + Y."""
    return k * n // 2 + 2 * 2 * (k // 128) * n + 2 * m * k + 2 * m * n


def load_peaks():
    p = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(p):
        d = json.load(open(p))
        return {'hbm_gbs': d['hbm_gbs'], 'bf16_tflops': d['bf16_tflops'],
                'bf16_tflops_sustained': d.get('bf16_tflops_sustained', d['bf16_tflops']), 'source': 'measured'}
    return {'hbm_gbs': 6650.0, 'bf16_tflops': 1590.0, 'bf16_tflops_sustained': 1400.0, 'source': 'fallback'}


# --------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------
class ClockSampler:
    Q = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,'
         'clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
         'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index):
        self.gpu, self.proc, self.rows = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(['nvidia-smi', f'--query-gpu={self.Q}', '--format=csv,noheader,nounits',
                                          '-i', str(self.gpu), '-lms', '100'], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(',')])

    def stop(self):
        if not self.proc:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except Exception:
                continue
            for name, col in (('hw_slowdown', 5), ('hw_thermal_slowdown', 6), ('sw_thermal_slowdown', 7),
                              ('sw_power_cap', 8)):
                if len(r) > col and r[col].lower().startswith('active'):
                    reasons.add(name)
        top = sorted(sm)[len(sm) // 2:] if sm else []       # the upper half = samples under load
        return {'sm_mhz': statistics.median(top) if top else None, 'sm_max_mhz': max(mx) if mx else None,
                'reasons': sorted(reasons), 'samples': len(sm)}


# --------------------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle port on the host cores
# --------------------------------------------------------------------------------------
CPU_SAMPLE = [((4096, 4096), 16), ((4096, 4096), 256), ((4096, 1024), 1024)]


def cpu_pass(cases):
    """One pass of the reference's CPU path over the sample: dequantize + matmul for the W4A16
    points, activation quantization + int8 conversion + integer matmul + rescale for M >= 256
    (the regime where the shipped LUTs choose W8A8)."""
    from oracle import kairos_oracle as ko
    flops = 0
    t0 = time.perf_counter()
    for (k, n), m, x, res in cases:
        if m >= 256:
            ko.y_w8a8(x, res)
        else:
            ko.y_w4a16(x, res)
        flops += 2 * m * k * n
    return flops, time.perf_counter() - t0


def cpu_cases():
    from oracle import kairos_oracle as ko
    cases = []
    for (k, n), m in CPU_SAMPLE:
        x, w = ko.make_case(m, k, n, seed=0)
        cases.append(((k, n), m, x, ko.from_module(w)))
    return cases


def cpu_baseline(repeats=2):
    cases = cpu_cases()
    cpu_pass(cases)                       # warm-up (BLAS threads, page faults)
    best = None
    for _ in range(repeats):
        flops, dt = cpu_pass(cases)
        v = flops / dt / 1e12
        best = v if best is None else max(best, v)
    return {'value': best, 'unit': 'TFLOPS', 'cores': os.cpu_count(), 'kind': 'port',
            'sample': 'oracle/kairos_oracle.py (numpy, BLAS on all host threads) incl. dequant/act-quant on '
                      + ', '.join(f'M={m} K={k} N={n}' for (k, n), m in CPU_SAMPLE)}


def run_reference_arm(args):
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    cases = cpu_cases()
    for _ in range(min(args.warmup, 1) or 1):
        cpu_pass(cases)
    steps = max(1, min(args.steps, 5))
    t_tot, f_tot = 0.0, 0
    for _ in range(steps):
        f, dt = cpu_pass(cases)
        t_tot += dt
        f_tot += f
    v = f_tot / t_tot / 1e12
    sample = ('numpy port of the reference torch path on the host cores; each step = '
              + ', '.join(f'M={m} K={k} N={n}' for (k, n), m in CPU_SAMPLE) + ' incl. dequant/act-quant')
    print(json.dumps({
        'impl': 'reference', 'metric': METRIC, 'value': v, 'unit': 'TFLOPS', 'n_gpus': args.gpus, 'steps': steps,
        'warmup': args.warmup, 'ms_per_step': 1e3 * t_tot / steps, 'higher_is_better': True,
        'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f16/int8', 'data': 'synthetic',
        'config': {'workload': 'llama3-8b-linear-sweep (bounded CPU sample)'},
        'cpu_baseline': {'value': v, 'unit': 'TFLOPS', 'cores': os.cpu_count(), 'kind': 'port', 'sample': sample},
        'e2e': {'value': v, 'unit': 'TFLOPS', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0}))


# --------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------
def build_layers(torch, kb, tp, rank, world, device):
    """One switched linear per (K,N) of the sweep (per-rank shard under tensor parallelism)."""
    from kairos_b200.synthetic import make_case
    layers = []
    for (k, n) in SHAPES_KN:
        _, w = make_case(1, k, n, seed=0)
        w = torch.from_numpy(w)
        if world > 1:
            layers.append(tp.shard_linear(w, kind=tp.layer_kind(SHAPE_ROLE[(k, n)]), rank=rank, world=world, device=device))
        else:
            lin = torch.nn.Linear(k, n, bias=False, dtype=torch.float16)
            lin.weight.data = w
            layers.append(kb.DynamicLinear.from_module(lin.to(device), device))
    return layers


def make_inputs(torch, device, world, rank, tp):
    from kairos_b200.synthetic import make_case
    xs = {}
    for (k, n) in SHAPES_KN:
        x, _ = make_case(max(M_LIST), k, 4, seed=1)
        x = torch.from_numpy(x)
        if world > 1 and tp.layer_kind(SHAPE_ROLE[(k, n)]) == 'row':
            ks = k // world
            x = x[:, rank * ks:(rank + 1) * ks].contiguous()
        xs[(k, n)] = x
    return xs


def graph_us_per_call(torch, calls, reps=5):
    """Device microseconds per call: the calls are captured once into a CUDA graph (no host launch
    gaps) and the graph is replayed `reps` times between two events."""
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for c in calls:
            c()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        for c in calls:
            c()
    g.replay()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(reps):
        g.replay()
    e.record()
    torch.cuda.synchronize()
    return 1e3 * s.elapsed_time(e) / (reps * len(calls))


class RotatingWeights:
    """Copies of a layer's resident tensors whose total size exceeds twice the L2, so that back-to-back
    calls on successive copies stream the weights from HBM."""

    def __init__(self, torch, mod, l2_bytes):
        per = mod.qweight.numel() * 2 + 2 * mod.scales.numel() * 2
        self.n = max(2, min(160, int(2.5 * l2_bytes / per) + 1))
        self.qw = [mod.qweight.clone() for _ in range(self.n)]
        self.sc = [mod.scales.clone() for _ in range(self.n)]
        self.sz = [mod.scaled_zeros.clone() for _ in range(self.n)]


def measure_int8_peak(torch, device):
    """Dense int8 tensor-core throughput of this GPU as a library GEMM reaches it (torch._int_mm, 8192^3):
    a burst (20 back-to-back calls) and a sustained figure (about a second of calls).  The denominator of
    the int8 roofline; the measured-peaks file of the pool has no int8 entry."""
    n = 8192
    try:
        a = torch.randint(-8, 8, (n, n), dtype=torch.int8, device=device)
        b = torch.randint(-8, 8, (n, n), dtype=torch.int8, device=device)
        for _ in range(3):
            torch._int_mm(a, b)
        torch.cuda.synchronize()

        def run(reps):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(reps):
                torch._int_mm(a, b)
            e.record()
            torch.cuda.synchronize()
            return 2 * n ** 3 * reps / (s.elapsed_time(e) * 1e-3) / 1e12

        burst = max(run(20) for _ in range(3))
        sustained = run(max(20, int(1.0 / (2 * n ** 3 / (burst * 1e12)))))
        return {'int8_tops_measured': burst, 'int8_tops_sustained': sustained, 'int8_source': 'torch._int_mm 8192^3'}
    except Exception as exc:       # no int8 library GEMM on this build: fall back to the nominal ratio
        return {'int8_tops_measured': None, 'int8_source': f'unavailable ({type(exc).__name__})'}


def rank0_decides(dist, flag, more):
    """Every rank must run the same number of timed blocks, because a block holds collectives: a rank that went on
    for one more block on its own clock would wait for its peers forever.  Rank 0's verdict is broadcast; `flag` is
    a one-element tensor on the backend's device."""
    flag.fill_(1.0 if more else 0.0)
    dist.broadcast(flag, src=0)
    return bool(flag.item())


def timed_blocks(torch, dist, world, device, fn, steps, warmup, min_seconds=1.0, max_blocks=400, mark=False):
    """Device time of `steps` calls of fn, repeated as blocks until the timed region is at least `min_seconds`
    long (so that clock samples fall inside it); every block is bracketed by events, barrier + synchronize
    on both sides of the whole region, max over ranks.  Returns (median ms per step, all block values)."""
    for _ in range(max(3, warmup)):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    blocks, t_start = [], time.perf_counter()
    if mark:
        torch.cuda.profiler.start()      # lets `ncu --profile-from-start off` see exactly the timed steps
    go_on = torch.ones(1, device=device) if world > 1 else None
    while True:
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(steps):
            fn()
        e.record()
        e.synchronize()
        blocks.append(s.elapsed_time(e) / steps)
        more = len(blocks) < max_blocks and time.perf_counter() - t_start < min_seconds
        if world > 1:
            more = rank0_decides(dist, go_on, more)
        if not more:
            break
    torch.cuda.synchronize()
    if mark:
        torch.cuda.profiler.stop()
    if world > 1:
        dist.barrier()
        t = torch.tensor([statistics.median(blocks)], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), blocks
    return statistics.median(blocks), blocks


def llm_block(torch, kb, runtime, device, saved_prof, saved_ctx):
    """TTFT / TPOT of a random-init Llama-3-8B decoder (the second half of the metric): prompts of 1024 random
    token ids, 64 new tokens, batch 2 and 32, protocol of the reference's utils/perf_eval.py:236-275."""
    from kairos_b200 import llm
    out = {'model': 'llama3-8b (random init, uint4 g128 linears, fp16 lm_head)', 'prompt_len': 1024, 'new_tokens': 64}
    try:
        t0 = time.perf_counter()
        ctx = runtime.Context(device, cache_bytes=24 << 30)
        kb.DynamicLinear.context = ctx
        model = llm.Decoder(llm.PRESETS['llama3-8b'], device)
        prof = llm.build_lut(model.linear_shapes(), device=device, cache='warm', n=8,
                             m_grid=[1, 2, 4, 8, 16, 32, 64, 128, 512, 2048, 8192, 32768])
        out['setup_seconds'] = round(time.perf_counter() - t0, 1)
        out['lut'] = {str(s): [(r, name) for r, name, _ in prof.seg_perf_list[i]] for i, s in enumerate(prof.shape_list)}
        rows = []
        for b in (2, 32):
            r = llm.measure_ttft_tpot(model, b, 1024, 64, warmup=1, ttft_times=3)
            rows.append({k: (round(v, 3) if isinstance(v, float) else v) for k, v in r.items()})
        out['results'] = rows
        model.release_graphs()
        del model
        ctx.close()
    except Exception as exc:
        out['error'] = f'{type(exc).__name__}: {exc}'
    finally:
        kb.DynamicLinear.prof = saved_prof
        kb.DynamicLinear.context = saved_ctx
        torch.cuda.empty_cache()
    return out


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    import kairos_b200 as kb
    from kairos_b200 import ops, runtime
    from kairos_b200._lib import check, lib

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    device = torch.device('cuda', local)
    tp = None
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        dist.init_process_group('nccl', device_id=device)
        dist.all_reduce(torch.zeros(1, device=device))        # communicator up before any capture
        from kairos_b200 import tp as tp_mod
        tp = tp_mod
    peaks = load_peaks()
    if rank == 0:
        peaks.update(measure_int8_peak(torch, device))
    l2_bytes = torch.cuda.get_device_properties(device).L2_cache_size

    layers = build_layers(torch, kb, tp, rank, world, device)
    xs_host = make_inputs(torch, device, world, rank, tp)
    xs_dev = {kn: x.to(device) for kn, x in xs_host.items()}
    xs_pin = {kn: x.pin_memory() for kn, x in xs_host.items()}
    mods = [l.linear if world > 1 else l for l in layers]
    shapes = [m.shape for m in mods]                       # per-rank (N, K)
    reduced = [world > 1 and isinstance(l, tp.RowParallelLinear) for l in layers]

    # the bounded conversion cache: room for the converted forms of the sweep's four layers
    cache_bytes = 512 << 20
    ctx = runtime.Context(device, cache_bytes=cache_bytes)
    ctx_cold = runtime.Context(device, cache_bytes=0)      # the reference's regime: convert on every call
    kb.DynamicLinear.context = ctx
    for c in (ctx, ctx_cold):
        c.reserve(max(M_LIST), max(s[0] for s in shapes), max(s[1] for s in shapes))

    # ---- on-device profiler builds the LUTs.  'warm' = a layer whose converted weight stays in the cache
    # (the regime of this sweep: all four layers fit); 'cold' = conversion on every call, what the
    # reference's DynamicLinear pays (kairos/dynamic_linear.py:145-147) and what a model larger than the
    # cache sees.
    t_prof = time.perf_counter()
    prof = kb.Profiler(shapes, m_grid=M_LIST, n=args.prof_iters, warmup=3, cache='warm')
    prof.profiling(device=device)
    prof_cold = kb.Profiler(shapes, m_grid=M_LIST, n=args.prof_iters, warmup=3, cache='cold')
    prof_cold.profiling(device=device)
    t_prof = time.perf_counter() - t_prof
    if world > 1:
        dist.barrier()
    kb.DynamicLinear.prof = prof

    y_pin = {(k, n): torch.empty((max(M_LIST), n), dtype=torch.float16).pin_memory() for (k, n) in SHAPES_KN}
    total_flops = sum(2 * m * k * n for (k, n) in SHAPES_KN for m in M_LIST)

    # the cold regime runs on copies of the layers bound to the zero-byte cache, so that nothing the warm
    # regime's CUDA graph points to (its layers' cached conversions) is released in between
    from kairos_b200.perf_profiler import _clone_layer
    mods_cold = [_clone_layer(mod, ctx_cold) for mod in mods]
    regime = {'mods': mods, 'prof': prof}

    def use(which):
        """Switch the sweep between the warm regime (bounded cache, warm LUT) and the cold one."""
        regime['mods'], regime['prof'] = (mods, prof) if which == 'warm' else (mods_cold, prof_cold)

    def one_pass_host():
        for li, (k, n) in enumerate(SHAPES_KN):
            for m in M_LIST:
                x = xs_pin[(k, n)][:m]
                if world > 1:
                    layers[li].forward_host(x)
                else:
                    mod = mods[li]
                    if m != mod.pre_m:
                        mod.pre_m = m
                        mod.comp_type = prof.get_comp_type(mod.shape, m)
                    y = y_pin[(k, n)][:m]
                    check(lib.kairos_switched_linear_host(mod._native(), x.data_ptr(), y.data_ptr(), m,
                                                          mod.comp_type, runtime.stream_ptr()), 'host forward')

    # One pass of the sweep.  Row-parallel shapes come first and write their 14 outputs into ONE flat buffer
    # each, so a shape's partial sums cross NVLink in a single all-reduce, issued on a second stream: it runs
    # while the following shapes compute.  The whole pass, collectives included, is one CUDA graph.
    # With `--tp-collective reducescatter` (the default) the sum is left sharded over the tokens (rank r keeps rows
    # r * T / t .. (r + 1) * T / t of the shape's T = 16384 token rows: the sequence-sharded layout a following norm
    # or residual addition consumes under sequence parallelism), which moves half the bytes of an all-reduce;
    # `allreduce` leaves the full sum on every rank.  The run reports both step times.
    order = sorted(range(len(SHAPES_KN)), key=lambda li: not reduced[li])
    rows_pad = (sum(M_LIST) + world - 1) // world * world
    flat = {li: torch.zeros((rows_pad, shapes[li][0]), dtype=torch.float16, device=device) for li in order}
    shard = {li: torch.empty((rows_pad // world, shapes[li][0]), dtype=torch.float16, device=device)
             for li in order if reduced[li]} if world > 1 else {}
    tp_mode = {'collective': args.tp_collective}
    views = {}
    for li in order:
        off = 0
        for m in M_LIST:
            views[(li, m)] = flat[li][off:off + m]
            off += m
    comm = torch.cuda.Stream() if world > 1 else None

    def one_pass():
        main = torch.cuda.current_stream()
        for li in order:
            mod, kn = regime['mods'][li], SHAPES_KN[li]
            lut = regime['prof']
            for m in M_LIST:
                mod._forward(xs_dev[kn][:m], m, lut.get_comp_type(mod.shape, m), out=views[(li, m)])
            if reduced[li]:
                comm.wait_stream(main)
                with torch.cuda.stream(comm):
                    if tp_mode['collective'] == 'reducescatter':
                        dist.reduce_scatter_tensor(shard[li], flat[li], op=dist.ReduceOp.SUM)
                    else:
                        dist.all_reduce(flat[li], op=dist.ReduceOp.SUM)
        if world > 1:
            main.wait_stream(comm)

    def capture(label):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                one_pass()
        torch.cuda.synchronize()
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                one_pass()
            graph.replay()
            torch.cuda.synchronize()
            return graph.replay, 'cuda-graph' + (f" ({tp_mode['collective']} of the row-parallel shapes captured, second "
                                                 'stream)' if world > 1 else ''), graph
        except Exception as exc:       # keep measuring, say why the graph was not used
            torch.cuda.synchronize()
            return one_pass, f'eager ({label}: graph capture failed: {type(exc).__name__})', None

    def note(msg):
        if rank == 0 and os.environ.get('KAIROS_BENCH_VERBOSE'):
            print(f'[bench {time.strftime("%H:%M:%S")}] {msg}', file=sys.stderr, flush=True)

    note('layers, inputs and LUTs ready')
    ms_other = None
    if world > 1:
        # the other collective first, for the record; the headline uses args.tp_collective
        tp_mode['collective'] = 'allreduce' if args.tp_collective == 'reducescatter' else 'reducescatter'
        other_fn, _, other_graph = capture('other collective')
        ms_other, _ = timed_blocks(torch, dist, world, device, other_fn, args.steps, args.warmup, min_seconds=0.3)
        other_name = tp_mode['collective']
        del other_fn, other_graph
        tp_mode['collective'] = args.tp_collective
        note(f'other collective timed: {ms_other:.3f} ms per step')
    step_fn, mode, graph = capture('warm')
    note('warm pass captured: ' + mode)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    stats0 = ctx.stats()
    ms_step, blocks = timed_blocks(torch, dist, world, device, step_fn, args.steps, args.warmup, mark=True)
    stats1 = ctx.stats()
    clocks = sampler.stop() if rank == 0 else None
    n_timed_steps = len(blocks) * args.steps

    note(f'timed region done: {ms_step:.3f} ms per step')
    ms_eager, _ = timed_blocks(torch, dist, world, device, one_pass, max(1, args.steps // 4), 1, min_seconds=0.2)
    note('eager pass timed')
    ms_e2e, _ = timed_blocks(torch, dist, world, device, one_pass_host, max(1, args.steps // 4), 1, min_seconds=0.5)
    note('host-buffer pass timed')

    # ---- the cold regime: same pass, nothing cached (every W8A8 / W8A16 / FP16 call converts first) ----
    use('cold')
    cold_fn, cold_mode, cold_graph = capture('cold')
    ms_cold, _ = timed_blocks(torch, dist, world, device, cold_fn, max(1, args.steps // 2), 2, min_seconds=0.5)
    cold_graph = None
    use('warm')

    # ---- N > 1: the reduced and the sharded outputs of this pass against the per-shard oracle ----
    parity = None
    if world > 1:
        step_fn()
        torch.cuda.synchronize()
        results = dict(views)
        if args.tp_collective == 'reducescatter':
            # rank 0's token rows hold the three checked M (offsets 0, 63, 1023; 16384 / world >= 2048 rows)
            off = 0
            for m in M_LIST:
                for li in shard:
                    results[(li, m)] = shard[li][off:off + m] if off + m <= rows_pad // world else None
                off += m
        note('cold regime timed; checking parity')
        parity = check_parity(torch, dist, kb, rank, world, mods, reduced, results, xs_host, prof)
        note('parity checked')
        parity['row_parallel_collective'] = args.tp_collective

    # kernels launched per pass: one GEMV/GEMM per point (+1 split-K reduce where split), +1 activation
    # quantization for W8A8, +1 conversion per cache miss
    launches = 0
    for (n_, k_) in shapes:
        for m in M_LIST:
            cid = prof.get_comp_type((n_, k_), m)
            launches += 2 if cid == 2 else 1
            if cid != 1 and lib.kairos_gemm_workspace_bytes(m, n_, k_) > 0:
                launches += 1
    launches = launches * n_timed_steps + (stats1['misses'] - stats0['misses'])

    # ---- per-point table and rooflines (N = 1).  Every point is graph-timed: the profiler replays a CUDA
    # graph of calls that rotate over copies of the layer (> 2x L2), so there are no host gaps and the
    # weights come from HBM.
    points, roof, roof_gemv, same_cfg, llm_res = [], None, None, None, None
    if world == 1:
        for li, (k, n) in enumerate(SHAPES_KN):
            shape = shapes[li]
            for m in M_LIST:
                row, row_cold = prof.timings[shape][m], prof_cold.timings[shape][m]
                name = min(row, key=row.get)
                us = 1e3 * row[name]
                fl = 2 * m * k * n
                roof_us = max(algorithmic_bytes(m, k, n) / peaks['hbm_gbs'] / 1e3, fl / peaks['bf16_tflops'] / 1e6)
                points.append({'K': k, 'N': n, 'M': m, 'kernel': name, 'us': round(us, 2),
                               'tflops': round(fl / us / 1e6, 2),
                               'hbm_frac': round(algorithmic_bytes(m, k, n) / (us * 1e-6) / 1e9 / peaks['hbm_gbs'], 3),
                               'tensor_frac': round(fl / us / 1e6 / peaks['bf16_tflops'], 3),
                               'roof_frac': round(roof_us / us, 3),
                               'timing': 'graph + rotating layer copies',
                               'cold_kernel': min(row_cold, key=row_cold.get),
                               'cold_us': round(1e3 * min(row_cold.values()), 2)})
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
        roof, roof_gemv = dominant_rooflines(torch, kb, mods, xs_dev, prof, peaks, flush, l2_bytes)
        # the three points of the CPU arm, on the GPU, same LUT (one same-configuration ratio)
        cpu_fl = sum(2 * m * k * n for (k, n), m in CPU_SAMPLE)
        calls = []
        for (k, n), m in CPU_SAMPLE:
            mod = mods[SHAPES_KN.index((k, n))]
            calls.append(lambda mod=mod, k=k, n=n, m=m: mod._forward(xs_dev[(k, n)][:m], m, prof.get_comp_type(mod.shape, m)))
        us3 = graph_us_per_call(torch, calls, reps=20) * len(calls)
        same_cfg = {'points': [f'M={m} K={k} N={n}' for (k, n), m in CPU_SAMPLE], 'gpu_us': round(us3, 2),
                    'gpu_tflops': cpu_fl / us3 / 1e6, 'note': 'same three points as cpu_baseline / the reference arm'}
        del flush
        if not args.no_llm:
            del graph
            step_fn = None
            llm_res = llm_block(torch, kb, runtime, device, prof, ctx)

    if world > 1:
        # graphs with captured collectives must be gone before the process group is destroyed
        step_fn = cold_fn = graph = None
        import gc
        gc.collect()
        torch.cuda.synchronize()
        dist.barrier()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    h2d = sum(2 * m * (k // world if tp and tp.layer_kind(SHAPE_ROLE[(k, n)]) == 'row' else k)
              for (k, n) in SHAPES_KN for m in M_LIST)
    out = {
        'metric': METRIC, 'value': total_flops / (ms_step * 1e-3) / 1e12, 'unit': 'TFLOPS', 'n_gpus': world,
        'steps': args.steps, 'warmup': max(3, args.warmup), 'ms_per_step': ms_step, 'higher_is_better': True,
        'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f16/int8 (per LUT choice)',
        'data': 'synthetic',
        'config': {'workload': 'llama3-8b-linear-sweep', 'shapes_KN': SHAPES_KN, 'M': M_LIST,
                   'parallelism': f'tp{world}' if world > 1 else 'single', 'step_mode': mode,
                   'timed_region': f'{len(blocks)} blocks of {args.steps} steps ({sum(blocks) * args.steps / 1e3:.2f} s of device '
                                   'time), ms_per_step = median block, clocks sampled during the region',
                   'eager_ms_per_step': ms_eager,
                   'l2': 'inputs larger than L2: a pass touches >400 MB between two uses of any tensor; the '
                         'per-point table rotates layer copies (> 2x L2)',
                   'lut': 'profiled on device before the timed region; value = warm regime (the four layers fit the '
                          'bounded cache), value_cold = nothing cached, conversion inside every W8A8/W8A16/FP16 call',
                   'cache_bytes': cache_bytes, 'profile_seconds': round(t_prof, 1)},
        'value_cold': total_flops / (ms_cold * 1e-3) / 1e12, 'ms_per_step_cold': ms_cold, 'step_mode_cold': cold_mode,
        'e2e': {'value': total_flops / (ms_e2e * 1e-3) / 1e12, 'unit': 'TFLOPS', 'h2d_bytes_per_step': h2d,
                'd2h_bytes_per_step': sum(2 * m * n for (k, n) in SHAPES_KN for m in M_LIST),
                'ms_per_step': ms_e2e},
        'gpu_launches': int(launches),
        'clocks': clocks,
        'lut': {str(s): prof.seg_perf_list[i] for i, s in enumerate(shapes)},
        'lut_cold': {str(s): prof_cold.seg_perf_list[i] for i, s in enumerate(shapes)},
        'profile_us': {str(s): {str(m): {k2: round(v * 1e3, 2) for k2, v in row.items()}
                                for m, row in prof.timings[s].items()} for s in shapes},
        'profile_us_cold': {str(s): {str(m): {k2: round(v * 1e3, 2) for k2, v in row.items()}
                                     for m, row in prof_cold.timings[s].items()} for s in shapes},
        'peaks': peaks,
    }
    if parity is not None:
        out['parity_checked'] = parity['ok']
        out['parity'] = parity
        out['config']['row_parallel_collective'] = (
            'reduce-scatter over the token rows (sum left sequence-sharded; half the bytes of an all-reduce)'
            if args.tp_collective == 'reducescatter' else 'all-reduce (full sum on every rank)')
        out['ms_per_step_other_collective'] = {other_name: ms_other}
    if roof:
        out['roofline'] = roof
        out['roofline_gemv'] = roof_gemv
    if world == 1:
        out['cpu_baseline'] = cpu_baseline()
        out['same_config'] = same_cfg
        if same_cfg and out['cpu_baseline']['value']:
            same_cfg['gpu_over_cpu'] = same_cfg['gpu_tflops'] / out['cpu_baseline']['value']
        out['points'] = points
        if llm_res is not None:
            out['ttft_tpot'] = llm_res
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def check_parity(torch, dist, kb, rank, world, mods, reduced, views, xs_host, prof):
    """Outputs of the tensor-parallel pass against the CPU oracle, on sampled output channels: every
    row-parallel output (after the all-reduce) against the sum of the per-shard oracle results, every
    column-parallel shard against its own oracle; M in {1, 64, 1024}; tolerance |y - ref| <= 1e-2 |ref| +
    1e-2 RMS(ref).  Each rank reports the kernel ids its LUT chose, so the oracle evaluates the same kernels."""
    from kairos_b200.synthetic import make_case
    from oracle import kairos_oracle as ko
    ms = (1, 64, 1024)
    mine = {li: {m: int(prof.get_comp_type(mods[li].shape, m)) for m in ms} for li in range(len(mods))}
    gathered = [None] * world
    dist.all_gather_object(gathered, mine)
    got = {(li, m): views[(li, m)].float().cpu().numpy() for li in range(len(mods)) for m in ms}
    res = {'ok': True, 'checked': 0, 'worst': 0.0, 'points': []}
    if rank != 0:
        return res
    rng = np.random.default_rng(7)
    for li, (k, n) in enumerate(SHAPES_KN):
        _, w = make_case(1, k, n, seed=0)
        x_full, _ = make_case(max(M_LIST), k, 4, seed=1)
        if reduced[li]:
            cols = np.sort(rng.choice(n, size=32, replace=False))
            ks = k // world
            for m in ms:
                ref = np.zeros((m, len(cols)), np.float32)
                for r in range(world):
                    shard = ko.from_module(np.ascontiguousarray(w[cols][:, r * ks:(r + 1) * ks]))
                    ref += ko.forward(np.ascontiguousarray(x_full[:m, r * ks:(r + 1) * ks]), shard, gathered[r][li][m]).astype(np.float32)
                y = got[(li, m)][:, cols]
                bad, rms = ko.within_tolerance(y, ref.astype(np.float16))
                res['points'].append({'K': k, 'N': n, 'M': m, 'kind': 'row+allreduce', 'bad': int(bad)})
                res['checked'] += y.size
                res['ok'] = res['ok'] and bad == 0
        else:
            ns = n // world
            cols = np.sort(rng.choice(ns, size=32, replace=False))        # rank 0 holds rows 0 .. n/world
            shard = ko.from_module(np.ascontiguousarray(w[cols]))
            for m in ms:
                ref = ko.forward(np.ascontiguousarray(x_full[:m]), shard, gathered[0][li][m])
                y = got[(li, m)][:, cols]
                bad, rms = ko.within_tolerance(y, ref)
                res['points'].append({'K': k, 'N': n, 'M': m, 'kind': 'column shard', 'bad': int(bad)})
                res['checked'] += y.size
                res['ok'] = res['ok'] and bad == 0
    return res


# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) as ONE ncu capture of the same kernel
# and shape recorded it (the summaries under profiles/ name command and values); not measured by this run.
PROFILE_TRAFFIC = {
    'umma_gemm_pair_kernel<int8> (cta_group::2, 256x256)': (152148992 + 191360768, 'profiles/umma_gemm_pair_int8_M8192_K4096_N14336.md'),
    'umma_gemm_pair_kernel<f16> (cta_group::2, 256x256)': (372429056 + 216130304, 'profiles/umma_gemm_pair_f16_M8192_K4096_N14336.md'),
    'decode': (31241216, 'profiles/decode_split_M1_K4096_N14336.md'),
}


def dominant_rooflines(torch, kb, mods, xs_dev, prof, peaks, flush, l2_bytes):
    """Roofline of the kernel that dominates the pass (the M=8192 GEMM of the gate/up shape, in
    the precision the LUT chose) and of the decode kernel at M=1 on every shape."""
    from kairos_b200 import ops
    li = 2
    k, n = SHAPES_KN[li]
    mod = mods[li]
    m = max(M_LIST)
    x = xs_dev[(k, n)][:m]
    cid = prof.get_comp_type(mod.shape, m)
    name = kb.COMP_TYPE_ID[cid]
    pair_ok = m >= 512 and ((n + 255) // 256) * ((m + 255) // 256) >= torch.cuda.get_device_properties(x.device).multi_processor_count // 2

    def time_call(fn, reps=10):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(reps):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        return statistics.mean(ts) * 1e-3

    int8_peak = peaks.get('int8_tops_measured')
    if cid == 2:
        w8 = mod._trans_weight_to_8()
        xq = torch.empty((m, k), dtype=torch.int8, device=x.device)
        sx = torch.empty((m,), dtype=torch.float16, device=x.device)
        ops.quant_fp16_to_int8(xq, x, sx)
        y = torch.empty((m, n), dtype=torch.float16, device=x.device)
        t = time_call(lambda: ops.w8a8_gemm_forward_cuda(xq, w8, mod.scales_1, sx, y))
        if int8_peak:
            peak, peak_note = int8_peak, 'measured in this run: torch._int_mm 8192^3, burst'
        else:
            peak, peak_note = 2 * peaks['bf16_tflops'], '2 x measured bf16 burst (no int8 library GEMM to measure)'
        kern = 'umma_gemm_pair_kernel<int8> (cta_group::2, 256x256)' if pair_ok else 'umma_gemm_kernel<int8, BT=256>'
    elif cid == 5:
        w16 = mod._trans_weight_to_16()
        t = time_call(lambda: ops.f16_gemm(x, w16))
        peak, peak_note = peaks['bf16_tflops'], f'{peaks["source"]}: bf16 burst'
        kern = 'umma_gemm_pair_kernel<f16> (cta_group::2, 256x256)' if pair_ok else 'umma_gemm_kernel<f16, BT=256>'
    elif cid == 3:
        w8 = mod._trans_weight_to_8()
        t = time_call(lambda: ops.w8a16_gemm(x, w8, mod.scales_1))
        peak, peak_note = peaks['bf16_tflops'], f'{peaks["source"]}: bf16 burst'
        kern = 'umma_gemm_kernel<f16, w8-expand, BT=256>'
    else:
        t = time_call(lambda: ops.gemm_forward_cuda_new(x, mod.qweight, mod.scales, mod.scaled_zeros))
        peak, peak_note = peaks['bf16_tflops'], f'{peaks["source"]}: bf16 burst'
        kern = 'umma_gemm_kernel<f16, w4-expand, BT=256>'
    ach = 2 * m * k * n / t / 1e12
    tr = PROFILE_TRAFFIC.get(kern)
    roof = {'bound': 'tensor', 'kernel': kern, 'lut_choice': name, 'point': {'M': m, 'K': k, 'N': n},
            'achieved': ach, 'peak': peak, 'unit': 'TFLOP/s', 'frac': ach / peak,
            'traffic': tr[0] if tr else None, 'traffic_source': (tr[1] + ' (one ncu capture, not this run)') if tr else None,
            'peak_source': peak_note, 'frac_of_2x_bf16_burst': ach / (2 * peaks['bf16_tflops']) if cid == 2 else None,
            'us_per_launch': t * 1e6}
    # kernel id 1 at M = 1 on every shape of the sweep
    table, main = [], None
    for (kk, nn), mo in zip(SHAPES_KN, mods):
        x1 = xs_dev[(kk, nn)][:1]
        rot = RotatingWeights(torch, mo, l2_bytes)
        calls = [lambda i=i: ops.gemv_forward_cuda_new(x1, rot.qw[i], rot.sc[i], rot.sz[i], 1, nn, kk, 128) for i in range(rot.n)]
        us1 = graph_us_per_call(torch, calls)
        ach1 = algorithmic_bytes(1, kk, nn) / us1 / 1e3
        rowd = {'K': kk, 'N': nn, 'us_per_launch': round(us1, 2), 'achieved_gbs': round(ach1, 1),
                'frac': round(ach1 / peaks['hbm_gbs'], 3), 'algorithmic_bytes': algorithmic_bytes(1, kk, nn), 'copies': rot.n}
        table.append(rowd)
        if (kk, nn) == (k, n):
            main = (us1, ach1, rot.n)
        del rot
    us1, ach1, copies = main
    tr = PROFILE_TRAFFIC['decode']
    roof_gemv = {'bound': 'hbm', 'kernel': 'decode_split_kernel<1, 2, 1> (kernel id 1 at M=1)', 'point': {'M': 1, 'K': k, 'N': n},
                 'achieved': ach1, 'peak': peaks['hbm_gbs'], 'unit': 'GB/s', 'frac': ach1 / peaks['hbm_gbs'],
                 'traffic': tr[0], 'traffic_source': tr[1] + ' (one ncu capture, not this run)',
                 'algorithmic_bytes': algorithmic_bytes(1, k, n),
                 'peak_source': f'{peaks["source"]}: stream copy', 'us_per_launch': us1,
                 'timing': f'CUDA graph over {copies} weight copies (> 2x L2)', 'per_shape_M1': table}
    return roof, roof_gemv


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='kairos_b200', choices=['kairos_b200', 'reference'])
    ap.add_argument('--prof-iters', type=int, default=20)
    ap.add_argument('--no-llm', action='store_true', help='skip the TTFT/TPOT block (N = 1)')
    ap.add_argument('--tp-collective', default='reducescatter', choices=['reducescatter', 'allreduce'],
                    help='N > 1: how the partial outputs of the row-parallel shapes are summed')
    args = ap.parse_args()
    if args.impl == 'reference':
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == '__main__':
    main()
