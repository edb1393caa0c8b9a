#!/usr/bin/env python
"""Kernel-switch frequency under continuous batching (the reference's switch-frequency experiment, Qwen2-7B geometry).

64 requests with prompt lengths drawn lognormal(mu = ln 512, sigma = 1.0), clipped to 16..8192, 256 output
tokens each, are scheduled by a token-budget continuous batcher (prefill chunks and decode tokens share a
step).  Every step presents M_t = prefill tokens + running sequences to the decoder's linears, so M changes
almost every step and the per-layer LUT lookup and kernel switch are exercised the way a serving engine
would.  Only the switched linears run (they are the path under test; attention and sampling do not depend
on the kernel choice): per step, one stack of the model's four stacked linears per layer.

Stands in for the reference's request traces (eval/switch_frequency.py:13-33: BurstGPT / ShareGPT /
LongBench input lengths), which are not available here; the seeded lognormal draw has their heavy tail.

Prints one JSON line: steps, distinct M values, switches per layer and per linear shape, selection counts
per kernel, time spent in LUT lookups, and the linear time per generated token.
"""
import argparse
import collections
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def make_trace(n_req=64, out_tokens=256, budget=1024, max_running=64, mean_gap=6.0, seed=0):
    """Token-budget continuous batching with Poisson arrivals (mean `mean_gap` steps apart): each step
    first serves one decode token for every running sequence, then fills the remaining budget with
    prefill chunks of the requests that have arrived (FIFO).  Returns (prompt lengths, M per step)."""
    rng = np.random.default_rng(seed)
    prompts = np.clip(np.exp(rng.normal(np.log(512.0), 1.0, n_req)), 16, 8192).astype(int)
    arrivals = np.floor(np.cumsum(rng.exponential(mean_gap, n_req))).astype(int)
    pending = collections.deque(zip(arrivals.tolist(), prompts.tolist()))
    waiting = collections.deque()
    running = []          # remaining output tokens
    prefilling = None     # remaining prompt tokens of the request being prefilled
    steps, step = [], 0
    while pending or waiting or running or prefilling is not None:
        while pending and pending[0][0] <= step:
            waiting.append(pending.popleft()[1])
        m = len(running)
        room = budget - m
        newly = 0
        while room > 0 and (prefilling is not None or (waiting and len(running) + newly < max_running)):
            if prefilling is None:
                prefilling = waiting.popleft()
            take = min(room, prefilling)
            prefilling -= take
            room -= take
            m += take
            if prefilling == 0:
                newly += 1
                prefilling = None
            else:
                break
        running = [r - 1 for r in running if r > 1] + [out_tokens] * newly
        if m > 0:
            steps.append(m)
        step += 1
    return prompts.tolist(), steps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='qwen2-7b')
    ap.add_argument('--layers', type=int, default=None)
    ap.add_argument('--budget', type=int, default=1024)
    args = ap.parse_args()

    import torch
    import kairos_b200 as kb
    from kairos_b200 import llm, runtime

    torch.cuda.set_device(0)
    cfg = llm.PRESETS[args.model]
    ctx = runtime.Context('cuda:0', cache_bytes=24 << 30)
    kb.DynamicLinear.context = ctx
    model = llm.Decoder(cfg, 'cuda:0', layers=args.layers)
    prof = llm.build_lut(model.linear_shapes(), m_grid=[1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192])
    prompts, steps = make_trace(budget=args.budget)
    ctx.reserve(max(steps), max(s[0] for s in model.linear_shapes()), max(s[1] for s in model.linear_shapes()))

    layers = []
    for layer in model.model.layers:
        layers.append([m for m in layer.modules() if isinstance(m, kb.DynamicLinear)])
    k_in = {lin: lin.in_features for lin in layers[0]}
    xs = {k: torch.randn((max(steps), k), dtype=torch.float16, device='cuda:0') for k in set(k_in.values())}

    # LUT lookup cost alone (host), over the trace
    t0 = time.perf_counter()
    for m in steps:
        for lin in layers[0]:
            prof.get_comp_type(lin.shape, m)
    lut_us = 1e6 * (time.perf_counter() - t0) / (len(steps) * len(layers[0]))

    switches = collections.Counter()
    picks = collections.Counter()
    last = {}
    for _ in range(2):                                   # warm the conversion cache
        for lins in layers:
            for lin in lins:
                lin(xs[lin.in_features][:64].unsqueeze(0))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for m in steps:
        for li, lins in enumerate(layers):
            for lin in lins:
                lin(xs[lin.in_features][:m].unsqueeze(0))
                if li == 0:
                    picks[kb.COMP_TYPE_ID[lin.comp_type]] += 1
                    if last.get(lin.shape) is not None and last[lin.shape] != lin.comp_type:
                        switches[str(lin.shape)] += 1
                    last[lin.shape] = lin.comp_type
    torch.cuda.synchronize()
    total = time.perf_counter() - t0
    tokens_out = 64 * 256
    print(json.dumps({
        'model': cfg.name, 'layers': len(layers), 'requests': 64, 'prompt_len_median': int(np.median(prompts)),
        'prompt_len_max': int(max(prompts)), 'steps': len(steps), 'distinct_M': len(set(steps)),
        'M_changes': int(sum(1 for a, b in zip(steps, steps[1:]) if a != b)), 'M_min': min(steps), 'M_max': max(steps),
        'kernel_switches_per_layer': dict(switches), 'selections_per_layer': dict(picks),
        'lut_lookup_us': round(lut_us, 3), 'linear_seconds_total': round(total, 3),
        'linear_ms_per_step': round(1e3 * total / len(steps), 3),
        'linear_us_per_generated_token': round(1e6 * total / tokens_out, 1),
        'lut': {str(s): [(r, n) for r, n, _ in prof.seg_perf_list[i]] for i, s in enumerate(prof.shape_list)}}))


if __name__ == '__main__':
    main()
