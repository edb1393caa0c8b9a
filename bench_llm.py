#!/usr/bin/env python
"""TTFT / TPOT of a random-init decoder whose linears are switched linears (the reference's end-to-end latency benchmark: Llama-3-8B, Qwen2-7B, Llama-3-70B geometries).

    python bench_llm.py --model llama3-8b --batches 2,4,8,16,32 --prompt 1024 --new 512
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        bench_llm.py --model llama3-70b --batches 1,8,32,64           # tensor parallel, one rank per GPU

Prints one JSON line per batch size: ttft_ms, tpot_ms, tokens_per_s, plus the LUT in use.  Protocol of
the reference (utils/perf_eval.py:236-275): warm-up generations, TTFT = mean prefill + first token,
TPOT = (t_generate - TTFT) / (new - 1).  Prompts are uniform random token ids (no dataset needed).
"""
import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='llama3-8b')
    ap.add_argument('--batches', default='2,4,8,16,32')
    ap.add_argument('--prompt', type=int, default=1024)
    ap.add_argument('--new', type=int, default=512)
    ap.add_argument('--layers', type=int, default=None, help='build only the first L layers (smoke runs)')
    ap.add_argument('--cache-gb', type=float, default=24.0, help='bound of the conversion cache')
    ap.add_argument('--lut', default='warm', choices=['warm', 'cold'])
    ap.add_argument('--no-fuse', action='store_true', help='keep q/k/v and gate/up as separate linears (7 per layer)')
    ap.add_argument('--compare-allreduce', action='store_true',
                    help='tensor parallel: measure a second time with the small all-reduces through NCCL')
    ap.add_argument('--glue', default='cuda', choices=['cuda', 'torch'], help="'torch' = stock torch ops around the linears")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist
    import kairos_b200 as kb
    from kairos_b200 import llm, runtime

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    dev = f'cuda:{local}'
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        dist.init_process_group('nccl', device_id=torch.device(dev))
        dist.all_reduce(torch.zeros(1, device=dev))          # communicator set up before any capture
    cfg = llm.PRESETS[args.model]
    ctx = runtime.Context(dev, cache_bytes=int(args.cache_gb * (1 << 30)))
    kb.DynamicLinear.context = ctx
    t0 = time.perf_counter()
    model = llm.Decoder(cfg, dev, layers=args.layers, fuse_linears=not args.no_fuse, glue=args.glue,
                        tp_rank=rank, tp_world=world)
    t_build = time.perf_counter() - t0
    t0 = time.perf_counter()
    prof = llm.build_lut(model.linear_shapes(), device=dev, cache=args.lut)
    t_lut = time.perf_counter() - t0
    if world > 1:
        dist.barrier()
    lut = {str(s): [(r, name) for r, name, _ in prof.seg_perf_list[i]] for i, s in enumerate(prof.shape_list)}
    say = (lambda *a, **k: print(*a, **k)) if rank == 0 else (lambda *a, **k: None)
    say(json.dumps({'model': model.cfg.name, 'tp': world, 'layers': len(model.model.layers), 'lut_seconds': round(t_lut, 1),
                      'build_seconds': round(t_build, 1), 'lut_mode': args.lut, 'lut': lut, 'fused_linears': not args.no_fuse, 'glue': args.glue,
                      'weights_gb': round(sum(b.numel() * b.element_size() for b in model.buffers()) / 2**30, 2)}))
    def sweep(label):
        for b in [int(v) for v in args.batches.split(',')]:
            r = llm.measure_ttft_tpot(model, b, args.prompt, args.new)
            r.update({'model': model.cfg.name, 'tp': world, 'small_allreduce': label, 'cache': ctx.stats(),
                      'peak_gb': round(torch.cuda.max_memory_allocated() / 2**30, 2)})
            say(json.dumps(r), flush=True)

    sweep('none' if world == 1 else ('peer-memory kernel' if model.peer_ar is not None else 'nccl'))
    if world > 1 and model.peer_ar is not None and args.compare_allreduce:
        # the same model with every all-reduce through NCCL (the decode graph is captured again)
        model.release_graphs()
        model.peer_ar = None
        sweep('nccl')
    if world > 1:
        model.release_graphs()      # captured collectives must be gone before the group is destroyed
        dist.barrier()
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
