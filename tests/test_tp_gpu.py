"""Tensor parallelism on real GPUs (needs two): NCCL all-reduce after the row-parallel layer, per-rank
quantization, per-rank kernels; checked against the per-shard oracle."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import kairos_oracle as ko

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ['NCCL_NVLS_ENABLE'] = '0'
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    import kairos_b200 as kb
    from kairos_b200 import tp
    dev = torch.device('cuda', rank)
    x, w = ko.make_case(24, 1024, 512, seed=13)
    xt, wt = torch.from_numpy(x), torch.from_numpy(w)
    col = tp.shard_linear(wt, 'col', rank, world, dev)
    row = tp.shard_linear(wt, 'row', rank, world, dev)
    prof = kb.Profiler([col.linear.shape, row.linear.shape])
    prof.load_table({col.linear.shape: [(8, 'w4a16_gemv'), (30720, 'w4a16_gemm')],
                     row.linear.shape: [(8, 'w4a16_gemv'), (30720, 'w8a8')]})
    kb.DynamicLinear.prof = prof
    col.gather_output = True
    ks = 1024 // world
    res = {}
    for m in (4, 24):
        xm = xt[:m].to(dev)
        res[f'col{m}'] = col(xm.unsqueeze(0))[0].cpu().numpy()
        res[f'row{m}'] = row(xm[:, rank * ks:(rank + 1) * ks].contiguous().unsqueeze(0))[0].cpu().numpy()
    torch.cuda.synchronize()
    if rank == 0:
        out.update(res)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs two GPUs')
def test_two_gpu_tensor_parallel_matches_per_shard_oracle():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    x, w = ko.make_case(24, 1024, 512, seed=13)
    for m in (4, 24):
        xm = x[:m]
        col = np.concatenate([ko.y_w4a16(xm, ko.from_module(w[r * 256:(r + 1) * 256])) for r in range(world)], axis=1)
        bad, _ = ko.within_tolerance(out[f'col{m}'], col)
        assert bad == 0, f'column parallel m={m}'
        comp = 1 if m <= 8 else 2
        parts = [ko.forward(xm[:, r * 512:(r + 1) * 512], ko.from_module(np.ascontiguousarray(w[:, r * 512:(r + 1) * 512])), comp)
                 for r in range(world)]
        row = (parts[0].astype(np.float32) + parts[1].astype(np.float32)).astype(np.float16)
        bad, _ = ko.within_tolerance(out[f'row{m}'], row)
        assert bad == 0, f'row parallel m={m}'


def _decoder_worker(rank, world, port, out):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ['NCCL_NVLS_ENABLE'] = '0'
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    dist.all_reduce(torch.zeros(1, device=dev))
    import kairos_b200 as kb
    from kairos_b200 import llm
    cfg = llm.DecoderConfig('tiny', 2, 512, 8, 4, 64, 1024, 1000)
    model = llm.Decoder(cfg, dev, layers=2, tp_rank=rank, tp_world=world)
    assert model.cfg.n_heads == 4 and model.cfg.n_kv_heads == 2 and model.cfg.inter == 512
    prof = kb.Profiler(model.linear_shapes())
    prof.load_table({s: [(4, 'w4a16_gemv'), (16, 'w4a16_gemm'), (30720, 'w8a8')] for s in model.linear_shapes()})
    kb.DynamicLinear.prof = prof
    tokens = torch.randint(0, cfg.vocab, (2, 24), generator=torch.Generator(device=dev).manual_seed(3), device=dev)
    model.allocate(2, 64)
    eager = model.generate(tokens, 6, use_graph=False)
    model.allocate(2, 64)
    graphed = model.generate(tokens, 6, use_graph=True)      # the all-reduces are captured with the step
    torch.cuda.synchronize()
    gathered = [torch.empty_like(graphed) for _ in range(world)]
    dist.all_gather(gathered, graphed)
    # the same step with the peer sum as a kernel of its own instead of inside the RMSNorm, and through NCCL
    assert model.peer_ar is not None and model.fuse_peer_sum
    model.release_graphs()
    model.fuse_peer_sum = False
    model.allocate(2, 64)
    unfused = model.generate(tokens, 6, use_graph=True)
    model.release_graphs()
    model.peer_ar = None
    model.allocate(2, 64)
    by_nccl = model.generate(tokens, 6, use_graph=True)
    torch.cuda.synchronize()
    if rank == 0:
        out['eager'] = eager.cpu().numpy()
        out['graphed'] = graphed.cpu().numpy()
        out['unfused'] = unfused.cpu().numpy()
        out['by_nccl'] = by_nccl.cpu().numpy()
        out['ranks_agree'] = all(torch.equal(g, graphed) for g in gathered)
        out['status'] = kb.runtime.device_status()
    model.release_graphs()      # graphs with captured collectives must be gone before the group is destroyed
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs two GPUs')
def test_two_gpu_tensor_parallel_decoder_graph_matches_eager():
    """A two-rank tensor-parallel decoder (sharded heads and inner channels, all-reduce after o_proj and
    down_proj): the CUDA-graph path with the collectives captured gives the eager path's tokens, and every
    rank ends with the same tokens.  Small row-parallel outputs are summed over NVLink peer memory inside the
    RMSNorm that consumes them; the stand-alone peer kernel and NCCL give the same tokens."""
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_decoder_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert out['ranks_agree']
    assert np.array_equal(out['eager'], out['graphed'])
    # sum inside the RMSNorm == stand-alone peer kernel == NCCL (two ranks: one fp16 rounding of a + b either way)
    assert np.array_equal(out['graphed'], out['unfused'])
    assert np.array_equal(out['graphed'], out['by_nccl'])
    assert out['status'] == 0


def _peer_allreduce_worker(rank, world, port, out):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ['NCCL_NVLS_ENABLE'] = '0'
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    dist.all_reduce(torch.zeros(1, device=dev))
    import kairos_b200 as kb
    from kairos_b200 import tp
    ar = tp.PeerAllReduce(None, dev, 64 * 1024)
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    ok = True

    def expected(part):
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part.contiguous())
        acc = torch.zeros(part.shape, dtype=torch.float32, device=dev)
        for p in parts:                       # rank order, fp32, one rounding at the end
            acc += p.float()
        return acc.half()

    for (m, n) in [(1, 8), (1, 4096), (24, 512), (3, 1000), (64, 1024)] * 2:    # eager, slots alternate
        part = ar.partial(m, n)
        part.copy_(torch.randn((m, n), generator=gen, device=dev, dtype=torch.float32).half())
        want = expected(part)
        got = ar.reduce(m, n)
        torch.cuda.synchronize()
        ok = ok and torch.equal(got, want)
    # four calls captured in one graph and replayed: sequence numbers advance on the device
    m, n = 8, 2048
    srcs = [torch.randn((m, n), generator=gen, device=dev, dtype=torch.float32).half() for _ in range(4)]
    wants = [expected(s) for s in srcs]
    outs = [torch.empty((m, n), dtype=torch.float16, device=dev) for _ in range(4)]
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for s, o in zip(srcs, outs):
                ar.partial(m, n).copy_(s)
                ar.reduce(m, n, out=o)
    for _ in range(3):
        for o in outs:
            o.zero_()
        graph.replay()
        torch.cuda.synchronize()
        ok = ok and all(torch.equal(o, w) for o, w in zip(outs, wants))
    # the sum folded into the RMSNorm that consumes it == stand-alone sum, then the norm with a local delta
    from kairos_b200 import ops
    for (m, k, quant) in [(1, 512, False), (5, 4096, True), (64, 1024, False), (8, 8192, True)] * 2:
        part = ar.partial(m, k)
        part.copy_(torch.randn((m, k), generator=gen, device=dev, dtype=torch.float32).half())
        want_delta = expected(part)
        x0 = torch.randn((m, k), generator=torch.Generator(device=dev).manual_seed(7), device=dev, dtype=torch.float32).half()
        w = torch.randn((k,), generator=torch.Generator(device=dev).manual_seed(8), device=dev, dtype=torch.float32).half()
        xa, xb = x0.clone(), x0.clone()
        pending = ar.defer(m, k)
        if quant:
            qa, sa, ya = ops.rms_norm_quant(xa, w, 1e-5, want_f16=True, residual_delta=pending)
            qb, sb, yb = ops.rms_norm_quant(xb, w, 1e-5, want_f16=True, residual_delta=want_delta)
            same = torch.equal(qa, qb) and torch.equal(sa, sb) and torch.equal(ya, yb)
        else:
            ya = ops.rms_norm(xa, w, 1e-5, residual_delta=pending)
            yb = ops.rms_norm(xb, w, 1e-5, residual_delta=want_delta)
            same = torch.equal(ya, yb)
        torch.cuda.synchronize()
        ok = ok and same and torch.equal(xa, xb)          # x += delta in place, both ways
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        out['ok'] = bool(flag.item())
        out['status'] = kb.runtime.device_status()
    del graph
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs two GPUs')
def test_two_gpu_peer_memory_allreduce_is_the_rank_ordered_sum():
    """The library's all-reduce over peer memory: bit-identical to the fp32 sum of the partials in rank order
    on every rank, eagerly with alternating slots and replayed from a CUDA graph."""
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_peer_allreduce_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert out['ok']
    assert out['status'] == 0
