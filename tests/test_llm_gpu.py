"""Decoder harness: the fused CUDA glue (RMSNorm, rotary + KV write, SiLU*up) against stock torch ops on
the same quantized model, prefill and graph-replayed decode."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _act_quant(y):
    """The stand-alone activation-quantization operator: int8 values and one fp16 scale per token."""
    from kairos_b200 import ops
    k = y.shape[-1]
    q = torch.empty(y.shape, dtype=torch.int8, device=y.device)
    s = torch.empty((y.numel() // k,), dtype=torch.float16, device=y.device)
    ops.quant_fp16_to_int8(q, y, s)
    return q, s


def test_glue_ops_match_torch():
    from kairos_b200 import ops
    torch.manual_seed(0)
    x = (torch.randn(37, 4096, device='cuda') * 3).half()
    w = (1 + 0.1 * torch.randn(4096, device='cuda')).half()
    v = x.float()
    ref = (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()).half()
    got = ops.rms_norm(x, w, 1e-5)
    assert (got.float() - ref.float()).abs().max() <= 2e-3 * ref.float().abs().max()
    gu = torch.randn(19, 2 * 1024, device='cuda').half()
    ref = torch.nn.functional.silu(gu[:, :1024]) * gu[:, 1024:]
    got = ops.silu_mul(gu)
    assert (got.float() - ref.float()).abs().max() <= 4e-3


def test_decoder_cuda_glue_matches_torch_glue():
    import kairos_b200 as kb
    from kairos_b200 import llm, runtime
    cfg = llm.DecoderConfig('tiny', 2, 512, 8, 2, 64, 1024, 1000, 1e-5, 10000.0, True)
    ctx = runtime.Context('cuda', cache_bytes=None)
    kb.DynamicLinear.context = ctx
    try:
        model = llm.Decoder(cfg, 'cuda', fuse_linears=True, glue='cuda')
        prof = kb.Profiler(model.linear_shapes())
        prof.load_table({s: [(4, 'w4a16_gemv'), (16, 'w4a16_gemm'), (30720, 'w8a8')] for s in model.linear_shapes()})
        kb.DynamicLinear.prof = prof
        tokens = torch.randint(0, cfg.vocab, (3, 40), device='cuda', generator=torch.Generator('cuda').manual_seed(1))
        outs = {}
        for glue in ('torch', 'cuda'):
            model.glue = glue
            model.allocate(3, 64)
            logits = model.prefill(tokens, return_logits=True).float()
            nxt = logits.argmax(dim=-1, keepdim=True)
            steps = []
            for _ in range(5):
                model.tok.copy_(nxt)
                model.decode_step(use_graph=(glue == 'cuda'))
                steps.append(model.logits.float().clone())
                nxt = model.next_tok.clone()
            outs[glue] = (logits, steps)
        ref, got = outs['torch'], outs['cuda']
        scale = ref[0].abs().max().item()
        assert (ref[0] - got[0]).abs().max().item() <= 3e-2 * scale
        # decode logits: compare the first step (same input token), loosely (fp16 glue rounding differs)
        assert (ref[1][0] - got[1][0]).abs().max().item() <= 5e-2 * scale
        assert torch.isfinite(got[1][-1]).all()
    finally:
        kb.DynamicLinear.context = None
        kb.DynamicLinear.prof = None


@pytest.mark.parametrize('m,k', [(1, 512), (37, 4096), (5, 3584), (3, 8192)])
def test_rms_norm_quant_equals_norm_then_act_quant(m, k):
    """The fused operator writes exactly what RMSNorm followed by the activation-quantization kernel writes."""
    from kairos_b200 import ops
    g = torch.Generator('cuda').manual_seed(m * 131 + k)
    x = (torch.randn(m, k, device='cuda', generator=g) * 2.5).half()
    w = (1 + 0.1 * torch.randn(k, device='cuda', generator=g)).half()
    y = ops.rms_norm(x, w, 1e-5)
    q_ref, s_ref = _act_quant(y)
    xq, sx, yf = ops.rms_norm_quant(x, w, 1e-5, want_f16=True)
    assert torch.equal(yf, y)
    assert torch.equal(sx.view(-1), s_ref.view(-1))
    assert torch.equal(xq, q_ref.view_as(xq))
    xq2, sx2, none = ops.rms_norm_quant(x, w, 1e-5)
    assert none is None and torch.equal(xq2, xq) and torch.equal(sx2, sx)


@pytest.mark.parametrize('m,i', [(1, 1024), (19, 14336), (4, 18944), (2, 28672)])
def test_silu_mul_quant_equals_act_then_act_quant(m, i):
    from kairos_b200 import ops
    g = torch.Generator('cuda').manual_seed(m * 17 + i)
    gu = (torch.randn(m, 2 * i, device='cuda', generator=g) * 2).half()
    y = ops.silu_mul(gu)
    q_ref, s_ref = _act_quant(y)
    xq, sx, yf = ops.silu_mul_quant(gu, want_f16=True)
    assert torch.equal(yf, y)
    assert torch.equal(sx.view(-1), s_ref.view(-1))
    assert torch.equal(xq, q_ref.view_as(xq))


def test_forward_q8_equals_forward_on_w8a8():
    """A layer fed pre-quantized activations gives the bits of the same layer quantizing them itself."""
    import kairos_b200 as kb
    from kairos_b200 import ops, runtime, synthetic
    ctx = runtime.Context('cuda', cache_bytes=None)
    kb.DynamicLinear.context = ctx
    try:
        _, w = synthetic.make_case(1, 1024, 768, seed=3)
        ref_lin = torch.nn.Linear(1024, 768, bias=True, dtype=torch.float16)
        ref_lin.weight.data = torch.from_numpy(w.copy())
        lin = kb.DynamicLinear.from_module(ref_lin.cuda(), 'cuda')
        prof = kb.Profiler([lin.shape])
        prof.load_table({lin.shape: [(30720, 'w8a8')]})
        kb.DynamicLinear.prof = prof
        x = torch.randn(2, 45, 1024, device='cuda').half()
        ref = lin(x)
        assert lin.wants_int8(90)
        xq, sx = _act_quant(x)
        got = lin.forward_q8(xq.view(2, 45, 1024), sx.view(-1))
        assert torch.equal(ref, got)
        prof.load_table({lin.shape: [(30720, 'w4a16_gemm')]})
        lin.pre_m = None
        assert not lin.wants_int8(90)
    finally:
        kb.DynamicLinear.context = None
        kb.DynamicLinear.prof = None


def test_decoder_fused_quant_is_bit_identical():
    """Letting the norm / activation emit int8 changes no output bit of prefill or decode."""
    import kairos_b200 as kb
    from kairos_b200 import llm, runtime
    cfg = llm.DecoderConfig('tiny', 2, 512, 8, 2, 64, 1024, 1000, 1e-5, 10000.0, True)
    ctx = runtime.Context('cuda', cache_bytes=None)
    kb.DynamicLinear.context = ctx
    try:
        model = llm.Decoder(cfg, 'cuda', fuse_linears=True, glue='cuda')
        prof = kb.Profiler(model.linear_shapes())
        prof.load_table({s: [(2, 'w4a16_gemv'), (30720, 'w8a8')] for s in model.linear_shapes()})
        kb.DynamicLinear.prof = prof
        tokens = torch.randint(0, cfg.vocab, (3, 40), device='cuda', generator=torch.Generator('cuda').manual_seed(1))
        outs = {}
        for fq in (False, True):
            model.fuse_quant = fq
            model.allocate(3, 64)
            logits = model.prefill(tokens, return_logits=True).clone()
            model.tok.copy_(logits.argmax(dim=-1, keepdim=True))
            model.decode_step(use_graph=False)
            outs[fq] = (logits, model.logits.clone())
        assert torch.equal(outs[False][0], outs[True][0])
        assert torch.equal(outs[False][1], outs[True][1])
    finally:
        kb.DynamicLinear.context = None
        kb.DynamicLinear.prof = None


def test_add_rms_norm_carries_the_residual_addition():
    """x <- x + h in place (fp16 addition, as torch does it), then the norm; also in the int8-emitting form."""
    from kairos_b200 import ops
    g = torch.Generator('cuda').manual_seed(5)
    x = (torch.randn(9, 4096, device='cuda', generator=g) * 2).half()
    h = torch.randn(9, 4096, device='cuda', generator=g).half()
    w = (1 + 0.1 * torch.randn(4096, device='cuda', generator=g)).half()
    summed = x + h
    ref = ops.rms_norm(summed, w, 1e-5)
    x1 = x.clone()
    got = ops.rms_norm(x1, w, 1e-5, residual_delta=h)
    assert torch.equal(x1, summed) and torch.equal(got, ref)
    x2 = x.clone()
    xq, sx, y = ops.rms_norm_quant(x2, w, 1e-5, want_f16=True, residual_delta=h)
    q_ref, s_ref = _act_quant(ref)
    assert torch.equal(x2, summed) and torch.equal(y, ref)
    assert torch.equal(xq, q_ref) and torch.equal(sx, s_ref)


def test_chained_launches_give_the_same_bits_as_ordinary_launches():
    """A decode-like chain (norm -> small-batch W4A16 -> SiLU*up -> W4A16, repeated) under programmatic
    stream serialization, replayed from a CUDA graph, equals the same chain run with a device
    synchronization after every operator (where no kernel can overlap its predecessor)."""
    import kairos_b200 as kb
    from kairos_b200 import ops, runtime, synthetic
    ctx = runtime.Context('cuda', cache_bytes=None)
    kb.DynamicLinear.context = ctx
    try:
        lins = []
        for i, (k, n) in enumerate(((1024, 2048), (1024, 1024))):
            _, w = synthetic.make_case(1, k, n, seed=20 + i)
            ref_lin = torch.nn.Linear(k, n, bias=False, dtype=torch.float16)
            ref_lin.weight.data = torch.from_numpy(w.copy()) * 3
            lins.append(kb.DynamicLinear.from_module(ref_lin.cuda(), 'cuda'))
        prof = kb.Profiler([l.shape for l in lins])
        prof.load_table({l.shape: [(30720, 'w4a16_gemv')] for l in lins})
        kb.DynamicLinear.prof = prof
        w = torch.ones(1024, device='cuda', dtype=torch.float16)
        x0 = torch.randn(4, 1, 1024, device='cuda', generator=torch.Generator('cuda').manual_seed(2)).half()

        def chain(x, sync):
            delta = None
            for _ in range(6):
                h = ops.rms_norm(x, w, 1e-5, residual_delta=delta)
                if sync: torch.cuda.synchronize()
                gu = lins[0](h)
                if sync: torch.cuda.synchronize()
                act = ops.silu_mul(gu)
                if sync: torch.cuda.synchronize()
                delta = lins[1](act)
                if sync: torch.cuda.synchronize()
            return ops.rms_norm(x, w, 1e-5, residual_delta=delta)

        ref = chain(x0.clone(), True)
        eager = chain(x0.clone(), False)
        assert torch.equal(ref, eager)
        xs = x0.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            chain(xs.clone(), False)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            xin = xs.clone()
            out = chain(xin, False)
        for _ in range(3):
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(out, ref)
        assert runtime.device_status() == 0
    finally:
        kb.DynamicLinear.context = None
        kb.DynamicLinear.prof = None


def test_prefill_graph_equals_eager_prefill():
    """Replaying the captured prefill of a (B, S) gives the bits of the eager prefill, also for a second
    prompt of the same shape."""
    import kairos_b200 as kb
    from kairos_b200 import llm, runtime
    cfg = llm.DecoderConfig('tiny', 2, 512, 8, 2, 64, 1024, 1000, 1e-5, 10000.0, True)
    ctx = runtime.Context('cuda', cache_bytes=None)
    kb.DynamicLinear.context = ctx
    try:
        model = llm.Decoder(cfg, 'cuda', fuse_linears=True, glue='cuda')
        prof = kb.Profiler(model.linear_shapes())
        prof.load_table({s: [(8, 'w4a16_gemv'), (64, 'w4a16_gemm'), (30720, 'w8a8')] for s in model.linear_shapes()})
        kb.DynamicLinear.prof = prof
        gen = torch.Generator('cuda').manual_seed(4)
        model.allocate(2, 96)
        for _ in range(2):
            tokens = torch.randint(0, cfg.vocab, (2, 48), device='cuda', generator=gen)
            eager = model.prefill(tokens, return_logits=True).clone()
            kv_eager = model.kv.clone()
            model.kv.zero_()
            replay = model.prefill(tokens, return_logits=True, use_graph=True).clone()
            assert torch.equal(eager, replay)
            assert torch.equal(kv_eager, model.kv)
            assert int(model.pos.item()) == 48
    finally:
        kb.DynamicLinear.context = None
        kb.DynamicLinear.prof = None
