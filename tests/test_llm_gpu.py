"""Decoder harness: the fused CUDA glue (RMSNorm, rotary + KV write, SiLU*up) against stock torch ops on
the same quantized model, prefill and graph-replayed decode."""
import pytest
import torch

pytestmark = pytest.mark.gpu


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
