"""Gated MLP with the gate and up rows of the stacked weight in blocks of 16: the SiLU * up kernels for that layout,
and the decode kernel that applies SiLU(gate) * up in its epilogue, against the unfused sequence, bit for bit."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import kairos_oracle as ko  # noqa: E402


def _block(gu_plain):
    """[m, 2 I] with gate | up one after the other -> the blocked order (16 gate, their 16 up, ...)."""
    m, i2 = gu_plain.shape
    i = i2 // 2
    g = gu_plain[:, :i].reshape(m, i // 16, 1, 16)
    u = gu_plain[:, i:].reshape(m, i // 16, 1, 16)
    return torch.cat((g, u), dim=2).reshape(m, i2).contiguous()


@pytest.mark.parametrize('m,i', [(1, 1024), (19, 14336), (4, 18944), (2, 28672), (3, 48)])
def test_blocked_silu_kernels_equal_the_plain_ones(m, i):
    from kairos_b200 import ops
    gu = (torch.randn((m, 2 * i), device='cuda', generator=torch.Generator('cuda').manual_seed(m + i)) * 2).half()
    plain = ops.silu_mul(gu)
    assert torch.equal(ops.silu_mul(_block(gu), blocked=True), plain)
    if i % 16 == 0 and i >= 64:
        q0, s0, y0 = ops.silu_mul_quant(gu, want_f16=True)
        q1, s1, y1 = ops.silu_mul_quant(_block(gu), want_f16=True, blocked=True)
        assert torch.equal(q0, q1) and torch.equal(s0, s1) and torch.equal(y0, y1) and torch.equal(y0, plain)


@pytest.mark.parametrize('m,k,n', [(1, 4096, 28672), (2, 512, 64), (5, 1024, 2048), (8, 4096, 28672), (16, 2048, 4096),
                                   (32, 1024, 1056), (3, 8192, 7168), (13, 256, 96), (1, 14336, 8192)])
def test_decode_kernel_with_gated_epilogue_equals_decode_then_silu(m, k, n):
    """Every cluster size and both rows-per-warp variants; N = 1056 and 96 leave a row tile partly outside."""
    from kairos_b200 import ops
    x, w = ko.make_case(m, k, n, seed=m + n)
    res = ko.from_module(w)
    t = {key: torch.from_numpy(np.ascontiguousarray(res[key])).cuda() for key in ('qweight', 'scales', 'scaled_zeros')}
    xd = torch.from_numpy(x).cuda()
    y = ops.decode_forward(xd, t['qweight'], t['scales'], t['scaled_zeros'], m, n, k)
    want = ops.silu_mul(y, blocked=True)
    got = ops.decode_silu_forward(xd, t['qweight'], t['scales'], t['scaled_zeros'], m, n, k)
    assert got.shape == (m, n // 2)
    assert torch.equal(got, want)
    # and against the oracle, through the blocked pairing (tolerance of the fp16 kernels on the linear's output)
    ref = ko.y_w4a16(x, res).astype(np.float32).reshape(m, n // 32, 2, 16)
    ref_act = (ref[:, :, 0] / (1 + np.exp(-ref[:, :, 0])) * ref[:, :, 1]).reshape(m, n // 2)
    err = np.abs(got.float().cpu().numpy() - ref_act)
    assert (err <= 3e-2 * np.abs(ref_act) + 3e-2 * np.sqrt((ref_act ** 2).mean())).all()


def test_decoder_with_the_fused_gated_epilogue_generates_the_same_tokens():
    import kairos_b200 as kb
    from kairos_b200 import llm, runtime
    cfg = llm.DecoderConfig('tiny', 2, 512, 8, 2, 64, 1024, 1000, 1e-5, 10000.0, True)
    ctx = runtime.Context('cuda', cache_bytes=None)
    kb.DynamicLinear.context = ctx
    try:
        model = llm.Decoder(cfg, 'cuda', fuse_linears=True, glue='cuda')
        assert model.blocked_gate_up
        prof = kb.Profiler(model.linear_shapes())
        prof.load_table({s: [(8, 'w4a16_gemv'), (16, 'w4a16_gemm'), (30720, 'w8a8')] for s in model.linear_shapes()})
        kb.DynamicLinear.prof = prof
        tokens = torch.randint(0, cfg.vocab, (3, 40), device='cuda', generator=torch.Generator('cuda').manual_seed(1))
        outs = {}
        for fused in (True, False):
            model.fuse_gate_silu = fused
            model.release_graphs()
            model.allocate(3, 64)
            outs[fused] = model.generate(tokens, 8, use_graph=True).cpu()
        assert torch.equal(outs[True], outs[False])
    finally:
        kb.DynamicLinear.context = None
        kb.DynamicLinear.prof = None
