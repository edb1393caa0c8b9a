"""CPU-side checks: the shared library loads and exports exactly what include/kairos_b200.h
declares, argument validation answers with status codes before touching a device, the native
LUT gives the reference's known answers, and the torch weight preparation reproduces the
reference's resident tensors bit for bit."""
import glob
import json
import os
import re

import numpy as np
import pytest
import torch

import kairos_b200
from kairos_b200 import _lib
from kairos_b200.awq_format import pack_int_awq, unpack_int_awq
from kairos_b200.dynamic_linear import COMP_TYPE_NAME, DynamicLinear
from kairos_b200.perf_profiler import LUT, Profiler, collapse_segments
from kairos_b200.quant_model import quantize_model

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, 'tests', 'golden')
SMALL = sorted(glob.glob(os.path.join(GOLDEN, 'small_*.npz')))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, 'include', 'kairos_b200.h')).read()
    header = re.sub(r'/\*.*?\*/', '', header, flags=re.S)
    declared = set(re.findall(r'\b(kairos_[a-z0-9_]+)\s*\(', header))
    assert len(declared) >= 25
    for name in sorted(declared):
        assert hasattr(_lib.lib, name), f'{name} declared in the header but not exported'
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert _lib.lib.kairos_abi_version() == 1


def test_argument_validation_needs_no_device():
    L = _lib.lib
    assert L.kairos_act_quant_i8(16, 16, 16, 4, 100, None) == -1          # K % 16
    assert L.kairos_act_quant_i8(None, None, None, 0, 128, None) == 0     # M == 0 is a no-op
    assert L.kairos_act_quant_i8(None, 16, 16, 1, 128, None) == -2        # null pointer
    assert L.kairos_w4_to_w8(16, 16, 16, 16, 6, 128, None) == -1          # N % 4
    assert L.kairos_w4_to_f16(16, 16, 16, 16, 8, 192, None) == -1         # K % 128
    assert L.kairos_w4a16_gemv(16, 16, 16, 16, None, 16, 33, 8, 128, None) == -1   # M > 32
    assert L.kairos_w4a16_gemm(16, 16, 16, 16, None, 16, 4, 256, 4096, None, 0, None) == -4   # split-K, no workspace
    assert L.kairos_w4a16_gemm(16, 16, 16, 16, None, 16, 4, 12, 128, None, 0, None) == -1     # N % 8
    assert L.kairos_w8a8_gemm(16, 16, 16, 16, None, 16, None, 4, 8, 100, 16, 1 << 20, None) == -1
    assert L.kairos_awq_to_qserve(16, 16, 48, 64, None) == -1             # N % 32
    assert L.kairos_switched_linear(None, 16, 16, 1, 0, None) == -8
    assert b'kernel id' in L.kairos_status_str(-6)
    assert L.kairos_gemm_workspace_bytes(16, 4096, 4096) == 4 * 32 * 32 * 128 * 4     # 4 K runs x 32 tiles of 32 tokens
    assert L.kairos_gemm_workspace_bytes(8192, 4096, 4096) == 0


def test_gemm_plan_invariants_and_the_measured_choices():
    """The one-CTA GEMM's plan (token tile, K runs) for the TMA-fed modes: structural invariants over a grid of
    shapes, and the choices the cost model was fitted to make (graph-timed on B200, 148 SMs assumed without a GPU)."""
    import ctypes
    L = _lib.lib

    def plan(m, n, k, int8=1):
        bt, runs, tiles = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        assert L.kairos_gemm_plan_query(m, n, k, int8, ctypes.byref(bt), ctypes.byref(runs), ctypes.byref(tiles)) == 0
        return bt.value, runs.value, tiles.value

    for int8 in (0, 1):
        for k, n in [(4096, 4096), (4096, 1024), (4096, 14336), (14336, 4096), (512, 256), (8192, 28672)]:
            for m in (1, 16, 17, 64, 65, 100, 128, 192, 256, 300, 512, 777, 1024, 2048, 8192):
                bt, runs, tiles = plan(m, n, k, int8)
                assert bt in (16, 32, 64, 128, 256) and runs >= 1
                assert tiles == -(-n // 128) * -(-m // bt)
                assert bt >= min(m, 16) and (m <= 64 or bt >= 64)
                assert runs == 1 or tiles * runs <= 148           # a split never makes more units than SMs
                need = L.kairos_gemm_workspace_bytes(m, n, k)
                assert need >= (tiles * runs * bt * 128 * 4 if runs > 1 else 0)
    assert L.kairos_gemm_plan_query(0, 128, 128, 1, None, None, None) == -8
    # measured winners (W8A8): unsplit 128- / 64-token tiles where 256-token tiles leave SMs idle ...
    assert plan(512, 4096, 4096)[:2] == (128, 1)
    assert plan(256, 4096, 4096)[:2] == (64, 1)
    assert plan(2048, 1024, 4096)[:2] == (128, 1)
    assert plan(1024, 1024, 4096)[:2] == (64, 1)
    # ... 256-token tiles once they fill the GPU ...
    assert plan(1024, 4096, 4096)[:2] == (256, 1)
    assert plan(256, 14336, 4096)[:2] == (256, 1)
    # ... and a K split only for very few tiles or long K
    assert plan(128, 1024, 4096)[1] > 1
    assert plan(128, 4096, 14336)[:2] == (128, 4)
    assert plan(128, 4096, 4096)[1] == 1


def test_native_lut_known_answers():
    cases = json.load(open(os.path.join(GOLDEN, 'lut_known_answers.json')))
    for c in cases:
        t = LUT()
        for r, cid in c['records']:
            t.record(r, cid)
        assert len(t) == len(c['records'])
        assert [t.get(q) for q in c['queries']] == c['answers'], (c['profile'], c['table'])
    with pytest.raises(kairos_b200.KairosError):
        LUT().get(5)


def test_profiler_wire_format_round_trip(tmp_path):
    shapes = [(1024, 4096), (4096, 4096)]
    seg = [[[16, 'w4a16_gemv', 0.0], [64, 'w4a16_gemm', 0.0], [30720, 'fp16', 28.1]],
           [[8, 'w4a16_gemv', 0.0], [256, 'w4a16_marlin', 0.0], [30720, 'w8a8', 30.2]]]
    d = str(tmp_path) + '/'
    with open(d + 'seg_perf_list.pt', 'w') as f:
        json.dump(seg, f)
    p = Profiler(shapes)
    p.load(d)
    assert p.get_comp_type((1024, 4096), 16) == COMP_TYPE_NAME['w4a16_gemv']
    assert p.get_comp_type((1024, 4096), 17) == COMP_TYPE_NAME['w4a16_gemm']
    assert p.get_comp_type((1024, 4096), 65) == COMP_TYPE_NAME['fp16']
    assert p.get_comp_type((4096, 4096), 100) == COMP_TYPE_NAME['w4a16_gemm']   # marlin -> in-library W4A16 GEMM
    assert p.get_comp_type((4096, 4096), 99999) == COMP_TYPE_NAME['w8a8']
    p.save(d + 'again/')
    assert json.load(open(d + 'again/seg_perf_list.pt')) == seg
    perf = [(1, 'a', 0), (2, 'a', 0), (4, 'b', 1), (8, 'b', 2), (16, 'a', 3)]
    assert collapse_segments(perf) == [[2, 'a', 0], [8, 'b', 2], [16, 'a', 3]]


@pytest.mark.parametrize('path', SMALL, ids=[os.path.basename(p)[6:-4] for p in SMALL])
def test_from_module_matches_reference(path):
    g = dict(np.load(path))
    n, k = g['W'].shape
    lin = torch.nn.Linear(k, n, bias='bias' in g, dtype=torch.float16)
    lin.weight.data = torch.from_numpy(g['W'].copy())
    if 'bias' in g:
        lin.bias.data = torch.from_numpy(g['bias'].copy())
    q = DynamicLinear.from_module(lin, 'cpu')
    for key in ('qweight', 'scales', 'scaled_zeros', 'scales_to8', 'scaled_zeros_to8', 'scales_1'):
        got = getattr(q, key).numpy()
        ref = g[key]
        if ref.dtype == np.float16:
            got, ref = got.view(np.uint16), ref.view(np.uint16)
        assert np.array_equal(got, ref), key
    assert np.array_equal(unpack_int_awq(q.qweight).numpy().astype(np.uint8), g['Q4'])
    assert torch.equal(pack_int_awq(torch.from_numpy(g['Q4'].astype(np.int32))), q.qweight)
    assert set(q.state_dict()) >= {'qweight', 'scales', 'scaled_zeros', 'scales_to8', 'scaled_zeros_to8', 'scales_1'}
    assert q.shape == (n, k) and q.pre_m == 0 and q.group_size == 128


def test_forward_without_cuda_fails_loudly():
    lin = torch.nn.Linear(128, 8, bias=False, dtype=torch.float16)
    q = DynamicLinear.from_module(lin, 'cpu')
    with pytest.raises(kairos_b200.KairosError):
        q._forward(torch.zeros(1, 128, dtype=torch.float16), 1, 0)


class _TinyBlock(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.self_attn = torch.nn.Module()
        self.self_attn.q_proj = torch.nn.Linear(128, 128, bias=True, dtype=torch.float16)
        self.mlp = torch.nn.Module()
        self.mlp.up_proj = torch.nn.Linear(128, 256, bias=False, dtype=torch.float16)


class _TinyModel(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.model = torch.nn.Module()
        self.model.layers = torch.nn.ModuleList([_TinyBlock(), _TinyBlock()])
        self.lm_head = torch.nn.Linear(128, 64, bias=False, dtype=torch.float16)


def test_quantize_model_swaps_decoder_linears():
    m = _TinyModel()
    cfg = quantize_model(m, quant_strategy='DynamicLinear')
    assert cfg == [{'self_attn.q_proj': 'DynamicLinear', 'mlp.up_proj': 'DynamicLinear'}] * 2
    assert isinstance(m.model.layers[1].mlp.up_proj, DynamicLinear)
    assert isinstance(m.lm_head, torch.nn.Linear)
    assert m.model.layers[0].self_attn.q_proj.bias is not None
    # checkpoint flow: init-only skeleton + state_dict restores the resident tensors
    m2 = _TinyModel()
    quantize_model(m2, init_only=True, _quant_config=cfg)
    m2.load_state_dict(m.state_dict())
    assert torch.equal(m2.model.layers[0].mlp.up_proj.qweight, m.model.layers[0].mlp.up_proj.qweight)
    with pytest.raises(ValueError):
        quantize_model(_TinyModel(), quant_strategy='W4A8Linear')


def test_first_argmax_is_torch_argmax():
    """The decoder's two-level argmax returns torch's answer (first maximum), ties and odd vocabularies included."""
    from kairos_b200.llm import first_argmax
    g = torch.Generator().manual_seed(0)
    for rows, vocab in [(2, 128256), (3, 152064), (1, 1000), (4, 1024), (5, 2048)]:
        x = torch.randn(rows, vocab, generator=g).half()
        assert torch.equal(first_argmax(x), x.argmax(-1, keepdim=True))
        top = x.max(dim=-1).values
        for r in range(rows):
            x[r, torch.randint(0, vocab, (5,), generator=g)] = top[r]
        assert torch.equal(first_argmax(x), x.argmax(-1, keepdim=True))
    z = torch.zeros(2, 128256).half()
    assert torch.equal(first_argmax(z), z.argmax(-1, keepdim=True))
