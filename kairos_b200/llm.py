"""Random-init decoder harness around the switched linear: the measurement vehicle for TTFT / TPOT.

The reference measures end to end with a HuggingFace Llama/Qwen checkpoint and ``generate()``
(utils/perf_eval.py:236-275, kairos/main_ablation.py:108-140).  Checkpoints are not available here,
so this module builds the same decoder geometry with random weights (N(0, 0.02)), swaps every linear of
the decoder layers through ``quantize_model`` exactly as the reference does (lm_head stays fp16), and
runs prefill + greedy decode with a static KV cache.  Everything that is not a linear (RMSNorm, RoPE,
attention, SiLU) is stock torch, as it is stock HuggingFace code in the reference.  The decode step is
captured into a CUDA graph, so the per-token host cost is one graph launch.
"""
from __future__ import annotations

import os

import math
import time
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import ops
from .dynamic_linear import COMP_TYPE_NAME, DynamicLinear
from .perf_profiler import Profiler
from .quant_model import quantize_model


@dataclass
class DecoderConfig:
    name: str
    layers: int
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    inter: int
    vocab: int
    rms_eps: float = 1e-5
    rope_theta: float = 500000.0
    qkv_bias: bool = False

    def shard(self, world):
        """This geometry as ONE rank of `world` tensor-parallel ranks sees it (Megatron split): the attention
        heads, the KV heads and the MLP's inner channels are divided, the hidden size is not.  q|k|v and
        gate|up become column-parallel (N / world), o and down row-parallel (K / world, one all-reduce each):
        e.g. Llama-3-70B on 8 ranks runs (1280, 8192), (8192, 1024), (7168, 8192), (8192, 3584) per rank
        with q|k|v and gate|up stacked."""
        if world == 1:
            return self
        if self.n_heads % world or self.n_kv_heads % world or self.inter % (128 * world):
            raise ValueError(f'{self.name} does not split over {world} ranks (heads {self.n_heads}/{self.n_kv_heads}, '
                             f'inner size {self.inter}: every shard must keep whole heads and quantization groups)')
        return DecoderConfig(f'{self.name}-tp{world}', self.layers, self.hidden, self.n_heads // world,
                             self.n_kv_heads // world, self.head_dim, self.inter // world, self.vocab, self.rms_eps,
                             self.rope_theta, self.qkv_bias)

    def linear_shapes(self):
        """Distinct (N, K) of the decoder linears, the key set of the profiler's LUT."""
        q = self.n_heads * self.head_dim
        kv = self.n_kv_heads * self.head_dim
        shapes = [(q, self.hidden), (kv, self.hidden), (self.hidden, q), (self.inter, self.hidden),
                  (self.hidden, self.inter)]
        return list(dict.fromkeys(shapes))


LLAMA3_8B = DecoderConfig('llama3-8b', 32, 4096, 32, 8, 128, 14336, 128256, 1e-5, 500000.0, False)
QWEN2_7B = DecoderConfig('qwen2-7b', 28, 3584, 28, 4, 128, 18944, 152064, 1e-6, 1e6, True)
LLAMA3_70B = DecoderConfig('llama3-70b', 80, 8192, 64, 8, 128, 28672, 128256, 1e-5, 500000.0, False)
PRESETS = {c.name: c for c in (LLAMA3_8B, QWEN2_7B, LLAMA3_70B)}


class RMSNorm(torch.nn.Module):
    def __init__(self, dim, eps, device):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.ones(dim, dtype=torch.float16, device=device), requires_grad=False)
        self.eps = eps

    def forward(self, x):
        v = x.float()
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)
        return (v * self.weight.float()).to(torch.float16)


class Attention(torch.nn.Module):
    def __init__(self, cfg, device, fuse):
        super().__init__()
        h, q, kv = cfg.hidden, cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
        mk = dict(dtype=torch.float16, device=device)
        if fuse:
            # q, k and v read the same activation: one switched linear with the three weights stacked
            # along N.  Quantization is per output row, so the result equals the three separate layers.
            self.qkv_proj = torch.nn.Linear(h, q + 2 * kv, bias=cfg.qkv_bias, **mk)
        else:
            self.q_proj = torch.nn.Linear(h, q, bias=cfg.qkv_bias, **mk)
            self.k_proj = torch.nn.Linear(h, kv, bias=cfg.qkv_bias, **mk)
            self.v_proj = torch.nn.Linear(h, kv, bias=cfg.qkv_bias, **mk)
        self.o_proj = torch.nn.Linear(q, h, bias=False, **mk)


class MLP(torch.nn.Module):
    def __init__(self, cfg, device, fuse):
        super().__init__()
        mk = dict(dtype=torch.float16, device=device)
        if fuse:
            self.gate_up_proj = torch.nn.Linear(cfg.hidden, 2 * cfg.inter, bias=False, **mk)
        else:
            self.gate_proj = torch.nn.Linear(cfg.hidden, cfg.inter, bias=False, **mk)
            self.up_proj = torch.nn.Linear(cfg.hidden, cfg.inter, bias=False, **mk)
        self.down_proj = torch.nn.Linear(cfg.inter, cfg.hidden, bias=False, **mk)


class DecoderLayer(torch.nn.Module):
    def __init__(self, cfg, device, fuse):
        super().__init__()
        self.self_attn = Attention(cfg, device, fuse)
        self.mlp = MLP(cfg, device, fuse)
        self.input_layernorm = RMSNorm(cfg.hidden, cfg.rms_eps, device)
        self.post_attention_layernorm = RMSNorm(cfg.hidden, cfg.rms_eps, device)


class _Inner(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.layers = torch.nn.ModuleList()


def _rope_tables(cfg, max_len, device):
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, device=device, dtype=torch.float32) / cfg.head_dim))
    ang = torch.arange(max_len, device=device, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cos(ang).to(torch.float16).contiguous(), torch.sin(ang).to(torch.float16).contiguous()


def _apply_rope(x, cos, sin):
    # x [B, S, H, D]; cos/sin [S, D/2] (rotate-half convention)
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1)


def first_argmax(logits):
    """``logits.argmax(dim=-1, keepdim=True)`` (index of the FIRST maximum) for [rows, vocab] with few rows.
    torch reduces each row in one CTA, which takes ~40 us for two rows of 128 k entries; here the row is cut into
    chunks of 256 (a [rows, vocab / 256, 256] view), the maxima of the chunks and then of their maxima are taken,
    both reductions spread over many CTAs, and ties resolve to the first index at both levels."""
    rows, vocab = logits.shape
    chunk = 256
    if vocab % chunk != 0 or vocab < 4 * chunk:
        return logits.argmax(dim=-1, keepdim=True)
    v, i = logits.view(rows, vocab // chunk, chunk).max(dim=-1)       # per chunk: maximum, first index of it
    _, j = v.max(dim=-1, keepdim=True)                                # first chunk that holds the row's maximum
    return j * chunk + i.gather(1, j)


class Decoder(torch.nn.Module):
    """``model.model.layers`` holds the decoder layers (the attribute path ``quantize_model`` walks).

    fuse_linears: stack q|k|v and gate|up into one switched linear each (4 instead of 7 per layer).
    glue: 'cuda' runs RMSNorm, rotary + KV write and SiLU*up as one library kernel each; 'torch' runs
    them as stock torch ops (what a HuggingFace model does)."""

    def __init__(self, cfg: DecoderConfig, device='cuda', seed=0, quant_strategy='DynamicLinear', layers=None,
                 fuse_linears=True, glue='cuda', tp_rank=0, tp_world=1, tp_group=None, peer_allreduce_tokens=64):
        super().__init__()
        # Tensor parallelism (new; the reference is single-GPU): every rank builds the decoder of the SHARDED
        # geometry -- its own heads and inner channels, quantized locally, with its own LUT -- and the outputs
        # of the two row-parallel linears of a layer (o_proj, down_proj) are summed over the group with one
        # all-reduce each.  Embedding, norms and lm_head are replicated (same seed on every rank).
        self.full_cfg = cfg
        self.tp_rank, self.tp_world, self.tp_group = tp_rank, tp_world, tp_group
        cfg = cfg.shard(tp_world)
        self.cfg = cfg
        self.device = torch.device(device)
        self.fuse, self.glue = fuse_linears, glue
        self.fuse_quant = True       # let RMSNorm / SiLU*up emit int8 when the next linear runs W8A8
        # gate and up rows of the stacked weight in blocks of 16 (SiLU * up inside the decode kernel's epilogue)
        self.blocked_gate_up = os.environ.get('KAIROS_BLOCKED_GATE_UP', '1') != '0' and cfg.inter % 16 == 0
        self.fuse_gate_silu = True   # False: the same layout, SiLU * up as a kernel of its own (for comparison)
        n_layers = cfg.layers if layers is None else layers
        gen = torch.Generator(device=self.device).manual_seed(seed)
        self.model = _Inner()
        self.embed = (torch.randn((cfg.vocab, cfg.hidden), generator=gen, device=self.device, dtype=torch.float32)
                      * 0.02).to(torch.float16)
        self.lm_head = (torch.randn((cfg.vocab, cfg.hidden), generator=gen, device=self.device, dtype=torch.float32)
                        * 0.02).to(torch.float16)
        self.norm = RMSNorm(cfg.hidden, cfg.rms_eps, self.device)
        if tp_world > 1:
            gen = torch.Generator(device=self.device).manual_seed(seed + 1000 * (tp_rank + 1))   # the rank's own shards
        # build and quantize layer by layer so that at most one fp16 layer is alive
        for _ in range(n_layers):
            layer = DecoderLayer(cfg, self.device, fuse_linears)
            for mod in layer.modules():
                if isinstance(mod, torch.nn.Linear):
                    mod.weight.data = (torch.randn(mod.weight.shape, generator=gen, device=self.device,
                                                   dtype=torch.float32) * 0.02).to(torch.float16)
                    if mod.bias is not None:
                        mod.bias.data = (torch.randn(mod.bias.shape, generator=gen, device=self.device,
                                                     dtype=torch.float32) * 0.02).to(torch.float16)
            holder = _Inner()
            holder.layers.append(layer)
            wrap = torch.nn.Module()
            wrap.model = holder
            quantize_model(wrap, quant_strategy=quant_strategy, device=self.device)
            self.model.layers.append(layer)
        self.kv = None
        self.graph = None
        self._prefill_graphs = {}
        # Row-parallel outputs of up to `peer_allreduce_tokens` tokens are summed by the library's own kernel
        # over NVLink peer memory (latency-bound sizes: decode steps); larger ones by NCCL.  0 = NCCL always.
        self.peer_ar = None
        self.fuse_peer_sum = os.environ.get('KAIROS_FUSE_PEER_SUM', '1') != '0'   # fold that sum into the next RMSNorm
        if tp_world > 1 and peer_allreduce_tokens > 0 and os.environ.get('KAIROS_PEER_ALLREDUCE', '1') != '0':
            from .tp import PeerAllReduce
            self.peer_ar = PeerAllReduce(tp_group, self.device, peer_allreduce_tokens * cfg.hidden)

    def linear_shapes(self):
        """Distinct (N, K) of this model's switched linears (the LUT's key set)."""
        shapes = []
        for mod in self.model.layers[0].modules():
            if isinstance(mod, DynamicLinear) and mod.shape not in shapes:
                shapes.append(mod.shape)
        return shapes

    # ---- state ------------------------------------------------------------------------------
    def allocate(self, batch, max_len, max_tokens=None):
        """Static state for `batch` sequences of up to `max_len` positions.  `max_tokens` (default
        batch * max_len) sizes the library's activation / split-K workspaces once, so that no later call
        reallocates a buffer a captured CUDA graph still points to."""
        cfg = self.cfg
        from .runtime import default_context
        ctx = DynamicLinear.context or default_context(self.device)
        shapes = self.linear_shapes()
        ctx.reserve(max_tokens or batch * max_len, max(s[0] for s in shapes), max(s[1] for s in shapes))
        shape = (len(self.model.layers), 2, batch, cfg.n_kv_heads, max_len, cfg.head_dim)
        self.kv = torch.zeros(shape, dtype=torch.float16, device=self.device)
        self.max_len = max_len
        self.cos, self.sin = _rope_tables(cfg, max_len, self.device)
        # decode-step buffers (static addresses for the CUDA graph)
        self.tok = torch.zeros((batch, 1), dtype=torch.long, device=self.device)
        self.pos = torch.zeros((1,), dtype=torch.long, device=self.device)
        self.mask = torch.full((1, 1, 1, max_len), float('-inf'), dtype=torch.float16, device=self.device)
        self.next_tok = torch.zeros((batch, 1), dtype=torch.long, device=self.device)
        self.graph = None
        self._prefill_graphs = {}

    def release_graphs(self):
        """Drop the captured CUDA graphs.  With tensor parallelism they hold the captured collectives, and a
        process group must not be destroyed while such a graph is alive (its teardown then never returns):
        call this, synchronize, and only then ``destroy_process_group``."""
        import gc
        self.graph = None
        self._prefill_graphs = {}
        gc.collect()
        torch.cuda.synchronize(self.device)

    # ---- layers -----------------------------------------------------------------------------
    def _norm(self, mod, x, delta=None):
        """RMSNorm of the residual stream; a pending `delta` (output of the block before) is added to x in
        place by the same pass."""
        if self.glue == 'cuda':
            return ops.rms_norm(x, mod.weight, mod.eps, residual_delta=delta)
        if delta is not None:
            x.add_(self._as_tensor(delta))
        return mod(x)

    def _reduce(self, y):
        """Sum of a row-parallel linear's partial outputs over the tensor-parallel group (fp16, in place;
        NCCL over NVLink, on the compute stream, so it is captured into the step's CUDA graph)."""
        if self.tp_world > 1:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.tp_group)
        return y

    def _row_parallel(self, lin, x, q8=None):
        """A row-parallel linear (o_proj, down_proj) and the sum of its partial outputs over the group.  Small
        outputs are written straight into the peer-addressable buffer and summed by the library's peer-memory
        kernel; `q8` = (int8 activations, scales) when the operator before already quantized them."""
        lead = (q8[0] if q8 is not None else x).shape[:-1]
        m, n = 1, lin.out_features
        for d in lead:
            m *= d
        ar = self.peer_ar
        if ar is not None and ar.fits(m * n):
            part = ar.partial(m, n)
            if q8 is not None:
                lin.forward_q8(q8[0], q8[1], out=part)
            else:
                lin(x if x.dim() == 3 else x.reshape(1, m, -1), out=part)
            if self.glue == 'cuda' and self.fuse_peer_sum and m <= 128:
                return ar.defer(m, n, lead)          # summed by the RMSNorm that consumes it
            return ar.reduce(m, n).view(*lead, n)
        y = lin.forward_q8(*q8) if q8 is not None else lin(x)
        return self._reduce(y)

    @staticmethod
    def _as_tensor(delta):
        return delta.materialize() if hasattr(delta, 'materialize') else delta

    def _norm_then_linear(self, mod, x, delta, lin):
        """lin(norm(x + delta)); when the LUT sends this M to W8A8 the norm emits the int8 activations that
        kernel consumes, with no fp16 round trip."""
        m = x.numel() // x.shape[-1]
        if self.glue == 'cuda' and self.fuse_quant and lin.wants_int8(m):
            xq, sx, _ = ops.rms_norm_quant(x, mod.weight, mod.eps, residual_delta=delta)
            return lin.forward_q8(xq, sx)
        return lin(self._norm(mod, x, delta))

    def _layer(self, li, layer, x, delta, pos0, decode):
        """One decoder layer on the residual stream x (updated in place).  `delta` is the output of the
        previous layer's MLP, not yet added; returns this layer's MLP output in the same way, so that each
        residual addition is carried by the norm that follows it."""
        cfg = self.cfg
        b, s, _ = x.shape
        nh, nkv, d = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        a = layer.self_attn
        if self.fuse:
            qkv = self._norm_then_linear(layer.input_layernorm, x, delta, a.qkv_proj)   # [B, S, (H + 2 Hkv) D]
        else:
            h = self._norm(layer.input_layernorm, x, delta)
            qkv = torch.cat((a.q_proj(h), a.k_proj(h), a.v_proj(h)), dim=-1)
        kc, vc = self.kv[li, 0], self.kv[li, 1]
        if self.glue == 'cuda':
            q = torch.empty((b, nh, s, d), dtype=torch.float16, device=x.device)
            ops.rope_kv(qkv, self.cos, self.sin, q, kc, vc, b, s, nh, nkv, d,
                        pos_dev=self.pos if decode else None, pos0=pos0)
        else:
            qh, kh, vh = qkv.split((nh * d, nkv * d, nkv * d), dim=-1)
            if decode:
                cos, sin = self.cos.index_select(0, self.pos), self.sin.index_select(0, self.pos)
            else:
                cos, sin = self.cos[pos0:pos0 + s], self.sin[pos0:pos0 + s]
            q = _apply_rope(qh.reshape(b, s, nh, d), cos, sin).transpose(1, 2)
            k = _apply_rope(kh.reshape(b, s, nkv, d), cos, sin).transpose(1, 2)
            v = vh.reshape(b, s, nkv, d).transpose(1, 2)
            if decode:
                idx = self.pos.view(1, 1, 1, 1).expand(b, nkv, 1, d)
                kc.scatter_(2, idx, k)
                vc.scatter_(2, idx, v)
            else:
                kc[:, :, pos0:pos0 + s] = k
                vc[:, :, pos0:pos0 + s] = v
        if decode:
            o = F.scaled_dot_product_attention(q, kc, vc, attn_mask=self.mask, enable_gqa=True)
        else:
            o = F.scaled_dot_product_attention(q, kc[:, :, pos0:pos0 + s], vc[:, :, pos0:pos0 + s], is_causal=True,
                                               enable_gqa=True)
        o = o.transpose(1, 2).reshape(b, s, nh * d)
        attn_out = self._row_parallel(a.o_proj, o)
        m = layer.mlp
        if not self.fuse:
            h = self._norm(layer.post_attention_layernorm, x, attn_out)
            return self._row_parallel(m.down_proj, F.silu(m.gate_proj(h)) * m.up_proj(h))
        # The rows of the stacked gate|up weight are read in the BLOCKED order (16 gate rows, their 16 up rows,
        # ...; for random weights that is only a naming of rows, a checkpoint loader would interleave them),
        # so that the decode kernel can apply SiLU(gate) * up in its epilogue.
        blocked = self.blocked_gate_up
        tokens = b * s
        down_q8 = self.glue == 'cuda' and self.fuse_quant and m.down_proj.wants_int8(tokens)
        gup = m.gate_up_proj
        if (blocked and self.glue == 'cuda' and self.fuse_gate_silu and not down_q8 and tokens <= 32
                and gup.out_features % 32 == 0 and gup.bias is None
                and not gup.wants_int8(tokens) and gup.comp_type == COMP_TYPE_NAME['w4a16_gemv']):
            # (wants_int8 refreshed gup.comp_type for this token count)
            h = self._norm(layer.post_attention_layernorm, x, attn_out)
            act = ops.decode_silu_forward(h, gup.qweight, gup.scales, gup.scaled_zeros, tokens, gup.out_features,
                                          gup.in_features).view(b, s, -1)
            return self._row_parallel(m.down_proj, act)
        gu = self._norm_then_linear(layer.post_attention_layernorm, x, attn_out, gup)
        if down_q8:
            aq, sa, _ = ops.silu_mul_quant(gu, blocked=blocked)
            return self._row_parallel(m.down_proj, None, (aq, sa))
        if self.glue == 'cuda':
            act = ops.silu_mul(gu, blocked=blocked)
        elif blocked:
            pairs = gu.view(*gu.shape[:-1], cfg.inter // 16, 2, 16)
            act = (F.silu(pairs[..., 0, :]) * pairs[..., 1, :]).reshape(*gu.shape[:-1], cfg.inter)
        else:
            act = F.silu(gu[..., :cfg.inter]) * gu[..., cfg.inter:]
        return self._row_parallel(m.down_proj, act)

    def _stack(self, x, decode):
        """All layers, then the final norm (which carries the last residual addition)."""
        delta = None
        for li, layer in enumerate(self.model.layers):
            delta = self._layer(li, layer, x, delta, 0, decode)
        return x, delta

    def _prefill_body(self, tokens):
        b, s = tokens.shape
        x, delta = self._stack(self.embed[tokens], False)
        delta = self._as_tensor(delta)
        last = self._norm(self.norm, x[:, -1:, :].contiguous(), None if delta is None else delta[:, -1:, :].contiguous())
        logits = last.reshape(b, -1) @ self.lm_head.t()
        self.mask.fill_(float('-inf'))
        self.mask[..., :s] = 0
        self.pos.fill_(s)
        return logits

    @torch.no_grad()
    def prefill(self, tokens, return_logits=False, use_graph=False):
        """tokens [B, S] -> next token ids [B, 1]; fills the KV cache for positions 0..S-1.

        use_graph: replay a CUDA graph captured for this (B, S) (the ~500 launches of a prefill are then off
        the host's critical path); the prompt is copied into the graph's static token buffer.  The graph is
        captured after two eager passes, so every converted weight it needs is in the conversion cache."""
        if not use_graph:
            logits = self._prefill_body(tokens)
        else:
            key = tuple(tokens.shape)
            entry = self._prefill_graphs.get(key)
            if entry is None:
                static_tokens = tokens.clone()
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    for _ in range(2):
                        self._prefill_body(static_tokens)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    static_logits = self._prefill_body(static_tokens)
                torch.cuda.synchronize()
                entry = self._prefill_graphs[key] = (graph, static_tokens, static_logits)
            graph, static_tokens, static_logits = entry
            static_tokens.copy_(tokens)
            graph.replay()
            logits = static_logits
        if return_logits:
            return logits
        return first_argmax(logits)

    def _decode_body(self):
        self.mask.index_fill_(3, self.pos, 0.0)
        x, delta = self._stack(self.embed[self.tok], True)
        self.logits = self._norm(self.norm, x, delta).reshape(x.shape[0], -1) @ self.lm_head.t()
        self.next_tok.copy_(first_argmax(self.logits))
        self.pos.add_(1)

    @torch.no_grad()
    def decode_step(self, use_graph=True):
        """One token for every sequence: reads self.tok, writes self.next_tok, advances self.pos."""
        if not use_graph:
            self._decode_body()
            return
        if self.graph is None:
            pos0 = self.pos.clone()
            mask0 = self.mask.clone()
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._decode_body()
            torch.cuda.synchronize()
            self.pos.copy_(pos0)
            self.mask.copy_(mask0)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side):
                self._decode_body()
            self.pos.copy_(pos0)
            self.mask.copy_(mask0)
            torch.cuda.synchronize()
        self.graph.replay()

    @torch.no_grad()
    def generate(self, tokens, max_new_tokens, use_graph=True):
        nxt = self.prefill(tokens, use_graph=use_graph)
        out = [nxt]
        for _ in range(max_new_tokens - 1):
            self.tok.copy_(nxt)
            self.decode_step(use_graph)
            nxt = self.next_tok.clone()
            out.append(nxt)
        return torch.cat(out, dim=1)


@torch.no_grad()
def measure_ttft_tpot(model, batch, prompt_len=1024, new_tokens=512, warmup=2, ttft_times=5, seed=0):
    """TTFT = mean wall time of prefill + first token over `ttft_times` runs; TPOT = (time of a full
    generation - TTFT) / (new_tokens - 1); throughput = batch * new_tokens / (TTFT + (new_tokens-1) * TPOT)
    (utils/perf_eval.py:236-275 and kairos/main_ablation.py:111-125 of the reference)."""
    dev = model.device
    gen = torch.Generator(device=dev).manual_seed(seed)
    tokens = torch.randint(0, model.cfg.vocab, (batch, prompt_len), generator=gen, device=dev)
    model.allocate(batch, prompt_len + new_tokens + 8)
    for _ in range(warmup):
        model.generate(tokens, 4)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(ttft_times):
        model.prefill(tokens, use_graph=True)
        torch.cuda.synchronize()
    ttft = (time.perf_counter() - t0) / ttft_times
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    out = model.generate(tokens, new_tokens)
    torch.cuda.synchronize()
    total = time.perf_counter() - t0
    tpot = (total - ttft) / (new_tokens - 1)
    return {'batch': batch, 'prompt_len': prompt_len, 'new_tokens': int(out.shape[1]), 'ttft_ms': 1e3 * ttft,
            'tpot_ms': 1e3 * tpot, 'tokens_per_s': batch * new_tokens / (ttft + (new_tokens - 1) * tpot)}


def build_lut(shapes, device='cuda', m_grid=None, cache='warm', n=20):
    """Profile the given (N, K) linear shapes on the device and install the LUT on DynamicLinear."""
    grid = m_grid or [1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192, 16384, 32768]
    prof = Profiler(list(shapes), m_grid=grid, n=n, warmup=3, cache=cache)
    prof.profiling(device=device)
    DynamicLinear.prof = prof
    return prof
