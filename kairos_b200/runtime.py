"""Per-device contexts (conversion cache + workspaces) and small torch<->C-ABI helpers."""
from __future__ import annotations

import ctypes
import os

import torch

from ._lib import KairosError, SIZE_MAX, check, lib

DEFAULT_CACHE_BYTES = int(os.environ.get('KAIROS_CACHE_BYTES', str(1 << 30)))


class Context:
    """Owns one kairos_ctx: the bounded LRU cache of converted weights, the activation
    workspace and the split-K scratch of one device."""

    def __init__(self, device, cache_bytes=DEFAULT_CACHE_BYTES):
        self.device = torch.device(device)
        self.cache_bytes = SIZE_MAX if cache_bytes is None else int(cache_bytes)
        with torch.cuda.device(self.device):
            self.handle = lib.kairos_ctx_create(self.cache_bytes)
        if not self.handle:
            raise KairosError('kairos_ctx_create failed')

    def reserve(self, max_m, max_n, max_k):
        with torch.cuda.device(self.device):
            check(lib.kairos_ctx_reserve(self.handle, max_m, max_n, max_k), 'kairos_ctx_reserve')

    def stats(self):
        v = [ctypes.c_uint64() for _ in range(4)]
        check(lib.kairos_ctx_stats(self.handle, *[ctypes.byref(x) for x in v]), 'kairos_ctx_stats')
        return dict(zip(('hits', 'misses', 'evictions', 'bytes_in_use'), (x.value for x in v)))

    def clear_cache(self):
        lib.kairos_ctx_clear_cache(self.handle)

    def close(self):
        if getattr(self, 'handle', None):
            lib.kairos_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_default_ctx = {}


def default_context(device):
    """The shared context of `device` (created on first use with DEFAULT_CACHE_BYTES)."""
    device = torch.device(device)
    if device.type != 'cuda':
        raise KairosError('the switched linear runs on CUDA devices only; there is no CPU path')
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _default_ctx:
        _default_ctx[idx] = Context(torch.device('cuda', idx))
    return _default_ctx[idx]


def set_default_cache_bytes(device, cache_bytes):
    """Replace the shared context of `device` by one with another cache bound
    (0 = convert on every call; None = unbounded)."""
    device = torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    _default_ctx[idx] = Context(torch.device('cuda', idx), cache_bytes)
    return _default_ctx[idx]


def stream_ptr(device=None):
    return torch.cuda.current_stream(device).cuda_stream


def device_status(clear=True):
    """KAIROS_OK (0) or KAIROS_ERR_DEVICE after the caller synchronised."""
    return lib.kairos_device_status(1 if clear else 0)


ARITHMETIC = {'torch': 0, 'reference_cuda': 1}


def set_arithmetic(rule):
    """Select the arithmetic of activation quantization and the two weight conversions, process-wide:
    'torch' (default; the reference's torch functions: IEEE division, product and sum rounded separately)
    or 'reference_cuda' (the reference's CUDA kernels as its build compiles them: approximate division, one
    fused multiply-add; bit-identical to its extension on the same GPU).  Returns the previous rule's name."""
    prev = lib.kairos_set_arithmetic(ARITHMETIC[rule])
    check(prev, 'kairos_set_arithmetic')
    return {v: k for k, v in ARITHMETIC.items()}[prev]


def get_arithmetic():
    return {v: k for k, v in ARITHMETIC.items()}[lib.kairos_get_arithmetic()]


class arithmetic:
    """``with runtime.arithmetic('reference_cuda'): ...`` -- the rule inside the block, restored after it."""

    def __init__(self, rule):
        self.rule = rule

    def __enter__(self):
        self.prev = set_arithmetic(self.rule)
        return self

    def __exit__(self, *exc):
        set_arithmetic(self.prev)
        return False


_gemm_ws = {}


def gemm_workspace(device, m, n, k):
    """A zero-initialised split-K workspace for the primitive GEMM entry points."""
    need = lib.kairos_gemm_workspace_bytes(m, n, k)
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    ws = _gemm_ws.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(int(need * 1.25) + 256, dtype=torch.uint8, device=device)
        _gemm_ws[key] = ws
    return ws
