"""Seeded synthetic activations and weights with the benchmark's value distributions."""
from __future__ import annotations

import numpy as np


def make_case(m, k, n, seed=0, outlier_frac=0.01, outlier_gain=20.0, w_std=0.02):
    """X [m,k] ~ N(0,1) fp16 with ceil(outlier_frac*k) seeded input channels scaled by
    outlier_gain; W [n,k] ~ N(0, w_std) fp16.  Stands in for real activations/checkpoints
    (the reference benchmarks on torch.randn inputs, kairos/perf_profiler.py:116)."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((m, k), dtype=np.float32)
    cols = rng.permutation(k)[:int(np.ceil(outlier_frac * k))]
    x[:, cols] *= np.float32(outlier_gain)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(w_std)
    return x.astype(np.float16), w.astype(np.float16)
