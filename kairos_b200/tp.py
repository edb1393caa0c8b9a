"""Megatron-style tensor parallelism for the switched linear (one process per GPU).

Column-parallel layers (q/k/v, gate, up) hold W[N/t, K]: replicated input, sharded output, no
collective.  Row-parallel layers (o_proj, down_proj) hold W[N, K/t]: sharded input, partial
output, ONE all-reduce (sum, fp16) over the process group -- NCCL over NVLink on GPUs.  Each rank
quantizes its own fp16 shard, so a rank is a self-contained ``DynamicLinear`` with its own
per-channel / per-token scales and its own LUT entry for the sharded shape.

The reference is single-GPU (kairos/main.py:19-23); this module is the multi-GPU extension of
its ``DynamicLinear`` and keeps that class as the per-rank compute.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .dynamic_linear import DynamicLinear


# Megatron split of a decoder layer's linears: the projections that read the replicated hidden state
# are column-parallel, the two that produce it are row-parallel (one all-reduce each).
LAYER_KIND = {'q_proj': 'col', 'k_proj': 'col', 'v_proj': 'col', 'gate_proj': 'col', 'up_proj': 'col',
              'o_proj': 'row', 'down_proj': 'row'}


def layer_kind(name):
    """'col' or 'row' for a projection name such as 'self_attn.o_proj' or 'down_proj'."""
    return LAYER_KIND[name.split('.')[-1]]


def shard_bounds(size, rank, world, multiple):
    if size % (world * multiple) != 0:
        raise ValueError(f'dimension {size} does not split into {world} shards that are multiples of {multiple}')
    per = size // world
    return rank * per, (rank + 1) * per


def shard_weight(weight, kind, rank, world):
    """[N, K] fp16 -> this rank's shard: rows for 'col' (N % (4t) == 0), columns for 'row'
    (K % (128t) == 0, so every shard keeps whole quantization groups)."""
    n, k = weight.shape
    if kind == 'col':
        lo, hi = shard_bounds(n, rank, world, 4)
        return weight[lo:hi, :].contiguous()
    lo, hi = shard_bounds(k, rank, world, 128)
    return weight[:, lo:hi].contiguous()


class ColumnParallelLinear(torch.nn.Module):
    def __init__(self, linear, rank, world, group=None, gather_output=False):
        super().__init__()
        self.linear, self.rank, self.world, self.group = linear, rank, world, group
        self.gather_output = gather_output

    def forward(self, x):
        y = self.linear(x)
        if self.gather_output and self.world > 1:
            parts = [torch.empty_like(y) for _ in range(self.world)]
            dist.all_gather(parts, y.contiguous(), group=self.group)
            y = torch.cat(parts, dim=-1)
        return y

    def forward_host(self, x_host):
        """Host buffer in, host buffer out (benchmark end-to-end leg)."""
        dev = self.linear.qweight.device
        y = self.forward(x_host.to(dev, non_blocking=True).unsqueeze(0))
        return y.squeeze(0).to('cpu', non_blocking=True)


class RowParallelLinear(torch.nn.Module):
    def __init__(self, linear, rank, world, group=None, bias=None):
        super().__init__()
        self.linear, self.rank, self.world, self.group = linear, rank, world, group
        self.bias = bias            # applied once, after the reduction

    def forward(self, x_shard):
        y = self.linear(x_shard)
        if self.world > 1:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        if self.bias is not None:
            y = y + self.bias
        return y

    def forward_host(self, x_host):
        dev = self.linear.qweight.device
        y = self.forward(x_host.to(dev, non_blocking=True).unsqueeze(0))
        return y.squeeze(0).to('cpu', non_blocking=True)


@torch.no_grad()
def shard_linear(weight, kind, rank, world, device, bias=None, group=None, linear_cls=DynamicLinear):
    """Build this rank's parallel layer from the full fp16 weight [N, K]."""
    w = shard_weight(weight, kind, rank, world)
    n, k = w.shape
    lin = torch.nn.Linear(k, n, bias=False, dtype=torch.float16)
    lin.weight.data = w
    if kind == 'col':
        b = None
        if bias is not None:
            lo, hi = shard_bounds(bias.shape[0], rank, world, 4)
            lin = torch.nn.Linear(k, n, bias=True, dtype=torch.float16)
            lin.weight.data = w
            lin.bias.data = bias[lo:hi].clone().half()
        q = linear_cls.from_module(lin.to(device), device)
        return ColumnParallelLinear(q, rank, world, group)
    q = linear_cls.from_module(lin.to(device), device)
    return RowParallelLinear(q, rank, world, group, None if bias is None else bias.to(device).half())
