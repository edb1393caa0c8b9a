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

import time

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


class PeerLost(RuntimeError):
    """A rank of the tensor-parallel group did not reach the step the others are about to run."""

    def __init__(self, step, missing, waited_s):
        super().__init__(f'ranks {missing} did not reach step {step} within {waited_s:.1f} s')
        self.step, self.missing = step, missing


class StepGuard:
    """Host-side liveness check between steps of a tensor-parallel job.

    A rank that died, hung in its own code or left the job is found out ON THE HOST, before the surviving
    ranks enqueue the next collective: an all-reduce that a peer never joins cannot be recalled once it is
    on the GPU.  Every rank publishes the number of the step it is about to run in the job's key-value store
    (the store torch.distributed was initialised with: no GPU and no collective involved) and then waits,
    with a limit, until all peers have published at least that number.  On a timeout it raises `PeerLost`;
    the caller then stops launching work.  Ranks leave only between steps, with nothing in flight.

    The second line of defence is the process group's own timeout: create the group with a short
    ``timeout=`` (and, for NCCL, ``TORCH_NCCL_ASYNC_ERROR_HANDLING=1``, which makes torch's watchdog poll
    ``ncclCommGetAsyncError`` and abort the communicator), so that a collective a peer never joins ends with
    an error instead of blocking forever.  `collective_errors()` reports what that watchdog has seen.
    """

    def __init__(self, store, rank, world, timeout_s=5.0, prefix='kairos/step', poll_s=0.01):
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s, self.prefix, self.poll_s = timeout_s, prefix, poll_s

    def _key(self, r):
        return f'{self.prefix}/{r}'

    def arrive(self, step):
        self.store.set(self._key(self.rank), str(int(step)))

    def reached(self, r, step):
        key = self._key(r)
        if not self.store.check([key]):
            return False
        return int(self.store.get(key)) >= step

    def wait_all(self, step):
        """Publish `step` and return once every peer has; raise PeerLost after `timeout_s`."""
        self.arrive(step)
        t0 = time.monotonic()
        pending = [r for r in range(self.world) if r != self.rank]
        while pending:
            pending = [r for r in pending if not self.reached(r, step)]
            if not pending:
                break
            waited = time.monotonic() - t0
            if waited > self.timeout_s:
                raise PeerLost(step, pending, waited)
            time.sleep(self.poll_s)

    @staticmethod
    def collective_errors(group=None):
        """Asynchronous errors the backend's watchdog recorded for `group` (NCCL: the result of its
        ncclCommGetAsyncError polling); an empty list when there are none or the backend keeps none."""
        pg = group if group is not None else dist.distributed_c10d._get_default_group()
        errs = []
        try:
            backend = pg._get_backend(torch.device('cuda')) if torch.cuda.is_available() else None
            if backend is not None and hasattr(backend, 'get_error'):
                e = backend.get_error()
                if e is not None and 'NO_ERROR' not in str(e).upper() and 'SUCCESS' not in str(e).upper():
                    errs.append(str(e))
        except Exception:                 # a backend without error reporting is not an error of the job
            pass
        return errs


class PeerAllReduce:
    """All-reduce of small row-parallel outputs by this library's own kernel over NVLink peer memory
    (``kairos_peer_allreduce_f16``: one flag exchange, then every rank sums all partials with plain peer
    loads), for the sizes where a library all-reduce is pure latency (decode steps).

    The partial outputs must live in memory the peers can address: two slots of ``max_elems`` fp16 values
    allocated through ``torch.distributed._symmetric_memory`` (CUDA virtual-memory handles exchanged over the
    group's store; multicast binding is switched off, the kernel uses plain loads).  ``partial(m, n)`` is the
    view a row-parallel linear writes into (``DynamicLinear._forward(..., out=...)``), ``reduce(m, n)`` sums it
    over the group into a fresh local tensor and flips the slot.  Consecutive calls alternate the slots, so a
    CUDA graph that captures calls must hold an even number of them.  Larger messages go to NCCL.
    """

    def __init__(self, group, device, max_elems):
        import ctypes
        import os
        os.environ.setdefault('TORCH_SYMM_MEM_DISABLE_MULTICAST', '1')
        import torch.distributed._symmetric_memory as symm_mem
        from ._lib import check, lib
        self._lib, self._check = lib, check
        self.group = group if group is not None else dist.distributed_c10d._get_default_group()
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.device = torch.device(device)
        self.max_elems = (int(max_elems) + 127) // 128 * 128
        sig = lib.kairos_peer_allreduce_signal_bytes()
        slot_bytes = self.max_elems * 2
        self.buf = symm_mem.empty(2 * slot_bytes + sig, dtype=torch.uint8, device=self.device)
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        self.handle = symm_mem.rendezvous(self.buf, self.group.group_name)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        dist.barrier(self.group)                      # every pad is zero before any rank signals
        arr = ctypes.c_void_p * self.world
        self._in = [arr(*[p + s * slot_bytes for p in ptrs]) for s in (0, 1)]
        self._sig = arr(*[p + 2 * slot_bytes for p in ptrs])
        self._slots = [self.buf[s * slot_bytes:(s + 1) * slot_bytes].view(torch.float16) for s in (0, 1)]
        self.turn = 0
        self.calls = 0

    def fits(self, n_elems):
        return n_elems <= self.max_elems and n_elems % 8 == 0

    def partial(self, m, n):
        """The [m, n] fp16 view of the slot the next `reduce` will sum."""
        return self._slots[self.turn][:m * n].view(m, n)

    def _launch(self, peer_in, m, n, out=None):
        if out is None:
            out = torch.empty((m, n), dtype=torch.float16, device=self.device)
        self._check(self._lib.kairos_peer_allreduce_f16(peer_in, self._sig, self.world, self.rank, out.data_ptr(), m * n,
                                                        torch.cuda.current_stream(self.device).cuda_stream),
                    'kairos_peer_allreduce_f16')
        return out

    def reduce(self, m, n, out=None):
        """Sum the current slot over the group with the stand-alone kernel; flips the slot."""
        out = self._launch(self._in[self.turn], m, n, out)
        self.turn ^= 1
        self.calls += 1
        return out

    def defer(self, m, n, lead=None):
        """Leave the sum to the RMSNorm that consumes the output (at most 128 tokens); flips the slot."""
        pending = PendingPeerSum(self, self.turn, m, n, tuple(lead) if lead is not None else (m,))
        self.turn ^= 1
        self.calls += 1
        return pending


class PendingPeerSum:
    """A row-parallel output whose sum over the group has not been formed yet: every rank's partial sits in its
    peer-addressable slot.  The RMSNorm that consumes it (``ops.rms_norm`` / ``ops.rms_norm_quant`` with this
    object as ``residual_delta``) sums the partials while it loads them, so the all-reduce costs no kernel of
    its own; `materialize()` forms the sum with the stand-alone kernel instead.  Consume exactly once, in the
    same order on every rank."""

    def __init__(self, ar, turn, m, n, lead):
        self.ar, self.turn, self.m, self.n, self.lead = ar, turn, m, n, lead
        self.done = False

    def peer_args(self):
        assert not self.done, 'a pending peer sum is consumed once'
        self.done = True
        return self.ar._in[self.turn], self.ar._sig, self.ar.world, self.ar.rank

    def materialize(self):
        return self.ar._launch(self.peer_args()[0], self.m, self.n).view(*self.lead, self.n)


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
