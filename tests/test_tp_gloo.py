"""Tensor-parallel host logic on CPU: two gloo ranks shard a layer column- and row-wise, run their
shards (the per-rank compute is the CPU oracle here, standing in for the CUDA layer), all-reduce the
row-parallel partials and must agree with the per-shard oracle sum and, loosely, with the unsharded
layer."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import kairos_oracle as ko


class OracleLinear(torch.nn.Module):
    """Test stand-in with the DynamicLinear interface: quantizes its fp16 weight like from_module and
    evaluates kernel id 0 with the numpy oracle."""

    def __init__(self, weight):
        super().__init__()
        self.res = ko.from_module(weight.numpy())
        self.shape = tuple(weight.shape)
        self.qweight = torch.from_numpy(self.res['qweight'])

    @classmethod
    def from_module(cls, linear, device, **_):
        return cls(linear.weight.data)

    def forward(self, x):
        shape = x.shape
        y = ko.y_w4a16(x.reshape(-1, shape[-1]).numpy(), self.res)
        return torch.from_numpy(y).reshape(*shape[:-1], -1)


def _free_port():
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    from kairos_b200 import tp
    x, w = ko.make_case(6, 512, 256, seed=9)
    xt, wt = torch.from_numpy(x), torch.from_numpy(w)
    # column parallel: replicated input, sharded output, gathered for the check
    col = tp.shard_linear(wt, 'col', rank, world, 'cpu', linear_cls=OracleLinear)
    col.gather_output = True
    y_col = col(xt.unsqueeze(0))[0]
    # row parallel: sharded input, all-reduced output
    row = tp.shard_linear(wt, 'row', rank, world, 'cpu', linear_cls=OracleLinear)
    ks = 512 // world
    y_row = row(xt[:, rank * ks:(rank + 1) * ks].contiguous().unsqueeze(0))[0]
    if rank == 0:
        out['y_col'] = y_col.numpy()
        out['y_row'] = y_row.numpy()
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_column_and_row_parallel():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    x, w = ko.make_case(6, 512, 256, seed=9)
    # expected: every rank quantizes its own shard
    col_parts = [ko.y_w4a16(x, ko.from_module(w[r * 128:(r + 1) * 128])) for r in range(world)]
    assert np.array_equal(out['y_col'].view(np.uint16), np.concatenate(col_parts, axis=1).view(np.uint16))
    row_parts = [ko.y_w4a16(x[:, r * 256:(r + 1) * 256], ko.from_module(np.ascontiguousarray(w[:, r * 256:(r + 1) * 256])))
                 for r in range(world)]
    expect = (row_parts[0].astype(np.float32) + row_parts[1].astype(np.float32)).astype(np.float16)
    bad, _ = ko.within_tolerance(out['y_row'], expect)
    assert bad == 0
    # and both are close to the unquantized product (quantization noise only)
    ref = (x.astype(np.float32) @ w.astype(np.float32).T)
    for y in (out['y_col'], out['y_row']):
        rel = np.abs(y.astype(np.float32) - ref).sum() / np.abs(ref).sum()
        assert rel < 0.2


def test_shard_rules():
    from kairos_b200 import tp
    assert tp.layer_kind('self_attn.o_proj') == 'row' and tp.layer_kind('mlp.down_proj') == 'row'
    assert all(tp.layer_kind(n) == 'col' for n in ('q_proj', 'k_proj', 'v_proj', 'gate_proj', 'mlp.up_proj'))
    w = torch.zeros(64, 512, dtype=torch.float16)
    assert tp.shard_weight(w, 'col', 1, 4).shape == (16, 512)
    assert tp.shard_weight(w, 'row', 3, 4).shape == (64, 128)
    with pytest.raises(ValueError):
        tp.shard_weight(w, 'row', 0, 8)           # 64-wide K shards would split a quantization group
    with pytest.raises(ValueError):
        tp.shard_weight(torch.zeros(20, 512), 'col', 0, 8)


# ---------------------------------------------------------------------------- failure detection (host side)
def _guard_worker(rank, world, port, out):
    """Rank 1 runs step 1 and then never arrives at step 2 (it stays alive, idle: a rank hung in its own
    code); rank 0 must learn that on the host within the limit, and a collective it starts anyway must end
    with an error through the group's timeout."""
    import datetime
    import time
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    from kairos_b200 import tp
    store = dist.distributed_c10d._get_default_store()
    guard = tp.StepGuard(store, rank, world, timeout_s=1.0)
    guard.wait_all(1)                                   # both ranks are there
    y = torch.ones(4)
    dist.all_reduce(y)
    assert float(y[0]) == world
    if rank == 1:
        # never reaches step 2; leaves only after rank 0 has finished its checks
        t0 = time.monotonic()
        while not store.check(['kairos/test/done']) and time.monotonic() - t0 < 30:
            time.sleep(0.05)
        return
    t0 = time.monotonic()
    try:
        guard.wait_all(2)
        out['guard'] = 'no error'
    except tp.PeerLost as e:
        out['guard'] = ('lost', list(e.missing), e.step, time.monotonic() - t0)
    # a collective the peer never joins: the short group timeout turns it into an error
    t0 = time.monotonic()
    try:
        dist.all_reduce(torch.ones(4))
        out['collective'] = 'no error'
    except Exception as e:                               # noqa: BLE001 (backend-specific exception type)
        out['collective'] = ('error', type(e).__name__, time.monotonic() - t0)
    store.set('kairos/test/done', '1')


def test_rank_that_never_arrives_is_detected_on_the_host():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_guard_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    kind, missing, step, waited = out['guard']
    assert (kind, missing, step) == ('lost', [1], 2)
    assert 0.9 < waited < 3.0
    assert out['collective'][0] == 'error' and out['collective'][2] < 15.0


def _block_count_worker(rank, world, port, out):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    import bench
    flag = torch.ones(1)
    # the ranks' own clocks disagree about going on (rank 1 would run one more block): rank 0's verdict holds
    mine = [(True, True, False), (True, False, True)][rank]          # what each rank's own clock says, block by block
    verdicts = [bench.rank0_decides(dist, flag, m) for m in mine]
    out[rank] = verdicts
    dist.barrier()
    dist.destroy_process_group()


def test_timed_blocks_agree_on_the_block_count():
    """bench.py's timed region: both ranks follow rank 0's clock, whatever their own says."""
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_block_count_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert out[0] == [True, True, False]
    assert out[1] == [True, True, False]
