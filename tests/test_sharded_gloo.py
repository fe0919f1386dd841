"""CPU, world_size 2 over gloo: the host logic of the column-sharded layer (slice bounds, gather
layout).  The local forward is replaced by a plain matmul: the CUDA path itself is covered by the
GPU tests; what is checked here is that shards assemble into the unsharded result."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from segquant_b200.sharded import ColumnShardedSegLinear, HostRowPipeline, all_gather_slices, assemble, row_range, shard_range


def test_shard_range_and_assemble():
    assert shard_range(1536, 8, 3) == (576, 768)
    assert [shard_range(1280, 8, r)[1] - shard_range(1280, 8, r)[0] for r in range(8)] == [160] * 8
    with pytest.raises(ValueError):
        shard_range(1000, 3, 0)
    parts = torch.arange(2 * 3 * 4).view(2, 3, 4)
    full = assemble(parts)
    assert full.shape == (3, 8) and torch.equal(full[:, :4], parts[0]) and torch.equal(full[:, 4:], parts[1])
    assert [row_range(5, 2, r) for r in range(2)] == [(0, 3), (3, 5)] and row_range(2, 4, 3) == (2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _PlainSlice:
    def __init__(self, w, b):
        self.w, self.b = w, b

    def __call__(self, x):
        return x @ self.w.t() + self.b


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        x = torch.randn(5, 3, 16, generator=g)
        w = torch.randn(12, 16, generator=g)
        b = torch.randn(12, generator=g)
        lo, hi = shard_range(12, world, rank)
        layer = ColumnShardedSegLinear(_PlainSlice(w[lo:hi], b[lo:hi]), rank, world, 12)
        y = layer(x)
        ok = torch.allclose(y, x @ w.t() + b, atol=1e-6) and y.shape == (5, 3, 12)
        # host-sharded input: every rank brings its own row block, the blocks are gathered, then the sharded forward runs
        x2 = torch.randn(5, 16, generator=g)                       # 5 rows over 2 ranks: blocks of 3 and 2
        r0, r1 = row_range(5, world, rank)
        y2 = layer.forward_from_host_rows(x2[r0:r1].clone(), 5, exchange="nccl")
        ok = ok and y2.shape == (5, 12) and torch.allclose(y2, x2 @ w.t() + b, atol=1e-6)
        # the same through the step pipeline (on CPU its three stages run one after the other)
        pipe = HostRowPipeline(layer, 5, 16, torch.float32, torch.float32, exchange="nccl")
        y_rows = torch.empty((r1 - r0, 12))
        x3 = torch.randn(5, 16, generator=g)
        pipe.run(3, [x2[r0:r1].clone(), x3[r0:r1].clone()], y_rows)     # steps 0, 1, 2 -> the last one used x2 again
        ok = ok and torch.allclose(y_rows, (x2 @ w.t() + b)[r0:r1], atol=1e-6)
        pipe.run(2, [x2[r0:r1].clone(), x3[r0:r1].clone()], y_rows)
        ok = ok and torch.allclose(y_rows, (x3 @ w.t() + b)[r0:r1], atol=1e-6)
        with pytest.raises(RuntimeError):
            layer.forward_push(x2)                                  # symmetric buffers were never set up
        buf = all_gather_slices(torch.full((2, 3), float(rank)))
        ok = ok and buf.shape == (world, 2, 3) and all(bool((buf[r] == r).all()) for r in range(world))
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_rank_column_shard_over_gloo():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}
