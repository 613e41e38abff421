"""Batch sharding across ranks: world_size-2 gloo processes on the CPU.  The
per-rank compute is the CPU oracle here (the GPU kernels are exercised by the
-m gpu tests); what is checked is that shard -> per-rank product -> gather
reproduces the unsharded result exactly, for even and uneven splits."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ksmm_b200.sharding import gather_output, shard_batch, shard_range


def test_shard_ranges_cover_batch():
    for batch in (0, 1, 7, 25088, 200704, 25089):
        for world in (1, 2, 3, 8):
            spans = [shard_range(batch, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == batch
            for (a0, a1), (b0, b1) in zip(spans[:-1], spans[1:]):
                assert a1 == b0 and a0 <= a1
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    assert shard_range(200704, 3, 8) == (3 * 25088, 4 * 25088)
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, batch, bs_last, ret):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    from oracle import ksmm_oracle as ko
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.RandomState(5)
        pats = [(2, 8, 4, 2), (4, 6, 4, 2)]
        ws = [rng.uniform(-0.5, 0.5, size=p) for p in pats]
        x = rng.standard_normal((16, batch) if bs_last else (batch, 16))
        full = ko.chain_apply(x, ws, bs_last)
        xl = shard_batch(torch.from_numpy(x), bs_last, rank, world)
        yl = torch.from_numpy(ko.chain_apply(xl.numpy(), ws, bs_last))
        y = gather_output(yl, bs_last, batch)
        ok = bool(np.array_equal(y.numpy(), full)) and xl.is_contiguous()
        flag = torch.tensor([1 if ok else 0])
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            ret.put(int(flag.item()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("batch,bs_last", [(10, True), (10, False), (7, True), (7, False)])
def test_shard_compute_gather_world2(batch, bs_last):
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, batch, bs_last, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert ret.get(timeout=5) == 1
