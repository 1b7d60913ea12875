"""Multi-rank host logic on CPU: gloo process groups of two and three ranks.
The local weight gradients come from the oracle (the GPU kernels cannot run
here); what is under test is the sharding arithmetic and the single all-reduce
of the weight-update pass."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from oracle import ConvSpec
from poplibs_b200 import parallel


def test_shard_range_partitions_in_order():
    for total in (0, 1, 7, 32, 256, 257):
        for world in (1, 2, 3, 8):
            ranges = [parallel.shard_range(total, r, world) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == total
            for (a0, a1), (b0, b1) in zip(ranges, ranges[1:]):
                assert a1 == b0 and a0 <= a1
            sizes = [e - b for b, e in ranges]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        parallel.shard_range(8, 2, 2)


def test_local_conv_params_slice_the_batch():
    kw = dict(batch=32, field=[56, 56], kernel=[3, 3], in_chans=64, out_chans=64, padding=1)
    seen = 0
    for r in range(3):
        p, b, e = parallel.local_conv_params(kw, r, 3)
        assert p.batch == e - b and b == seen
        seen = e
    assert seen == 32


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _wu_worker(rank, world, port, spec_kw, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        spec = ConvSpec.simple(**spec_kw)
        r = np.random.default_rng(5)  # every rank draws the same global data
        xs, ws, ys = oracle._shapes(spec)
        x = r.integers(-2, 3, xs).astype(np.float64)
        dy = r.integers(-2, 3, ys).astype(np.float64)
        begin, end = parallel.shard_range(spec.batch, rank, world)
        local = ConvSpec.simple(**{**spec_kw, "batch": end - begin})
        if end > begin:
            dw_local, _ = oracle.conv_wu(local, x[begin:end], dy[begin:end], threads=1)
        else:
            dw_local = np.zeros(ws)
        t = torch.from_numpy(dw_local.astype(np.float32))
        parallel.allreduce_weight_grads(t)
        full, _ = oracle.conv_wu(spec, x, dy, threads=1)
        out[rank] = bool((t.numpy().astype(np.float64) == full).all())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_weight_update_allreduce_matches_unsharded_gradient(world):
    spec_kw = dict(batch=5, field=[6, 6], kernel=[3, 3], in_chans=4, out_chans=3, padding=1)
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        out = manager.dict()
        port = _free_port()
        procs = [ctx.Process(target=_wu_worker, args=(r, world, port, spec_kw, out)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert all(out[r] for r in range(world))
