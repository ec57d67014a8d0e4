"""Token sharding host logic with two gloo ranks on CPU (the layer itself is replaced by the CPU oracle,
which is legitimate here: what is under test is the partition / gather plumbing, not the kernels)."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from mamba_tuckermoe_b200.sharding import all_shard_bounds, shard_bounds, sharded_forward  # noqa: E402


def test_shard_bounds_cover_and_balance():
    for n in (0, 1, 7, 64, 1000, 32768):
        for w in (1, 2, 3, 4, 8):
            b = all_shard_bounds(n, w)
            assert b[0][0] == 0 and b[-1][1] == n
            assert all(b[i][1] == b[i + 1][0] for i in range(w - 1))
            sizes = [h - l for l, h in b]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(10, 2, 2)


def _worker(rank, world, port, n_tokens, chunks, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle.tucker_moe_oracle import LayerShape, layer_forward, make_factors, make_tokens
        shape = LayerShape(64, 96, 8, 2, 4, 32, 64, 1e-5)
        f = make_factors(shape, 3, torch.float32, 0.02, 0.1)
        x = make_tokens(n_tokens, shape.d_in, 3)
        layer = lambda t: layer_forward(t, f, shape.top_k, shape.eps)
        lo, hi = shard_bounds(n_tokens, world, rank)
        y_local = sharded_forward(layer, x[lo:hi], n_tokens=n_tokens)
        y_full = sharded_forward(layer, x[lo:hi], n_tokens=n_tokens, gather=True, chunks=chunks)
        ref = layer(x)
        ok = torch.allclose(y_local, ref[lo:hi], atol=1e-5) and torch.allclose(y_full, ref, atol=1e-5)
        ok = ok and y_full.shape == ref.shape
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_tokens,chunks", [(37, 1), (37, 3), (64, 4), (2, 2)])
def test_two_rank_shard_and_gather(n_tokens, chunks):
    world = 2
    port = 29500 + (os.getpid() + n_tokens * 7 + chunks) % 2000
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, n_tokens, chunks, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)
