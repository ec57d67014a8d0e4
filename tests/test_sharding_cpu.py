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

from mamba_tuckermoe_b200.sharding import (all_shard_bounds, cyclic_rows, local_tokens, shard_bounds,  # noqa: E402
                                            sharded_forward)


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


def test_block_cyclic_rows_partition_the_tokens():
    for n, w, c in ((64, 2, 4), (32768, 8, 4), (48, 4, 1), (131072, 8, 4)):
        seen = torch.zeros(n, dtype=torch.int32)
        for r in range(w):
            rows = cyclic_rows(n, w, r, c)
            assert len(rows) == c and all(h - l == n // (w * c) for l, h in rows)
            for l, h in rows:
                seen[l:h] += 1
        assert bool((seen == 1).all())
        # chunk c of all ranks is one contiguous block of the output
        for ci in range(c):
            los = sorted(cyclic_rows(n, w, r, c)[ci][0] for r in range(w))
            assert los == [ci * n // c + r * (n // (w * c)) for r in range(w)]
    assert cyclic_rows(48, 4, 1, 1) == [shard_bounds(48, 4, 1)]
    with pytest.raises(ValueError):
        cyclic_rows(37, 2, 0, 3)


class _IntoLayer:
    """Stand-in with the module's two entry points (the CPU oracle does the arithmetic)."""

    def __init__(self, fn, d_out):
        self.fn, self.d_out, self.into_calls = fn, d_out, 0

    def __call__(self, t):
        return self.fn(t)

    def forward_into(self, t, out):
        self.into_calls += 1
        out.copy_(self.fn(t))


def _worker(rank, world, port, n_tokens, chunks, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle.tucker_moe_oracle import LayerShape, layer_forward, make_factors, make_tokens
        shape = LayerShape(64, 96, 8, 2, 4, 32, 64, 1e-5)
        f = make_factors(shape, 3, torch.float32, 0.02, 0.1)
        x = make_tokens(n_tokens, shape.d_in, 3)
        fn = lambda t: layer_forward(t, f, shape.top_k, shape.eps)
        layer = _IntoLayer(fn, shape.d_out)
        lo, hi = shard_bounds(n_tokens, world, rank)
        y_local = sharded_forward(layer, x[lo:hi], n_tokens=n_tokens)
        mine = local_tokens(x, world, rank, chunks)
        y_full = sharded_forward(layer, mine, n_tokens=n_tokens, gather=True, chunks=chunks, d_out=shape.d_out)
        ref = fn(x)
        ok = torch.allclose(y_local, ref[lo:hi], atol=1e-5) and torch.allclose(y_full, ref, atol=1e-5)
        ok = ok and y_full.shape == ref.shape and layer.into_calls > 0
        # caller-provided result buffer, plain callable as the layer
        buf = torch.full((n_tokens, shape.d_out), float("nan"))
        got = sharded_forward(fn, mine, n_tokens=n_tokens, gather=True, chunks=chunks, out=buf, d_out=shape.d_out)
        ok = ok and got.data_ptr() == buf.data_ptr() and torch.allclose(buf, ref, atol=1e-5)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_tokens,chunks", [(37, 1), (37, 3), (64, 4), (64, 1), (2, 2), (48, 3)])
def test_two_rank_shard_and_gather(n_tokens, chunks):
    """Even splits take the block-cyclic in-place gather, ragged ones the padded staging path."""
    world = 2
    port = 29500 + (os.getpid() + n_tokens * 7 + chunks) % 2000
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, n_tokens, chunks, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)


def test_in_kernel_gather_rule():
    """The GEMM writes the peers' buffers itself only with one peer and a contraction deep enough to hide the stores."""
    from types import SimpleNamespace as NS
    from mamba_tuckermoe_b200.sharding import in_kernel_gather_pays
    deep, shallow = NS(U_out=torch.empty(2048, 8)), NS(U_out=torch.empty(1024, 8))
    assert in_kernel_gather_pays(deep, 2) and not in_kernel_gather_pays(deep, 4)
    assert not in_kernel_gather_pays(shallow, 2)
    assert not in_kernel_gather_pays(lambda x: x, 2)
    from mamba_tuckermoe_b200.sharding import push_chunks
    assert [push_chunks(t) for t in (1, 4096, 8192, 16384, 32768, 65536, 1 << 20)] == [1, 1, 1, 2, 4, 4, 4]


def _peer_failure_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import contextlib
        from mamba_tuckermoe_b200 import sharding
        # no GPU here: the allocation fails on every rank; what is checked is that all ranks leave the constructor with
        # the same error after the same collectives (nobody is left waiting) and that the group still works afterwards
        real = torch.cuda.device
        torch.cuda.device = lambda d: contextlib.nullcontext()
        try:
            try:
                sharding.PeerBuffers(64, 96, torch.bfloat16, torch.device("cuda", 0))
                ret[rank] = "constructed"
            except RuntimeError as e:
                ret[rank] = str(e)
        finally:
            torch.cuda.device = real
        t = torch.ones(1)
        dist.all_reduce(t)
        ret[f"sum{rank}"] = float(t)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.is_available(), reason="needs a machine on which the device allocation fails")
def test_peer_buffers_fail_on_every_rank_alike():
    world = 2
    port = 29500 + (os.getpid() + 911) % 2000
    ret = mp.Manager().dict()
    mp.spawn(_peer_failure_worker, args=(world, port, ret), nprocs=world, join=True)
    for r in range(world):
        assert "tmoe_peer_alloc" in ret[r] and "rank 0" in ret[r] and "rank 1" in ret[r], dict(ret)
        assert ret[f"sum{r}"] == world
