"""Token sharding with the NCCL all-gather of y on real GPUs (needs two; skipped otherwise).

Every rank runs the layer on its share of the tokens and gathers the output into a [T, d_out] buffer, once with NCCL in
place (block-cyclic share) and once through the peers' mapped buffers (contiguous share) -- written by the
out-projection GEMM itself, or copied chunk by chunk with the copy engines; the result on every rank must be bit-identical to one GPU running all tokens (the layer is token-wise
independent, so the split changes nothing).  NVLS is switched off for the test processes: a rank that dies while its
memory is bound to an NVLink multicast object disturbs the other ranks' GPUs.
"""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, T, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from gpu_util import build_module
        from mamba_tuckermoe_b200.sharding import PeerBuffers, local_tokens, shard_bounds, sharded_forward
        from mamba_tuckermoe_b200 import _lib
        from oracle.tucker_moe_oracle import LayerShape, make_factors, make_tokens
        lib = _lib.load()
        shape = LayerShape(256, 264, 8, 2, 4, 128, 256, 1e-5)
        f = make_factors(shape, 55, torch.bfloat16, 0.02, 0.1)
        m = build_module(shape, f, torch.bfloat16, device=dev)
        x = make_tokens(T, shape.d_in, 55, torch.bfloat16).to(dev)
        with torch.no_grad():
            ref = m(x)                                               # all tokens on this GPU
            ok = True
            lo, hi = shard_bounds(T, world, rank)
            ok &= torch.equal(sharded_forward(m, x[lo:hi].contiguous(), n_tokens=T), ref[lo:hi])
            for chunks in (1, 4, 3):
                mine = local_tokens(x, world, rank, chunks).contiguous()
                out = torch.full((T, shape.d_out), float("nan"), dtype=torch.bfloat16, device=dev)
                got = sharded_forward(m, mine, n_tokens=T, gather=True, chunks=chunks, out=out)
                torch.cuda.synchronize()
                ok &= got.data_ptr() == out.data_ptr() and torch.equal(out, ref)
                ok &= torch.equal(sharded_forward(m, mine, n_tokens=T, gather=True, chunks=chunks), ref)
            # the copy-engine push into mapped peer buffers: contiguous shards, any T; the buffer is poisoned between the
            # calls, so a push that overtook the previous call's readers, or one that never landed, shows
            for buffers in (2, 1):
                peers = PeerBuffers(T, shape.d_out, torch.bfloat16, dev, buffers=buffers)
                try:
                    launches = []
                    for in_kernel, chunks in ((True, 1), (False, 1), (False, 3), (True, 1), (None, 4)):
                        n0 = lib.tmoe_launch_count()
                        got = sharded_forward(m, x[lo:hi].contiguous(), n_tokens=T, gather=True, chunks=chunks, peers=peers,
                                              in_kernel=in_kernel)
                        launches.append(lib.tmoe_launch_count() - n0)
                        ok &= got.data_ptr() == peers.out.data_ptr() and torch.equal(got, ref)
                        peers.out.fill_(float("nan"))
                    ok &= launches[0] == launches[1] and launches[2] == 3 * launches[0]   # in-kernel: one forward, no copies
                finally:
                    peers.close()
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("T", [4096, 4100])      # divisible (in-place block-cyclic gather) and ragged (staged path)
def test_sharded_forward_with_nccl_all_gather(T):
    import torch.multiprocessing as mp
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip("needs two GPUs")
    port = 29700 + (os.getpid() + T) % 1000
    ret = mp.Manager().dict()
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    mp.spawn(_worker, args=(world, port, T, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)
