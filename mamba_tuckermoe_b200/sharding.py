"""Token sharding of the layer across the GPUs of one node.

Every token's output depends only on its own row of ``x`` and on the (replicated) factors
(``pure_torch_mlx/model.py:71-102`` has no cross-token operation), so the forward needs no
collective: each rank runs the layer on a contiguous range of tokens.  The only exchange is the
optional all-gather of the output shards, which is issued per token chunk on a side stream so
that it overlaps the kernels of the next chunk.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(n_tokens: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced token range [lo, hi) of `rank`; the first n_tokens % world ranks get one more."""
    if world <= 0 or not 0 <= rank < world or n_tokens < 0:
        raise ValueError("invalid shard request")
    base, extra = divmod(n_tokens, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def all_shard_bounds(n_tokens: int, world: int) -> List[Tuple[int, int]]:
    return [shard_bounds(n_tokens, world, r) for r in range(world)]


def sharded_forward(layer: Callable[[torch.Tensor], torch.Tensor], x_local: torch.Tensor, *, n_tokens: int,
                    gather: bool = False, chunks: int = 1, group=None) -> torch.Tensor:
    """Runs `layer` on this rank's tokens ``x_local`` ([T_local, d_in], the range shard_bounds gives).

    gather=False: returns the local output shard [T_local, d_out]; nothing is communicated.
    gather=True : returns the full [n_tokens, d_out] output on every rank.  The local shard is processed in
    `chunks` pieces; the all-gather of piece i runs on a side stream (CUDA) while piece i+1 is computed.
    Shards may have unequal sizes (n_tokens not divisible by the world size).
    """
    if not gather or not dist.is_initialized() or dist.get_world_size(group) == 1:
        y = layer(x_local)
        if gather and n_tokens != x_local.shape[0]:
            raise ValueError("single-rank gather needs the whole token range")
        return y
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    bounds = all_shard_bounds(n_tokens, world)
    lo, hi = bounds[rank]
    if x_local.shape[0] != hi - lo:
        raise ValueError(f"rank {rank} holds {x_local.shape[0]} tokens, its shard is [{lo},{hi})")
    max_len = max(h - l for l, h in bounds)
    chunks = max(1, min(chunks, max_len))
    step = -(-max_len // chunks)
    out: Optional[torch.Tensor] = None
    on_cuda = x_local.is_cuda
    comm = torch.cuda.Stream(device=x_local.device) if on_cuda else None
    pending = []
    for c in range(chunks):
        c_lo, c_hi = c * step, min((c + 1) * step, max_len)   # offsets inside a shard, same on every rank
        mine = x_local[min(c_lo, hi - lo):min(c_hi, hi - lo)]
        y = layer(mine) if mine.shape[0] else None
        if out is None:
            d_out = y.shape[-1] if y is not None else layer(x_local[:1]).shape[-1]
            dtype = y.dtype if y is not None else x_local.dtype
            out = torch.empty((n_tokens, d_out), dtype=dtype, device=x_local.device)
        # every rank contributes a piece padded to the common length c_hi - c_lo
        piece = torch.zeros((c_hi - c_lo, out.shape[1]), dtype=out.dtype, device=out.device)
        if y is not None:
            piece[: y.shape[0]] = y
        recv = torch.empty((world, c_hi - c_lo, out.shape[1]), dtype=out.dtype, device=out.device)
        if on_cuda:
            comm.wait_stream(torch.cuda.current_stream(x_local.device))
            with torch.cuda.stream(comm):
                dist.all_gather_into_tensor(recv.view(-1, out.shape[1]), piece, group=group)
                for r, (l, h) in enumerate(bounds):
                    n = max(0, min(c_hi, h - l) - c_lo)
                    if n:
                        out[l + c_lo:l + c_lo + n] = recv[r, :n]
            piece.record_stream(comm); recv.record_stream(comm)
        else:
            dist.all_gather_into_tensor(recv.view(-1, out.shape[1]), piece, group=group)
            for r, (l, h) in enumerate(bounds):
                n = max(0, min(c_hi, h - l) - c_lo)
                if n:
                    out[l + c_lo:l + c_lo + n] = recv[r, :n]
        pending.append((piece, recv))
    if on_cuda:
        torch.cuda.current_stream(x_local.device).wait_stream(comm)
    return out
