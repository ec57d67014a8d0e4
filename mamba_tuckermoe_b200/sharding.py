"""Token sharding of the layer across the GPUs of one node.

Every token's output depends only on its own row of ``x`` and on the (replicated) factors
(``pure_torch_mlx/model.py:71-102`` has no cross-token operation), so the forward needs no
collective: each rank runs the layer on its own tokens.  The only exchange is the optional
all-gather of the output, which is issued per token chunk on a side stream so that it overlaps
the kernels of the next chunk.

Two token-to-rank maps:

* ``shard_bounds``  one contiguous range per rank -- what ``gather=False`` and ``chunks=1`` use.
* ``cyclic_rows``   block-cyclic: with ``chunks`` chunks of ``L = n_tokens / (world * chunks)`` tokens per rank, chunk c
  of rank r is the global rows ``[(c * world + r) * L, (c * world + r + 1) * L)``.  The chunk-c blocks of all ranks
  are then adjacent in the output, so every chunk's all-gather is ONE in-place NCCL all-gather that lands in the final
  ``[n_tokens, d_out]`` buffer: the layer writes its block straight into that buffer, nothing is staged, padded or
  copied afterwards, and no memory is allocated per chunk.

When ``n_tokens`` does not divide evenly the shards are contiguous and unequal; the chunks are then padded to a common
length in two staging buffers that are allocated once per call.
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


def cyclic_rows(n_tokens: int, world: int, rank: int, chunks: int) -> List[Tuple[int, int]]:
    """Global row ranges of `rank`, chunk by chunk, in the block-cyclic map (n_tokens divisible by world * chunks).
    With chunks == 1 this is the contiguous range of shard_bounds."""
    if chunks <= 0 or world <= 0 or not 0 <= rank < world or n_tokens % (world * chunks):
        raise ValueError("block-cyclic sharding needs n_tokens divisible by world * chunks")
    L = n_tokens // (world * chunks)
    return [((c * world + rank) * L, (c * world + rank + 1) * L) for c in range(chunks)]


def local_tokens(x_all: torch.Tensor, world: int, rank: int, chunks: int = 1) -> torch.Tensor:
    """The rows of a full ``[n_tokens, d_in]`` activation that `rank` processes in ``sharded_forward(gather=True,
    chunks=chunks)``, in the order it processes them."""
    n = x_all.shape[0]
    if n % (world * chunks) == 0:
        return torch.cat([x_all[lo:hi] for lo, hi in cyclic_rows(n, world, rank, chunks)])
    lo, hi = shard_bounds(n, world, rank)
    return x_all[lo:hi]


def _into(layer, x: torch.Tensor, dst: torch.Tensor) -> None:
    """Runs the layer on x with its output in dst (written in place when the layer offers forward_into)."""
    if hasattr(layer, "forward_into"):
        layer.forward_into(x, dst)
    else:
        dst.copy_(layer(x))


def sharded_forward(layer: Callable[[torch.Tensor], torch.Tensor], x_local: torch.Tensor, *, n_tokens: int,
                    gather: bool = False, chunks: int = 1, group=None, out: Optional[torch.Tensor] = None,
                    d_out: Optional[int] = None) -> torch.Tensor:
    """Runs `layer` on this rank's tokens ``x_local`` ([T_local, d_in]).

    gather=False: returns the local output shard [T_local, d_out]; nothing is communicated.
    gather=True : returns the full [n_tokens, d_out] output on every rank (in `out` when given).  The local tokens are
    processed in `chunks` pieces; the all-gather of piece i runs on a side stream (CUDA) while piece i+1 is computed.
    With n_tokens divisible by world * chunks, ``x_local`` holds the rank's rows in the block-cyclic order of
    ``cyclic_rows`` (``local_tokens`` cuts them out of a full activation) and every piece is gathered in place into the
    result; otherwise the shards are the contiguous ranges of ``shard_bounds`` and the pieces go through two staging
    buffers.  ``d_out`` spares a probing call when `layer` is not a module with ``U_out``.
    """
    if not gather or not dist.is_initialized() or dist.get_world_size(group) == 1:
        if gather and n_tokens != x_local.shape[0]:
            raise ValueError("single-rank gather needs the whole token range")
        if out is not None:
            _into(layer, x_local, out)
            return out
        return layer(x_local)
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    if d_out is None:
        d_out = layer.U_out.shape[1] if hasattr(layer, "U_out") else layer(x_local[:1]).shape[-1]
    dev, dtype = x_local.device, x_local.dtype
    if out is None:
        out = torch.empty((n_tokens, d_out), dtype=dtype, device=dev)
    elif out.shape != (n_tokens, d_out) or out.dtype != dtype or out.device != dev or not out.is_contiguous():
        raise ValueError("`out` must be a contiguous [n_tokens, d_out] tensor of x's dtype on x's device")
    on_cuda = x_local.is_cuda
    cur = torch.cuda.current_stream(dev) if on_cuda else None
    comm = _comm_stream(dev) if on_cuda else None
    if on_cuda:
        comm.wait_stream(cur)   # `out` may be a fresh block whose previous owner's work is ordered on the current stream

    chunks = max(1, chunks)
    if n_tokens % (world * chunks) == 0 and n_tokens > 0:
        L = n_tokens // (world * chunks)
        if x_local.shape[0] != L * chunks:
            raise ValueError(f"rank {rank} holds {x_local.shape[0]} tokens, the block-cyclic map gives it {L * chunks}")
        for c in range(chunks):
            block = out[c * world * L:(c + 1) * world * L]           # chunk c of every rank, adjacent
            mine = block[rank * L:(rank + 1) * L]
            _into(layer, x_local[c * L:(c + 1) * L], mine)
            if on_cuda:
                done = torch.cuda.Event()
                done.record(cur)
                with torch.cuda.stream(comm):
                    comm.wait_event(done)
                    dist.all_gather_into_tensor(block, mine, group=group)   # in place: `mine` is block's slot of this rank
            else:
                dist.all_gather_into_tensor(block, mine.clone(), group=group)
        if on_cuda:
            cur.wait_stream(comm)
        return out

    # unequal shards: contiguous ranges, pieces padded to a common length in two staging buffers used in turn
    bounds = all_shard_bounds(n_tokens, world)
    lo, hi = bounds[rank]
    if x_local.shape[0] != hi - lo:
        raise ValueError(f"rank {rank} holds {x_local.shape[0]} tokens, its shard is [{lo},{hi})")
    max_len = max(h - l for l, h in bounds)
    chunks = max(1, min(chunks, max_len))
    step = -(-max_len // chunks)
    piece = [torch.zeros((step, d_out), dtype=dtype, device=dev) for _ in range(min(2, chunks))]
    recv = [torch.empty((world, step, d_out), dtype=dtype, device=dev) for _ in range(min(2, chunks))]
    free = [None, None]   # event after which staging slot b may be overwritten
    for c in range(chunks):
        b = c & 1
        c_lo, c_hi = c * step, min((c + 1) * step, max_len)   # offsets inside a shard, same on every rank
        mine = x_local[min(c_lo, hi - lo):min(c_hi, hi - lo)]
        if on_cuda and free[b] is not None:
            cur.wait_event(free[b])
        if mine.shape[0]:
            _into(layer, mine, piece[b][:mine.shape[0]])
        if on_cuda:
            done = torch.cuda.Event()
            done.record(cur)
        with (torch.cuda.stream(comm) if on_cuda else _nullcontext()):
            if on_cuda:
                comm.wait_event(done)
            dist.all_gather_into_tensor(recv[b].view(-1, d_out), piece[b], group=group)   # whole slots, also for a short last chunk
            got = recv[b]
            for r, (l, h) in enumerate(bounds):
                n = max(0, min(c_hi, h - l) - c_lo)
                if n:
                    out[l + c_lo:l + c_lo + n] = got[r, :n]
            if on_cuda:
                free[b] = torch.cuda.Event()
                free[b].record(comm)
    if on_cuda:
        cur.wait_stream(comm)
        for t in piece + recv:
            t.record_stream(comm)
    return out


class _nullcontext:
    def __enter__(self):
        return None

    def __exit__(self, *a):
        return False


_comm_streams = {}


def _comm_stream(dev: torch.device):
    """One communication stream per device, created on first use."""
    s = _comm_streams.get(dev.index)
    if s is None:
        s = torch.cuda.Stream(device=dev)
        _comm_streams[dev.index] = s
    return s
