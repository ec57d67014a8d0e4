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

``PeerBuffers`` is the second way to gather: every rank's ``[n_tokens, d_out]`` result buffer is mapped into every other
rank's process, and a finished token block is copied to the same rows of all peer buffers by the copy engines over
NVLink (``tmoe_peer_push``).  No SM takes part, so the copies run beside the tensor-core kernels of the next block --
an NCCL all-gather launched there has to wait for SMs that the one-CTA-per-SM kernels hold -- and any token-to-rank
map works: the push path uses the contiguous ranges of ``shard_bounds``, divisible or not.
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


class _DevicePointer:
    """Lets torch wrap a raw device pointer (CUDA array interface, version 3) without copying."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class PeerBuffers:
    """This rank's ``[n_tokens, d_out]`` result buffers plus the mapped result buffers of the other ranks.

    Creating one is a collective over `group` (every rank allocates, the 64-byte handles travel through
    ``all_gather_object``); keep it for the life of the model and pass it to ``sharded_forward(peers=...)``.  ``close()``
    is a collective too: it unmaps the peers' buffers, waits for every rank to have done so, then frees its own.

    ``buffers=2`` (default): consecutive calls alternate between two result buffers, so a call needs ONE rendezvous of
    the ranks (after its last write) instead of two: when rank r starts writing buffer A again in call k+2 it has passed
    the rendezvous of call k+1, which every rank q enqueued behind its reads of call k's result in A.  The result of a
    call therefore stays valid until the call after next.  ``buffers=1`` keeps one buffer (valid until the next call) and
    adds a rendezvous in front of the first write.  ``.out`` is the buffer of the latest call.  The buffers belong to this
    object: ``close()`` (or dropping the object) frees them, tensors obtained from ``.out`` must not be used afterwards.
    """

    def __init__(self, n_tokens: int, d_out: int, dtype: torch.dtype, device: torch.device, group=None, buffers: int = 2):
        import ctypes as C
        from . import _lib
        if buffers not in (1, 2):
            raise ValueError("buffers must be 1 or 2")
        lib = _lib.load()
        self.group, self.world, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        self.n_tokens, self.d_out, self.dtype, self.device = n_tokens, d_out, dtype, torch.device(device)
        self.row_bytes = d_out * torch.empty((), dtype=dtype).element_size()
        self.buffers = buffers
        self._stride = -(-max(1, n_tokens) * self.row_bytes // 256) * 256     # bytes between the two buffers
        nbytes = self._stride * buffers
        with torch.cuda.device(self.device):
            # every step that can fail on one rank alone is followed by an agreement of all ranks, so that a failure raises
            # everywhere instead of leaving the others inside a collective
            own, handle = C.c_void_p(), (C.c_ubyte * _lib.PEER_HANDLE_BYTES)()
            rc = lib.tmoe_peer_alloc(nbytes, C.byref(own), handle)
            self._base = own.value if rc == 0 else None
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle) if rc == 0 else None, group=group)
            # the peers in the order rank+1, rank+2, ...: when every rank copies to its peers in this order, one after the
            # other, each GPU receives from one sender at a time.  Measured on 4 B200s (302 MB per copy): 748 GB/s leave
            # every GPU this way, 369-388 GB/s when the copies to all peers run at once or all ranks start with rank 0.
            self.peer_ranks = [(self.rank + k) % self.world for k in range(1, self.world)]
            self._peer_base = []
            failed = "tmoe_peer_alloc" if rc else None
            if all(h is not None for h in handles):
                for r in self.peer_ranks:
                    p = C.c_void_p()
                    h = (C.c_ubyte * _lib.PEER_HANDLE_BYTES).from_buffer_copy(handles[r])
                    rc = lib.tmoe_peer_open(h, C.byref(p))
                    if rc:
                        failed = f"tmoe_peer_open(rank {r})"
                        break
                    self._peer_base.append(p.value)
            elif failed is None:
                failed = "tmoe_peer_alloc on another rank"
            verdicts = [None] * self.world
            dist.all_gather_object(verdicts, failed, group=group)
            if any(v is not None for v in verdicts):
                for p in self._peer_base:
                    lib.tmoe_peer_close(p)
                self._peer_base = []
                dist.barrier(group=group)
                if self._base is not None:
                    lib.tmoe_peer_free(self._base)
                    self._base = None
                raise RuntimeError("PeerBuffers: mapping the result buffers across the ranks failed: " +
                                   "; ".join(f"rank {r}: {v}" for r, v in enumerate(verdicts) if v is not None))
            flat = torch.as_tensor(_DevicePointer(self._base, nbytes), device=self.device)
            self._outs = [flat[i * self._stride:i * self._stride + n_tokens * self.row_bytes].view(dtype).view(n_tokens, d_out)
                          for i in range(buffers)]
            self._which = 0
            self.comm = torch.cuda.Stream(device=self.device)
            self.push_stream = torch.cuda.Stream(device=self.device)
            self._stream_ptrs = (C.c_void_p * max(1, len(self.peer_ranks)))(*[self.push_stream.cuda_stream] * len(self.peer_ranks))
            self._token = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._lib, self._C = lib, C

    @property
    def out(self) -> torch.Tensor:
        """The result buffer of the latest call (of the next one right after ``next_buffer``)."""
        return self._outs[self._which]

    def next_buffer(self) -> torch.Tensor:
        """Moves on to the other result buffer (with ``buffers=2``) and returns it."""
        self._which = (self._which + 1) % self.buffers
        return self._outs[self._which]

    @property
    def _own(self) -> int:
        return self._base + self._which * self._stride

    def peer_pointers(self):
        """Device addresses, in this process, of the other ranks' copies of ``.out``, in the order of ``peer_ranks``."""
        return [p + self._which * self._stride for p in self._peer_base]

    def push(self, row_lo: int, row_hi: int) -> None:
        """Enqueues the copies of rows [row_lo, row_hi) of ``.out`` to the same rows of every peer on ``push_stream``, one
        after the other in the order of ``peer_ranks``.  The caller orders that stream (``sharded_forward`` does)."""
        if row_hi <= row_lo or not self.peer_ranks:
            return
        from . import _lib
        C, off = self._C, row_lo * self.row_bytes
        dst = (C.c_void_p * len(self._peer_base))(*[p + off for p in self.peer_pointers()])
        _lib.check(self._lib.tmoe_peer_push(dst, len(self._peer_base), self._own + off, (row_hi - row_lo) * self.row_bytes,
                                            self._stream_ptrs), "tmoe_peer_push")

    def rendezvous(self, stream) -> None:
        """A one-element all-reduce on `stream`: when it has run here, every rank's work enqueued before its own
        rendezvous has finished."""
        with torch.cuda.stream(stream):
            dist.all_reduce(self._token, group=self.group)

    def __del__(self):
        # not a substitute for close() (which agrees with the other ranks first): last-resort release of this rank's memory
        try:
            if getattr(self, "_base", None) is not None:
                for p in self._peer_base:
                    self._lib.tmoe_peer_close(p)
                self._lib.tmoe_peer_free(self._base)
                self._base = None
        except Exception:
            pass

    def close(self) -> None:
        if self._base is None:
            return
        from . import _lib
        torch.cuda.synchronize(self.device)
        with torch.cuda.device(self.device):
            for p in self._peer_base:
                _lib.check(self._lib.tmoe_peer_close(p), "tmoe_peer_close")
            self._peer_base = []
            dist.barrier(group=self.group)
            self._outs = []
            _lib.check(self._lib.tmoe_peer_free(self._base), "tmoe_peer_free")
        self._base = None


def push_chunks(local_tokens: int) -> int:
    """Chunks of the copy-engine push when the caller leaves the choice open: about 8192 tokens per chunk, at most 4 -- below
    that a chunk's copies are too short to stay ahead of the host's per-chunk work (measured optimum at 4096 ... 65536
    tokens per GPU on 2, 4 and 8 GPUs: 1, 1, 2, 4, 4)."""
    return max(1, min(4, local_tokens // 8192))


def in_kernel_gather_pays(layer, world: int) -> bool:
    """Whether the out-projection GEMM should write the peers' buffers itself.  It produces 2 * d_out bytes of y per
    2 * r2 * d_out flops, i.e. (world - 1) / r2 bytes per flop have to leave through NVLink while it runs: at ~1.4 PFLOP/s
    and ~0.75 TB/s that keeps up with the GEMM only up to (world - 1) * 1900 / r2 ~ 1.  Beyond that, and whenever a GPU
    would receive tiles from several senders at once (measured: the inbound rate halves), the copy engines do better:
    they run beside ALL kernels of the next chunk, not only beside the GEMM."""
    r2 = getattr(layer, "r2", None)
    if r2 is None and hasattr(layer, "U_out"):
        r2 = layer.U_out.shape[0]
    return world == 2 and r2 is not None and 1900.0 / r2 <= 1.0


def _push_gather(layer, x_local: torch.Tensor, n_tokens: int, chunks: int, peers: "PeerBuffers", in_kernel) -> torch.Tensor:
    """The layer on this rank's contiguous token range into ``peers.out`` and into the same rows of every peer's buffer.
    in_kernel: the out-projection GEMM stores each finished tile to all of them itself (tensor-core path; one call, no
    copies).  Otherwise, and for calls that path does not take, block by block: every finished block is pushed to the
    peers by the copy engines while the next one is computed.  in_kernel=None picks by ``in_kernel_gather_pays``."""
    if peers.n_tokens != n_tokens or peers.dtype != x_local.dtype or peers.device != x_local.device:
        raise ValueError("`peers` was made for another token count, dtype or device")
    lo, hi = shard_bounds(n_tokens, peers.world, peers.rank)
    if x_local.shape[0] != hi - lo:
        raise ValueError(f"rank {peers.rank} holds {x_local.shape[0]} tokens, its shard is [{lo},{hi})")
    if in_kernel is None:
        in_kernel = in_kernel_gather_pays(layer, peers.world)
    cur = torch.cuda.current_stream(peers.device)
    out = peers.next_buffer()
    # Every call makes the same rendezvous on every rank, whichever form a rank ends up using (the ranks' token counts may
    # differ by one, and with them the path): one after this rank's last write and, with a single result buffer, one
    # before anything is written into a peer's buffer -- nobody may still read what the previous call left there.
    lead = peers.buffers == 1
    if in_kernel and hi > lo and hasattr(layer, "forward_into") and len(peers.peer_ranks) <= _lib_max_peers():
        from ._lib import ERR_UNSUPPORTED, TmoeError
        off = lo * peers.row_bytes
        if lead:
            peers.rendezvous(cur)
            lead = False
        try:
            # validation comes before the first launch: a refusal leaves nothing enqueued
            layer.forward_into(x_local, out[lo:hi], peer_ptrs=[p + off for p in peers.peer_pointers()])
            peers.rendezvous(cur)
            return out
        except TmoeError as e:
            if e.status != ERR_UNSUPPORTED:
                raise
    if lead:
        # the copies wait for the rendezvous on a side stream; the kernels do not
        peers.comm.wait_stream(cur)
        peers.rendezvous(peers.comm)
        peers.push_stream.wait_stream(peers.comm)
    n = hi - lo
    chunks = max(1, min(chunks, n)) if n else 1
    step = -(-n // chunks) if n else 0
    for c in range(chunks):
        a, b = lo + c * step, min(lo + (c + 1) * step, hi)
        if b <= a:
            break
        _into(layer, x_local[a - lo:b - lo], out[a:b])
        done = torch.cuda.Event()
        done.record(cur)
        peers.push_stream.wait_event(done)
        peers.push(a, b)
    cur.wait_stream(peers.push_stream)
    peers.rendezvous(cur)   # every rank's pushes have landed behind this point
    return out


def _lib_max_peers() -> int:
    from ._lib import MAX_PEERS
    return MAX_PEERS


def _into(layer, x: torch.Tensor, dst: torch.Tensor) -> None:
    """Runs the layer on x with its output in dst (written in place when the layer offers forward_into)."""
    if hasattr(layer, "forward_into"):
        layer.forward_into(x, dst)
    else:
        dst.copy_(layer(x))


def sharded_forward(layer: Callable[[torch.Tensor], torch.Tensor], x_local: torch.Tensor, *, n_tokens: int,
                    gather: bool = False, chunks: Optional[int] = None, group=None, out: Optional[torch.Tensor] = None,
                    d_out: Optional[int] = None, peers: Optional[PeerBuffers] = None, in_kernel: Optional[bool] = None) -> torch.Tensor:
    """Runs `layer` on this rank's tokens ``x_local`` ([T_local, d_in]).

    gather=False: returns the local output shard [T_local, d_out]; nothing is communicated.
    gather=True : returns the full [n_tokens, d_out] output on every rank (in `out` when given).  The local tokens are
    processed in `chunks` pieces; the all-gather of piece i runs on a side stream (CUDA) while piece i+1 is computed.
    With n_tokens divisible by world * chunks, ``x_local`` holds the rank's rows in the block-cyclic order of
    ``cyclic_rows`` (``local_tokens`` cuts them out of a full activation) and every piece is gathered in place into the
    result; otherwise the shards are the contiguous ranges of ``shard_bounds`` and the pieces go through two staging
    buffers.  ``d_out`` spares a probing call when `layer` is not a module with ``U_out``.
    peers=PeerBuffers(...): gathers through the mapped peer buffers instead of NCCL (CUDA only).  ``x_local`` is then the
    contiguous ``shard_bounds`` range for any n_tokens, and the result is ``peers.out`` (see ``PeerBuffers`` for how long
    it stays valid).  With in_kernel=True the out-projection GEMM itself stores every output tile to all ranks' buffers
    when the call takes the tensor-core path; in_kernel=False, or a call on another path, copies finished chunks with the
    copy engines instead (`chunks` applies to this form only; None = ``push_chunks``); None (default) decides by
    ``in_kernel_gather_pays``.  With NCCL `chunks` defaults to 1.
    """
    if peers is not None:
        if not gather or out is not None:
            raise ValueError("`peers` is the gathered result buffer: pass gather=True and no `out`")
        if chunks is None:
            chunks = push_chunks(x_local.shape[0])
        return _push_gather(layer, x_local, n_tokens, chunks, peers, in_kernel)
    if chunks is None:
        chunks = 1
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
