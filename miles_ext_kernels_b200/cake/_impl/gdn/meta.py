"""Chunk tables of a call: which tokens form each 64-token chunk and which chunks form each sequence.

Two routes, as in the reference (reference: miles_ext_kernels/cake/_impl/gdn/ops.py:201-251 host route, :311-376
device route, :1808-1858 selection):

* host route -- equal-length batches and calls that pass ``cu_seqlens_cpu``: the exact tables are built on the host
  once per layout, copied to the device from pinned memory and kept in an LRU cache shared by every layer;
* device route -- a device-only ``cu_seqlens``: the tables are computed on the GPU without a device-to-host
  synchronisation, padded to the most chunks the layout can have (``ceil(T / 64) + N``); pad chunks have length 0
  and every kernel skips them.

Chunks never straddle a sequence; the last chunk of a sequence may be partial.
"""

from __future__ import annotations

from collections import OrderedDict
from collections.abc import Sequence
from dataclasses import dataclass
from typing import Any

import torch

CHUNK = 64
_CACHE_LIMIT = 64

__all__ = ["CHUNK", "ChunkMeta", "UploadGuard", "chunk_meta", "device_index", "host_cache_clear", "host_meta_builds",
           "host_tables", "upload"]


def device_index(device: torch.device) -> int | None:
    """The ordinal a cache key uses: ``torch.device("cuda")`` means the current device, whichever that is now."""
    if device.type != "cuda":
        return None
    return torch.cuda.current_device() if device.index is None else device.index


class UploadGuard:
    """Orders later users of a cached device table after its one host-to-device copy.  The copy is enqueued on the
    stream that was current when the table was built; a later call on ANOTHER stream waits for the copy's event (on
    the device, no host synchronisation) until the copy is seen to be complete, after which the guard costs nothing."""

    def __init__(self, device: torch.device) -> None:
        self.device = device
        stream = torch.cuda.current_stream(device)
        self.stream_id = stream.cuda_stream
        self.event: torch.cuda.Event | None = torch.cuda.Event()
        self.event.record(stream)

    def wait(self) -> None:
        event = self.event
        if event is None:
            return
        current = torch.cuda.current_stream(self.device)
        if current.cuda_stream == self.stream_id:
            return  # stream order already covers it
        if event.query():
            self.event = None
        else:
            current.wait_event(event)


def upload(table: torch.Tensor, device: torch.device) -> tuple[torch.Tensor, UploadGuard | None]:
    """A host table on ``device`` (through pinned memory, asynchronously) and the guard its cache entry keeps."""
    if device.type != "cuda":
        return table, None
    on_device = table.pin_memory().to(device, non_blocking=True)
    return on_device, UploadGuard(device)


@dataclass(frozen=True)
class ChunkMeta:
    """int32 device tables of one layout (``chunk_start, chunk_len, chunk_seq [NC]``, ``seq_chunk_start [N + 1]``)."""

    chunk_start: torch.Tensor
    chunk_len: torch.Tensor
    chunk_seq: torch.Tensor
    seq_chunk_start: torch.Tensor
    num_chunks: int  # launch extent (an upper bound on the device route)
    num_seqs: int
    total_tokens: int
    exact: bool  # False: built on the device, padded
    max_seq_chunks: int  # most chunks of one sequence (an upper bound on the device route)
    host_seq_chunk_start: tuple[int, ...] | None = None  # the host route's copy of seq_chunk_start (scan planner)
    seq_order: torch.Tensor | None = None  # int32 [N]: sequences by falling chunk count, when they differ (host route)
    guard: Any = None  # UploadGuard of a cached host-route table


def host_tables(seq_lens: Sequence[int]) -> tuple[list[int], list[int], list[int], list[int]]:
    """``(chunk_start, chunk_len, chunk_seq, seq_chunk_start)`` of the sequence lengths, as Python lists."""
    starts: list[int] = []
    lens: list[int] = []
    seqs: list[int] = []
    first = [0]
    token = 0
    for n, length in enumerate(seq_lens):
        if length < 0:
            raise ValueError(f"cu_seqlens must not decrease; sequence {n} has length {length}")
        for offset in range(0, length, CHUNK):
            starts.append(token + offset)
            lens.append(min(CHUNK, length - offset))
            seqs.append(n)
        token += length
        first.append(len(starts))
    return starts, lens, seqs, first


_HOST_CACHE: OrderedDict[tuple[Any, ...], ChunkMeta] = OrderedDict()
_HOST_BUILDS = 0


def host_meta_builds() -> int:
    """How many layouts the host route has built in this process (a counter the tests read)."""
    return _HOST_BUILDS


def host_cache_clear() -> None:
    _HOST_CACHE.clear()


def _from_host(seq_lens: tuple[int, ...], device: torch.device) -> ChunkMeta:
    global _HOST_BUILDS
    key = (seq_lens, device.type, device_index(device))
    cached = _HOST_CACHE.get(key)
    if cached is not None:
        _HOST_CACHE.move_to_end(key)
        if cached.guard is not None:
            cached.guard.wait()
        return cached
    starts, lens, seqs, first = host_tables(seq_lens)
    nc = len(starts)
    # the scans take one CTA per (sequence, head) and a CTA's duration is its sequence's chunk count: with uneven
    # documents the longest go first, so that no long walk starts when the others are done
    counts = [first[n + 1] - first[n] for n in range(len(seq_lens))]
    order = sorted(range(len(counts)), key=lambda n: -counts[n]) if len(set(counts)) > 1 else []
    flat, guard = upload(torch.tensor([*starts, *lens, *seqs, *first, *order], dtype=torch.int32), device)
    ends = 3 * nc + len(first)
    meta = ChunkMeta(
        flat[:nc], flat[nc : 2 * nc], flat[2 * nc : 3 * nc], flat[3 * nc : ends], nc, len(seq_lens), sum(seq_lens), True,
        max(counts, default=0), tuple(first), flat[ends:] if order else None, guard,
    )
    _HOST_BUILDS += 1
    _HOST_CACHE[key] = meta
    while len(_HOST_CACHE) > _CACHE_LIMIT:
        _HOST_CACHE.popitem(last=False)
    return meta


def _from_device(cu_seqlens: torch.Tensor, total_tokens: int) -> ChunkMeta:
    """Tables from a device ``cu_seqlens``: no synchronisation, padded extents (``ceil(T / 64) + N`` chunks, the
    surplus being pad chunks of length 0).  On a GPU one launch of the library's ``chunk_meta`` kernel; for a host
    tensor (the CPU tests of the layout logic) the same tables by torch integer ops."""
    if cu_seqlens.is_cuda:
        from . import native

        num_seqs = cu_seqlens.numel() - 1
        bound = (total_tokens + CHUNK - 1) // CHUNK + num_seqs
        cu = cu_seqlens.contiguous()
        flat = torch.empty(3 * bound + num_seqs + 1, dtype=torch.int32, device=cu.device)
        with torch.cuda.device(cu.device):
            native.launch("gdn_chunk_meta", cu, int(cu.dtype == torch.int64), num_seqs, bound, flat[:bound],
                          flat[bound : 2 * bound], flat[2 * bound : 3 * bound], flat[3 * bound :], device=cu.device)
        return ChunkMeta(flat[:bound], flat[bound : 2 * bound], flat[2 * bound : 3 * bound], flat[3 * bound :], bound,
                         num_seqs, total_tokens, False, (total_tokens + CHUNK - 1) // CHUNK + 1)
    cu = cu_seqlens.to(torch.int64)
    num_seqs = cu.numel() - 1
    bound = (total_tokens + CHUNK - 1) // CHUNK + num_seqs
    lens = cu[1:] - cu[:-1]
    per_seq = (lens + (CHUNK - 1)) // CHUNK
    first = torch.zeros(num_seqs + 1, dtype=torch.int64, device=cu.device)
    first[1:] = torch.cumsum(per_seq, 0)
    ids = torch.arange(bound, dtype=torch.int64, device=cu.device)
    seq = torch.searchsorted(first[1:].contiguous(), ids, right=True).clamp_(max=num_seqs - 1)
    start = cu[:-1][seq] + (ids - first[:-1][seq]) * CHUNK
    length = (cu[1:][seq] - start).clamp_(min=0, max=CHUNK)
    length = torch.where(ids < first[-1], length, torch.zeros_like(length))
    start = torch.where(length > 0, start, torch.zeros_like(start))
    as32 = lambda t: t.to(torch.int32).contiguous()  # noqa: E731
    return ChunkMeta(as32(start), as32(length), as32(seq), as32(first), bound, num_seqs, total_tokens, False,
                     (total_tokens + CHUNK - 1) // CHUNK + 1)


def _seq_lens_from_host(cu_seqlens_cpu: Any) -> tuple[int, ...]:
    offsets = cu_seqlens_cpu.tolist() if isinstance(cu_seqlens_cpu, torch.Tensor) else list(cu_seqlens_cpu)
    if not offsets or offsets[0] != 0:
        raise ValueError(f"cu_seqlens_cpu must start at 0; it starts at {offsets[0] if offsets else 'nothing'}")
    return tuple(int(b) - int(a) for a, b in zip(offsets[:-1], offsets[1:]))


def chunk_meta(cu_seqlens, cu_seqlens_cpu, batch: int, seq_len: int, device) -> ChunkMeta:
    """The tables of a call, without a device-to-host synchronisation.

    ``cu_seqlens is None``: ``batch`` sequences of ``seq_len`` tokens.  With ``cu_seqlens_cpu`` the host copy decides
    (it must start at 0, not decrease, and end at the ``batch * seq_len`` tokens of q: tokens past its last offset
    would never be written).  A device-only ``cu_seqlens`` takes the device route.
    """
    device = torch.device(device)
    total = int(batch) * int(seq_len)
    if cu_seqlens is None:
        return _from_host((int(seq_len),) * int(batch), device)
    if batch != 1:
        raise ValueError("cu_seqlens requires a leading batch dimension of 1")
    if cu_seqlens_cpu is None:
        return _from_device(cu_seqlens, total)
    seq_lens = _seq_lens_from_host(cu_seqlens_cpu)
    if sum(seq_lens) != total:
        raise ValueError(f"cu_seqlens_cpu must end at the {total} tokens of q; it ends at {sum(seq_lens)}")
    return _from_host(seq_lens, device)
