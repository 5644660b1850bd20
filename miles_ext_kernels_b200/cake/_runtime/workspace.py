"""One bounded pool of scratch device buffers shared by the ops.

An op asks for scratch with :func:`take` under a key ``(op, role)``.  The pool holds at most
``--cake-workspace-pool-bytes`` per device.  At the default 0 nothing is held: every ``take`` is a plain
``torch.empty``.  With a positive bound the pool keeps one byte buffer per ``(op, role)`` and CUDA stream, hands out
typed views of it while it is large enough, and drops the least recently used buffers to stay under the bound; a
request larger than the bound is served by a plain allocation.  While the current stream captures a CUDA graph the
pool is bypassed, so a graph never records memory the pool may free later.

A buffer from :func:`take` stays valid until the next :func:`take` of the same key on the same stream, or
:func:`release`.  Use it on that stream only; never save it for backward and never return it to a caller.

Same contract as the reference's pool (reference: miles_ext_kernels/cake/_runtime/workspace.py:77-141).  Importing
this module does not import torch.
"""

from __future__ import annotations

import math
import threading
from collections import OrderedDict
from collections.abc import Sequence
from typing import Any

from . import config

__all__ = ["release", "stats", "take"]


class _DevicePool:
    """The buffers of one device, least recently used first, and its counters."""

    def __init__(self) -> None:
        self.buffers: OrderedDict[tuple[str, str, Any], Any] = OrderedDict()
        self.hits = self.misses = self.evictions = 0

    def held(self) -> int:
        return sum(buffer.numel() for buffer in self.buffers.values())

    def shrink_to(self, room: int) -> None:
        held = self.held()
        while self.buffers and held > room:
            _, dropped = self.buffers.popitem(last=False)
            held -= dropped.numel()
            self.evictions += 1


_pools: dict[Any, _DevicePool] = {}
_lock = threading.Lock()


def _locate(device: Any) -> tuple[Any, Any]:
    """``(pool key, torch.device)``: the CUDA index (current device for a bare ``"cuda"``), else the device name."""
    import torch

    where = torch.device(device)
    if where.type != "cuda":
        return str(where), where
    index = where.index if where.index is not None else torch.cuda.current_device()
    return index, torch.device("cuda", index)


def _current_stream(key: Any) -> tuple[Any, bool]:
    """``(stream handle, capturing)`` on the CUDA device ``key``; ``(None, False)`` off CUDA."""
    if not isinstance(key, int):
        return None, False
    import torch

    with torch.cuda.device(key):
        if torch.cuda.is_current_stream_capturing():
            return None, True
        return torch.cuda.current_stream().cuda_stream, False


def take(op: str, role: str, shape: Sequence[int], dtype: Any, device: Any) -> Any:
    """A tensor of ``shape`` / ``dtype`` on ``device`` with undefined content: a view of the pooled buffer of
    ``(op, role)`` on the current stream, or a plain ``torch.empty`` when the pool does not serve the request."""
    import torch

    bound = config.option(None, "cake_workspace_pool_bytes")
    key, where = _locate(device)
    with _lock:
        pool = _pools.setdefault(key, _DevicePool())
        unpooled = not bound and not pool.buffers
        if unpooled:
            pool.misses += 1
    if unpooled:
        return torch.empty(shape, dtype=dtype, device=where)

    stream, capturing = _current_stream(key)
    if capturing:
        with _lock:
            pool.misses += 1
        return torch.empty(shape, dtype=dtype, device=where)

    nbytes = math.prod(shape) * dtype.itemsize
    slot = (op, role, stream)
    with _lock:
        buffer = pool.buffers.get(slot)
        if buffer is not None and nbytes <= buffer.numel() <= bound:
            pool.hits += 1
            pool.buffers.move_to_end(slot)
            pool.shrink_to(bound)
        else:
            pool.misses += 1
            if buffer is not None:  # too small, or larger than a bound that was lowered since
                del pool.buffers[slot]
            if nbytes <= 0 or nbytes > bound:
                pool.shrink_to(bound)
                return torch.empty(shape, dtype=dtype, device=where)
            pool.shrink_to(bound - nbytes)
            buffer = pool.buffers[slot] = torch.empty(nbytes, dtype=torch.uint8, device=where)
    flat = buffer[:nbytes]
    if dtype is not torch.uint8:
        flat = flat.view(dtype)
    return flat.view(shape)


def release(op: str | None = None) -> int:
    """Drop the pooled buffers of every op, or of ``op``, on every device and stream; returns the bytes dropped."""
    freed = 0
    with _lock:
        for pool in _pools.values():
            for slot in [slot for slot in pool.buffers if op is None or slot[0] == op]:
                freed += pool.buffers.pop(slot).numel()
    return freed


def stats() -> dict[Any, dict[str, int]]:
    """``{device: {"bytes", "entries", "hits", "misses", "evictions"}}``; ``device`` is the CUDA index."""
    with _lock:
        return {
            key: {
                "bytes": pool.held(),
                "entries": len(pool.buffers),
                "hits": pool.hits,
                "misses": pool.misses,
                "evictions": pool.evictions,
            }
            for key, pool in sorted(_pools.items(), key=lambda item: str(item[0]))
        }
