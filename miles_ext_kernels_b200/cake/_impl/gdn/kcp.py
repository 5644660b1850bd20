"""Context parallelism of the GDN op: one packed batch split into contiguous token slices, one per rank of a process
group; the chunk state crosses rank boundaries.

:class:`KcpContext` is one rank's view of the partition (reference: miles_ext_kernels/cake/_impl/gdn/kcp.py:71-169):
``rank``, ``world_size``, ``num_tokens`` (this rank's), ``cu_seqlens`` / ``cu_seqlens_cpu`` (local boundaries: one
sequence per document fragment), ``layout``, ``group`` and ``fla_compatible``.  :func:`build_kcp_context` builds and
caches it (reference: kcp.py:185-226).

Contract under a context (FLA's): no ``initial_state``, no final state; tokens never move, only ``[HV, 128, 128]``
fp32 states.  Forward: the state at the end of this rank's last fragment goes to the next rank when the document
continues there; backward: the adjoint state at the start of this rank's first fragment goes to the previous rank.
States travel point to point on the group's backend (NCCL over NVLink between GPUs; gloo in the CPU tests) and land
in this GPU's own memory before any kernel reads them.

Only the ``"contiguous"`` layout is served; the load-balanced layouts of the reference (zigzag, per-document
zigzag, explicit fragments) raise ``NotImplementedError``.
"""

from __future__ import annotations

from collections import OrderedDict
from collections.abc import Sequence
from typing import Any

import torch

LAYOUTS = ("contiguous",)
_CACHE_LIMIT = 32
_CONTEXTS: OrderedDict[tuple[Any, ...], KcpContext] = OrderedDict()

__all__ = ["KcpContext", "build_kcp_context", "local_partition", "release"]


def local_partition(cu_global: Sequence[int], rank: int, world_size: int):
    """This rank's slice of a contiguous partition.

    Returns ``(local_cu, continues_in, continues_out)``: the local boundaries (starting at 0; one entry per document
    fragment that has tokens here), whether the first fragment continues a document begun on an earlier rank, and
    whether the last fragment's document continues on a later rank.  The token count must divide by the world size.
    """
    total = int(cu_global[-1])
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} is not in a world of {world_size}")
    if total % world_size:
        raise ValueError(f"a contiguous partition needs the token count ({total}) to divide by the world size "
                         f"({world_size})")
    part = total // world_size
    lo, hi = rank * part, (rank + 1) * part
    cuts = sorted({min(max(int(b), lo), hi) for b in cu_global} | {lo, hi})
    local = tuple(b - lo for b in cuts)
    bounds = set(int(b) for b in cu_global)
    continues_in = part > 0 and lo not in bounds
    continues_out = part > 0 and hi not in bounds
    return local, continues_in, continues_out


class _Exchange:
    """The state hand-over of one call: receive before the scan, send after it (forward: to the next rank; backward:
    to the previous one).  The hand-over is sequential along the rank chain, which reproduces the single-rank
    recurrence exactly."""

    def __init__(self, context: KcpContext) -> None:
        self.context = context

    def _peer(self, offset: int) -> int:
        import torch.distributed as dist

        ctx = self.context
        peer = ctx.rank + offset
        return peer if ctx.group is None else dist.get_global_rank(ctx.group, peer)

    def incoming_state(self, num_local_seqs: int, num_v_heads: int, device) -> torch.Tensor | None:
        """``h0 [N_local, HV, 128, 128]``: zero, except the first fragment's when its document began earlier."""
        ctx = self.context
        if not ctx.continues_in or ctx.world_size == 1:
            return None
        import torch.distributed as dist

        h0 = torch.zeros(num_local_seqs, num_v_heads, 128, 128, dtype=torch.float32, device=device)
        dist.recv(h0[0], src=self._peer(-1), group=ctx.group)
        return h0

    def outgoing_state(self, final_state: torch.Tensor) -> None:
        ctx = self.context
        if not ctx.continues_out or ctx.world_size == 1:
            return
        import torch.distributed as dist

        dist.send(final_state[-1].contiguous(), dst=self._peer(+1), group=ctx.group)

    def incoming_adjoint(self, num_local_seqs: int, num_v_heads: int, device) -> torch.Tensor | None:
        """``dht [N_local, HV, 128, 128]``: zero, except the last fragment's when its document continues later."""
        ctx = self.context
        if not ctx.continues_out or ctx.world_size == 1:
            return None
        import torch.distributed as dist

        dht = torch.zeros(num_local_seqs, num_v_heads, 128, 128, dtype=torch.float32, device=device)
        dist.recv(dht[-1], src=self._peer(+1), group=ctx.group)
        return dht

    def outgoing_adjoint(self, dh0: torch.Tensor) -> None:
        ctx = self.context
        if not ctx.continues_in or ctx.world_size == 1:
            return
        import torch.distributed as dist

        dist.send(dh0[0].contiguous(), dst=self._peer(-1), group=ctx.group)


class KcpContext:
    """One rank's view of a contiguous partition of a packed batch."""

    def __init__(self, cu_seqlens_global, group, rank: int, world_size: int, device, conv_kernel_size: int = 4,
                 layout: str = "contiguous", fragments=None) -> None:
        if layout not in LAYOUTS or fragments is not None:
            raise NotImplementedError(
                f"KcpContext: only the {LAYOUTS} layout without explicit fragments is served, not {layout!r}"
            )
        self.cu_seqlens_global = tuple(int(b) for b in cu_seqlens_global)
        if not self.cu_seqlens_global or self.cu_seqlens_global[0] != 0:
            raise ValueError("KcpContext: cu_seqlens_global must start at 0")
        self.group = group
        self.rank, self.world_size = int(rank), int(world_size)
        self.device = torch.device(device)
        self.conv_kernel_size = int(conv_kernel_size)
        self.layout = layout
        local, self.continues_in, self.continues_out = local_partition(self.cu_seqlens_global, self.rank,
                                                                       self.world_size)
        self.cu_seqlens_cpu = local
        self.num_tokens = local[-1]
        self.cu_seqlens = torch.tensor(local, dtype=torch.int32, device=self.device)
        self.fla_compatible = True  # a contiguous partition is FLA's

    def exchange(self) -> _Exchange:
        return _Exchange(self)

    def __repr__(self) -> str:
        return (f"KcpContext(rank={self.rank}, world_size={self.world_size}, num_tokens={self.num_tokens}, "
                f"layout={self.layout!r}, cu_seqlens_cpu={self.cu_seqlens_cpu})")


def build_kcp_context(cu_seqlens_global, group=None, *, device=None, conv_kernel_size: int = 4,
                      layout: str = "contiguous", fragments=None) -> KcpContext:
    """The :class:`KcpContext` of this process for the global boundaries ``cu_seqlens_global`` (a sequence of ints or
    a CPU tensor) and the process group ``group`` (default: the world).  Cached per layout, so every layer of a
    micro-batch shares one context."""
    import torch.distributed as dist

    if isinstance(cu_seqlens_global, torch.Tensor):
        if cu_seqlens_global.is_cuda:
            raise ValueError("build_kcp_context: cu_seqlens_global must be on the host (a tuple or a CPU tensor)")
        cu_seqlens_global = cu_seqlens_global.tolist()
    boundaries = tuple(int(b) for b in cu_seqlens_global)
    if dist.is_available() and dist.is_initialized():
        rank, world = dist.get_rank(group), dist.get_world_size(group)
    else:
        rank, world = 0, 1
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu"
    device = torch.device(device)
    key = (boundaries, id(group), rank, world, str(device), conv_kernel_size, layout)
    found = _CONTEXTS.get(key)
    if found is not None:
        _CONTEXTS.move_to_end(key)
        return found
    context = KcpContext(boundaries, group, rank, world, device, conv_kernel_size, layout, fragments)
    _CONTEXTS[key] = context
    while len(_CONTEXTS) > _CACHE_LIMIT:
        _CONTEXTS.popitem(last=False)
    return context


def release() -> None:
    _CONTEXTS.clear()
