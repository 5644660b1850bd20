"""Forward + backward of the gated-delta-rule ops for callers whose tensors live in HOST memory.

The ops' sequences are independent of one another, so a call whose operands sit in pinned host memory does not have to
wait for all of them to cross PCIe before the first kernel runs: :class:`HostPipeline` cuts the call into parts (batch
rows, or runs of whole sequences of a packed call), and keeps three streams busy at once --

    copy-in stream     part p+1's operands, host -> device
    compute stream     part p through the op's public entry point (forward and backward)
    copy-out stream    part p-1's output and gradients, device -> host

PCIe is full duplex, so with enough parts a step costs about max(bytes in, bytes out) / link bandwidth instead of the
sum of both copies and the kernels.  The results are the bits of the undivided call: a sequence's chunks never mix
with another sequence's.

The reference has no host-memory entry point (its callers hold device tensors); this one exists for embedding the
kernels behind a C ABI whose callers hold host buffers, and it is what the benchmark's end-to-end figure times.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Sequence

import torch

__all__ = ["Part", "HostPipeline", "batch_parts", "packed_parts"]


@dataclass(frozen=True)
class Part:
    """One slice of a call: ``rows`` of the leading dimension and ``tokens`` of the second; for a packed call the
    sequences ``seqs`` it holds and their boundaries relative to the slice."""

    rows: slice
    tokens: slice
    seqs: slice
    cu_seqlens: tuple[int, ...] | None = None


def batch_parts(batch: int, parts: int | None = None) -> list[Part]:
    """Parts of a ``[B, T, ...]`` call: runs of batch rows, ``parts`` of them (default: one per row)."""
    if batch < 1:
        raise ValueError(f"batch_parts: batch must be positive, got {batch}")
    n = min(batch, parts or batch)
    edges = [round(i * batch / n) for i in range(n + 1)]
    return [Part(slice(a, b), slice(None), slice(a, b)) for a, b in zip(edges, edges[1:]) if b > a]


def packed_parts(cu_seqlens: Sequence[int], parts: int) -> list[Part]:
    """Parts of a packed ``[1, S, ...]`` call: runs of whole sequences holding about ``S / parts`` tokens each."""
    cu = [int(x) for x in cu_seqlens]
    if len(cu) < 2 or cu[0] != 0 or any(b < a for a, b in zip(cu, cu[1:])):
        raise ValueError("packed_parts: cu_seqlens must start at 0 and not decrease")
    total, n = cu[-1], len(cu) - 1
    out, first = [], 0
    for p in range(1, parts + 1):
        goal = total * p / parts
        last = first
        while last < n and (cu[last + 1] <= goal or last == first):
            last += 1
        if p == parts:
            last = n
        if last > first:
            base = cu[first]
            out.append(Part(slice(0, 1), slice(base, cu[last]), slice(first, last),
                            tuple(x - base for x in cu[first:last + 1])))
            first = last
        if first >= n:
            break
    return out


class HostPipeline:
    """Runs ``step(part, operands on the device) -> outputs on the device`` over the parts of a call whose operands
    are pinned host tensors, and lands every output in pinned host memory.

    ``per_token`` names the operands (and ``token_outputs`` the indices of the outputs) that are sliced by rows and
    tokens; every other operand / output is per sequence (initial states, their gradients, final states) and is
    sliced by ``Part.seqs`` along its first dimension.

    Device staging buffers and host landing buffers are allocated once, on the first call, and reused; a part's
    staging buffers are not overwritten before the kernels that read them in the previous call have finished.
    """

    def __init__(self, device: torch.device, parts: Sequence[Part], per_token: Sequence[str]):
        if not parts:
            raise ValueError("HostPipeline: no parts")
        self.device = device
        self.parts = list(parts)
        self.per_token = frozenset(per_token)
        self.copy_in = torch.cuda.Stream(device)
        self.copy_out = torch.cuda.Stream(device)
        self._staging: list[dict[str, torch.Tensor]] | None = None
        self._consumed: list[torch.cuda.Event] = [torch.cuda.Event() for _ in self.parts]
        self._landing: list[torch.Tensor] | None = None
        self._landed: torch.cuda.Event | None = None

    def _cut(self, name: str, t: torch.Tensor, part: Part) -> torch.Tensor:
        return t[part.rows, part.tokens] if name in self.per_token else t[part.seqs]

    def run(self, host: dict[str, torch.Tensor], step: Callable[[Part, dict[str, torch.Tensor]], Sequence[torch.Tensor]],
            token_outputs: Sequence[int], total: tuple[int, int, int]) -> list[torch.Tensor]:
        """``total = (rows, tokens, sequences)`` of the whole call sizes the landing buffers.  Returns the landing
        buffers (pinned host tensors); they are complete once the calling stream's work is done
        (``torch.cuda.current_stream().synchronize()``)."""
        for name, t in host.items():
            if t.device.type != "cpu" or not t.is_pinned():
                raise ValueError(f"HostPipeline: operand {name!r} must be a pinned host tensor")
        main = torch.cuda.current_stream(self.device)
        if self._staging is None:
            self._staging = [
                {n: torch.empty(self._cut(n, t, p).shape, dtype=t.dtype, device=self.device) for n, t in host.items()}
                for p in self.parts
            ]
        if self._landed is not None:  # the previous call's results may still be on their way into the landing buffers
            self.copy_out.wait_event(self._landed)
        token_set = frozenset(token_outputs)
        rows, tokens, seqs = total
        ready: list[torch.cuda.Event] = []
        with torch.cuda.stream(self.copy_in):
            for p, part in enumerate(self.parts):
                self.copy_in.wait_event(self._consumed[p])
                for n, t in host.items():
                    self._staging[p][n].copy_(self._cut(n, t, part), non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.copy_in)
                ready.append(ev)
        for p, part in enumerate(self.parts):
            main.wait_event(ready[p])
            outs = list(step(part, self._staging[p]))
            self._consumed[p].record(main)
            done = torch.cuda.Event()
            done.record(main)
            if self._landing is None:
                shapes = []
                for i, x in enumerate(outs):
                    lead = (rows, tokens) if i in token_set else (seqs,)
                    shapes.append(lead + tuple(x.shape[len(lead):]))
                self._landing = [torch.empty(s, dtype=x.dtype, pin_memory=True) for s, x in zip(shapes, outs)]
            with torch.cuda.stream(self.copy_out):
                self.copy_out.wait_event(done)
                for i, x in enumerate(outs):
                    dst = self._landing[i]
                    dst = dst[part.rows, part.tokens] if i in token_set else dst[part.seqs]
                    dst.copy_(x.detach(), non_blocking=True)
                    x.record_stream(self.copy_out)
        self._landed = torch.cuda.Event()
        self._landed.record(self.copy_out)
        main.wait_event(self._landed)
        return self._landing
