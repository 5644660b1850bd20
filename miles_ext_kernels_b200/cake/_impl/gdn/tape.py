"""Keeping a forward's tape on an autograd node.

Every tensor the backward reads -- inputs, intermediates, the kernels' status word, boundary states -- goes through
``ctx.save_for_backward`` (as the reference's autograd function does; reference:
miles_ext_kernels/cake/_impl/gdn/ops.py:1953), so that autograd's version counters catch an in-place write to an
operand between forward and backward, and ``torch.autograd.graph.saved_tensors_hooks`` (activation checkpointing, CPU
offload) see the whole tape.  Only non-tensor metadata stays on the node as plain attributes.
"""

from __future__ import annotations

import dataclasses
from typing import Any

import torch

__all__ = ["keep", "restore"]


def keep(ctx: Any, tape: Any, **extra: torch.Tensor | None) -> None:
    """Save the tensor fields of the dataclass ``tape`` and the ``extra`` tensors on ``ctx``; remember the rest."""
    names: list[str] = []
    tensors: list[torch.Tensor] = []
    plain: dict[str, Any] = {}
    for field in dataclasses.fields(tape):
        value = getattr(tape, field.name)
        if isinstance(value, torch.Tensor):
            names.append(field.name)
            tensors.append(value)
        else:
            plain[field.name] = value
    extras = []
    for name, value in extra.items():
        if value is not None:
            extras.append(name)
            tensors.append(value)
    ctx.save_for_backward(*tensors)
    ctx.tape_layout = (type(tape), tuple(names), plain, tuple(extras), tuple(extra))


def restore(ctx: Any) -> tuple[Any, dict[str, torch.Tensor | None]]:
    """``(tape, extra)`` as :func:`keep` took them (unpacked through any active saved-tensor hooks)."""
    cls, names, plain, extras, all_extra = ctx.tape_layout
    saved = ctx.saved_tensors
    values = dict(plain)
    values.update(zip(names, saved[: len(names)]))
    extra: dict[str, torch.Tensor | None] = dict.fromkeys(all_extra)
    extra.update(zip(extras, saved[len(names):]))
    return cls(**values), extra
