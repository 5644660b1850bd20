"""``tape.keep`` / ``tape.restore`` on the CPU: the tensors of a dataclass go through ``save_for_backward`` (version
checks and saved-tensor hooks apply), everything else stays on the node."""

from __future__ import annotations

from dataclasses import dataclass

import pytest
import torch

from miles_ext_kernels_b200.cake._impl.gdn import tape as tape_module


@dataclass
class _Tape:
    x: torch.Tensor
    hidden: torch.Tensor
    absent: torch.Tensor | None
    factor: float


class _Square(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias):
        tape_module.keep(ctx, _Tape(x, x * 3.0, None, 2.0), bias=bias, nothing=None)
        return x * x

    @staticmethod
    def backward(ctx, grad):
        tape, extra = tape_module.restore(ctx)
        assert tape.absent is None and tape.factor == 2.0 and extra["nothing"] is None
        assert torch.equal(tape.hidden, tape.x * 3.0) and extra["bias"] is not None
        return grad * tape.factor * tape.x, None


def test_round_trip_and_gradient():
    x = torch.arange(4.0, requires_grad=True)
    _Square.apply(x, torch.ones(1)).sum().backward()
    assert torch.equal(x.grad, 2.0 * torch.arange(4.0))


def test_an_inplace_write_after_forward_is_caught():
    x = torch.arange(4.0, requires_grad=True)
    y = x * 1.0
    out = _Square.apply(y, torch.ones(1)).sum()
    with torch.no_grad():
        y.add_(1.0)
    with pytest.raises(RuntimeError, match="modified by an inplace operation"):
        out.backward()


def test_saved_tensor_hooks_see_every_tensor():
    seen = []
    x = torch.arange(4.0, requires_grad=True)
    with torch.autograd.graph.saved_tensors_hooks(lambda t: (seen.append(t.shape), t)[1], lambda t: t):
        out = _Square.apply(x, torch.ones(1)).sum()
    out.backward()
    assert len(seen) == 3  # x, hidden, bias
