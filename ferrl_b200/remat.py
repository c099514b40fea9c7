"""Activation rematerialisation: keep only segment boundaries, replay in backward.

A segment is a pure function of its boundary activation (plus closed-over
parameters).  Forward runs it without an autograd tape and keeps just the
boundary; backward replays the segment with a tape, takes the vector-Jacobian
product against the incoming cotangent and hands back the boundary cotangent
and the parameter gradients.  This is the same contract as the reference's
``RematTape`` + ``stitched_backward`` (``crates/ferrl/src/remat.rs:108-313``),
expressed as one ``torch.autograd.Function`` so it composes with ordinary
autograd above and below.

Under tensor parallelism a replayed segment re-issues its forward collectives
in the same order on every rank, and ``cot_transform`` (a sum-all-reduce) is
applied to the boundary cotangent before it flows to the previous segment
(reference ``remat.rs:172-264``, ``gemma4.rs:2136-2169``).
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch


class _RematSegment(torch.autograd.Function):
    @staticmethod
    def forward(ctx, fn, cot_transform, n_params, x, *params):
        ctx.fn = fn
        ctx.cot_transform = cot_transform
        ctx.save_for_backward(x, *params)
        with torch.no_grad():
            return fn(x)

    @staticmethod
    def backward(ctx, gout):
        x, *params = ctx.saved_tensors
        xin = x.detach().requires_grad_(True)
        with torch.enable_grad():
            out = ctx.fn(xin)
        wanted = [xin] + [p for p in params if p.requires_grad]
        grads = torch.autograd.grad(out, wanted, gout, allow_unused=True)
        gx = grads[0]
        if gx is not None and ctx.cot_transform is not None:
            gx = ctx.cot_transform(gx)
        it = iter(grads[1:])
        gp = [next(it) if p.requires_grad else None for p in params]
        return (None, None, None, gx, *gp)


def remat_segment(fn: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor,
                  params: Sequence[torch.Tensor],
                  cot_transform: Optional[Callable[[torch.Tensor], torch.Tensor]] = None) -> torch.Tensor:
    """Run ``fn(x)`` keeping only ``x``.  ``params`` are the trainable tensors
    ``fn`` reads (they must be listed so autograd routes their gradients)."""
    if not torch.is_grad_enabled():
        return fn(x)
    params = [p for p in params if p.requires_grad]
    if not x.requires_grad and not params:
        return fn(x)
    if not x.requires_grad:
        x = x.detach().requires_grad_(True)  # keeps the Function differentiable w.r.t. params
    return _RematSegment.apply(fn, cot_transform, len(params), x, *params)


class RematTape:
    """Explicit boundary list for callers that want to inspect what is kept
    (memory telemetry and tests)."""

    def __init__(self):
        self.boundaries: list[torch.Tensor] = []

    def capture(self, h: torch.Tensor) -> torch.Tensor:
        self.boundaries.append(h.detach())
        return h

    def bytes_held(self) -> int:
        return sum(b.numel() * b.element_size() for b in self.boundaries)
