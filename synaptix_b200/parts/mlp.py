"""Dense gated feed-forward (SwiGLU): ``down( silu(x Wg^T) * (x Wu^T) )``,
``silu(x) = x / (1 + exp(-x))`` (crates/synaptix-models/llm/common/src/model.rs:1670-1691;
crates/synaptix-kernels-cuda/src/cu/fused/mlp/silu_and_mul.cu:11-25).  Gate and up
run as one product; the activation is computed in 32-bit.

``CappedGLU``: ``down( g sigmoid(alpha g) (u + 1) )`` with ``g = min(x Wg^T, limit)`` and
``u = clamp(x Wu^T, -limit, limit)``; ``alpha`` and ``limit`` are parameters.
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from .. import ops
from .base import FeedForward, Part, StepContext
from .linear import Linear


class SwiGLU(FeedForward):
    accepts_lazy_input = True      # x goes straight into the fused gate/up product
    can_defer_output = True        # the down projection may be handed on unrun

    def __init__(self, prefix: str, width: int, intermediate: int):
        self.width, self.intermediate = width, intermediate
        self.gate_up = Linear([prefix + "gate_proj.weight", prefix + "up_proj.weight"], width,
                              [intermediate, intermediate])
        self.down = Linear(prefix + "down_proj.weight", intermediate, width)

    def children(self) -> List[Part]:
        return [self.gate_up, self.down]

    def forward(self, x: torch.Tensor, ctx: StepContext, defer_output: bool = False) -> torch.Tensor:
        z = self.gate_up.forward(x, epilogue="silu_mul")
        return self.down.deferred(z) if defer_output else self.down.forward(z)


class CappedGLU(FeedForward):
    accepts_lazy_input = False
    can_defer_output = True

    NAMES = {"gate": "gate", "up": "up", "down": "down"}

    def __init__(self, prefix: str, width: int, intermediate: int, *, limit: float, alpha: float = 1.702,
                 names: Optional[Mapping[str, str]] = None):
        self.width, self.intermediate = width, intermediate
        self.limit, self.alpha = float(limit), float(alpha)
        n = dict(self.NAMES, **(names or {}))
        self.gate_up = Linear([prefix + n["gate"], prefix + n["up"]], width, [intermediate, intermediate])
        self.down = Linear(prefix + n["down"], intermediate, width)

    def children(self) -> List[Part]:
        return [self.gate_up, self.down]

    def forward(self, x: torch.Tensor, ctx: StepContext, defer_output: bool = False) -> torch.Tensor:
        with ops.gate_activation(self.alpha, self.limit):          # the gate/up product's epilogue applies it
            z = self.gate_up.forward(x, epilogue="silu_mul")
        return self.down.deferred(z) if defer_output else self.down.forward(z)
