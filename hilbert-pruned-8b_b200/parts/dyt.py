"""Dynamic tanh in the place of a norm: ``y = tanh(alpha * x) * w + b`` with a learned scalar
``alpha`` and vectors ``w`` and ``b``.  It takes no mean and no variance of ``x``, so it has no
epsilon and nothing to reduce over; computed in 32-bit, written in the dtype the next product
reads.  Tensor names below the part's prefix: the weight is the prefix itself, then ``.b`` and
``.alpha`` (a tensor without dimensions).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import NORMS, Norm, ParamSpec


@NORMS.register("dyt")
class DynamicTanh(Norm):
    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.size = int(spec.params["size"])
        self.weight = self.bias = self.alpha = None

    def params(self) -> List[ParamSpec]:
        return [ParamSpec("", (self.size,), kind="vector", init="ones"),
                ParamSpec(".b", (self.size,), kind="vector", init="zeros"),
                ParamSpec(".alpha", (), kind="vector", init="ones")]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        f32 = lambda t, n: t.reshape(n).to(torch.float32).contiguous()        # widened once, exactly
        self.weight, self.bias, self.alpha = f32(tensors[""], self.size), f32(tensors[".b"], self.size), f32(tensors[".alpha"], 1)

    def weight_bytes(self) -> int:
        return (2 * self.size + 1) * 4

    def forward(self, x, out, rows=None) -> None:
        """``out[i] = dyt(x[rows[i]])`` (``rows`` None: every row of ``x``)."""
        self.ctx.ops.dyt(x, self.weight, self.bias, self.alpha, out, rows)

    def as_arguments(self):
        """``(weight, bias, alpha)`` for a kernel that applies this norm to its own input."""
        return (self.weight, self.bias, self.alpha)
