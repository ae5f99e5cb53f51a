"""A short causal convolution over time on what a mixer reads: ``h <- h + conv(h)`` with
``conv(h)[t] = sum_j w[:, j] * h[t - taps + 1 + j]`` per channel, zeros before a sequence's first
token.  The last ``taps - 1`` inputs of every sequence are its state (32-bit), carried from
step to step, so a prompt cut anywhere gives the same values.  The weight ``[channels, taps]`` is
the tensor named by the part's prefix itself; there is no bias.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .base import TOKEN_FILTERS, ParamSpec, StateNeed, TokenFilter


@TOKEN_FILTERS.register("short_conv")
class ShortConvolution(TokenFilter):
    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.size = int(spec.params["size"])
        self.taps = int(spec.params["taps"])
        if self.taps < 1:
            raise ValueError("short_conv: at least one tap")
        self.weight = None

    def params(self) -> List[ParamSpec]:
        return [ParamSpec("", (self.size, self.taps))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[""].reshape(self.size, self.taps).to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.size * self.taps * 4

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed(((self.taps - 1) * self.size,), torch.float32) if self.taps > 1 else None

    def fuses_norm(self, norm) -> bool:
        return hasattr(norm, "as_arguments") and getattr(norm, "size", None) == self.size

    def forward(self, x, out, step, state, norm=None) -> None:
        """``out = h + conv(h)``; ``x`` is ``h`` (32-bit), or with ``norm`` the residual stream."""
        if state is None:           # a single tap keeps nothing
            state = torch.empty((1, 0), dtype=torch.float32, device=x.device)
        self.ctx.ops.short_conv(x, self.weight, state, step, out, norm.as_arguments() if norm is not None else None)
