"""Dense feed-forward with one up and one down projection: ``residual += Wd act(Wu h)``.
Activations: ``relu2`` (the square of ``max(z, 0)``).  The up projection's result is kept in
32-bit until the activation has been applied, so the square sees unrounded values.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import FEED_FORWARDS, FeedForward, ParamSpec


@FEED_FORWARDS.register("dense")
class DenseFeedForward(FeedForward):
    ACTIVATIONS = ("relu2",)

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.activation = spec.get("activation", "relu2")
        if self.activation not in self.ACTIVATIONS:
            raise ValueError(f"dense feed-forward: activation {self.activation!r} ({', '.join(self.ACTIVATIONS)})")
        self.w_up = self.w_down = None

    def params(self) -> List[ParamSpec]:
        return [ParamSpec("up", (self.inter, self.hidden)), ParamSpec("down", (self.hidden, self.inter))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        pack = self.ctx.ops.pack_weight
        self.w_up, self.w_down = pack(tensors["up"].contiguous()), pack(tensors["down"].contiguous())

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_up, self.w_down))

    def forward(self, h, residual, step):
        ops, ws, T, cap = self.ctx.ops, self.ctx.workspace, step.num_tokens, self.ctx.max_step_tokens
        up = ws.buffer("dense_ffn.up", (cap, self.inter), torch.float32)[:T]
        ops.linear(h, self.w_up, up)
        act = ws.buffer("dense_ffn.act", (cap, self.inter), self.ctx.dtype)[:T]
        ops.relu2(up, act)
        ops.linear(act, self.w_down, residual, accumulate=True)
