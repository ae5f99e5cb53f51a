"""Mixture of experts with a clamped gated unit, and an optional shared expert.

Router: ``z = W_router h`` in 32-bit; the ``top`` experts with the largest logits are chosen per
token and weighted by the softmax over the chosen logits alone.  Expert (no biases):
``g = min(W_gate h, limit)``, ``u = clamp(W_up h, -limit, limit)``, ``y = g sigmoid(alpha g) (u + 1)``,
output ``W_down y``; ``alpha`` is 1.702 unless the spec says otherwise.  The layer's result is the
weighted sum of the chosen experts' outputs, plus the shared expert's (same form, own sizes and
limit), which runs for every token.

Tensors below the part's prefix: ``router``, ``e<i>.gate|up|down``, ``shared.gate|up|down``.  The
experts' matrices are stacked at load time; the routed products gather their rows on the device
from a plan that a kernel makes, so a step reads nothing back and decode steps can be captured.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import FEED_FORWARDS, FeedForward, ParamSpec


@FEED_FORWARDS.register("moe")
class MixtureOfExperts(FeedForward):
    can_overwrite = True

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.n_experts = int(p["num_experts"])
        self.top = int(p["top"])
        self.ff = int(p["expert_size"])
        self.limit = float(p["limit"])
        self.alpha = float(p.get("alpha", 1.702))
        self.shared_ff = int(p.get("shared_size") or 0)
        self.shared_limit = float(p.get("shared_limit", self.limit))
        if not 1 <= self.top <= self.n_experts:
            raise ValueError(f"moe: top {self.top} of {self.n_experts} experts")
        self.w_router = self.w_gate = self.w_up = self.w_down = self.ws_gate_up = self.ws_down = None

    def params(self) -> List[ParamSpec]:
        W, F = self.hidden, self.ff
        out = [ParamSpec("router", (self.n_experts, W))]
        for e in range(self.n_experts):
            out += [ParamSpec(f"e{e}.gate", (F, W)), ParamSpec(f"e{e}.up", (F, W)), ParamSpec(f"e{e}.down", (W, F))]
        if self.shared_ff:
            S = self.shared_ff
            out += [ParamSpec("shared.gate", (S, W)), ParamSpec("shared.up", (S, W)), ParamSpec("shared.down", (W, S))]
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        t, E = tensors, self.n_experts
        self.w_router = t["router"].to(torch.float32).contiguous()
        self.w_gate = torch.stack([t[f"e{e}.gate"] for e in range(E)]).contiguous()
        self.w_up = torch.stack([t[f"e{e}.up"] for e in range(E)]).contiguous()
        self.w_down = torch.stack([t[f"e{e}.down"] for e in range(E)]).contiguous()
        if self.shared_ff:
            pack = self.ctx.ops.pack_weight
            self.ws_gate_up = pack(torch.cat([t["shared.gate"], t["shared.up"]], dim=0).contiguous())
            self.ws_down = pack(t["shared.down"].contiguous())

    def weight_bytes(self) -> int:
        # what a decode step of one token reads: the router, `top` experts, the shared expert
        per = 3 * self.ff * self.hidden * self.w_gate.element_size()
        shared = sum(w.numel() * w.element_size() for w in (self.ws_gate_up, self.ws_down)) if self.shared_ff else 0
        return self.w_router.numel() * 4 + self.top * per + shared

    def forward(self, h, residual, step, accumulate: bool = True):
        ops, ws, T, cap = self.ctx.ops, self.ctx.workspace, step.num_tokens, self.ctx.max_step_tokens
        experts = ws.buffer("moe.experts", (cap, self.top), torch.int32)[:T]
        weights = ws.buffer("moe.weights", (cap, self.top), torch.float32)[:T]
        ops.moe_route(h, self.w_router, self.top, experts, weights)
        ops.moe_experts(h, experts, weights, self.w_gate, self.w_up, self.w_down, self.limit, self.alpha, residual, accumulate, ws, cap)
        if self.shared_ff:
            S = self.shared_ff
            gu = ws.buffer("moe.shared_gate_up", (cap, 2 * S), torch.float32)[:T]
            ops.linear(h, self.ws_gate_up, gu)
            act = ws.buffer("moe.shared_act", (cap, S), self.ctx.dtype)[:T]
            ops.glu_clamp(gu, act, self.shared_limit, self.alpha)
            ops.linear(act, self.ws_down, residual, accumulate=True)
