"""mLSTM mixer: a recurrent layer whose memory per head is a matrix.

Per token, from the mixer's input ``h``: ``q = Wq h / sqrt(d)``, ``k = Wk h`` (heads x d),
``v = Wv h`` (heads x dv), and per head the log gates ``i = cap tanh((Wi h + bi) / cap)`` and
``f = logsigmoid(cap tanh((Wf h + bf) / cap))``.  With the running maximum ``m`` (from 0):
``m' = max(f + m, i)``, ``S' = exp(f + m - m') S + exp(i - m') k v^T``, ``n'`` the same with ``k``
alone, ``o = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)``.  Each head's ``o`` is divided by its root
mean square, the heads are concatenated, multiplied by a weight and by ``sigmoid(Wg h)``, and
projected by ``Wo`` into the residual stream.  ``S``, ``n`` and ``m`` start at zero, are 32-bit and
are the sequence's state; so are the gates and everything else that enters the recurrence.  The
six input projections are one matrix product with a 32-bit result.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .base import MIXERS, Mixer, ParamSpec, StateNeed


@MIXERS.register("mlstm")
class MLSTM(Mixer):
    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.d = int(p["head_dim"])
        self.dv = int(p["v_head_dim"])
        self.cap = float(p["gate_cap"])
        self.eps = float(p["eps"])
        H, d, dv = self.heads, self.d, self.dv
        self.proj_width = 2 * H * d + 2 * H * dv + 2 * H
        self.proj_ld = (self.proj_width + 7) // 8 * 8            # rows of the 32-bit result start on 32 bytes
        self.w_in = self.w_o = self.gate_bias = self.norm_weight = None

    def params(self) -> List[ParamSpec]:
        H, d, dv, W = self.heads, self.d, self.dv, self.hidden
        return [ParamSpec("q", (H * d, W)), ParamSpec("k", (H * d, W)), ParamSpec("v", (H * dv, W)), ParamSpec("g", (H * dv, W)),
                ParamSpec("o", (W, H * dv)), ParamSpec("norm", (H * dv,), kind="vector", init="ones"),
                ParamSpec("i", (H, W)), ParamSpec("i.b", (H,), kind="vector", init="zeros"),
                ParamSpec("f", (H, W)), ParamSpec("f.b", (H,), kind="vector", init="zeros")]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        t = tensors
        rows = [t["q"], t["k"], t["v"], t["g"], t["i"], t["f"]]
        if len({r.dtype for r in rows}) != 1:
            raise ValueError("mlstm: the input projections are stored in different dtypes")
        pad = self.proj_ld - self.proj_width
        if pad:
            rows.append(torch.zeros(pad, self.hidden, dtype=rows[0].dtype, device=rows[0].device))
        pack = self.ctx.ops.pack_weight
        self.w_in = pack(torch.cat(rows, dim=0).contiguous())
        self.w_o = pack(t["o"].contiguous())
        self.gate_bias = torch.cat([t["i.b"].reshape(-1), t["f.b"].reshape(-1)]).to(torch.float32).contiguous()
        self.norm_weight = t["norm"].reshape(-1).to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o))

    def state_need(self) -> Optional[StateNeed]:
        H, d, dv = self.heads, self.d, self.dv
        return StateNeed((H * d * dv + H * d + H,), torch.float32)

    def forward(self, h, residual, step, cache, state, append: bool):
        ops, ws, T, cap = self.ctx.ops, self.ctx.workspace, step.num_tokens, self.ctx.max_step_tokens
        H, d, dv = self.heads, self.d, self.dv
        proj = ws.buffer("mlstm.proj", (cap, self.proj_ld), torch.float32)[:T]
        ops.linear(h, self.w_in, proj)
        o = ws.buffer("mlstm.o", (cap, H * dv), torch.float32)[:T]
        ops.mlstm_scan(proj, self.gate_bias, self.cap, float(d) ** -0.5, state, step, o, H, d, dv)
        gated = ws.buffer("mlstm.gated", (cap, H * dv), self.ctx.dtype)[:T]
        ops.mlstm_output(o, proj[:, 2 * H * d + H * dv: 2 * H * d + 2 * H * dv], self.norm_weight, self.eps, gated, H, dv)
        ops.linear(gated, self.w_o, residual, accumulate=True)
