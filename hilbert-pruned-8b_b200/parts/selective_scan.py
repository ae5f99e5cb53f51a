"""Selective state-space mixer (Mamba).

``W_in h = [x | z]`` (``inner`` each).  ``x`` passes a causal convolution per channel (``conv``
``[inner, taps]``, the last column the current token's, with bias ``conv.b``, zeros before the
sequence's start) and silu, giving ``u``.  ``W_x u = [dt_low (dt_rank) | B (state) | C (state)]``;
``dt = softplus(W_dt dt_low + dt.b)`` per channel; ``A = -exp(A_log)`` (``inner x state``).  Per
channel c and state index n: ``S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c u_c B_n`` and
``y_c = sum_n S[c, n] C_n + D_c u_c``; the mixer's result is ``W_o (y * silu(z))``.

32-bit: the results of ``W_x`` (B, C) and of ``W_dt``, the softplus, A, the exponentials, S, y and the
gate.  The step-size projection is a matrix product like the others: where the tensor-core product
takes its sizes (bfloat16, ``dt_rank`` a multiple of 8) ``W_x``'s low-rank rows form a product of their
own with a bfloat16 result that ``W_dt`` reads; otherwise ``W_dt`` reads the 32-bit low-rank values
through the general product.  The sequence's state is one flat run of 32-bit values
``[last taps - 1 convolution inputs | S]``, zero at the start.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .base import MIXERS, Mixer, ParamSpec, StateNeed


@MIXERS.register("selective_scan")
class SelectiveScan(Mixer):
    can_overwrite = True

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.inner = int(p["inner"])
        self.n_state = int(p["state"])
        self.dt_rank = int(p["dt_rank"])
        self.taps = int(p["conv"])
        if self.taps < 1:
            raise ValueError("selective_scan: at least one convolution tap")
        self.x_width = self.dt_rank + 2 * self.n_state
        self.x_ld = (self.x_width + 7) // 8 * 8
        self.conv_state = (self.taps - 1) * self.inner
        self.w_in = self.w_x = self.w_o = self.w_dt = self.b_dt = self.a_log = self.d_skip = self.conv_w = self.conv_b = None
        self.w_x_low = self.w_x_bc = None       # the two halves of W_x, when the step sizes run through the tensor-core products
        self.split_low_rank = ctx.dtype == torch.bfloat16 and self.dt_rank % 8 == 0 and self.inner % 8 == 0
        self.bc_ld = (2 * self.n_state + 7) // 8 * 8

    def params(self) -> List[ParamSpec]:
        I, N, R, W = self.inner, self.n_state, self.dt_rank, self.hidden
        return [ParamSpec("in", (2 * I, W)), ParamSpec("conv", (I, self.taps)), ParamSpec("conv.b", (I,), kind="vector", init="zeros"),
                ParamSpec("x", (R + 2 * N, I)), ParamSpec("dt", (I, R)), ParamSpec("dt.b", (I,), kind="vector", init="zeros"),
                ParamSpec("A_log", (I, N), init="zeros"), ParamSpec("D", (I,), kind="vector", init="ones"), ParamSpec("o", (W, I))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        t = tensors
        pack = self.ctx.ops.pack_weight
        f32 = lambda x: x.to(torch.float32).contiguous()
        self.w_in = pack(t["in"].contiguous())
        wx = t["x"]
        pad = lambda w, rows: torch.cat([w, torch.zeros(rows - w.shape[0], w.shape[1], dtype=w.dtype, device=w.device)], dim=0) if rows > w.shape[0] else w
        if self.split_low_rank:
            self.w_x_low = pack(wx[: self.dt_rank].contiguous())
            self.w_x_bc = pack(pad(wx[self.dt_rank:], self.bc_ld).contiguous())
        else:
            self.w_x = pack(pad(wx, self.x_ld).contiguous())
        self.w_o = pack(t["o"].contiguous())
        # (the general product reads the matrix as it is stored; only the tensor-core product wants it in tiles)
        self.w_dt, self.b_dt = (pack(t["dt"].contiguous()) if self.split_low_rank else t["dt"].contiguous()), f32(t["dt.b"].reshape(-1))
        self.a_log, self.d_skip = f32(t["A_log"]), f32(t["D"].reshape(-1))
        self.conv_w, self.conv_b = f32(t["conv"].reshape(self.inner, self.taps)), f32(t["conv.b"].reshape(-1))

    def weight_bytes(self) -> int:
        big = sum(w.numel() * w.element_size() for w in (self.w_in, self.w_x, self.w_x_low, self.w_x_bc, self.w_dt, self.w_o) if w is not None)
        return big + 4 * (self.a_log.numel() + self.conv_w.numel() + 3 * self.inner)

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.conv_state + self.inner * self.n_state,), torch.float32)

    def forward(self, h, residual, step, cache, state, append: bool, accumulate: bool = True):
        ops, ws, T, cap = self.ctx.ops, self.ctx.workspace, step.num_tokens, self.ctx.max_step_tokens
        I = self.inner
        xz = ws.buffer("selective_scan.xz", (cap, 2 * I), torch.float32)[:T]
        ops.linear(h, self.w_in, xz)
        u = ws.buffer("selective_scan.u", (cap, I), self.ctx.dtype)[:T]
        ops.conv_act(xz[:, :I], self.conv_w, self.conv_b, state[:, : self.conv_state], step, u, "silu")
        R, N = self.dt_rank, self.n_state
        dt_raw = ws.buffer("selective_scan.dt", (cap, I), torch.float32)[:T]
        if self.split_low_rank:
            low = ws.buffer("selective_scan.low", (cap, R), self.ctx.dtype)[:T]
            ops.linear(u, self.w_x_low, low)
            bc = ws.buffer("selective_scan.bc", (cap, self.bc_ld), torch.float32)[:T]
            ops.linear(u, self.w_x_bc, bc)
            ops.linear(low, self.w_dt, dt_raw)
            bc = bc[:, : 2 * N]
        else:
            dbc = ws.buffer("selective_scan.dbc", (cap, self.x_ld), torch.float32)[:T]
            ops.linear(u, self.w_x, dbc)
            ops.linear(dbc[:, :R], self.w_dt, dt_raw)
            bc = dbc[:, R: R + 2 * N]
        y = ws.buffer("selective_scan.y", (cap, I), self.ctx.dtype)[:T]
        ops.selective_scan(u, bc, xz[:, I:], dt_raw, self.b_dt, self.a_log, self.d_skip, state[:, self.conv_state:], step, y, N, workspace=ws)
        ops.linear(y, self.w_o, residual, accumulate=accumulate)
