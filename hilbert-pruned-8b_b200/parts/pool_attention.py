"""Grouped-query attention over a sliding window of tokens plus pooled summaries of what lies
before it, with sigmoid weights.

Per token: ``q, k, v = Wq h, Wk h, Wv h`` (no biases, no rotation: positions enter only through
what a query sees).  With ``qk_norm`` the token's whole query projection (all heads together) is
divided by its root mean square and multiplied by a weight of that size, the key projection
likewise.  ``k`` and ``v`` go to the cache.  A query at position p sees token j if
``0 <= p - j < window`` and, with ``pool = P``, one key and one value per block of P tokens that
lies wholly before the window (block e, tokens ``e P .. e P + P - 1``, is seen once
``e P + P - 1 <= p - window``): the mean of the block's keys and the mean of its values as the cache
holds them.  Tokens that have left the window while their block is still incomplete or not yet
wholly before the window are not seen.  The weight of a visible key is
``sigmoid(q . k * scale + bias[head])`` (``head_bias``), not normalised over the keys; the heads'
results are concatenated, multiplied element by element by ``sigmoid(Wg h)`` (``gate``) and
projected by ``Wo``.  The four input projections are one matrix product with a 32-bit result.

Storage: the token keys and values live in a windowed cache group that keeps ``max(window, P)``
tokens back (the newest block is averaged from it); the pooled ones in a second group with one
32-bit entry per block (``CacheNeed.stride``), filled as soon as a block's last token is cached.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .base import MIXERS, CacheNeed, Mixer, ParamSpec


@MIXERS.register("pool_attention")
class PoolAttention(Mixer):
    can_overwrite = True

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.v_dim = int(p.get("v_head_dim") or self.head_dim)
        self.scale = float(p["scale"]) if p.get("scale") is not None else float(self.head_dim) ** -0.5
        self.window: Optional[int] = int(p["window"]) if p.get("window") else None
        self.pool = int(p.get("pool") or 0)
        self.qk_norm = bool(p.get("qk_norm", False))
        self.eps = float(p.get("eps", 1e-6))
        self.head_bias = bool(p.get("head_bias", False))
        self.gate = bool(p.get("gate", False))
        if self.heads % self.kv_heads:
            raise ValueError("pool_attention: heads must be a multiple of kv heads")
        if self.pool and not self.window:
            raise ValueError("pool_attention: pooled blocks lie before a window; without a window every token is seen")
        self.q_width, self.k_width, self.v_width = self.heads * self.head_dim, self.kv_heads * self.head_dim, self.kv_heads * self.v_dim
        self.out_width = self.heads * self.v_dim
        self.gate_at = self.q_width + self.k_width + self.v_width
        self.proj_width = self.gate_at + (self.out_width if self.gate else 0)
        self.proj_ld = (self.proj_width + 7) // 8 * 8
        self.w_in = self.w_o = self.q_weight = self.k_weight = self.bias = None

    def params(self) -> List[ParamSpec]:
        W = self.hidden
        out = [ParamSpec("q", (self.q_width, W)), ParamSpec("k", (self.k_width, W)), ParamSpec("v", (self.v_width, W)),
               ParamSpec("o", (W, self.out_width))]
        if self.qk_norm:
            out += [ParamSpec("q.norm", (self.q_width,), kind="vector", init="ones"), ParamSpec("k.norm", (self.k_width,), kind="vector", init="ones")]
        if self.head_bias:
            out.append(ParamSpec("pb", (self.heads,), kind="vector", init="zeros"))
        if self.gate:
            out.append(ParamSpec("g", (self.out_width, W)))
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        t = tensors
        rows = [t["q"], t["k"], t["v"]] + ([t["g"]] if self.gate else [])
        if len({r.dtype for r in rows}) != 1:
            raise ValueError("pool_attention: the input projections are stored in different dtypes")
        if self.proj_ld > self.proj_width:
            rows.append(torch.zeros(self.proj_ld - self.proj_width, self.hidden, dtype=rows[0].dtype, device=rows[0].device))
        pack = self.ctx.ops.pack_weight
        self.w_in = pack(torch.cat(rows, dim=0).contiguous())
        self.w_o = pack(t["o"].contiguous())
        f32 = lambda x: x.reshape(-1).to(torch.float32).contiguous()
        if self.qk_norm:
            self.q_weight, self.k_weight = f32(t["q.norm"]), f32(t["k.norm"])
        if self.head_bias:
            self.bias = f32(t["pb"])

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o))

    def cache_need(self):
        if not self.pool:
            return CacheNeed(self.kv_heads, self.head_dim, self.window, v_head_dim=self.v_dim)
        return (CacheNeed(self.kv_heads, self.head_dim, max(self.window, self.pool), v_head_dim=self.v_dim),
                CacheNeed(self.kv_heads, self.head_dim, None, v_head_dim=self.v_dim, stride=self.pool, store_f32=True))

    def forward(self, h, residual, step, cache, state, append: bool, accumulate: bool = True):
        ops, ws, T, cap = self.ctx.ops, self.ctx.workspace, step.num_tokens, self.ctx.max_step_tokens
        H, G, d, dv = self.heads, self.kv_heads, self.head_dim, self.v_dim
        tokens, pooled = cache if self.pool else (cache, None)
        proj = ws.buffer("pool_attention.proj", (cap, self.proj_ld), torch.float32)[:T]
        ops.linear(h, self.w_in, proj)
        q = ws.buffer("pool_attention.q", (cap, self.q_width), self.ctx.dtype)[:T]
        ops.qk_norm_append(proj, self.q_weight, self.k_weight, self.eps, H, G, d, dv, q, tokens, step, append)
        if self.pool and append:
            ops.pool_blocks(tokens, pooled, step, self.pool, G, d, dv)
        attn = ws.buffer("pool_attention.out", (cap, self.out_width), self.ctx.dtype)[:T]
        gate = proj[:, self.gate_at: self.gate_at + self.out_width] if self.gate else None
        ops.attention_pool(q, tokens, pooled, step, self.bias, gate, attn, H, G, d, dv, self.scale, self.window, self.pool, workspace=ws)
        ops.linear(attn, self.w_o, residual, accumulate=accumulate)
