"""A plain, slow Vuladra decoder: the oracle of the tests.

One function per mechanism, written from the design's equations in torch on the CPU (float64
unless another dtype is asked for); it shares no code with the library.  ``PlainVuladra`` feeds a
whole sequence at once and recomputes everything from the first token: attention through an
explicit mask over tokens and pooled blocks, the recurrent layers as token-by-token loops.

Notation: ``x`` residual stream, ``h`` what a sublayer reads, ``S`` a recurrent state, ``P`` the
tokens of a pooled block, ``w`` the size of a window.  With ``round_to`` the values are rounded
where the library rounds them in bfloat16 (what a matrix product reads, cached keys and values).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def window_mask(n: int, w: int) -> torch.Tensor:
    """[n, n]: query i sees token j if 0 <= i - j < w."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return (j <= i) & (i - j < w)


def pooled_mask(n: int, w: int, P: int) -> torch.Tensor:
    """[n, n // P]: query i sees block b if the block's last token b P + P - 1 <= i - w."""
    i = torch.arange(n)[:, None]
    b = torch.arange(n // P)[None, :]
    return b * P + P - 1 <= i - w


def pool_blocks(t: torch.Tensor, P: int) -> torch.Tensor:
    """t [n, ...] -> [n // P, ...]: the mean of each whole block of P tokens."""
    n = t.shape[0] // P
    return t[: n * P].reshape((n, P) + tuple(t.shape[1:])).mean(1)


def sigmoid_pool_attention(q, k, v, bias, scale: float, w: int, P: Optional[int]):
    """q [T, H, d], k [T, G, d], v [T, G, dv], bias [H] -> [T, H, dv].  The weight of a visible key is
    sigmoid(q . k * scale + bias[h]); nothing is normalised over the keys.  Visible: the last w tokens
    and, with P, the mean key and value of every block of P tokens that lies wholly before them."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    keys, vals, mask = k, v, window_mask(T, w)
    if P:
        keys = torch.cat([pool_blocks(k, P), k], 0)
        vals = torch.cat([pool_blocks(v, P), v], 0)
        mask = torch.cat([pooled_mask(T, w, P), mask], 1)
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // rep
        s = q[:, h] @ keys[:, g].T * scale + bias[h]
        wgt = torch.sigmoid(s) * mask.to(q.dtype)
        out[:, h] = wgt @ vals[:, g]
    return out


def softmax_window_attention(q, k, v, scale: float, w: int):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]: softmax over the last w tokens."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    mask = window_mask(T, w)
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // rep
        s = (q[:, h] @ k[:, g].T * scale).masked_fill(~mask, float("-inf"))
        out[:, h] = torch.softmax(s, -1) @ v[:, g]
    return out


def decayed_memory(q, k, v, decay):
    """q, k [T, H, d], v [T, H, dv], decay [H] -> [T, H, dv]: S_t = decay S_{t-1} + k_t v_t^T, o_t = S_t^T q_t."""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[2], dtype=q.dtype)
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def causal_conv_bias(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """y[t] = b + sum_j w[:, j] x[t - taps + 1 + j], zeros before the start.  x [T, C], w [C, taps]."""
    T, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], 0)
    out = b.expand(T, C).clone()
    for j in range(taps):
        out = out + w[:, j] * padded[j: j + T]
    return out


def selective_scan(u, dt, A, B, C, D):
    """u, dt [T, I], A [I, N], B, C [T, N], D [I] -> y [T, I]:
    S <- exp(dt A) S + dt u B,  y = S C + D u  per channel."""
    T, I = u.shape
    S = torch.zeros(I, A.shape[1], dtype=u.dtype)
    y = torch.zeros(T, I, dtype=u.dtype)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * u[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + D * u[t]
    return y


def clamped_glu(h, wg, wu, wd, limit: float, r=lambda t: t):
    """W_d y with g = min(W_g h, limit), u = clamp(W_u h, -limit, limit), y = g sigmoid(1.702 g) (u + 1)."""
    g = torch.clamp(h @ wg.T, max=limit)
    u = torch.clamp(h @ wu.T, -limit, limit)
    return r(g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ wd.T


def route(z: torch.Tensor, top: int):
    """z [T, E] -> (experts [T, top], weights [T, top]): the largest logits, softmax over them alone."""
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, -1)


class PlainVuladra:
    def __init__(self, config: dict, tensors: Dict[str, torch.Tensor], dtype=torch.float64, round_to=None):
        self.cfg = config
        self.dtype = dtype
        self.w = {n: (t.to(dtype) if t.is_floating_point() else t) for n, t in tensors.items()}
        self.eps = float(config["norm"]["eps"])
        self.round_to = round_to
        self.trace: List[torch.Tensor] = []

    def r(self, t):
        return t if self.round_to is None else t.to(self.round_to).to(self.dtype)

    # ------------------------------------------------------------------ mixers
    def attention(self, p: str, m: dict, h):
        w, T = self.w, h.shape[0]
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        hr = self.r(h)
        q = rms_norm(hr @ w[p + "q"].T, w[p + "q.norm"], self.eps)
        k = rms_norm(hr @ w[p + "k"].T, w[p + "k.norm"], self.eps)
        v = hr @ w[p + "v"].T
        q, k, v = self.r(q).view(T, H, d), self.r(k).view(T, G, d), self.r(v).view(T, G, dv)
        o = sigmoid_pool_attention(q, k, v, w[p + "pb"], float(m["scale"]), int(m["mask"]["size"]), m["mask"].get("pool"))
        o = o.reshape(T, H * dv) * torch.sigmoid(hr @ w[p + "g"].T)
        return self.r(o) @ w[p + "o"].T

    def parallel(self, p: str, m: dict, h):
        w, T = self.w, h.shape[0]
        hr = self.r(h)
        a, b = m["left"], m["right"]
        H, G, d, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
        q = self.r(hr @ w[p + "left.q"].T).view(T, H, d)
        k = self.r(hr @ w[p + "left.k"].T).view(T, G, d)
        v = self.r(hr @ w[p + "left.v"].T).view(T, G, dv)
        left = self.r(softmax_window_attention(q, k, v, float(a["scale"]), int(a["mask"]["size"])).reshape(T, H * dv)) @ w[p + "left.o"].T
        H2, d2, dv2 = b["heads"], b["dim"], b["vdim"]
        q2 = silu(hr @ w[p + "right.q"].T).view(T, H2, d2)
        k2 = silu(hr @ w[p + "right.k"].T).view(T, H2, d2)
        v2 = silu(hr @ w[p + "right.v"].T).view(T, H2, dv2)
        o = decayed_memory(q2, k2, v2, torch.tensor(b["decay"], dtype=self.dtype)).reshape(T, H2 * dv2)
        o = rms_norm(o, w[p + "right.norm"], self.eps) * torch.sigmoid(hr @ w[p + "right.g"].T)
        right = self.r(o) @ w[p + "right.o"].T
        return float(m["left_scale"]) * left + float(m["right_scale"]) * right

    def mamba1(self, p: str, m: dict, h):
        w = self.w
        I, N, R = m["inner"], m["state"], m["dt_rank"]
        xz = self.r(h) @ w[p + "in"].T
        x, z = xz[:, :I], xz[:, I:]
        u = self.r(silu(causal_conv_bias(x, w[p + "conv"], w[p + "conv.b"])))
        dbc = u @ w[p + "x"].T
        dt = softplus(dbc[:, :R] @ w[p + "dt"].T + w[p + "dt.b"])
        y = selective_scan(u, dt, -torch.exp(w[p + "A_log"]), dbc[:, R:R + N], dbc[:, R + N:R + 2 * N], w[p + "D"])
        return self.r(y * silu(z)) @ w[p + "o"].T

    # ------------------------------------------------------------------ feed-forwards
    def feed_forward(self, p: str, f: dict, h):
        w = self.w
        hr = self.r(h)
        if f["kind"] == "dense":
            return self.r(silu(hr @ w[p + "gate"].T) * (hr @ w[p + "up"].T)) @ w[p + "down"].T
        E, top = f["router"]["experts"], f["router"]["top"]
        idx, wgt = route(hr @ w[p + "router"].T, top)
        out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=self.dtype)
        limit = float(f["expert"]["limit"])
        for e in range(E):
            rows, slot = (idx == e).nonzero(as_tuple=True)
            if rows.numel():
                y = clamped_glu(hr[rows], w[f"{p}e{e}.gate"], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"], limit, self.r)
                out[rows] += wgt[rows, slot][:, None] * y
        if f.get("shared"):
            out = out + clamped_glu(hr, w[p + "shared.gate"], w[p + "shared.up"], w[p + "shared.down"], float(f["shared"]["limit"]), self.r)
        return out

    # ------------------------------------------------------------------ the stack
    def hidden(self, tokens) -> torch.Tensor:
        w = self.w
        x = w["embed"][torch.as_tensor(list(tokens), dtype=torch.long)]
        self.trace = []
        for i, layer in enumerate(self.cfg["layers"]):
            p = f"l{i}."
            h = rms_norm(x, w[p + "norm1"], self.eps)
            y = getattr(self, layer["type"])(p + "mix.", layer["mixer"], h)
            x = x + rms_norm(y, w[p + "norm1b"], self.eps)
            if layer.get("mlp") is not None:
                h = rms_norm(x, w[p + "norm2"], self.eps)
                x = x + rms_norm(self.feed_forward(p + "mlp.", layer["mlp"], h), w[p + "norm2b"], self.eps)
            self.trace.append(x)
        return x

    def logits(self, tokens) -> torch.Tensor:
        """[len(tokens), vocab]: the logits at every position."""
        x = self.hidden(tokens)
        return self.r(rms_norm(x, self.w["final.norm"], self.eps)) @ self.w["embed"].T


def generate_greedy(model: PlainVuladra, prompt, n: int) -> List[int]:
    toks, out = list(prompt), []
    for _ in range(n):
        t = int(torch.argmax(model.logits(toks)[-1]))
        out.append(t)
        toks.append(t)
    return out
