"""A plain, slow Pogezen decoder: the oracle of the tests.

One function per mechanism, written from the design's equations in torch on the CPU (float64
unless another dtype is asked for); it shares no code with the library.  ``PlainPogezen`` keeps the
whole history of a sequence and recomputes nothing cleverly: attention looks at every earlier
key through an explicit mask, the matrix memory is a token-by-token loop, the short convolution
reads the earlier inputs from a list.

Notation: ``x`` residual stream, ``h`` what a mixer reads, ``P`` softmax weights, ``S, n, m`` the
matrix memory, its normaliser and the running maximum of the log gates.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def dyt(x, w, b, alpha):
    """Dynamic tanh: tanh(alpha x) w + b (no statistics of x)."""
    return torch.tanh(alpha * x) * w + b


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def causal_conv(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """conv(h)[t] = sum_j w[:, j] h[t - taps + 1 + j], zeros before the start.  h [T, C], w [C, taps]."""
    T, C = h.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=h.dtype), h], 0)
    out = torch.zeros_like(h)
    for j in range(taps):
        out = out + w[:, j] * padded[j: j + T]
    return out


def yarn_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(frequency per pair [dims/2], amplitude that multiplies cos and sin)."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, amplitude: float, dims: int) -> torch.Tensor:
    """x [T, heads, dim]: the pair (i, i + dims/2) of every head is turned by positions * freq[i]."""
    half = dims // 2
    a = positions.to(x.dtype)[:, None] * freq.to(x.dtype)[None, :]
    c, s = (torch.cos(a) * amplitude)[:, None, :], (torch.sin(a) * amplitude)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def visible(n: int, size: int, keep_first: int) -> torch.Tensor:
    """[n, n] mask: query i sees key j if j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def talking_attention(q, k, v, talk, scale: float, size: int, keep_first: int):
    """q [T, H, d], k [T, G, d], v [T, G, dv], talk [H, H] -> [T, H, dv].
    P_g = softmax of head g's masked scores; head h uses sum_g talk[h, g] P_g on the values of
    ITS key/value head."""
    T, H, _ = q.shape
    G = k.shape[1]
    group = H // G
    mask = visible(T, size, keep_first)
    P = []
    for g in range(H):
        s = (q[:, g] @ k[:, g // group].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        P.append(torch.softmax(s, -1))
    P = torch.stack(P, 0)                                   # [H, T, T]
    mixed = torch.einsum("hg,gij->hij", talk, P)
    return torch.stack([mixed[h] @ v[:, h // group] for h in range(H)], 1)


def mlstm_scan(q, k, v, log_i, log_f):
    """The matrix memory, token by token.  q, k [T, H, d] (q already scaled), v [T, H, dv],
    log_i, log_f [T, H].  S, n and m start at zero."""
    T, H, d = q.shape
    dv = v.shape[2]
    S = torch.zeros(H, d, dv, dtype=q.dtype)
    n = torch.zeros(H, d, dtype=q.dtype)
    m = torch.zeros(H, dtype=q.dtype)
    out = []
    for t in range(T):
        m_new = torch.maximum(log_f[t] + m, log_i[t])
        keep = torch.exp(log_f[t] + m - m_new)
        take = torch.exp(log_i[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        m = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out.append(num / den[:, None])
    return torch.stack(out, 0)                               # [T, H, dv]


def soft_cap(z, cap: float):
    return cap * torch.tanh(z / cap)


class PlainPogezen:
    def __init__(self, config: dict, tensors: Dict[str, torch.Tensor], dtype=torch.float64, round_to=None):
        """``round_to`` (torch.bfloat16): what a matrix product reads, and the cached keys and values,
        are rounded to that type first, as a library that serves in it does; all else stays ``dtype``."""
        self.c = config
        self.dtype = dtype
        self.round_to = round_to
        self.w = {n: t.to(dtype) for n, t in tensors.items()}
        self.eps = float(config["norm"]["eps"])
        self.taps = int(config["canon"]["taps"])
        self.mix_layers = [i for i, l in enumerate(config["layers"]) if l["type"] == "attention" and l["mixer"].get("v_mix")]

    def r(self, x):
        return x if self.round_to is None else x.to(self.round_to).to(self.dtype)

    def norm(self, x, name):
        return dyt(x, self.w[name], self.w[name + ".b"], self.w[name + ".alpha"])

    def attention(self, i: int, h, positions, shared):
        w, p = self.w, self.c["layers"][i]["mixer"]
        pre = f"l{i}.mix."
        H, G, d, dv = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
        T = h.shape[0]
        q = (h @ w[pre + "q"].T + w[pre + "q.b"]).view(T, H, d)
        k = (h @ w[pre + "k"].T + w[pre + "k.b"]).view(T, G, d)
        v = (h @ w[pre + "v"].T + w[pre + "v.b"]).view(T, G, dv)
        rot = p["rot"]
        freq, amp = yarn_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
        q = self.r(rms_unit(rotate(q, positions, freq, amp, int(rot["dims"])), self.eps))
        k = self.r(rms_unit(rotate(k, positions, freq, amp, int(rot["dims"])), self.eps))
        if p.get("v_mix"):
            if i == self.mix_layers[0]:
                shared["v_first"] = v
            else:
                lam = w[pre + "vmix"]
                v = (1.0 - lam) * v + lam * shared["v_first"]
        v = self.r(v)
        o = talking_attention(q, k, v, w[pre + "talk"], float(p["scale"]), int(p["mask"]["size"]), int(p["mask"]["keep_first"]))
        return self.r(o.reshape(T, H * dv)) @ w[pre + "o"].T + w[pre + "o.b"]

    def mlstm(self, i: int, h):
        w, p = self.w, self.c["layers"][i]["mixer"]
        pre = f"l{i}.mix."
        H, d, dv, cap = p["heads"], p["dim"], p["vdim"], float(p["gate_cap"])
        T = h.shape[0]
        q = (h @ w[pre + "q"].T).view(T, H, d) * d ** -0.5
        k = (h @ w[pre + "k"].T).view(T, H, d)
        v = (h @ w[pre + "v"].T).view(T, H, dv)
        log_i = soft_cap(h @ w[pre + "i"].T + w[pre + "i.b"], cap)
        log_f = torch.nn.functional.logsigmoid(soft_cap(h @ w[pre + "f"].T + w[pre + "f.b"], cap))
        o = rms_unit(mlstm_scan(q, k, v, log_i, log_f), self.eps).reshape(T, H * dv)
        o = o * w[pre + "norm"] * torch.sigmoid(h @ w[pre + "g"].T)
        return self.r(o) @ w[pre + "o"].T

    def feed_forward(self, i: int, h):
        w = self.w
        return self.r(torch.relu(h @ w[f"l{i}.mlp.up"].T) ** 2) @ w[f"l{i}.mlp.down"].T

    def forward(self, tokens: List[int], return_layers: bool = False):
        """Logits [T, vocab] of one sequence from its first token on."""
        w = self.w
        T = len(tokens)
        positions = torch.arange(T)
        x = w["embed"][torch.tensor(tokens)] * float(self.c["embedding"]["scale"])
        shared, layers = {}, []
        for i, layer in enumerate(self.c["layers"]):
            h = self.norm(x, f"l{i}.norm1")
            h = self.r(h + causal_conv(h, w[f"l{i}.canon1"]))
            x = x + (self.attention(i, h, positions, shared) if layer["type"] == "attention" else self.mlstm(i, h))
            if layer.get("mlp") is not None:
                x = x + self.feed_forward(i, self.r(self.norm(x, f"l{i}.norm2")))
            layers.append(x)
        logits = self.r(self.norm(x, "final.norm")) @ w["embed"].T
        return (logits, torch.stack(layers, 0)) if return_layers else logits
