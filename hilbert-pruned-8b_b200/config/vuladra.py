"""Typed configuration of the Vuladra decoder: a stack whose layers each have a norm before and
after every sublayer, one of three mixers (attention over a window plus pooled blocks with sigmoid
weights; a softmax window attention beside a matrix memory with fixed decays; a selective
state-space scan), and a dense feed-forward, a mixture of experts, or none.

config.json keys (every size and every constant that may differ between models comes from here):
``architecture`` ("Vuladra"), ``vocab``, ``width``, ``norm.eps`` and ``layers``: a list of
``{"type", "mixer", "mlp"}`` with ``type``

* "attention": ``mixer`` = ``heads, kv_heads, dim, vdim, scale, mask {size, pool}``;
* "parallel": ``mixer`` = ``left {heads, kv_heads, dim, vdim, scale, mask {size}}``,
  ``right {heads, dim, vdim, decay [per head]}``, ``left_scale``, ``right_scale``;
* "mamba1": ``mixer`` = ``inner, state, dt_rank, conv``;

and ``mlp`` null, ``{"kind": "dense", "ff"}`` or ``{"kind": "moe", "router {experts, top}", "expert {ff,
limit}", "shared {ff, limit} | null"}``.  Tensor names: ``embed``, ``l<i>.norm1|norm1b|norm2|norm2b``,
``l<i>.mix.*`` (``left.*`` / ``right.*`` below it for the parallel mixer), ``l<i>.mlp.*``,
``final.norm``; the head is the embedding table.
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, PlanEntry


def _number(v: Any) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


def _int(d: Any, key: str, where: str, least: int = 1) -> int:
    v = d.get(key) if isinstance(d, dict) else None
    if not _number(v) or v != math.floor(v) or v < least or v > 1e9:
        raise ConfigError(f"config: missing or bad {where}{key}")
    return int(v)


def _float(d: Any, key: str, where: str) -> float:
    v = d.get(key) if isinstance(d, dict) else None
    if not _number(v) or not math.isfinite(v):
        raise ConfigError(f"config: missing or bad {where}{key}")
    return float(v)


def _heads(m: Any, where: str, kv: bool) -> Dict[str, Any]:
    out = {"heads": _int(m, "heads", where), "dim": _int(m, "dim", where), "vdim": _int(m, "vdim", where)}
    if kv:
        out["kv_heads"] = _int(m, "kv_heads", where)
        if out["heads"] % out["kv_heads"]:
            raise ConfigError(f"config: {where}heads is no multiple of kv_heads")
        out["scale"] = _float(m, "scale", where)
    return out


def _mlp(mlp: Any, where: str) -> Optional[Dict[str, Any]]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"config: {where}kind must be dense or moe (or mlp null)")
    if mlp["kind"] == "dense":
        return {"kind": "dense", "ff": _int(mlp, "ff", where)}
    router, expert, shared = mlp.get("router"), mlp.get("expert"), mlp.get("shared")
    out = {"kind": "moe",
           "router": {"experts": _int(router, "experts", where + "router."), "top": _int(router, "top", where + "router.")},
           "expert": {"ff": _int(expert, "ff", where + "expert."), "limit": _float(expert, "limit", where + "expert.")},
           "shared": None}
    if out["router"]["top"] > out["router"]["experts"]:
        raise ConfigError(f"config: {where}router.top is larger than router.experts")
    if shared is not None:
        out["shared"] = {"ff": _int(shared, "ff", where + "shared."), "limit": _float(shared, "limit", where + "shared.")}
    return out


@dataclass(frozen=True)
class VuladraConfig:
    vocab: int
    width: int
    eps: float
    layers: List[Dict[str, Any]] = field(default_factory=list)       # the validated entries of config.json
    eos_token_ids: List[int] = field(default_factory=list)
    max_position_embeddings: Optional[int] = None

    architecture = "Vuladra"
    model_type = "vuladra"

    # llama-style names that the generic entry points and the benchmark read
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, root: Dict[str, Any]) -> "VuladraConfig":
        if not isinstance(root, dict):
            raise ConfigError("config: config.json is not an object")
        vocab, width = _int(root, "vocab", ""), _int(root, "width", "")
        eps = _float(root.get("norm"), "eps", "norm.")
        raw = root.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config: layers must be a list with at least one entry")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(entry, dict) or entry.get("type") not in ("attention", "parallel", "mamba1"):
                raise ConfigError(f"config: {where}type must be attention, parallel or mamba1")
            m = entry.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config: missing {where}mixer")
            mw = where + "mixer."
            if entry["type"] == "attention":
                mixer = _heads(m, mw, kv=True)
                mask = m.get("mask")
                mixer["mask"] = {"size": _int(mask, "size", mw + "mask.")}
                if isinstance(mask, dict) and mask.get("pool") is not None:
                    mixer["mask"]["pool"] = _int(mask, "pool", mw + "mask.")
            elif entry["type"] == "parallel":
                left = _heads(m.get("left"), mw + "left.", kv=True)
                left["mask"] = {"size": _int(m["left"].get("mask"), "size", mw + "left.mask.")}
                right = _heads(m.get("right"), mw + "right.", kv=False)
                decay = m["right"].get("decay")
                if not isinstance(decay, list) or len(decay) != right["heads"] or not all(_number(x) and 0.0 <= x <= 1.0 for x in decay):
                    raise ConfigError(f"config: {mw}right.decay must give a number in [0, 1] per head")
                right["decay"] = [float(x) for x in decay]
                mixer = {"left": left, "right": right, "left_scale": _float(m, "left_scale", mw), "right_scale": _float(m, "right_scale", mw)}
            else:
                mixer = {"inner": _int(m, "inner", mw), "state": _int(m, "state", mw), "dt_rank": _int(m, "dt_rank", mw),
                         "conv": _int(m, "conv", mw)}
            layers.append({"type": entry["type"], "mixer": mixer, "mlp": _mlp(entry.get("mlp"), where + "mlp.")})
        eos = root.get("eos_token_id")
        eos_ids = [int(eos)] if _number(eos) else [int(e) for e in eos if _number(e)] if isinstance(eos, list) else []
        for e in eos_ids:
            if not 0 <= e < vocab:
                raise ConfigError(f"config: eos_token_id {e} is outside the vocabulary")
        max_pos = root.get("max_position_embeddings")
        return cls(vocab=vocab, width=width, eps=eps, layers=layers, eos_token_ids=eos_ids,
                   max_position_embeddings=int(max_pos) if _number(max_pos) and max_pos >= 1 else None)

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "layers": copy.deepcopy(self.layers), "norm": {"eps": self.eps},
                             "vocab": self.vocab, "width": self.width}
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        if self.max_position_embeddings is not None:
            d["max_position_embeddings"] = self.max_position_embeddings
        return d

    # ------------------------------------------------------------------ model description
    def model_spec(self) -> ModelSpec:
        W = self.width
        norm = PartSpec("rmsnorm", {"size": W, "eps": self.eps, "tensor_name": ""})
        layers: List[LayerSpec] = []
        for i, l in enumerate(self.layers):
            m = l["mixer"]
            if l["type"] == "attention":
                mixer = PartSpec("pool_attention", {
                    "hidden_size": W, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_head_dim": m["vdim"],
                    "scale": m["scale"], "window": m["mask"]["size"], "pool": m["mask"].get("pool"), "qk_norm": True, "eps": self.eps,
                    "head_bias": True, "gate": True})
            elif l["type"] == "parallel":
                a, b = m["left"], m["right"]
                left = PartSpec("sink_attention", {
                    "hidden_size": W, "num_heads": a["heads"], "num_kv_heads": a["kv_heads"], "head_dim": a["dim"], "v_head_dim": a["vdim"],
                    "window": a["mask"]["size"], "keep_first": 0, "scale": a["scale"], "bias": False, "qk_unit_norm": False, "talk": False,
                    "v_mix": None, "position": None})
                right = PartSpec("decay_memory", {"hidden_size": W, "num_heads": b["heads"], "head_dim": b["dim"], "v_head_dim": b["vdim"],
                                                  "decay": tuple(b["decay"]), "eps": self.eps, "activation": "silu"})
                mixer = PartSpec("parallel", {"hidden_size": W, "branches": (
                    {"prefix": "left.", "mixer": left, "scale": m["left_scale"]},
                    {"prefix": "right.", "mixer": right, "scale": m["right_scale"]})})
            else:
                mixer = PartSpec("selective_scan", {"hidden_size": W, "inner": m["inner"], "state": m["state"], "dt_rank": m["dt_rank"],
                                                    "conv": m["conv"]})
            parts = {"mixer_norm": norm, "mixer": mixer, "mixer_post_norm": norm}
            prefixes = {"mixer_norm": "norm1", "mixer": "mix.", "mixer_post_norm": "norm1b"}
            f = l["mlp"]
            if f is not None:
                if f["kind"] == "dense":
                    ff = PartSpec("swiglu", {"hidden_size": W, "intermediate_size": f["ff"], "tensor_names": ("gate", "up", "down")})
                else:
                    shared = f["shared"]
                    ff = PartSpec("moe", {"hidden_size": W, "num_experts": f["router"]["experts"], "top": f["router"]["top"],
                                          "expert_size": f["expert"]["ff"], "limit": f["expert"]["limit"], "alpha": 1.702,
                                          "shared_size": shared["ff"] if shared else 0,
                                          "shared_limit": shared["limit"] if shared else f["expert"]["limit"]})
                parts.update({"feed_forward_norm": norm, "feed_forward": ff, "feed_forward_post_norm": norm})
                prefixes.update({"feed_forward_norm": "norm2", "feed_forward": "mlp.", "feed_forward_post_norm": "norm2b"})
            layers.append(LayerSpec(prefix=f"l{i}.", block="sandwich", parts=parts, part_prefixes=prefixes))
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=W, vocab_size=self.vocab, layers=layers,
            plan=[PlanEntry(i) for i in range(len(layers))],
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": W, "tensor_name": "embed"}),
            final_norm=norm,
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": W, "tied": True}),
            weight_prefixes=[""], embedding_prefix="", final_norm_prefix="final.norm", head_prefix="lm_head.",
            stop_token_ids=list(self.eos_token_ids), max_position=self.max_position_embeddings)
        spec.validate()
        return spec
