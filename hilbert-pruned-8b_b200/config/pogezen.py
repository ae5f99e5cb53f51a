"""Typed configuration of the Pogezen decoder: a stack whose layers are either attention with a
sliding window that keeps the first tokens, or an mLSTM matrix memory, each behind a dynamic-tanh
norm and a short causal convolution, some followed by a dense feed-forward.

config.json keys (every size and every constant that may differ between models comes from here):
``architecture`` ("Pogezen"), ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``,
``canon.taps`` and ``layers``: a list of ``{"type", "mixer", "mlp"}`` with ``type`` "attention"
(``mixer``: ``heads, kv_heads, dim, vdim, scale, v_mix, mask {size, keep_first}, rot {base, dims,
scaling {factor, original, fast, slow} | null}``) or "mlstm" (``mixer``: ``heads, dim, vdim,
gate_cap``), and ``mlp`` null or ``{"kind": "dense", "ff"}``.  Tensor names: ``embed``,
``l<i>.norm1|norm2[.b|.alpha]``, ``l<i>.canon1``, ``l<i>.mix.*``, ``l<i>.mlp.up|down``,
``final.norm[.b|.alpha]``; the head is the embedding table.
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


def _int(d: Dict[str, Any], key: str, where: str, least: int = 1) -> int:
    v = d.get(key) if isinstance(d, dict) else None
    if not _number(v) or v != math.floor(v) or v < least or v > 1e9:
        raise ConfigError(f"config: missing or bad {where}{key}")
    return int(v)


def _float(d: Dict[str, Any], key: str, where: str) -> float:
    v = d.get(key) if isinstance(d, dict) else None
    if not _number(v) or not math.isfinite(v):
        raise ConfigError(f"config: missing or bad {where}{key}")
    return float(v)


@dataclass(frozen=True)
class PogezenConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    taps: int
    layers: List[Dict[str, Any]] = field(default_factory=list)       # the validated entries of config.json
    eos_token_ids: List[int] = field(default_factory=list)
    max_position_embeddings: Optional[int] = None

    architecture = "Pogezen"
    model_type = "pogezen"

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
    def from_dict(cls, root: Dict[str, Any]) -> "PogezenConfig":
        if not isinstance(root, dict):
            raise ConfigError("config: config.json is not an object")
        vocab, width = _int(root, "vocab", ""), _int(root, "width", "")
        eps = _float(root.get("norm"), "eps", "norm.")
        scale = _float(root.get("embedding"), "scale", "embedding.")
        taps = _int(root.get("canon"), "taps", "canon.")
        raw = root.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config: layers must be a list with at least one entry")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(entry, dict) or entry.get("type") not in ("attention", "mlstm"):
                raise ConfigError(f"config: {where}type must be attention or mlstm")
            m = entry.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config: missing {where}mixer")
            mw = where + "mixer."
            if entry["type"] == "attention":
                mixer = {"heads": _int(m, "heads", mw), "kv_heads": _int(m, "kv_heads", mw), "dim": _int(m, "dim", mw),
                         "vdim": _int(m, "vdim", mw), "scale": _float(m, "scale", mw), "v_mix": bool(m.get("v_mix", False))}
                if mixer["heads"] % mixer["kv_heads"]:
                    raise ConfigError(f"config: {mw}heads is no multiple of kv_heads")
                mask = m.get("mask")
                mixer["mask"] = {"size": _int(mask, "size", mw + "mask."), "keep_first": _int(mask, "keep_first", mw + "mask.", 0)}
                rot = m.get("rot")
                dims = _int(rot, "dims", mw + "rot.", 0)
                if dims % 2 or dims > mixer["dim"]:
                    raise ConfigError(f"config: {mw}rot.dims must be even and at most dim")
                r = {"base": _float(rot, "base", mw + "rot."), "dims": dims, "scaling": None}
                sc = rot.get("scaling")
                if sc is not None:
                    r["scaling"] = {k: _float(sc, k, mw + "rot.scaling.") for k in ("factor", "original", "fast", "slow")}
                mixer["rot"] = r
            else:
                mixer = {"heads": _int(m, "heads", mw), "dim": _int(m, "dim", mw), "vdim": _int(m, "vdim", mw),
                         "gate_cap": _float(m, "gate_cap", mw)}
                if mixer["gate_cap"] <= 0:
                    raise ConfigError(f"config: {mw}gate_cap must be positive")
            mlp = entry.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config: {where}mlp.kind must be dense (or mlp null)")
                mlp = {"kind": "dense", "ff": _int(mlp, "ff", where + "mlp.")}
            layers.append({"type": entry["type"], "mixer": mixer, "mlp": mlp})
        eos = root.get("eos_token_id")
        eos_ids = [int(eos)] if _number(eos) else [int(e) for e in eos if _number(e)] if isinstance(eos, list) else []
        for e in eos_ids:
            if not 0 <= e < vocab:
                raise ConfigError(f"config: eos_token_id {e} is outside the vocabulary")
        max_pos = root.get("max_position_embeddings")
        return cls(vocab=vocab, width=width, eps=eps, embedding_scale=scale, taps=taps, layers=layers, eos_token_ids=eos_ids,
                   max_position_embeddings=int(max_pos) if _number(max_pos) and max_pos >= 1 else None)

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "canon": {"taps": self.taps},
                             "embedding": {"scale": self.embedding_scale}, "layers": copy.deepcopy(self.layers),
                             "norm": {"eps": self.eps}, "vocab": self.vocab, "width": self.width}
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        if self.max_position_embeddings is not None:
            d["max_position_embeddings"] = self.max_position_embeddings
        return d

    # ------------------------------------------------------------------ model description
    def model_spec(self) -> ModelSpec:
        W = self.width
        norm = PartSpec("dyt", {"size": W})
        conv = PartSpec("short_conv", {"size": W, "taps": self.taps})
        first_mix = next((i for i, l in enumerate(self.layers) if l["type"] == "attention" and l["mixer"]["v_mix"]), None)
        layers: List[LayerSpec] = []
        for i, l in enumerate(self.layers):
            m = l["mixer"]
            if l["type"] == "attention":
                rot = m["rot"]
                position = None
                if rot["dims"] > 0:
                    rp: Dict[str, Any] = {"head_dim": m["dim"], "rotary_dim": rot["dims"], "theta": rot["base"], "frequencies_in_64_bit": True}
                    if rot["scaling"] is not None:
                        rp["yarn"] = dict(rot["scaling"])
                    position = PartSpec("rotary", rp)
                mixer = PartSpec("sink_attention", {
                    "hidden_size": W, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                    "v_head_dim": m["vdim"], "window": m["mask"]["size"], "keep_first": m["mask"]["keep_first"],
                    "scale": m["scale"], "bias": True, "qk_unit_norm": True, "eps": self.eps, "talk": True,
                    "v_mix": None if not m["v_mix"] else ("first" if i == first_mix else "mix"), "v_mix_key": "pogezen",
                    "position": position})
            else:
                mixer = PartSpec("mlstm", {"hidden_size": W, "num_heads": m["heads"], "head_dim": m["dim"],
                                           "v_head_dim": m["vdim"], "gate_cap": m["gate_cap"], "eps": self.eps})
            parts = {"mixer_norm": norm, "mixer_filter": conv, "mixer": mixer}
            prefixes = {"mixer_norm": "norm1", "mixer_filter": "canon1", "mixer": "mix."}
            if l["mlp"] is not None:
                parts["feed_forward_norm"] = norm
                parts["feed_forward"] = PartSpec("dense", {"hidden_size": W, "intermediate_size": l["mlp"]["ff"], "activation": "relu2"})
                prefixes.update({"feed_forward_norm": "norm2", "feed_forward": "mlp."})
            layers.append(LayerSpec(prefix=f"l{i}.", block="prenorm_filtered", parts=parts, part_prefixes=prefixes))
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=W, vocab_size=self.vocab, layers=layers,
            plan=[PlanEntry(i) for i in range(len(layers))],
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": W, "scale": self.embedding_scale,
                                             "tensor_name": "embed"}),
            final_norm=norm,
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": W, "tied": True}),
            weight_prefixes=[""], embedding_prefix="", final_norm_prefix="final.norm", head_prefix="lm_head.",
            stop_token_ids=list(self.eos_token_ids), max_position=self.max_position_embeddings)
        spec.validate()
        return spec
