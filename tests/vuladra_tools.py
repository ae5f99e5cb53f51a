"""Small Vuladra configurations and weights for the tests.

The weights are drawn so that every mechanism moves the logits: the norms on the sublayers'
outputs are far from zero, the per-head score biases, step-size biases, skip weights and
convolution biases are far from the values that would switch them off, and the router's logits
are spread out so that no choice of experts is a close call.  Stored in bfloat16, so that a 32-bit
engine and the 64-bit plain model read the same numbers.
"""
import json
import os

import torch


def attention(heads, kv_heads, dim, vdim, size, pool, scale=None):
    mask = {"size": size}
    if pool:
        mask["pool"] = pool
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                           "scale": scale if scale is not None else dim ** -0.5, "mask": mask}}


def parallel(left, right, left_scale=1.2, right_scale=0.9):
    heads, kv_heads, dim, vdim, size = left
    h2, d2, dv2, decay = right
    return {"type": "parallel", "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5, "mask": {"size": size}},
        "right": {"heads": h2, "dim": d2, "vdim": dv2, "decay": list(decay)}, "left_scale": left_scale, "right_scale": right_scale}}


def mamba(inner, state, dt_rank, conv):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, shared=None):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit},
            "shared": None if shared is None else {"ff": shared[0], "limit": shared[1]}}


def with_mlp(layer, mlp):
    return dict(layer, mlp=mlp)


def config(width, vocab, layers, eps=1e-5):
    return {"architecture": "Vuladra", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}


# every kind of mixer and of feed-forward; windows and pooled blocks that prompts pass; sizes that are no multiples of 8
MIXED = config(64, 200, [
    with_mlp(mamba(96, 8, 5, 3), dense(80)),
    with_mlp(attention(4, 2, 16, 8, 20, 6), moe(6, 2, 24, 1.5, (40, 1.0))),
    with_mlp(parallel((4, 2, 16, 16, 30), (2, 8, 16, (0.7, 0.98))), None),
    with_mlp(mamba(72, 20, 3, 4), moe(5, 3, 20, 2.5))])
# sizes that are equal or 1 where the others differ: one head, as many kv heads as heads, a window of one token, blocks of one
# token, one expert chosen, every expert chosen, one state value, step sizes of rank one, a single tap (no convolution state),
# a window longer than any prompt (no pooled block is ever seen), a decay of one (nothing is forgotten) and of zero
EDGES = config(48, 130, [
    with_mlp(attention(1, 1, 8, 12, 1, 1, scale=0.4), moe(3, 3, 16, 0.7, (8, 3.0))),
    with_mlp(mamba(40, 1, 1, 1), None),
    with_mlp(parallel((2, 2, 8, 4, 1000), (1, 4, 4, (1.0,)), 0.5, 1.5), moe(4, 1, 16, 1.0)),
    with_mlp(attention(3, 3, 4, 4, 1000, 7), dense(24)),
    with_mlp(parallel((3, 1, 8, 8, 1), (3, 8, 4, (0.0, 0.5, 0.9))), None)], eps=1e-6)
# widths the tensor-core products take; head sizes of 64 and 128 (the tensor-core prompt kernels of both kinds of attention);
# blocks that straddle page borders (48 does not divide 64), a window shorter than a block, state sizes above 32
WIDE = config(128, 300, [
    with_mlp(mamba(256, 40, 16, 4), moe(8, 2, 64, 2.0, (64, 1.5))),
    with_mlp(attention(4, 2, 64, 64, 33, 48), dense(192)),
    with_mlp(parallel((2, 1, 64, 64, 70), (2, 32, 64, (0.9, 0.999))), moe(8, 3, 32, 1.0)),
    with_mlp(attention(2, 1, 32, 64, 100, 16), None),
    with_mlp(parallel((2, 2, 128, 64, 40), (4, 16, 16, (0.5, 0.8, 0.95, 0.99))), dense(64))])
# recurrent layers only (no cache at all)
RECURRENT = config(40, 90, [with_mlp(mamba(56, 6, 4, 2), dense(48)), with_mlp(mamba(24, 33, 2, 5), None)])

CONFIGS = {"mixed": MIXED, "edges": EDGES, "wide": WIDE, "recurrent": RECURRENT}


def draw_tensors(cfg, seed):
    """name -> bfloat16 tensor for every tensor the configuration's model reads."""
    import hilbert_pruned_8b_b200 as hb
    from hilbert_pruned_8b_b200.engine.model import weight_table
    table = weight_table(hb.VuladraConfig.from_dict(cfg).model_spec(), "")
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, spec in table.items():
        if spec.optional and name.startswith("lm_head"):
            continue
        shape = tuple(spec.shape)
        n = lambda std=1.0, mean=0.0: torch.randn(shape, generator=g) * std + mean
        leaf = name.split(".")[-1]
        if leaf in ("norm1b", "norm2b"):
            t = n(0.15, 0.6)
        elif leaf in ("norm", "norm1", "norm2"):
            t = n(0.2, 1.0)
        elif leaf == "pb":
            t = n(1.0, -0.5)
        elif leaf == "A_log":
            t = torch.log(torch.rand(shape, generator=g) * 3.0 + 0.3)
        elif name.endswith("dt.b"):
            t = n(0.8, -1.5)
        elif leaf == "D":
            t = n(0.3, 1.0)
        elif name.endswith("conv.b"):
            t = n(0.3)
        elif leaf == "conv":
            t = n(0.5)
        elif leaf == "router":
            t = n(4.0 / shape[1] ** 0.5)
        elif name == "embed":
            t = n(1.0)
        elif len(shape) == 2:
            t = n(1.0 / shape[1] ** 0.5)
        else:
            t = n(1.0)
        out[name] = t.to(torch.bfloat16)
    return out


def write_model(folder, cfg, seed):
    from hilbert_pruned_8b_b200.weights.safetensors_io import write_safetensors
    os.makedirs(folder, exist_ok=True)
    tensors = draw_tensors(cfg, seed)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    return tensors
