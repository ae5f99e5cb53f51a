"""Small Pogezen configurations and weights for the tests.

The weights are drawn so that every mechanism moves the logits: biases, gate biases, the
norm's offsets, the value-mixing scalar and the head-mixing matrix are all far from the
values that would switch them off (a zero bias or a unit matrix would hide a fault).  Stored in
bfloat16, so that a 32-bit engine and the 64-bit plain model read the same numbers.
"""
import json
import os

import torch


def attention(heads, kv_heads, dim, vdim, size, keep_first, rot_dims, scaling=None, v_mix=True, base=10000.0, scale=None):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5,
                      "v_mix": v_mix, "mask": {"size": size, "keep_first": keep_first},
                      "rot": {"base": base, "dims": rot_dims, "scaling": scaling}}}


def mlstm(heads, dim, vdim, cap=10.0):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def with_mlp(layer, ff):
    return dict(layer, mlp=None if ff is None else {"kind": "dense", "ff": ff})


def config(width, vocab, taps, layers, eps=1e-5, scale=0.7):
    return {"architecture": "Pogezen", "canon": {"taps": taps}, "embedding": {"scale": scale}, "layers": layers,
            "norm": {"eps": eps}, "vocab": vocab, "width": width}


YARN = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}

# both kinds of layer, with and without a feed-forward, a window that prompts pass
MIXED = config(64, 200, 3, [
    with_mlp(attention(4, 2, 16, 8, 40, 3, 8, YARN), 96),
    with_mlp(mlstm(2, 8, 16, 8.0), None),
    with_mlp(attention(4, 2, 16, 8, 40, 3, 8, YARN), None),
    with_mlp(mlstm(2, 8, 16, 8.0), 80)])
# sizes that are equal or 1 where the others differ: one head, as many kv heads as heads, no kept
# tokens, every dimension rotated, no scaling, no value mixing, a window longer than any prompt
EDGES = config(48, 130, 2, [
    with_mlp(mlstm(1, 16, 16, 15.0), 64),
    with_mlp(attention(2, 2, 8, 8, 20, 0, 8, None, v_mix=False, base=500.0), None),
    with_mlp(attention(3, 1, 16, 24, 1000, 5, 4, {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 2.0}, v_mix=True, scale=0.5), 56)],
    eps=1e-6, scale=1.0)
# no attention at all (no cache), a single tap (no convolution state), sizes that are no multiples of 8 or 32
RECURRENT = config(40, 90, 1, [with_mlp(mlstm(3, 24, 40, 6.0), None), with_mlp(mlstm(2, 12, 20, 12.0), 50)])
# widths the tensor-core products take (rows of a multiple of 64 bytes), two value-mixing layers with different windows
WIDE = config(128, 300, 4, [
    with_mlp(attention(4, 2, 32, 64, 70, 2, 16, {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 1.0}), 192),
    with_mlp(mlstm(2, 32, 64, 10.0), None),
    with_mlp(attention(4, 2, 32, 64, 33, 7, 32, None), 128)], scale=0.5)

# sixteen heads: the sizes whose weights-times-values product runs on the tensor cores in bfloat16
MANY_HEADS = config(128, 250, 2, [
    with_mlp(attention(16, 4, 16, 32, 45, 2, 8, YARN), 160),
    with_mlp(mlstm(4, 16, 32, 9.0), None),
    with_mlp(attention(16, 4, 16, 32, 45, 2, 8, YARN), None)], scale=0.6)

# head sizes of 64 and 128: the flash-style kernel for prompts in bfloat16 (kept tokens beyond a page, windows of odd sizes)
BIG_HEADS = config(128, 220, 3, [
    with_mlp(attention(4, 2, 64, 64, 70, 3, 32, YARN), 160),
    with_mlp(mlstm(2, 16, 32, 9.0), None),
    with_mlp(attention(2, 1, 128, 64, 97, 66, 64, None, v_mix=False), None),
    with_mlp(attention(4, 2, 64, 64, 1000, 0, 16, YARN), 96)], scale=0.6)

CONFIGS = {"big_heads": BIG_HEADS, "mixed": MIXED, "edges": EDGES, "recurrent": RECURRENT, "wide": WIDE, "many_heads": MANY_HEADS}


def draw_tensors(cfg, seed):
    """name -> bfloat16 tensor for every tensor the configuration's model reads."""
    import hilbert_pruned_8b_b200 as hb
    from hilbert_pruned_8b_b200.engine.model import weight_table
    table = weight_table(hb.PogezenConfig.from_dict(cfg).model_spec(), "")
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, spec in table.items():
        if spec.optional and name.startswith("lm_head"):
            continue
        shape = tuple(spec.shape)
        n = lambda std=1.0, mean=0.0: torch.randn(shape, generator=g) * std + mean
        leaf = name.split(".")[-1]
        if name.endswith(".alpha"):
            t = torch.rand(shape, generator=g) * 0.8 + 0.4
        elif name.endswith("vmix"):
            t = torch.rand(shape, generator=g) * 0.5 + 0.2
        elif name.endswith("talk"):
            t = torch.eye(shape[0]) + n(0.4)
        elif name.endswith("f.b"):
            t = n(1.0, 2.0)
        elif name.endswith(".b"):
            t = n(0.5)
        elif "canon" in leaf:
            t = n(0.4)
        elif leaf in ("norm", "norm1", "norm2"):
            t = n(0.2, 1.0)
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
