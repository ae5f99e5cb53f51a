"""The Pogezen decoder against the plain implementation (tests/plain_pogezen.py): every mechanism
alone, then the engine: whole prompts, token-by-token decoding, prompts in portions, unequal
batches with slots and pages used again, windows' edges, long decoding, greedy generation through
the library's entry point and the replay program."""
import json
import math
import os

import pytest
import torch

import pogezen_tools as pt
import trace_tools as tt
from conftest import require_gpu
from plain_pogezen import (PlainPogezen, causal_conv, dyt, mlstm_scan, rms_unit, rotate, soft_cap, talking_attention, visible,
                           yarn_frequencies)

DTYPES = ["float32", "bfloat16"]
NAMES = ["mixed", "edges", "recurrent", "wide", "many_heads", "big_heads"]


# --------------------------------------------------------------------------- helpers
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (folder, config, {dtype: plain model}); the bfloat16 one rounds where the library does"""
    out = {}
    for i, (name, cfg) in enumerate(pt.CONFIGS.items()):
        d = str(tmp_path_factory.mktemp("pogezen_" + name))
        tensors = pt.write_model(d, cfg, 40 + i)
        out[name] = (d, cfg, {"float32": PlainPogezen(cfg, tensors), "bfloat16": PlainPogezen(cfg, tensors, round_to=torch.bfloat16)})
    return out


def _engine(folder, dtype, max_tokens, **kw):
    from hilbert_pruned_8b_b200.engine.step import Engine
    return Engine.from_folder(folder, dtype, max_tokens=max_tokens, **kw)


def _reference(plain, requests):
    ref = {}
    for rid, toks in requests.items():
        lg = plain.forward(toks)
        for p in range(len(toks)):
            ref[(rid, p)] = lg[p]
    return ref


# Fixed bounds.  float32: the largest difference of a position is at most 1e-4 of that position's largest
# logit (or of 1) against the 64-bit plain model: rounding errors grow with the size of the sums that make a
# logit, not with the logit that is left after cancellation.  bfloat16: at most 2 % of it, against the plain
# model that rounds what the matrix products read and what the cache holds to bfloat16 as the library does.
def _compare(got, ref, dtype, what):
    assert got, "nothing was compared"
    for key, g in got.items():
        r = ref[key]
        assert torch.isfinite(g).all(), f"{what}: non-finite logits at {key}"
        if dtype == "float32":
            err, bound = (g - r).abs().max().item() / max(1.0, r.abs().max().item()), 1e-4
        else:
            err, bound = (g - r).abs().max().item() / max(1e-3, r.abs().max().item()), 0.02
        assert err <= bound, f"{what}: {dtype} logits differ at request {key[0]} position {key[1]}: {err:.3e} > {bound}"


def _requests(cfg, lengths, seed):
    return {f"r{i}": tt.random_tokens(n, cfg["vocab"], seed + i) for i, n in enumerate(lengths)}


# --------------------------------------------------------------------------- without a GPU
def test_config_round_trip_and_weight_table():
    import hilbert_pruned_8b_b200 as hb
    from hilbert_pruned_8b_b200.config import ConfigError, config_class_for
    from hilbert_pruned_8b_b200.engine.model import weight_table
    for cfg in pt.CONFIGS.values():
        assert config_class_for(cfg) is hb.PogezenConfig
        c = hb.PogezenConfig.from_dict(cfg)
        assert hb.PogezenConfig.from_dict(c.to_dict()) == c
        table = weight_table(c.model_spec(), "")
        for i, layer in enumerate(cfg["layers"]):
            assert (f"l{i}.norm2.alpha" in table) == (layer["mlp"] is not None)
            assert table[f"l{i}.canon1"].shape == (cfg["width"], cfg["canon"]["taps"])
            assert (f"l{i}.mix.talk" in table) == (layer["type"] == "attention")
            assert (f"l{i}.mix.f.b" in table) == (layer["type"] == "mlstm")
        assert table["final.norm.alpha"].shape == () and table["embed"].shape == (cfg["vocab"], cfg["width"])
    # the first value-mixing layer never reads its scalar; later ones must have it
    table = weight_table(hb.PogezenConfig.from_dict(pt.MIXED).model_spec(), "")
    assert table["l0.mix.vmix"].optional and not table["l2.mix.vmix"].optional
    for bad in ({**pt.MIXED, "layers": []}, {**pt.MIXED, "width": 0}, {k: v for k, v in pt.MIXED.items() if k != "canon"},
                {**pt.MIXED, "layers": [{"type": "conv", "mixer": {}, "mlp": None}]},
                {**pt.MIXED, "layers": [pt.with_mlp(pt.attention(3, 2, 8, 8, 4, 0, 4), None)]},
                {**pt.MIXED, "layers": [pt.with_mlp(pt.attention(2, 2, 8, 8, 4, 0, 10), None)]}):
        with pytest.raises(ConfigError):
            hb.PogezenConfig.from_dict(bad)


def test_cache_keeps_the_pages_of_the_first_tokens():
    from hilbert_pruned_8b_b200.cache.manager import CacheManager
    from hilbert_pruned_8b_b200.parts.base import CacheNeed
    need = CacheNeed(2, 16, window=70, v_head_dim=8, keep_first=3)
    cache = CacheManager({0: need}, {}, 64 * 8, "cpu", torch.float32, allocate=True)
    assert cache.groups[0].v.shape[-1] == 8 and cache.groups[0].k.shape[-1] == 16
    seq = cache.open()
    cache.reserve([(seq, 300)])
    cache.commit(seq, 300)
    cache.reserve([(seq, 301)])                 # position 300 sees 231..300 and 0..2: pages 1 and 2 are given back
    pages = seq.pages[0]
    assert pages[0] is not None and pages[1] is None and pages[2] is None and pages[3] is not None
    assert cache.groups[0].pool.num_free == 8 - 3
    other = cache.open()
    cache.reserve([(other, 128)])               # the freed pages are used again
    assert sorted(other.pages[0]) == [1, 2]
    cache.close(seq)
    cache.close(other)
    assert cache.groups[0].pool.num_free == 8


def test_plain_mechanisms_agree_with_their_definitions():
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    # the stabilised matrix memory equals the unstabilised sums  S_t = sum_s exp(F_t - F_s + i_s) k_s v_s^T
    T, H, d, dv = 9, 2, 3, 4
    q, k, v, li, lf = r(T, H, d), r(T, H, d), r(T, H, dv), r(T, H), -torch.rand(T, H, generator=g, dtype=torch.float64)
    out = mlstm_scan(q, k, v, li, lf)
    F = lf.cumsum(0)
    for t in range(T):
        for h in range(H):
            w = torch.exp(F[t, h] - F[: t + 1, h] + li[: t + 1, h])
            S = torch.einsum("s,sd,sv->dv", w, k[: t + 1, h], v[: t + 1, h])
            n = (w[:, None] * k[: t + 1, h]).sum(0)
            m = max(0.0 + F[t, h].item(), (F[t, h] - F[: t + 1, h] + li[: t + 1, h]).max().item())
            want = S.T @ q[t, h] / (max(abs((n @ q[t, h]).item()), 1.0) * math.exp(-m) + 1e-6) * math.exp(-m)
            assert torch.allclose(out[t, h], want, rtol=1e-9, atol=1e-12)
    # the window with kept first tokens
    m = visible(12, 4, 2)
    assert m[10].tolist() == [True, True] + [False] * 5 + [True] * 4 + [False] and m[3].tolist() == [True] * 4 + [False] * 8
    # the convolution's taps: the last tap multiplies the token itself
    h, w = r(6, 2), r(2, 3)
    c = causal_conv(h, w)
    assert torch.allclose(c[0], w[:, 2] * h[0]) and torch.allclose(c[4], w[:, 0] * h[2] + w[:, 1] * h[3] + w[:, 2] * h[4])
    # YaRN: fast pairs keep their frequency, slow ones are divided by the factor
    f, amp = yarn_frequencies(16, 10000.0, {"factor": 4.0, "original": 64, "fast": 32.0, "slow": 0.01})
    base = 10000.0 ** (-torch.arange(8, dtype=torch.float64) / 8)
    assert torch.allclose(f[0], base[0]) and torch.allclose(f[-1], base[-1] / 4.0) and abs(amp - (0.1 * math.log(4.0) + 1.0)) < 1e-12


# --------------------------------------------------------------------------- mechanisms on the GPU
def _ops_and_step(lengths_new, lengths_before, needs, state_floats, dtype=torch.float32, slots=None):
    """A kernel library, a cache with one entry per need and a step of sequences that hold
    ``lengths_before`` tokens and bring ``lengths_new`` more."""
    from hilbert_pruned_8b_b200.cache.manager import CacheManager
    from hilbert_pruned_8b_b200.engine.batch import StepEntry, build_step
    from hilbert_pruned_8b_b200.engine.workspace import Workspace
    from hilbert_pruned_8b_b200.kernels.ops import Ops
    from hilbert_pruned_8b_b200.parts.base import StateNeed
    dev = torch.device("cuda:0")
    ops, ws = Ops(dev), Workspace(dev)
    cache = CacheManager(dict(enumerate(needs)), {0: StateNeed((state_floats,), torch.float32)} if state_floats else {},
                         64 * 16, dev, dtype)
    seqs = [cache.open() for _ in lengths_new]
    return ops, ws, cache, seqs


def _step(cache, ws, seqs, new):
    from hilbert_pruned_8b_b200.engine.batch import StepEntry, build_step
    entries = [StepEntry(s, [0] * n, []) for s, n in zip(seqs, new)]
    cache.reserve([(s, s.length + n) for s, n in zip(seqs, new)])
    step = build_step(entries, cache, ws, torch.device("cuda:0"))
    return step


def _commit(cache, seqs, new):
    for s, n in zip(seqs, new):
        cache.commit(s, s.length + n)


@pytest.mark.gpu
def test_dynamic_tanh_squared_relu_and_scaled_embedding():
    require_gpu()
    ops, ws, cache, seqs = _ops_and_step([1], [0], [], 0)
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(37, 72, generator=g) * 3).cuda()
    w, b, a = torch.randn(72, generator=g).cuda(), torch.randn(72, generator=g).cuda(), torch.tensor([0.37]).cuda()
    want = dyt(x.double(), w.double(), b.double(), a.double())
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-2)):
        out = torch.empty(37, 72, dtype=dtype, device="cuda")
        ops.dyt(x, w, b, a, out)
        assert (out.double() - want).abs().max() < tol * 4
        rows = torch.tensor([5, 0, 36], dtype=torch.int32, device="cuda")
        picked = torch.empty(3, 72, dtype=dtype, device="cuda")
        ops.dyt(x, w, b, a, picked, rows)
        assert torch.equal(picked, out[rows.long()])
    act = torch.empty(37, 72, dtype=torch.bfloat16, device="cuda")
    ops.relu2(x, act)
    assert torch.equal(act, (torch.relu(x) ** 2).to(torch.bfloat16))
    table = torch.randn(50, 24, generator=g).to(torch.bfloat16).cuda()
    toks = torch.tensor([3, 49, 0], dtype=torch.int32, device="cuda")
    emb = torch.empty(3, 24, device="cuda")
    ops.embed(toks, table, emb, 0.25)
    assert torch.equal(emb, table[toks.long()].float() * 0.25)
    ops.check_errors()


@pytest.mark.gpu
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
@pytest.mark.parametrize("fused", [True, False])
def test_short_convolution_carries_its_state_over_portions(taps, fused):
    """Two sequences of unequal lengths fed in portions of 1, 2, 3 ... tokens: the same values as the
    whole sequence at once, with the norm applied by the convolution kernel or in front of it."""
    require_gpu()
    C = 70
    ops, ws, cache, seqs = _ops_and_step([0, 0], [0, 0], [], max(1, (taps - 1) * C))
    g = torch.Generator().manual_seed(taps)   # (the cache of _ops_and_step holds 1024 tokens)
    total = [23, 9]
    x = [torch.randn(n, C, generator=g) * 2 for n in total]
    cw = (torch.randn(C, taps, generator=g) * 0.5).cuda()
    nw, nb, na = torch.randn(C, generator=g).cuda(), torch.randn(C, generator=g).cuda(), torch.tensor([0.8]).cuda()
    want = []
    for xs in x:
        h = dyt(xs.double(), nw.cpu().double(), nb.cpu().double(), 0.8)
        want.append(h + causal_conv(h, cw.cpu().double()))
    state = cache.state_view(0)[:, : (taps - 1) * C]
    got = [[], []]
    done = [0, 0]
    portion = 1
    while any(d < t for d, t in zip(done, total)):
        live = [i for i in range(2) if done[i] < total[i]]
        new = [min(portion, total[i] - done[i]) for i in live]
        step = _step(cache, ws, [seqs[i] for i in live], new)
        xin = torch.cat([x[i][done[i]: done[i] + n] for i, n in zip(live, new)]).cuda()
        out = torch.empty_like(xin)
        if fused:
            ops.short_conv(xin, cw, state, step, out, norm=(nw, nb, na))
        else:
            h = torch.empty_like(xin)
            ops.dyt(xin, nw, nb, na, h)
            ops.short_conv(h, cw, state, step, out)
        o = out.cpu()
        at = 0
        for i, n in zip(live, new):
            got[i].append(o[at: at + n])
            at += n
            done[i] += n
        _commit(cache, [seqs[i] for i in live], new)
        portion += 1
    for i in range(2):
        assert (torch.cat(got[i]).double() - want[i]).abs().max() < 2e-5
    # a slot that is used again starts from zeros; a long portion is cut over several blocks, then goes on
    for s in seqs:
        cache.close(s)
    again = cache.open()
    long_x = torch.randn(700, C, generator=g) * 2
    h = dyt(long_x.double(), nw.cpu().double(), nb.cpu().double(), 0.8)
    long_want = h + causal_conv(h, cw.cpu().double())
    at = 0
    for n in (total[1], 600, 700 - 600 - total[1]):
        step = _step(cache, ws, [again], [n])
        out = torch.empty(n, C, device="cuda")
        ops.short_conv(long_x[at: at + n].cuda(), cw, state, step, out, norm=(nw, nb, na))
        assert (out.cpu().double() - long_want[at: at + n]).abs().max() < 2e-5
        _commit(cache, [again], [n])
        at += n


@pytest.mark.gpu
@pytest.mark.parametrize("heads,d,dv", [(2, 8, 16), (1, 40, 33), (3, 64, 70)])
def test_matrix_memory_in_portions_equals_the_scan(heads, d, dv):
    require_gpu()
    H = heads
    n_state = H * d * dv + H * d + H
    ops, ws, cache, seqs = _ops_and_step([0, 0], [0, 0], [], n_state)
    g = torch.Generator().manual_seed(d)
    width = 2 * H * d + 2 * H * dv + 2 * H
    total = [75, 11]
    proj = [torch.randn(n, width + 3, generator=g) for n in total]          # rows longer than what is read
    for p in proj:
        p[:, -2 * H - 3: -3] *= 3.0                                          # gates that reach their cap
    bias = torch.cat([torch.randn(H, generator=g), torch.randn(H, generator=g) + 2.0])
    cap, eps = 5.0, 1e-5
    nw = torch.randn(H * dv, generator=g)
    want = []
    for p in proj:
        pd = p.double()
        T = p.shape[0]
        q = pd[:, : H * d].view(T, H, d) * d ** -0.5
        k = pd[:, H * d: 2 * H * d].view(T, H, d)
        v = pd[:, 2 * H * d: 2 * H * d + H * dv].view(T, H, dv)
        gate = pd[:, 2 * H * d + H * dv: 2 * H * d + 2 * H * dv]
        li = soft_cap(pd[:, width - 2 * H: width - H] + bias[:H].double(), cap)
        lf = torch.nn.functional.logsigmoid(soft_cap(pd[:, width - H: width] + bias[H:].double(), cap))
        o = rms_unit(mlstm_scan(q, k, v, li, lf), eps).reshape(T, H * dv)
        want.append(o * nw.double() * torch.sigmoid(gate))
    state = cache.state_view(0)
    got, done = [[], []], [0, 0]
    for portion in (1, 2, 1, 5, 64, 8):     # portions of 8 tokens and more run the chunked kernel
        live = [i for i in range(2) if done[i] < total[i]]
        if not live:
            break
        new = [min(portion, total[i] - done[i]) for i in live]
        step = _step(cache, ws, [seqs[i] for i in live], new)
        pin = torch.cat([proj[i][done[i]: done[i] + n] for i, n in zip(live, new)]).cuda()
        o = torch.empty(pin.shape[0], H * dv, device="cuda")
        ops.mlstm_scan(pin, bias.cuda(), cap, d ** -0.5, state, step, o, H, d, dv)
        out = torch.empty_like(o)
        ops.mlstm_output(o, pin[:, 2 * H * d + H * dv: 2 * H * d + 2 * H * dv], nw.cuda(), eps, out, H, dv)
        oc, at = out.cpu(), 0
        for i, n in zip(live, new):
            got[i].append(oc[at: at + n])
            at += n
            done[i] += n
        _commit(cache, [seqs[i] for i in live], new)
    for i in range(2):
        assert done[i] == total[i]
        err = (torch.cat(got[i]).double() - want[i]).abs().max().item()
        assert err < 5e-5 * max(1.0, want[i].abs().max().item()), err


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,size,keep,rot", [(4, 2, 16, 8, 70, 3, 8), (2, 2, 8, 24, 64, 0, 8), (3, 1, 32, 16, 129, 65, 0),
                                                     (6, 3, 64, 40, 5, 1, 32), (8, 4, 32, 256, 100, 2, 16), (3, 1, 20, 12, 40, 3, 4),
                                                     (16, 4, 32, 32, 70, 3, 16), (32, 8, 16, 24, 100, 2, 8), (32, 2, 64, 64, 33, 40, 32),
                                                     (4, 2, 64, 128, 70, 3, 32), (3, 1, 128, 64, 130, 65, 0), (8, 4, 128, 128, 64, 0, 64)])
def test_attention_sees_exactly_the_window_and_the_first_tokens(H, G, d, dv, size, keep, rot, dtype):
    """A prompt of 300 tokens, then tokens one by one.  For some queries one key is made to stand
    out (its score dwarfs the others): the key just inside the window, just outside it, the last
    kept first token, the first one that is not kept, a key on a page border.  The output then shows
    at once whether that key was seen."""
    require_gpu()
    from hilbert_pruned_8b_b200.parts.base import CacheNeed
    ops, ws, cache, seqs = _ops_and_step([0], [0], [CacheNeed(G, d, size, v_head_dim=dv, keep_first=keep)], 0, dtype)
    g = torch.Generator().manual_seed(H * 100 + size)
    T, tail = 300, 6
    n = T + tail
    width = H * d + G * d + G * dv
    proj = torch.randn(n, width, generator=g) * 0.3
    bias = torch.randn(width, generator=g) * 0.2
    talk = torch.eye(H) + torch.randn(H, H, generator=g) * 0.4
    # queries whose first head points at one chosen key
    probes = {}
    for qpos in (T - 1, T - 40, T + tail - 1, T + 2):
        for kpos in (qpos - size + 1, qpos - size, keep - 1, keep, 64, 63, qpos):
            if 0 <= kpos <= qpos and (qpos, 0) not in probes and torch.rand(1, generator=g).item() < 0.5:
                probes[(qpos, 0)] = kpos
    for (qpos, head), kpos in probes.items():
        direction = torch.randn(d, generator=g)
        proj[kpos, H * d: H * d + d] = direction * 3 - bias[H * d: H * d + d]
        proj[qpos, head * d: head * d + d] = direction * 3 - bias[head * d: head * d + d]
    freq, amp = yarn_frequencies(rot, 100.0, {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}) if rot else (None, 1.0)
    eps, scale = 1e-5, 8.0 / d ** 0.5
    pd = (proj + bias).double()
    q, k, v = pd[:, : H * d].view(n, H, d), pd[:, H * d: H * d + G * d].view(n, G, d), pd[:, H * d + G * d:].view(n, G, dv)
    pos = torch.arange(n)
    if rot:
        q, k = rotate(q, pos, freq, amp, rot), rotate(k, pos, freq, amp, rot)
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    if dtype == torch.bfloat16:          # what the cache and the query buffer hold
        q, k, v = (t.to(torch.bfloat16).double() for t in (q, k, v))
    want = talking_attention(q, k, v, talk.double(), scale, size, keep).reshape(n, H * dv)
    inv_freq = freq.float().cuda() if rot else None
    got = []
    for new in [T] + [1] * tail:
        step = _step(cache, ws, seqs, [new])
        lo = seqs[0].length
        pin = proj[lo: lo + new].cuda()
        table = None
        if rot:
            table = torch.empty(new, rot // 2, 2, device="cuda")
            ops.rope_table(step.positions, inv_freq, table, amp)
        qb = torch.empty(new, H * d, dtype=dtype, device="cuda")
        view = cache.view(0)
        ops.qkv_prepare(pin, bias.cuda(), table, rot, H, G, d, dv, True, eps, qb, view, step, True)
        partial = torch.empty(new, H * G * dv, device="cuda")
        ops.attention_sink(qb, H, G, d, dv, view, step, partial, scale, size, keep, True)
        out = torch.empty(new, H * dv + 8, dtype=dtype, device="cuda")
        ops.head_mix(partial, talk.reshape(-1).cuda(), out, H, G, dv, G, 8)
        assert torch.equal(out[:, H * dv:].float().cpu(), torch.tensor([1.0] + [0.0] * 7).expand(new, 8))
        got.append(out[:, : H * dv].float().cpu())
        # the flash-style kernel for steps of many tokens (it takes any step; here also the single tokens)
        if dtype == torch.bfloat16 and ops.lib.hb_attention_sink_prefill_supported(H, G, d, dv):
            flash = torch.full((new * H * G * dv,), float("nan"), device="cuda")
            ops.attention_sink_prefill(qb, H, G, d, dv, view, step, flash, scale, size, keep, True)
            again = torch.empty_like(out)
            ops.head_mix(flash, talk.reshape(-1).cuda(), again, H, G, dv, G, 8)
            assert (again.float() - out.float()).abs().max().item() <= 2e-2 * max(1.0, out.float().abs().max().item())
        # the kernel that serves all heads of a token in one block: key splits combined afterwards, or the output at once
        if ops.attention_heads_plan(new, H, G, d, dv, dtype, 10 ** 6) is not None:
            for splits in (1, 3, 8):
                part = torch.full((new * H * splits * G * dv,), float("nan"), device="cuda")
                ml = torch.empty(new * H * splits * 2, device="cuda")
                ops.attention_heads(qb, H, G, d, dv, view, step, scale, size, keep, splits, partial=part, ml=ml)
                again = torch.empty_like(out)
                ops.head_mix_splits(part, ml, talk.reshape(-1).cuda(), again, H, G, dv, splits, 8)
                assert (again.float() - out.float()).abs().max().item() <= (1e-5 if dtype == torch.float32 else 2e-2) * max(1.0, out.float().abs().max().item())
            for mma in (True, False):       # the weights-times-values product on the tensor cores, and on the FP32 pipe
                ops.use_mma_attention = mma
                if ops.attention_heads_whole(H, G, d, dv, dtype):
                    again = torch.empty_like(out)
                    ops.attention_heads(qb, H, G, d, dv, view, step, scale, size, keep, 1, mix=talk.reshape(-1).cuda(), out=again, ones=8)
                    assert (again.float() - out.float()).abs().max().item() <= (1e-5 if dtype == torch.float32 else 2e-2) * max(1.0, out.float().abs().max().item())
                    assert torch.equal(again[:, H * dv:].float().cpu(), torch.tensor([1.0] + [0.0] * 7).expand(new, 8))
                part = torch.full((new * H * 5 * G * dv,), float("nan"), device="cuda")
                ml = torch.empty(new * H * 5 * 2, device="cuda")
                ops.attention_heads(qb, H, G, d, dv, view, step, scale, size, keep, 5, partial=part, ml=ml)
                again = torch.empty_like(out)
                ops.head_mix_splits(part, ml, talk.reshape(-1).cuda(), again, H, G, dv, 5, 8)
                assert (again.float() - out.float()).abs().max().item() <= (1e-5 if dtype == torch.float32 else 2e-2) * max(1.0, out.float().abs().max().item())
            ops.use_mma_attention = True
        _commit(cache, seqs, [new])
    ops.check_errors()
    got = torch.cat(got).double()
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    err = (got - want).abs().max().item()
    assert err < tol * max(1.0, want.abs().max().item()), err
    assert probes, "no probe was placed"


@pytest.mark.gpu
def test_values_are_mixed_with_the_first_layers():
    require_gpu()
    from hilbert_pruned_8b_b200.parts.base import CacheNeed
    G, d, dv, H = 2, 8, 12, 2
    ops, ws, cache, seqs = _ops_and_step([0], [0], [CacheNeed(G, d, None, v_head_dim=dv), CacheNeed(G, d, 9, v_head_dim=dv)], 0)
    g = torch.Generator().manual_seed(5)
    n = 5
    width = H * d + G * d + G * dv
    p1, p2 = torch.randn(n, width, generator=g), torch.randn(n, width, generator=g)
    step = _step(cache, ws, seqs, [n])
    first = torch.empty(n, G * dv, device="cuda")
    q = torch.empty(n, H * d, device="cuda")
    lam = torch.tensor([0.3], device="cuda")
    ops.qkv_prepare(p1.cuda(), None, None, 0, H, G, d, dv, False, 0.0, q, cache.view(0), step, True, None, first, 1)
    ops.qkv_prepare(p2.cuda(), None, None, 0, H, G, d, dv, False, 0.0, q, cache.view(1), step, True, lam, first, 2)
    page = seqs[0].pages[1][0]
    stored = cache.view(1).v[page][:, :n].permute(1, 0, 2).reshape(n, G * dv).cpu()
    v1, v2 = p1[:, H * d + G * d:], p2[:, H * d + G * d:]
    assert torch.allclose(first.cpu(), v1) and torch.allclose(stored, 0.7 * v2 + 0.3 * v1, atol=1e-6)
    assert torch.allclose(q.cpu(), p2[:, : H * d])          # no rotation, no norm, no bias: the queries pass through


@pytest.mark.gpu
def test_yarn_rotation_table():
    require_gpu()
    from hilbert_pruned_8b_b200.parts.rope import yarn_amplitude, yarn_inv_freq
    ops, ws, cache, seqs = _ops_and_step([1], [0], [], 0)
    yarn = {"factor": 8.0, "original": 128, "fast": 16.0, "slow": 2.0}
    f = yarn_inv_freq(24, 3000.0, yarn)
    want_f, want_amp = yarn_frequencies(24, 3000.0, yarn)
    assert torch.allclose(torch.from_numpy(f).double(), want_f, rtol=1e-7) and abs(yarn_amplitude(yarn) - want_amp) < 1e-12
    assert torch.allclose(torch.from_numpy(yarn_inv_freq(24, 3000.0, None)).double(), yarn_frequencies(24, 3000.0, None)[0], rtol=1e-7)
    pos = torch.tensor([0, 1, 77, 4000], dtype=torch.int32, device="cuda")
    table = torch.empty(4, 12, 2, device="cuda")
    ops.rope_table(pos, torch.from_numpy(f).cuda(), table, want_amp)
    a = pos.cpu().double()[:, None] * torch.from_numpy(f).double()[None, :]
    assert (table[..., 0].cpu().double() - torch.cos(a) * want_amp).abs().max() < 5e-4       # a float32 angle near 4000
    assert (table[:3, :, 1].cpu().double() - (torch.sin(a) * want_amp)[:3]).abs().max() < 1e-5


# --------------------------------------------------------------------------- the engine
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts(models, name, dtype):
    require_gpu()
    folder, cfg, plain = models[name]
    reqs = _requests(cfg, [1, 2, 7, 70, 150], 100)
    steps, peak = tt.trace_whole(reqs)
    eng = _engine(folder, dtype, peak)
    _compare(tt.run_in_process(eng, steps), _reference(plain[dtype], reqs), dtype, "whole")
    assert all(f == eng.cache.num_pages for f in eng.cache.pages_free()) and eng.cache.slots.num_held == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_tokens_one_by_one(models, name, dtype):
    """The decoded tokens carry the window over the prompt's end and over page borders."""
    require_gpu()
    folder, cfg, plain = models[name]
    reqs = _requests(cfg, [3, 60, 130], 200)
    steps, peak = tt.trace_tail(reqs, tail=58)
    eng = _engine(folder, dtype, peak)
    _compare(tt.run_in_process(eng, steps), _reference(plain[dtype], reqs), dtype, "tail")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompts_in_portions(models, name, dtype):
    """A prompt cut into portions of 2, 3, 1, 64, 5 ... tokens, and cut by the engine itself when a
    step brings more tokens than it takes at once."""
    require_gpu()
    folder, cfg, plain = models[name]
    toks = tt.random_tokens(170, cfg["vocab"], 300)
    steps, at = [], 0
    for n in (2, 3, 1, 64, 5, 2, 40, 2, 51):
        steps.append({"step": len(steps), "entries": [{"id": "p", "tokens": toks[at: at + n], "want": list(range(n))}],
                      "end": ["p"] if at + n == len(toks) else []})
        at += n
    assert at == len(toks)
    ref = _reference(plain[dtype], {"p": toks})
    _compare(tt.run_in_process(_engine(folder, dtype, 192), steps), ref, dtype, "portions")
    whole = [{"step": 0, "entries": [{"id": "p", "tokens": toks, "want": list(range(len(toks)))}], "end": ["p"]}]
    _compare(tt.run_in_process(_engine(folder, dtype, 192, max_step_tokens=48), whole), ref, dtype, "cut by the engine")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_with_slots_and_pages_used_again(models, name, dtype):
    require_gpu()
    folder, cfg, plain = models[name]
    v = cfg["vocab"]
    batches = [{f"a{i}": (tt.random_tokens(n, v, 400 + i), p) for i, (n, p) in enumerate([(90, 70), (12, 1), (150, 129), (40, 39)])},
               {f"b{i}": (tt.random_tokens(n, v, 500 + i), p) for i, (n, p) in enumerate([(30, 2), (100, 64), (5, 5)])}]
    steps, peak = tt.trace_batches(batches)
    eng = _engine(folder, dtype, peak)
    reqs = {rid: t for b in batches for rid, (t, _) in b.items()}
    _compare(tt.run_in_process(eng, steps), _reference(plain[dtype], reqs), dtype, "batches")
    assert eng.graph_replays > 0
    assert all(f == eng.cache.num_pages for f in eng.cache.pages_free()) and eng.cache.slots.num_held == 0


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_long_decoding(models, name):
    """Hundreds of single-token steps through the captured graphs: windows slide off their pages,
    which are given back, the first tokens' page stays."""
    require_gpu()
    folder, cfg, plain = models[name]
    toks = tt.random_tokens(330, cfg["vocab"], 600)
    steps = [{"step": 0, "entries": [{"id": "l", "tokens": toks[:4], "want": [3]}], "end": []}]
    for p in range(4, len(toks)):
        steps.append({"step": len(steps), "entries": [{"id": "l", "tokens": [toks[p]], "want": [0]}],
                      "end": ["l"] if p == len(toks) - 1 else []})
    eng = _engine(folder, "float32", 384)
    got = tt.run_in_process(eng, steps)
    ref = _reference(plain["float32"], {"l": toks})
    _compare(got, {k: ref[k] for k in got}, "float32", "long decoding")
    assert eng.graph_replays > 300


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
def test_fused_norm_and_convolution_equal_the_two_kernels(models, name):
    require_gpu()
    folder, cfg, plain = models[name]
    reqs = _requests(cfg, [50, 3], 700)
    steps, peak = tt.trace_tail(reqs, tail=5)
    a = tt.run_in_process(_engine(folder, "float32", peak), steps)
    eng = _engine(folder, "float32", peak)
    for b in eng.model.blocks:
        b.fuse_norm_and_filter = False
    b = tt.run_in_process(eng, steps)
    for k in a:
        assert (a[k] - b[k]).abs().max() < 1e-4


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "edges", "wide", "many_heads", "big_heads"])
def test_attention_kernels_agree(models, name, dtype):
    """The kernel that serves all heads per block (with key splits in decode steps) against the general one."""
    require_gpu()
    folder, cfg, plain = models[name]
    v = cfg["vocab"]
    batches = [{f"k{i}": (tt.random_tokens(n, v, 950 + i), p) for i, (n, p) in enumerate([(160, 150), (20, 3)])}]
    steps, peak = tt.trace_batches(batches)
    a = tt.run_in_process(_engine(folder, dtype, peak), steps)
    eng = _engine(folder, dtype, peak)
    for blk in eng.model.blocks:
        if hasattr(blk.mixer, "use_heads_kernel"):
            blk.mixer.use_heads_kernel = False
    b = tt.run_in_process(eng, steps)
    for k in a:
        scale = max(1.0, b[k].abs().max().item())
        assert (a[k] - b[k]).abs().max().item() <= (1e-4 if dtype == "float32" else 2e-2) * scale, k


def _greedy(plain, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(plain.forward(toks)[-1].argmax()))
    return toks[len(prompt):]


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["mixed", "edges", "recurrent"])
def test_greedy_generation_through_the_library(models, name):
    """hb.load(...).generate(...): the scheduler's batches, the sampler and the captured decode steps."""
    require_gpu()
    import hilbert_pruned_8b_b200 as hb
    folder, cfg, plain = models[name]
    prompts = [tt.random_tokens(n, cfg["vocab"], 800 + i) for i, n in enumerate([1, 9, 45, 3, 66])]
    llm = hb.load(folder, dtype="float32", max_tokens=64 * 8, max_batch=3)       # two batches: slots are used again
    res = llm.generate(prompts, max_new_tokens=10, stop_token_ids=[])
    for r, p in zip(res, prompts):
        assert r.tokens == _greedy(plain["float32"], p, 10), f"prompt of {len(p)} tokens"
    assert llm.generator.stats.batches == 2
    assert all(f == llm.engine.cache.num_pages for f in llm.engine.cache.pages_free())


@pytest.mark.gpu
def test_replay_program(models, tmp_path):
    require_gpu()
    folder, cfg, plain = models["mixed"]
    batches = [{f"t{i}": (tt.random_tokens(n, cfg["vocab"], 900 + i), p) for i, (n, p) in enumerate([(70, 66), (9, 2)])}]
    steps, peak = tt.trace_batches(batches, want_all=False)
    reqs = {rid: t for rid, (t, _) in batches[0].items()}
    for dtype in DTYPES:
        ref = _reference(plain[dtype], reqs)
        got = tt.run_program(folder, dtype, steps, peak, str(tmp_path / dtype), cfg["vocab"])
        _compare(got, {k: ref[k] for k in got}, dtype, "trace_run")
