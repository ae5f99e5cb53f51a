"""The Vuladra decoder against the plain implementation (tests/plain_vuladra.py): every mechanism
alone, then the engine: whole prompts, token-by-token decoding, prompts in portions down to two
tokens, unequal batches with slots and pages used again, the edges of windows and pooled blocks,
long decoding, greedy generation through the library's entry point and the replay program."""
import pytest
import torch

import trace_tools as tt
import vuladra_tools as vt
from conftest import require_gpu
from plain_vuladra import (PlainVuladra, causal_conv_bias, clamped_glu, decayed_memory, pool_blocks, pooled_mask, rms_norm, route,
                           selective_scan, sigmoid_pool_attention, silu, softplus, window_mask)

DTYPES = ["float32", "bfloat16"]
NAMES = ["mixed", "edges", "wide", "recurrent"]


# --------------------------------------------------------------------------- helpers
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (folder, config, {dtype: plain model}); the bfloat16 one rounds where the library does"""
    out = {}
    for i, (name, cfg) in enumerate(vt.CONFIGS.items()):
        d = str(tmp_path_factory.mktemp("vuladra_" + name))
        tensors = vt.write_model(d, cfg, 70 + i)
        out[name] = (d, cfg, {"float32": PlainVuladra(cfg, tensors), "bfloat16": PlainVuladra(cfg, tensors, round_to=torch.bfloat16)})
    return out


def _engine(folder, dtype, max_tokens, **kw):
    from hilbert_pruned_8b_b200.engine.step import Engine
    return Engine.from_folder(folder, dtype, max_tokens=max_tokens, **kw)


def _reference(plain, requests):
    ref = {}
    for rid, toks in requests.items():
        lg = plain.logits(toks)
        for p in range(len(toks)):
            ref[(rid, p)] = lg[p]
    return ref


# Fixed bounds.  float32: the largest difference of a position is at most 1e-4 of that position's largest logit (or of 1)
# against the 64-bit plain model, at every position.  bfloat16: at most 3 % of it against the plain model that rounds what the
# matrix products read and what the cache holds to bfloat16.  There a router's near tie may fall the other way (the two
# sides' inputs differ by their rounding), which changes that token's experts and, through states and windows, what
# later tokens see: up to a tenth of the positions may therefore differ by more, none by more than half.
def _compare(got, ref, dtype, what):
    assert got, "nothing was compared"
    over = []
    for key, g in got.items():
        r = ref[key]
        assert torch.isfinite(g).all(), f"{what}: non-finite logits at {key}"
        if dtype == "float32":
            err = (g - r).abs().max().item() / max(1.0, r.abs().max().item())
            assert err <= 1e-4, f"{what}: float32 logits differ at request {key[0]} position {key[1]}: {err:.3e}"
        else:
            err = (g - r).abs().max().item() / max(1e-3, r.abs().max().item())
            assert err <= 0.5, f"{what}: bfloat16 logits differ at request {key[0]} position {key[1]}: {err:.3e}"
            if err > 0.03:
                over.append((key, err))
    assert len(over) <= 0.1 * len(got), f"{what}: bfloat16 logits differ by more than 3 % at {len(over)} of {len(got)} positions, first {over[0]}"


def _requests(cfg, lengths, seed):
    return {f"r{i}": tt.random_tokens(n, cfg["vocab"], seed + i) for i, n in enumerate(lengths)}


# --------------------------------------------------------------------------- without a GPU
def test_config_round_trip_and_weight_table():
    import hilbert_pruned_8b_b200 as hb
    from hilbert_pruned_8b_b200.config import ConfigError, config_class_for
    from hilbert_pruned_8b_b200.engine.model import weight_table
    for cfg in vt.CONFIGS.values():
        assert config_class_for(cfg) is hb.VuladraConfig
        c = hb.VuladraConfig.from_dict(cfg)
        assert hb.VuladraConfig.from_dict(c.to_dict()) == c
        table = weight_table(c.model_spec(), "")
        for i, layer in enumerate(cfg["layers"]):
            assert f"l{i}.norm1" in table and f"l{i}.norm1b" in table
            assert (f"l{i}.norm2b" in table) == (layer["mlp"] is not None)
            assert (f"l{i}.mix.pb" in table) == (layer["type"] == "attention")
            assert (f"l{i}.mix.right.norm" in table) == (layer["type"] == "parallel")
            assert (f"l{i}.mix.A_log" in table) == (layer["type"] == "mamba1")
            mlp = layer["mlp"]
            assert (f"l{i}.mlp.router" in table) == (mlp is not None and mlp["kind"] == "moe")
            assert (f"l{i}.mlp.shared.up" in table) == (mlp is not None and mlp["kind"] == "moe" and mlp["shared"] is not None)
            assert (f"l{i}.mlp.gate" in table) == (mlp is not None and mlp["kind"] == "dense")
        assert table["final.norm"].shape == (cfg["width"],) and table["embed"].shape == (cfg["vocab"], cfg["width"])
    m = vt.MIXED["layers"][0]["mixer"]
    table = weight_table(hb.VuladraConfig.from_dict(vt.MIXED).model_spec(), "")
    assert table["l0.mix.x"].shape == (m["dt_rank"] + 2 * m["state"], m["inner"]) and table["l0.mix.dt"].shape == (m["inner"], m["dt_rank"])
    assert table["l1.mlp.e5.down"].shape == (64, 24) and "l1.mlp.e6.down" not in table
    for bad in ({**vt.MIXED, "layers": []}, {**vt.MIXED, "width": 0}, {k: v for k, v in vt.MIXED.items() if k != "norm"},
                {**vt.MIXED, "layers": [{"type": "conv", "mixer": {}, "mlp": None}]},
                {**vt.MIXED, "layers": [vt.with_mlp(vt.attention(3, 2, 8, 8, 4, 2), None)]},
                {**vt.MIXED, "layers": [vt.with_mlp(vt.mamba(8, 2, 1, 2), vt.moe(2, 3, 4, 1.0))]},
                {**vt.MIXED, "layers": [vt.with_mlp(vt.parallel((2, 1, 4, 4, 5), (2, 4, 4, (0.5,))), None)]}):
        with pytest.raises(ConfigError):
            hb.VuladraConfig.from_dict(bad)


def test_cache_with_a_window_group_and_a_group_of_pooled_blocks():
    """A mixer that asks for two needs gets two groups; the pooled one holds one entry per whole block, the windowed
    one gives pages back, and everything returns when a sequence closes."""
    from hilbert_pruned_8b_b200.cache.manager import CacheManager
    from hilbert_pruned_8b_b200.parts.base import CacheNeed
    window, pooled = CacheNeed(2, 16, window=70, v_head_dim=8), CacheNeed(2, 16, None, v_head_dim=8, stride=6, store_f32=True)
    cache = CacheManager({0: (window, pooled), 1: CacheNeed(1, 8, None)}, {}, 64 * 8, "cpu", torch.bfloat16, max_sequences=4)
    views = cache.view(0)
    assert isinstance(views, tuple) and views[0].k.dtype == torch.bfloat16 and views[1].k.dtype == torch.float32
    assert views[1].v.shape[-1] == 8 and not isinstance(cache.view(1), tuple)
    gw, gp = views[0].group, views[1].group
    assert cache.groups[gp].pool.size == 64 * 8 // 6 // 64 + 1 + 4             # blocks of all tokens, and a partly used page per sequence
    seq = cache.open()
    cache.reserve([(seq, 300)])
    cache.commit(seq, 300)
    assert len(seq.pages[gw]) == 5 and len(seq.pages[gp]) == 1                  # 50 blocks fit one page
    cache.reserve([(seq, 400)])                                                 # position 300 sees 231 ..: pages 0 to 2 are given back
    cache.commit(seq, 400)
    assert seq.pages[gw][:3] == [None] * 3 and seq.pages[gw][3] is not None and len(seq.pages[gp]) == 2     # 66 blocks
    snap = cache.snapshot(seq)
    cache.reserve([(seq, 500)])
    cache.commit(seq, 500)
    cache.restore(seq, snap)
    assert seq.length == 400 and len(seq.pages[gp]) == 2 and len(seq.pages[gw]) == 7
    cache.close(seq)
    assert all(g.pool.num_free == g.pool.size for g in cache.groups)


def test_plain_mechanisms_agree_with_their_definitions():
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    # window and pooled blocks: query 20 with a window of 5 and blocks of 4 sees tokens 16..20 and blocks 0..3 (tokens 0..15)
    assert window_mask(24, 5)[20].tolist() == [False] * 16 + [True] * 5 + [False] * 3
    assert pooled_mask(24, 5, 4)[20].tolist() == [True] * 4 + [False] * 2 and pooled_mask(24, 5, 4)[19].tolist() == [True] * 3 + [False] * 3
    assert pooled_mask(24, 5, 4)[7].tolist() == [False] * 6 and pooled_mask(24, 5, 4)[8].tolist() == [True] + [False] * 5
    t = r(10, 2, 3)
    assert torch.allclose(pool_blocks(t, 4)[1], t[4:8].mean(0)) and pool_blocks(t, 4).shape == (2, 2, 3)
    # sigmoid attention: one query, by hand
    q, k, v, b = r(9, 2, 4), r(9, 1, 4), r(9, 1, 3), r(2)
    out = sigmoid_pool_attention(q, k, v, b, 0.3, 3, 2)
    keys = [(k[0:2, 0].mean(0), v[0:2, 0].mean(0)), (k[2:4, 0].mean(0), v[2:4, 0].mean(0)), (k[4:6, 0].mean(0), v[4:6, 0].mean(0))]
    keys += [(k[j, 0], v[j, 0]) for j in (6, 7, 8)]
    want = sum(torch.sigmoid(q[8, 1] @ kk * 0.3 + b[1]) * vv for kk, vv in keys)
    assert torch.allclose(out[8, 1], want)
    # the decayed memory equals the explicit sums
    q, k, v, lam = r(7, 2, 3), r(7, 2, 3), r(7, 2, 5), torch.tensor([0.8, 1.0], dtype=torch.float64)
    out = decayed_memory(q, k, v, lam)
    for h in range(2):
        want = sum(lam[h] ** (6 - s) * (q[6, h] @ k[s, h]) * v[s, h] for s in range(7))
        assert torch.allclose(out[6, h], want)
    # the selective scan equals the explicit sums
    u, dt, A, B, C, D = r(6, 3), torch.rand(6, 3, generator=g, dtype=torch.float64), -torch.rand(3, 2, generator=g, dtype=torch.float64), r(6, 2), r(6, 2), r(3)
    y = selective_scan(u, dt, A, B, C, D)
    for c in range(3):
        want = D[c] * u[5, c] + sum(torch.exp(dt[s + 1:, c].sum() * A[c, n]) * dt[s, c] * u[s, c] * B[s, n] * C[5, n] for s in range(6) for n in range(2))
        assert torch.allclose(y[5, c], want)
    # the convolution's last tap multiplies the token itself; the router's weights are a softmax over the chosen logits
    x, w, bias = r(5, 2), r(2, 3), r(2)
    c = causal_conv_bias(x, w, bias)
    assert torch.allclose(c[0], bias + w[:, 2] * x[0]) and torch.allclose(c[3], bias + w[:, 0] * x[1] + w[:, 1] * x[2] + w[:, 2] * x[3])
    idx, wgt = route(torch.tensor([[0.1, 2.0, -1.0, 1.5]], dtype=torch.float64), 2)
    assert idx.tolist() == [[1, 3]] and torch.allclose(wgt, torch.softmax(torch.tensor([[2.0, 1.5]], dtype=torch.float64), -1))
    h = r(1, 4)
    wg, wu, wd = r(3, 4) * 3, r(3, 4) * 3, r(2, 3)
    gg, uu = torch.clamp(h @ wg.T, max=0.5), torch.clamp(h @ wu.T, -0.5, 0.5)
    assert torch.allclose(clamped_glu(h, wg, wu, wd, 0.5), (gg * torch.sigmoid(1.702 * gg) * (uu + 1)) @ wd.T)


# --------------------------------------------------------------------------- mechanisms on the GPU
def _ops_and_cache(n_seqs, needs, state_floats, dtype=torch.float32, tokens=64 * 16):
    from hilbert_pruned_8b_b200.cache.manager import CacheManager
    from hilbert_pruned_8b_b200.engine.workspace import Workspace
    from hilbert_pruned_8b_b200.kernels.ops import Ops
    from hilbert_pruned_8b_b200.parts.base import StateNeed
    dev = torch.device("cuda:0")
    ops, ws = Ops(dev), Workspace(dev)
    cache = CacheManager(needs, {0: StateNeed((state_floats,), torch.float32)} if state_floats else {}, tokens, dev, dtype)
    return ops, ws, cache, [cache.open() for _ in range(n_seqs)]


def _step(cache, ws, seqs, new):
    from hilbert_pruned_8b_b200.engine.batch import StepEntry, build_step
    entries = [StepEntry(s, [0] * n, []) for s, n in zip(seqs, new)]
    cache.reserve([(s, s.length + n) for s, n in zip(seqs, new)])
    return build_step(entries, cache, ws, torch.device("cuda:0"))


def _commit(cache, seqs, new):
    for s, n in zip(seqs, new):
        cache.commit(s, s.length + n)


def _portions(total, sizes):
    """Per round the new tokens of every sequence that still has some: [(live indices, new tokens)]."""
    done, out = [0] * len(total), []
    for portion in sizes:
        live = [i for i in range(len(total)) if done[i] < total[i]]
        if not live:
            break
        new = [min(portion, total[i] - done[i]) for i in live]
        out.append((live, new, list(done)))
        for i, n in zip(live, new):
            done[i] += n
    assert done == list(total), "the portions do not cover the sequences"
    return out


@pytest.mark.gpu
def test_norm_on_a_sublayer_output_and_the_weighted_sum():
    require_gpu()
    ops, ws, cache, seqs = _ops_and_cache(0, {}, 0)
    g = torch.Generator().manual_seed(1)
    for width in (72, 2500):                 # rows that a thread keeps in registers, and longer ones
        y, x = (torch.randn(19, width, generator=g) * 3).cuda(), torch.randn(19, width, generator=g).cuda()
        w, w2 = torch.randn(width, generator=g).cuda(), torch.randn(width, generator=g).cuda()
        want_x = x.double() + rms_norm(y.double(), w.double(), 1e-5)
        want_h = rms_norm(want_x, w2.double(), 1e-6)
        x1 = x.clone()
        ops.rmsnorm_add(y, w, 1e-5, 0.0, x1)
        assert (x1.double() - want_x).abs().max() < 1e-5
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 4e-2)):
            x2, h = x.clone(), torch.empty(19, width, dtype=dtype, device="cuda")
            ops.rmsnorm_add(y, w, 1e-5, 0.0, x2, then=(w2, 1e-6, 0.0), then_out=h)
            assert torch.equal(x2, x1) and (h.double() - want_h).abs().max() < tol
        out = torch.empty_like(x)
        ops.scaled_sum(x, 1.2, y, -0.7, out)
        assert (out.double() - (1.2 * x.double() - 0.7 * y.double())).abs().max() < 1e-5
    ops.check_errors()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,size,P", [(4, 2, 16, 8, 20, 6), (1, 1, 8, 12, 1, 1), (3, 3, 4, 4, 1000, 7), (4, 2, 64, 40, 33, 48),
                                             (2, 1, 32, 64, 100, 16), (6, 2, 24, 40, 64, 64), (2, 2, 128, 256, 37, 5), (2, 1, 16, 16, 50, 0),
                                             (4, 2, 64, 64, 44, 12), (2, 1, 128, 128, 70, 48), (2, 2, 64, 128, 33, 5), (2, 1, 128, 64, 200, 0)])
def test_pooled_window_attention_sees_exactly_the_window_and_the_whole_blocks(H, G, d, dv, size, P, dtype):
    """A prompt of 300 tokens, then tokens one by one.  For some queries one key is made to stand out (its score is far above
    the others, which are pushed far below zero by the heads' biases): the token just inside the window, the one just outside
    it, the newest pooled block that is seen, the block that is complete but not yet wholly before the window, a token on a page
    border.  The output then shows at once whether that key was seen, and with which value."""
    require_gpu()
    from hilbert_pruned_8b_b200.parts.base import CacheNeed
    needs = (CacheNeed(G, d, max(size, P), v_head_dim=dv), CacheNeed(G, d, None, v_head_dim=dv, stride=P, store_f32=True)) if P else CacheNeed(G, d, size, v_head_dim=dv)
    ops, ws, cache, seqs = _ops_and_cache(2, {0: needs}, 0, dtype)
    views = cache.view(0)
    tokens, pooled = views if P else (views, None)
    g = torch.Generator().manual_seed(H * 100 + size)
    n, n2 = 420, 97                         # a second, shorter sequence shares every step
    scale = 0.5
    qn, kn, v = torch.randn(n, H, d, generator=g), torch.randn(n, G, d, generator=g), torch.randn(n, G, dv, generator=g)
    qw, kw = torch.rand(H * d, generator=g) + 0.5, torch.rand(G * d, generator=g) + 0.5
    bias = torch.randn(H, generator=g) - 6.0
    # queries at 299 (the prompt's end), 300 (the first decoded token), 383 and 384 (a page border): each asks for one key
    probes = {299: 299 - size + 1, 300: 300 - size, 383: 320, 384: 383, 411: 411 - size + 1}
    if P:
        probes.update({305: ((305 - size + 1) // P - 1) * P + P // 2 if (305 - size + 1) // P >= 1 else 0,      # inside the newest block that is seen
                       341: ((341 - size + 1) // P) * P})                                                 # the next block: not yet seen
    eps = 1e-5
    q_raw, k_raw = qn.clone(), kn.clone()
    for p, key in probes.items():
        if 0 <= key < n:
            k_raw[key] = k_raw[key] * 3.0
            # the query points at that key (after the norms' weights) for every head
            kk = rms_norm(k_raw[key].reshape(-1).double(), kw.double(), eps).reshape(G, d)
            for h in range(H):
                q_raw[p, h] = (kk[h // (H // G)] / qw.view(H, d)[h].double() * 4.0).float()
    gate = torch.randn(n, H * dv, generator=g)
    proj = torch.cat([q_raw.reshape(n, -1), k_raw.reshape(n, -1), v.reshape(n, -1), gate, torch.zeros(n, 3)], 1)     # rows longer than what is read
    r = (lambda t: t.to(torch.bfloat16).double()) if dtype == torch.bfloat16 else (lambda t: t.double())
    qd = r(rms_norm(q_raw.reshape(n, -1).double(), qw.double(), eps)).view(n, H, d)
    kd = r(rms_norm(k_raw.reshape(n, -1).double(), kw.double(), eps)).view(n, G, d)
    want = sigmoid_pool_attention(qd, kd, r(v), bias.double(), scale, size, P or None).reshape(n, H * dv) * torch.sigmoid(gate.double())
    got = torch.zeros(n, H * dv, dtype=torch.float64)
    at2 = 0
    for live, new, done in _portions([n, n2], [300] + [1] * 200):
        step = _step(cache, ws, [seqs[i] for i in live], new)
        pin = torch.cat([proj[done[i]: done[i] + m] for i, m in zip(live, new)]).cuda()
        T = pin.shape[0]
        qb = torch.empty(T, H * d, dtype=dtype, device="cuda")
        ops.qk_norm_append(pin, qw.cuda(), kw.cuda(), eps, H, G, d, dv, qb, tokens, step, True)
        if P:
            ops.pool_blocks(tokens, pooled, step, P, G, d, dv)
        out = torch.empty(T, H * dv, dtype=dtype, device="cuda")
        ops.attention_pool(qb, tokens, pooled, step, bias.cuda(), pin[:, H * d + G * d + G * dv: H * d + G * d + G * dv + H * dv], out,
                           H, G, d, dv, scale, size, P, workspace=ws)
        got[done[0]: done[0] + new[0]] = out[: new[0]].cpu().double()
        if len(live) > 1:                   # the second sequence repeats the first one's start
            assert (out[new[0]:].cpu().double() - got[done[1]: done[1] + new[1]]).abs().max() < (1e-4 if dtype == torch.float32 else 3e-2)
        _commit(cache, [seqs[i] for i in live], new)
    ops.check_errors()
    tol = 2e-4 if dtype == torch.float32 else 4e-2
    err = (got - want).abs().max(1).values / want.abs().max(1).values.clamp(min=1.0)
    assert err.max() < tol, f"position {int(err.argmax())}: {float(err.max()):.3e}"
    # enough of the probed keys are visible ones: leaving one out, or seeing one too many, changes the output
    hit = [p for p, key in probes.items() if 0 <= key < n and (p - key < size or (P and (key // P) * P + P - 1 <= p - size))]
    assert len(hit) >= 3
    if P:
        # the pooled store holds the mean of what the cache holds, block by block, for the first sequence
        blocks = n // P
        page = seqs[0].pages[pooled.group][0]
        stored = pooled.k[page][:, : min(blocks, 64)].permute(1, 0, 2).cpu().double()
        # (bfloat16: a cached key may differ from the plain one by one rounding step, where 32-bit and 64-bit norms fall on two sides of a tie)
        assert (stored - pool_blocks(kd, P)[: min(blocks, 64)]).abs().max() < (1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("heads,d,dv", [(2, 8, 16), (1, 40, 33), (3, 64, 70), (2, 128, 32)])
def test_decayed_memory_in_portions_equals_the_recurrence(heads, d, dv):
    require_gpu()
    H = heads
    ops, ws, cache, seqs = _ops_and_cache(2, {}, H * d * dv)
    g = torch.Generator().manual_seed(d)
    width = 2 * H * d + 2 * H * dv
    total = [150, 11]
    proj = [torch.randn(n, width + 5, generator=g) for n in total]
    decay = torch.tensor([1.0, 0.0, 0.93][:H] if H <= 3 else [0.5] * H)
    nw = torch.randn(H * dv, generator=g)
    want = []
    for p in proj:
        pd, T = p.double(), p.shape[0]
        q, k = silu(pd[:, : H * d]).view(T, H, d), silu(pd[:, H * d: 2 * H * d]).view(T, H, d)
        v = silu(pd[:, 2 * H * d: 2 * H * d + H * dv]).view(T, H, dv)
        o = decayed_memory(q, k, v, decay.double()).reshape(T, H * dv)
        want.append(rms_norm(o, nw.double(), 1e-5) * torch.sigmoid(pd[:, 2 * H * d + H * dv: width]) * 1.1)
    state = cache.state_view(0)
    got = [[], []]
    for live, new, done in _portions(total, [1, 2, 1, 5, 70, 33, 1, 1, 64]):
        step = _step(cache, ws, [seqs[i] for i in live], new)
        pin = torch.cat([proj[i][done[i]: done[i] + n] for i, n in zip(live, new)]).cuda()
        o = torch.empty(pin.shape[0], H * dv, device="cuda")
        ops.decay_memory(pin, decay.cuda(), state, step, o, H, d, dv, "silu")
        out = torch.empty_like(o)
        ops.gated_norm(o, pin[:, 2 * H * d + H * dv: width], nw.cuda(), 1e-5, out, 1.1)
        oc, at = out.cpu(), 0
        for i, n in zip(live, new):
            got[i].append(oc[at: at + n])
            at += n
        _commit(cache, [seqs[i] for i in live], new)
    for i in range(2):
        err = (torch.cat(got[i]).double() - want[i]).abs().max().item()
        assert err < 5e-5 * max(1.0, want[i].abs().max().item()), err
    # a slot that is used again starts from zeros
    for s in seqs:
        cache.close(s)
    again = cache.open()
    step = _step(cache, ws, [again], [total[1]])
    o = torch.empty(total[1], H * dv, device="cuda")
    ops.decay_memory(proj[1].cuda(), decay.cuda(), state, step, o, H, d, dv, "silu")
    out = torch.empty_like(o)
    ops.gated_norm(o, proj[1][:, 2 * H * d + H * dv: width].cuda(), nw.cuda(), 1e-5, out, 1.1)
    assert (out.cpu().double() - want[1]).abs().max() < 5e-5 * max(1.0, want[1].abs().max().item())


@pytest.mark.gpu
@pytest.mark.parametrize("inner,n_state,dt_rank,taps", [(96, 8, 5, 3), (40, 1, 1, 1), (70, 33, 2, 5), (256, 16, 16, 4), (24, 100, 3, 2)])
def test_convolution_and_selective_scan_carry_their_state_over_portions(inner, n_state, dt_rank, taps):
    """Two sequences of unequal lengths fed in portions of 1, 2, ... and of several hundred tokens (those run as chunks side by
    side): the values of the whole sequence at once.  Some channels forget almost nothing (step sizes near zero), some almost
    everything."""
    require_gpu()
    I, N, R = inner, n_state, dt_rank
    conv_state = (taps - 1) * I
    ops, ws, cache, seqs = _ops_and_cache(2, {}, conv_state + I * N)
    g = torch.Generator().manual_seed(inner + taps)
    total = [700, 23]
    xz = [torch.randn(n, 2 * I + 4, generator=g) for n in total]
    cw, cb = torch.randn(I, taps, generator=g) * 0.5, torch.randn(I, generator=g) * 0.3
    wx = torch.randn(R + 2 * N, I, generator=g) / I ** 0.5
    wdt, bdt = torch.randn(I, R, generator=g), torch.randn(I, generator=g) * 3.0 - 3.0
    a_log, D = torch.log(torch.rand(I, N, generator=g) * 3 + 0.2), torch.randn(I, generator=g)
    want = []
    for m in xz:
        md = m.double()
        u = silu(causal_conv_bias(md[:, :I], cw.double(), cb.double()))
        dbc = u @ wx.double().T
        dt = softplus(dbc[:, :R] @ wdt.double().T + bdt.double())
        y = selective_scan(u, dt, -torch.exp(a_log.double()), dbc[:, R:R + N], dbc[:, R + N:], D.double())
        want.append((u, y * silu(md[:, I:2 * I])))
    state = cache.state_view(0)
    got_u, got_y = [[], []], [[], []]
    for live, new, done in _portions(total, [1, 2, 3, 300, 1, 17, 2, 260, 200]):
        step = _step(cache, ws, [seqs[i] for i in live], new)
        pin = torch.cat([xz[i][done[i]: done[i] + n] for i, n in zip(live, new)]).cuda()
        T = pin.shape[0]
        u = torch.empty(T, I, device="cuda")
        ops.conv_act(pin[:, :I], cw.cuda(), cb.cuda(), state[:, :conv_state], step, u, "silu")
        dbc = (u.double() @ wx.double().cuda().T).float().contiguous()       # the projections themselves are not under test here
        dt_raw = (dbc[:, :R].double() @ wdt.double().cuda().T).float().contiguous()
        y = torch.empty(T, I, device="cuda")
        ops.selective_scan(u, dbc[:, R:], pin[:, I:2 * I], dt_raw, bdt.cuda(), a_log.cuda(), D.cuda(), state[:, conv_state:], step, y, N, workspace=ws,
                           chunked=max(new) >= 128)
        uc, yc, at = u.cpu(), y.cpu(), 0
        for i, n in zip(live, new):
            got_u[i].append(uc[at: at + n])
            got_y[i].append(yc[at: at + n])
            at += n
        _commit(cache, [seqs[i] for i in live], new)
    for i in range(2):
        assert (torch.cat(got_u[i]).double() - want[i][0]).abs().max() < 2e-5
        err = (torch.cat(got_y[i]).double() - want[i][1]).abs().max().item()
        assert err < 1e-4 * max(1.0, want[i][1].abs().max().item()), err


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,E,top,F,limit", [(64, 6, 2, 24, 1.5), (48, 3, 3, 16, 0.7), (40, 4, 1, 20, 1.0), (128, 40, 5, 70, 2.0), (192, 8, 2, 136, 2.0)])
def test_mixture_of_experts(W, E, top, F, limit, dtype):
    """Router, plan, the experts' products and the weighted sum for 1, a few and many tokens, written and added."""
    require_gpu()
    ops, ws, cache, seqs = _ops_and_cache(0, {}, 0)
    g = torch.Generator().manual_seed(E * 10 + top)
    rd = (lambda t: t.to(torch.bfloat16)) if dtype == torch.bfloat16 else (lambda t: t)
    wr = rd(torch.randn(E, W, generator=g) * 4 / W ** 0.5)
    wg, wu = rd(torch.randn(E, F, W, generator=g) * 2 / W ** 0.5), rd(torch.randn(E, F, W, generator=g) * 2 / W ** 0.5)
    wd = rd(torch.randn(E, W, F, generator=g) / F ** 0.5)
    for T in (1, 5, 333):
        h = rd(torch.randn(T, W, generator=g))
        experts = torch.empty(T, top, dtype=torch.int32, device="cuda")
        weights = torch.empty(T, top, device="cuda")
        ops.moe_route(h.cuda(), wr.float().cuda(), top, experts, weights)
        idx, wgt = route(h.double() @ wr.double().T, top)
        assert torch.equal(experts.cpu().long(), idx) and (weights.cpu().double() - wgt).abs().max() < 1e-5
        want = torch.zeros(T, W, dtype=torch.float64)
        r = (lambda t: t.to(torch.bfloat16).double()) if dtype == torch.bfloat16 else (lambda t: t)
        for e in range(E):
            rows, slot = (idx == e).nonzero(as_tuple=True)
            if rows.numel():
                want[rows] += wgt[rows, slot][:, None] * clamped_glu(h.double()[rows], wg[e].double(), wu[e].double(), wd[e].double(), limit, r)
        base = torch.randn(T, W, generator=g)
        out = base.clone().cuda()
        ops.moe_experts(h.cuda(), experts, weights, wg.cuda(), wu.cuda(), wd.cuda(), limit, 1.702, out, True, ws, 400)
        tol = 1e-4 if dtype == torch.float32 else 3e-2
        assert (out.cpu().double() - base.double() - want).abs().max() < tol * max(1.0, want.abs().max().item())
        ops.moe_experts(h.cuda(), experts, weights, wg.cuda(), wu.cuda(), wd.cuda(), limit, 1.702, out, False, ws, 400)
        assert (out.cpu().double() - want).abs().max() < tol * max(1.0, want.abs().max().item())
    gu = torch.randn(7, 2 * 30, generator=g) * 2
    act = torch.empty(7, 30, device="cuda")
    ops.glu_clamp(gu.cuda(), act, 0.8, 1.702)
    gg, uu = torch.clamp(gu[:, :30].double(), max=0.8), torch.clamp(gu[:, 30:].double(), -0.8, 0.8)
    assert (act.cpu().double() - gg * torch.sigmoid(1.702 * gg) * (uu + 1)).abs().max() < 1e-6
    ops.check_errors()


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
    assert all(g.pool.num_free == g.pool.size for g in eng.cache.groups) and eng.cache.slots.num_held == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_tokens_one_by_one(models, name, dtype):
    """The decoded tokens carry windows and blocks over the prompt's end and over page borders."""
    require_gpu()
    folder, cfg, plain = models[name]
    reqs = _requests(cfg, [3, 60, 190], 200)
    steps, peak = tt.trace_tail(reqs, tail=75)
    eng = _engine(folder, dtype, peak)
    _compare(tt.run_in_process(eng, steps), _reference(plain[dtype], reqs), dtype, "tail")
    assert eng.graph_replays > 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompts_in_portions(models, name, dtype):
    """A prompt cut into portions of 2, 3, 1, 64, 5 ... tokens, and cut by the engine itself when a step brings more tokens
    than it takes at once."""
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
    assert all(g.pool.num_free == g.pool.size for g in eng.cache.groups) and eng.cache.slots.num_held == 0


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_long_decoding(models, name):
    """Hundreds of single-token steps through the captured graphs: windows slide off their pages, which are given back,
    pooled blocks fill more than one page of their own."""
    require_gpu()
    folder, cfg, plain = models[name]
    toks = tt.random_tokens(460, cfg["vocab"], 600)
    steps = [{"step": 0, "entries": [{"id": "l", "tokens": toks[:4], "want": [3]}], "end": []}]
    for p in range(4, len(toks)):
        steps.append({"step": len(steps), "entries": [{"id": "l", "tokens": [toks[p]], "want": [0]}],
                      "end": ["l"] if p == len(toks) - 1 else []})
    eng = _engine(folder, "float32", 512)
    got = tt.run_in_process(eng, steps)
    ref = _reference(plain["float32"], {"l": toks})
    _compare(got, {k: ref[k] for k in got}, "float32", "long decoding")
    assert eng.graph_replays > 400


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
def test_the_two_norms_between_sublayers_in_one_pass_or_two(models, name):
    require_gpu()
    folder, cfg, plain = models[name]
    reqs = _requests(cfg, [50, 3], 700)
    steps, peak = tt.trace_tail(reqs, tail=5)
    a = tt.run_in_process(_engine(folder, "float32", peak), steps)
    eng = _engine(folder, "float32", peak)
    for b in eng.model.blocks:
        b.fuse_norms = False
    b = tt.run_in_process(eng, steps)
    for k in a:
        assert (a[k] - b[k]).abs().max() < 1e-4


@pytest.mark.gpu
def test_prompt_attention_on_the_tensor_cores_equals_the_fp32_kernel(models):
    """bfloat16 prompts with head sizes of 64: the window on the tensor cores plus the pooled blocks' share, against the
    kernel that does both on the FP32 pipe."""
    require_gpu()
    folder, cfg, plain = models["wide"]
    v = cfg["vocab"]
    batches = [{f"k{i}": (tt.random_tokens(n, v, 950 + i), p) for i, (n, p) in enumerate([(260, 250), (20, 17), (70, 64)])}]
    steps, peak = tt.trace_batches(batches)
    a = tt.run_in_process(_engine(folder, "bfloat16", peak), steps)
    eng = _engine(folder, "bfloat16", peak)
    eng.ctx.ops.use_mma_pool_attention = False
    b = tt.run_in_process(eng, steps)
    close = sum((a[k] - b[k]).abs().max().item() <= 2e-2 * max(1.0, b[k].abs().max().item()) for k in a)
    assert close >= 0.9 * len(a), f"{len(a) - close} of {len(a)} positions differ"      # (a router's near tie may fall the other way)


def _greedy(plain, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(plain.logits(toks)[-1].argmax()))
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
    assert all(g.pool.num_free == g.pool.size for g in llm.engine.cache.groups)


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
