"""Bizepel on the GPU against the plain implementation (tests/plain_bizepel.py): the new kernels alone, every mixer and
feed-forward as one-layer models, keys made to stand out at the edges of windows, kept positions and pages, states
that must survive hundreds of tokens, then whole models from small configurations with random weights: prompts,
token-by-token decoding, portions, batches of unequal requests, slots used again, long decoding, greedy generation,
trace replay."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT, close_enough, has_gpu
from bizepel_configs import CONFIGS, _attention, _delta, _dense, _layer, _mamba, _model, _moe

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not has_gpu(), reason="needs a CUDA device")]
DEV = "cuda:0"


def _ops():
    from ultima_b200.kernels import ops
    return ops


def rel_err(got, ref):
    got, ref = got.double().cpu(), ref.double().cpu()
    return float((got - ref).abs().max() / max(1e-30, float(ref.abs().max())))


def _ids(seed, n, vocab, avoid=()):
    ids = np.random.default_rng(seed).integers(0, vocab, size=n).tolist()
    if avoid:
        free = [t for t in range(vocab) if t not in avoid]
        ids = [free[t % len(free)] for t in ids]
    return ids


def _all(n):
    return list(range(n))


def agree(got, ref, dtype, layers, what):
    """float32: every position within rounding.  bfloat16: the same bound for all but a few positions, since a router
    whose two candidates lie within rounding of each other may choose the other one there."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    if dtype == "float32":
        err, bound = close_enough(got, ref, dtype, layers)
        assert err <= bound, (what, err, bound)
        return
    assert got.shape == ref.shape and np.isfinite(got).all(), what
    _, bound = close_enough(got, ref, dtype, layers)
    rows = np.abs(got - ref).max(axis=-1)
    over = int((rows > bound).sum())
    assert over <= max(1, len(rows) // 25) and float(np.median(rows)) <= bound / 2, (what, over, len(rows), float(rows.max()), bound)


class _Batch:
    """The step record's arrays that the row-wise kernels read, for sequences that bring ``lens`` tokens."""

    def __init__(self, lens, slots):
        start = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        self.n_seqs, self.n_tokens = len(lens), int(start[-1])
        self.seq_start = torch.tensor(start, dtype=torch.int32, device=DEV)
        self.seq_slot = torch.tensor(slots, dtype=torch.int32, device=DEV)
        self.tok_seq = torch.tensor(np.repeat(np.arange(len(lens)), lens), dtype=torch.int32, device=DEV)


# ---------------------------------------------------------------------------------------
# the row-wise kernels
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,width", [(1, 48), (37, 100), (5, 257), (3, 1024), (9, 2048), (2, 4100)])
def test_layer_norm_and_the_join_that_writes_the_next_norm(T, width, out_dtype):
    import plain_bizepel as P
    ops = _ops()
    g = torch.Generator().manual_seed(T * 7 + width)
    x = torch.randn(T, width, generator=g) * 3 + 1.5              # a mean far from zero: the variance is about the mean
    w = 1 + 0.2 * torch.randn(width, generator=g)
    eps = 1e-5
    tol = 1e-5 if out_dtype == torch.float32 else 2 ** -7
    out = torch.empty(T, width, dtype=out_dtype, device=DEV)
    ops.layernorm(x.to(DEV), w.to(DEV), out, eps)
    assert rel_err(out, P.layer_norm(x.double(), w.double(), eps)) < tol
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, width, dtype=out_dtype, device=DEV)
    ops.layernorm(x.to(DEV), w.to(DEV), out2, eps, rows)
    assert rel_err(out2, P.layer_norm(x.double(), w.double(), eps)[[T - 1, 0]]) < tol
    y = torch.randn(T, width, generator=g)
    s = torch.randn(width, generator=g)
    new = x.double() + s.double() * y.double()
    for mode, ref in ((ops.NEXT_NONE, None), (ops.NEXT_PLAIN, new), (ops.NEXT_RMS, P.rms_norm(new, w.double(), eps)),
                      (ops.NEXT_LAYER, P.layer_norm(new, w.double(), eps))):
        xd, yd = x.to(DEV), y.to(DEV)
        o = torch.empty(T, width, dtype=out_dtype, device=DEV) if ref is not None else None
        ops.scale_add_norm(yd, s.to(DEV), xd, mode, w.to(DEV) if mode >= ops.NEXT_RMS else None, eps, o)
        assert rel_err(xd, new) < 1e-6 and float(yd.abs().max()) == 0.0
        if ref is not None:
            assert rel_err(o, ref) < tol, mode


@pytest.mark.parametrize("long", [False, True])
@pytest.mark.parametrize("taps", [1, 2, 3, 4, 7])
@pytest.mark.parametrize("C", [5, 64, 300])
def test_the_causal_convolution_over_portions_with_its_state(taps, C, long):
    """Two sequences of unequal lengths in slots 3 and 1, cut into portions down to one token: the inputs of before a
    portion come from the state, zeros before the start; with a bias on the inputs, with the input added, with a bias
    of its own and SiLU, from a projection in K slices and from a column range of a wider row.  ``long``: portions of a
    hundred tokens and more, which take the kernels that walk tokens (a channel, or four neighbouring ones, a thread)."""
    import plain_bizepel as P
    ops = _ops()
    g = torch.Generator().manual_seed(taps * 100 + C)
    lens = [150, 90] if long else [23, 9]
    cuts = ([100, 64], [1, 1], [49, 25]) if long else ([4, 1], [1, 1], [2, 2], [10, 5], [6, 0])
    u = [torch.randn(n, C, generator=g) for n in lens]
    w = torch.randn(C, taps, generator=g)
    bias, ob = torch.randn(C, generator=g), torch.randn(C, generator=g)
    for variant in ("plain", "input_bias", "residual", "out_bias_silu", "slices"):
        refs = []
        for x in u:
            xin = (x + bias if variant == "input_bias" else x).double()
            r = P.causal_conv(xin, w.double())
            if variant == "residual":
                r = r + xin
            if variant == "out_bias_silu":
                r = P.silu(r + ob.double())
            refs.append(r)
        state = torch.full((5, max(taps - 1, 1), C), 9.0, device=DEV)
        state[[3, 1]] = 0.0                                        # a slot that is acquired starts at zero
        state = state[:, :taps - 1].contiguous() if taps > 1 else None
        at = [0, 0]
        got = [[], []]
        for cut in cuts:
            live = [i for i in (0, 1) if cut[i] > 0]
            b = _Batch([cut[i] for i in live], [[3, 1][i] for i in live])
            x = torch.cat([u[i][at[i]:at[i] + cut[i]] for i in live])
            off = 0
            if variant == "slices":                                # the sum of three slices, in columns 7.. (or 8..) of a wider row
                off = 8 if long and C % 4 == 0 else 7
                parts = torch.randn(3, x.shape[0], C + 12, generator=g)
                parts[2, :, off:off + C] = x - parts[0, :, off:off + C] - parts[1, :, off:off + C]
                x = parts
            xd = x.to(DEV)
            out = torch.empty(b.n_tokens, C, device=DEV)
            kw = {"bias": bias.to(DEV)} if variant == "input_bias" else {}
            one_each = all(cut[i] == 1 for i in live)              # one token a sequence: the kernel moves the state on itself
            ops.causal_conv(xd, w.to(DEV), state, b, out, col_off=off, add_input=variant == "residual", update_state=one_each,
                            silu=variant == "out_bias_silu", out_bias=ob.to(DEV) if variant == "out_bias_silu" else None, **kw)
            if taps > 1 and not one_each:
                ops.causal_conv_state(xd, state, b, col_off=off, **kw)
            o = 0
            for i in live:
                got[i].append(out[o:o + cut[i]].cpu())
                o += cut[i]
                at[i] += cut[i]
        for i in (0, 1):
            assert rel_err(torch.cat(got[i]), refs[i][:at[i]]) < (1e-5 if variant != "slices" else 1e-4), (variant, i)
        if taps > 1:
            assert float(state[0].min()) == 9.0                    # other slots are not touched


def test_values_handed_from_one_layer_to_another_and_blended():
    ops = _ops()
    g = torch.Generator().manual_seed(1)
    T, C, lo = 6, 40, 24
    x, y = torch.randn(T, C, generator=g), torch.randn(T, C, generator=g)
    lam = torch.tensor([0.3])
    b = _Batch([T], [0])
    shared = torch.zeros(T, C - lo, device=DEV)
    o1, o2 = torch.empty(T, C, device=DEV), torch.empty(T, C, device=DEV)
    ops.causal_conv(x.to(DEV), None, None, b, o1, mix=(1, lo, C, lam.to(DEV), shared))
    assert torch.equal(o1.cpu(), x) and torch.equal(shared.cpu(), x[:, lo:])
    ops.causal_conv(y.to(DEV), None, None, b, o2, mix=(2, lo, C, lam.to(DEV), shared))
    ref = y.clone()
    ref[:, lo:] = 0.7 * y[:, lo:] + 0.3 * x[:, lo:]
    assert rel_err(o2, ref) < 1e-6


@pytest.mark.parametrize("ne,groups,top,scale", [(6, (3, 2), 2, 1.7), (20, (4, 1), 4, 1.9), (5, None, 3, 1.0), (4, None, 1, 0.5),
                                                 (12, (4, 3), 4, 1.0), (8, (8, 2), 2, 3.0), (64, (8, 3), 6, 2.5), (3, (3, 3), 3, 1.0)])
def test_the_sigmoid_router_scores_groups_by_their_two_best_and_renormalises(ne, groups, top, scale):
    """The correction is larger than the scores and partly negative, so that choice scores are negative too: an expert
    outside the kept groups must count as minus infinity, not as 0; a group of one expert has one score to sum."""
    import plain_bizepel as P
    ops = _ops()
    T = 200
    g = torch.Generator().manual_seed(ne)
    z = (torch.randn(T, ne, generator=g) * 2).float()
    corr = (torch.randn(ne, generator=g) * 0.6 - 0.8).float()
    f = {"router": {"experts": ne, "top": top, "scale": scale}}
    if groups:
        f["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    ref_idx, ref_w = P.route(z.double(), {"r.router": torch.eye(ne, dtype=torch.float64), "r.correction": corr.double()}, f, "r.")
    mode = ops.ROUTE_SIGMOID | ops.ROUTE_GROUP_TOP2 | ops.ROUTE_NORMALISE
    idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, device=DEV)
    counts = torch.zeros(ne, dtype=torch.int32, device=DEV)
    ops.route(z.to(DEV), corr.to(DEV), ne, top, groups[0] if groups else 1, groups[1] if groups else 1, idx, wts, counts,
              mode=mode, wscale=scale)
    idx, wts = idx.cpu().long(), wts.cpu().double()
    for t in range(T):
        got = dict(zip(idx[t].tolist(), wts[t].tolist()))
        want = dict(zip(ref_idx[t].tolist(), ref_w[t].tolist()))
        assert set(got) == set(want), (t, got, want)
        assert all(abs(got[e] - want[e]) < 1e-6 * max(1.0, scale) for e in want), (t, got, want)
    assert counts.cpu().tolist() == torch.bincount(ref_idx.flatten(), minlength=ne).tolist()


# ---------------------------------------------------------------------------------------
# models
# ---------------------------------------------------------------------------------------
_TINY = _mamba(16, 2, 2, 2)
ONE_LAYER = {
    "attention_all": _model([_layer("attention", _attention(6, 2, 16, 24, 0.4, conv=3, rot=(100.0, 8), mask=(45, 5)))]),
    "attention_equal_heads_window_only": _model([_layer("attention", _attention(4, 2, 32, 32, 0.2, conv=2, rot=(1000.0, 32), mask=(40, 0)))]),
    "attention_equal_heads_kept": _model([_layer("attention", _attention(2, 1, 64, 64, 0.15, conv=4, rot=(10000.0, 32), mask=(30, 7)))]),
    "attention_bare": _model([_layer("attention", _attention(2, 2, 40, 8, 0.3))], width=72, taps=0, side=0),
    "attention_one_head_window_one": _model([_layer("attention", _attention(1, 1, 64, 64, 0.2, conv=1, rot=(50.0, 2), mask=(1, 0)))]),
    "mamba_small": _model([_layer("mamba1", _mamba(40, 7, 3, 4))]),
    "mamba_one_tap_wide_state": _model([_layer("mamba1", _mamba(24, 70, 9, 1))], width=56, taps=1),
    "mamba_state_of_one": _model([_layer("mamba1", _mamba(130, 1, 1, 5))]),
    "delta_small": _model([_layer("general_delta", _delta(3, 16, 4))]),
    "delta_one_head": _model([_layer("general_delta", _delta(1, 72, 16))], width=56, side=3),
    "delta_heads_of_six": _model([_layer("general_delta", _delta(5, 6, 1))], width=40),
    "dense": _model([_layer("mamba1", _TINY, _dense(70))]),
    "routed_groups": _model([_layer("mamba1", _TINY, _moe(10, 3, 24, scale=2.0, groups=(5, 2), shared=40))]),
    "routed_plain": _model([_layer("mamba1", _TINY, _moe(7, 7, 16))], width=48),
    "routed_groups_of_one": _model([_layer("mamba1", _TINY, _moe(6, 2, 32, scale=0.7, groups=(6, 3)))], taps=5),
}


def _sharpen(W):
    """Random weights changed so that faults show: projections large enough that states, experts and the token input
    carry weight against the skip paths, q/k norm weights large enough that attention weights are far from uniform,
    layer scales near one (a layer's result counts), value mixing between 0.2 and 0.8."""
    out = {}
    for n, t in W.items():
        leaf = n.split(".")[-1]
        if ".mix." in n and t.dim() == 2 and leaf not in ("conv", "A_log"):
            t = t * 4
        if ".mlp." in n and leaf in ("up", "down"):
            t = t * 6
        if n.endswith("side.gate"):
            t = t * 6
        if n.endswith("q.norm"):
            t = t * 1.8
        if leaf in ("ls1", "ls2"):
            t = t + 1.0
        if leaf == "vmix":
            t = t * 0 + (0.35 if "l1." in n or "l3." in n else 0.6)
        out[n] = t.to(torch.bfloat16)
    return out


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    import plain_bizepel as P
    import ultima_b200 as u
    from ultima_b200.weights.safetensors_io import write_safetensors
    base = tmp_path_factory.mktemp("bizepel")
    made = {}

    def get(name, raw=None, change=None):
        if name not in made:
            d = str(base / name.replace("/", "_"))
            plain_name = name.split("/")[0]
            raw = copy.deepcopy(raw or CONFIGS.get(plain_name) or ONE_LAYER[plain_name])
            if name.endswith("/all_chosen"):
                for L in raw["layers"]:
                    if L.get("mlp") and L["mlp"]["kind"] == "moe":
                        r = L["mlp"]["router"]
                        r["top"] = r["experts"]
                        if r.get("groups"):
                            r["groups"]["keep"] = r["groups"]["count"]
            u.write_random_model(d, u.config_from_dict(raw), seed=len(plain_name), dtype="bfloat16")
            cfg, W = P.read_folder(d)
            W = _sharpen(W)
            if change is not None:
                W = {n: t.to(torch.bfloat16) for n, t in change(cfg, {n: t.double() for n, t in W.items()}).items()}
            write_safetensors(os.path.join(d, "model.safetensors"), W)
            made[name] = (d,) + P.read_folder(d)
        return made[name]
    return get


_engines = {}


def _engine(folder, dtype, **kw):
    from ultima_b200.engine import Engine
    key = (folder, dtype, tuple(sorted(kw.items())))
    if key not in _engines:
        _engines[key] = Engine.from_dir(folder, dtype=dtype, with_sampler=False, **{"max_tokens": 2048, "max_seqs": 6, **kw})
    return _engines[key]


def _for(name, dtype):
    """The model's folder for a run in ``dtype``.  In bfloat16 a router's near tie between two experts may go either
    way, and one other choice reaches every later position through states and keys; so the bfloat16 runs of whole
    models use the same models with routers that choose every expert (the weights still differ from token to token).
    The choice itself is held to the plain implementation by the 32-bit runs of the same models, by the one-layer
    models in both types and by the router's own test."""
    return name + "/all_chosen" if dtype == "bfloat16" else name


def _whole(eng, ids, want=None):
    s = eng.open(1)
    got = eng.step(s, [ids], [want if want is not None else _all(len(ids))]).cpu().numpy()
    eng.close(s)
    eng.check_errors()
    return got


def _prompt_then_single_tokens(eng, ids, cut, want_from=0):
    s = eng.open(1)
    rows = [eng.step(s, [ids[:cut]], [list(range(want_from, cut))]).cpu().numpy()]
    for t in range(cut, len(ids)):
        rows.append(eng.step(s, [[ids[t]]]).cpu().numpy())
    eng.close(s)
    eng.check_errors()
    return np.concatenate(rows)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_one_layer_alone_in_a_prompt_and_token_by_token(folders, name, dtype):
    import plain_bizepel as P
    d, cfg, W = folders(name)
    eng = _engine(d, dtype, poison_cache=True)
    ids = _ids(len(name), 150, cfg["vocab"])
    ref = P.logits(cfg, W, ids)
    if dtype == "float32":
        taps, layers = [], []
        eng.model.tap = lambda i, x: taps.append(x.detach().double().cpu())
        got = _whole(eng, ids)
        eng.model.tap = None
        with torch.no_grad():
            P.forward(cfg, W, ids, torch.float64, layers)
        assert rel_err(taps[0], layers[0]) < 2e-5, name            # the stream behind the layer
    else:
        got = _whole(eng, ids)
    agree(got, ref, dtype, 2, (name, dtype, "prompt"))
    agree(_prompt_then_single_tokens(eng, ids, 70), ref, dtype, 2, (name, dtype, "decoded"))
    agree(_prompt_then_single_tokens(eng, ids[:40], 1), ref[:40], dtype, 2, (name, dtype, "from the first token"))


# ---------------------------------------------------------------------------------------
# one key made to stand out: it is seen exactly where the mask says so
# ---------------------------------------------------------------------------------------
ASKER, MARKED = 5, 11


def _stand_out(cfg, W):
    """Layer 0's queries of token ASKER are turned towards the keys of token MARKED (a rank-one change of W_q a head), so
    that this one score lies far above the others, and MARKED's values are made large.  In these models the input
    convolution and the convolutions of q and k look at the current token only (their earlier taps are zero), so that
    a token's key is the same wherever it stands; v's convolution stays as drawn."""
    import plain_bizepel as P
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    if "l0.canon1" in W:
        W["l0.canon1"][:, :-1] = 0
    for n in ("q", "k"):
        if f"l0.mix.{n}.conv" in W:
            W[f"l0.mix.{n}.conv"][:, :-1] = 0
            W[f"l0.mix.{n}.conv"][:, -1] = 1
    h = {}
    for t in (ASKER, MARKED):
        x = P.layer_norm(P.layer_norm(W["embed"][t], W["embed.norm"], eps), W["l0.norm1"], eps)
        h[t] = x * (1 + W["l0.canon1"][:, -1]) if "l0.canon1" in W else x
    towards = h[ASKER] / (h[ASKER] @ h[ASKER])
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    k = (W["l0.mix.k"] @ h[MARKED] + W["l0.mix.k.b"]).view(G, d)
    q = W["l0.mix.q"].clone()
    for a in range(H):
        kh = k[a // (H // G)]
        q[a * d:(a + 1) * d] += torch.outer(kh / kh.norm() * 40.0, towards)
    W["l0.mix.q"] = q
    W["l0.mix.q.norm"] = W["l0.mix.q.norm"] * 0 + 12.0 / (m["scale"] * d)     # a score of about 12 for the marked key
    W["l0.mix.k.norm"] = W["l0.mix.k.norm"] * 0 + 1.0
    W["l0.mix.v"] = W["l0.mix.v"] + torch.outer(torch.ones(W["l0.mix.v"].shape[0], dtype=torch.float64) * 4.0,
                                                h[MARKED] / (h[MARKED] @ h[MARKED]))
    return W


MARKED_MODELS = {
    # name: (model, window, kept first positions)
    "marked_window_kept": (_model([_layer("attention", _attention(4, 2, 32, 16, 0.2, conv=3, rot=(10000.0, 4), mask=(70, 9), v_mix=True)),
                                   _layer("mamba1", _mamba(32, 4, 2, 3))]), 70, 9),
    "marked_page_window": (_model([_layer("attention", _attention(2, 1, 16, 32, 0.3, conv=2, rot=(10000.0, 2), mask=(64, 64)))]), 64, 64),
    "marked_equal_heads": (_model([_layer("attention", _attention(2, 2, 64, 64, 0.12, conv=4, rot=(10000.0, 8), mask=(40, 3)))]), 40, 3),
    "marked_window_only": (_model([_layer("attention", _attention(3, 1, 32, 32, 0.2, conv=2, mask=(50, 0)))]), 50, 0),
    "marked_no_window": (_model([_layer("attention", _attention(3, 3, 32, 16, 0.25, conv=3, rot=(10000.0, 2)))]), None, 0),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(MARKED_MODELS))
def test_a_key_just_inside_and_outside_the_window_among_the_kept_positions_at_page_borders_and_far_away(folders, name, dtype):
    import plain_bizepel as P
    raw, window, keep = MARKED_MODELS[name]
    d, cfg, W = folders(name, raw, _stand_out)
    eng = _engine(d, dtype, poison_cache=True)
    cases = []                                                   # (place of the marked key, place of the asking token)
    if window is None:
        cases = [(0, 1), (3, 420), (63, 64), (64, 300), (0, 449)]
    else:
        for m in sorted({0, 1, 63, 64, 127, 200, max(keep - 1, 0), keep, keep + 1}):
            cases += [(m, m + window - 1), (m, m + window), (m, m + 1), (m, m + window + 1), (m, m + window + 130)]
    for m, p in cases:
        ids = _ids(m * 1000 + p, p + 1, cfg["vocab"], avoid=(ASKER, MARKED))
        ids[m], ids[p] = MARKED, ASKER
        ref = P.logits(cfg, W, ids)[p]
        seen = window is None or p - m < window or m < keep
        without = list(ids)
        without[m] = ids[m + 1] if m + 1 < p else ids[m - 1]
        bound = close_enough(ref[None], ref[None], dtype, 2)[1]
        moved = float(np.abs(P.logits(cfg, W, without)[p] - ref).max())
        assert moved > 0.06 or not seen, (name, m, p, moved)      # the test's weights do show the key where it is seen
        got = _whole(eng, ids, [p])[0]                             # the asking token in a prompt
        err = float(np.abs(got - ref).max())
        assert err <= bound, (name, dtype, m, p, "prompt", err, bound)
        cut = max(1, p - 3)                                         # and decoded alone, three tokens behind the prompt
        got = _prompt_then_single_tokens(eng, ids, cut, want_from=cut - 1)[-1]
        err = float(np.abs(got - ref).max())
        assert err <= bound, (name, dtype, m, p, "decoded", err, bound)


def test_states_keep_an_early_input_over_hundreds_of_tokens(folders):
    """A recurrent state that is lost would hide behind fast decays: here the decays are close to one, so the first
    tokens still count after hundreds, in a prompt and decoded token by token."""
    import plain_bizepel as P

    def slow_scan(cfg, W):
        W["l0.mix.A_log"] = W["l0.mix.A_log"] * 0 - 7.0
        W["l0.mix.x"] = W["l0.mix.x"] * 2.5                # the state's share of the output against the skip path
        return W

    def slow_delta(cfg, W):
        W["l0.mix.w0"] = W["l0.mix.w0"] * 0 - 8.0          # decays of exp(-0.0002)
        W["l0.mix.a.b"] = W["l0.mix.a.b"] * 0 - 4.0        # little is removed
        W["l0.mix.w2"] = W["l0.mix.w2"] * 0.1
        W["l0.mix.a"] = W["l0.mix.a"] * 0.1
        return W
    for name, raw, change in (("slow_scan", _model([_layer("mamba1", _mamba(48, 6, 4, 3))]), slow_scan),
                              ("slow_delta", _model([_layer("general_delta", _delta(2, 16, 4))]), slow_delta)):
        d, cfg, W = folders(name, raw, change)
        ids = _ids(2, 400, cfg["vocab"])
        ref = P.logits(cfg, W, ids)
        other = P.logits(cfg, W, _ids(3, 4, cfg["vocab"]) + ids[4:])
        assert np.abs(other[-1] - ref[-1]).max() > 1e-3, name       # the first four tokens still count at the end
        for dtype in ("float32", "bfloat16"):
            eng = _engine(d, dtype)
            agree(_whole(eng, ids), ref, dtype, 2, (name, dtype, "prompt"))
            agree(_prompt_then_single_tokens(eng, ids, 150)[-200:], ref[-200:], dtype, 2, (name, dtype, "decoded"))


# ---------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_a_prompt_in_one_step_every_position_and_every_layer(folders, name, dtype):
    import plain_bizepel as P
    d, cfg, W = folders(_for(name, dtype))
    eng = _engine(d, dtype, poison_cache=True)
    L = len(cfg["layers"])
    for seed, n in ((1, 1), (2, 2), (3, 277)):                 # 277: past window and page borders of every configuration
        ids = _ids(seed, n, cfg["vocab"])
        taps, layers = [], []
        eng.model.tap = lambda i, x: taps.append(x.detach().double().cpu())
        got = _whole(eng, ids)
        eng.model.tap = None
        with torch.no_grad():
            ref = P.forward(cfg, W, ids, torch.float64, layers).numpy()
        assert len(taps) == len(layers) == L
        if dtype == "float32":
            for i, (a, b) in enumerate(zip(taps, layers)):     # the stream behind every layer
                assert rel_err(a, b) < 2e-5, (name, n, i)
        agree(got, ref, dtype, 2 * L, (name, dtype, n))


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prompt_against_token_by_token_and_portions(folders, name):
    """float32: a sequence run whole, token by token, and in portions of several sizes gives the same logits
    up to rounding, and all of them the plain implementation's."""
    import plain_bizepel as P
    d, cfg, W = folders(name)
    eng = _engine(d, "float32", poison_cache=True)
    n = 150
    ids = _ids(11, n, cfg["vocab"])
    ref = P.logits(cfg, W, ids)
    for sizes in ([1] * n, [2] * 75, [3, 2, 64, 1, 65, 2, 13], [149, 1], [5] + [1] * 145):
        assert sum(sizes) == n
        s = eng.open(1)
        rows, at = [], 0
        for m in sizes:
            rows.append(eng.step(s, [ids[at:at + m]], [_all(m)]).cpu().numpy())
            at += m
        eng.close(s)
        eng.check_errors()
        agree(np.concatenate(rows), ref, "float32", 4, (name, sizes[:4]))
    # the same through passes inside one step (a step cut at 16 tokens)
    small = _engine(d, "float32", max_step_tokens=16)
    agree(_whole(small, ids), ref, "float32", 4, (name, "passes"))
    # and with passes shorter and longer than the windows
    for wp in (24, 2048):
        eng2 = _engine(d, "float32", window_pass=wp, poison_cache=True)
        agree(_whole(eng2, ids), ref, "float32", 4, (name, "window_pass", wp))
        agree(_prompt_then_single_tokens(eng2, ids, 97), ref, "float32", 4, (name, "window_pass then tokens", wp))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_unequal_requests_together_then_decoded_with_slots_used_again(folders, name, dtype):
    import plain_bizepel as P
    d, cfg, W = folders(_for(name, dtype))
    eng = _engine(d, dtype, poison_cache=True)
    L = len(cfg["layers"])
    for round_ in range(2):                                    # the second time on slots and pages just given back
        lens, tail = [1, 130, 66, 23], [3, 20, 9, 20]
        seqs = [_ids(20 + 10 * round_ + i, a + b, cfg["vocab"]) for i, (a, b) in enumerate(zip(lens, tail))]
        refs = [P.logits(cfg, W, s) for s in seqs]
        slots = eng.open(4)
        got = [dict() for _ in seqs]
        out = eng.step(slots, [s[:a] for s, a in zip(seqs, lens)], [_all(a) for a in lens]).cpu().numpy()
        o = 0
        for i, a in enumerate(lens):
            for p in range(a):
                got[i][p] = out[o]
                o += 1
        live = list(range(4))
        for t in range(max(tail)):
            live = [i for i in live if t < tail[i]]            # the shorter requests end earlier
            out = eng.step([slots[i] for i in live], [[seqs[i][lens[i] + t]] for i in live]).cpu().numpy()
            for r, i in enumerate(live):
                got[i][lens[i] + t] = out[r]
            for i in list(live):
                if t + 1 == tail[i]:
                    eng.close([slots[i]])
        eng.check_errors()
        for i, s in enumerate(seqs):
            g = np.stack([got[i][p] for p in range(len(s))])
            agree(g, refs[i], dtype, 2 * L, (name, dtype, round_, i))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "plain"])
def test_long_decoding_over_window_and_page_borders(folders, name, dtype):
    import plain_bizepel as P
    d, cfg, W = folders(_for(name, dtype))
    eng = _engine(d, dtype)
    ids = _ids(5, 210, cfg["vocab"])
    ref = P.logits(cfg, W, ids)
    agree(_prompt_then_single_tokens(eng, ids, 4), ref, dtype, 2 * len(cfg["layers"]), (name, dtype))


def test_greedy_generation_through_the_loop(folders):
    import plain_bizepel as P
    import ultima_b200 as u
    d, cfg, W = folders("mixed")
    llm = u.LLM(d, dtype="float32", n_ctx=128, max_batch=2)
    prompts = [_ids(1, 9, cfg["vocab"]), _ids(2, 30, cfg["vocab"])]
    outs = llm.generate(prompts, n_predict=8, temp=0.0)
    for p, g in zip(prompts, outs):
        ids = list(p)
        for _ in range(8):
            ids.append(int(np.argmax(P.logits(cfg, W, ids)[-1])))
        assert g.tokens == ids[len(p):], (g.tokens, ids[len(p):])


def test_trace_replay_and_the_command_line(folders, tmp_path):
    import plain_bizepel as P
    d, cfg, W = folders("odd")
    listed = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "ultima"), "archinfo", d], capture_output=True,
                            text=True, timeout=300)
    assert listed.returncode == 0 and "l0.mix.A_log" in listed.stdout and "all " in listed.stdout, listed.stderr[-1500:]
    a, b = _ids(3, 70, cfg["vocab"]), _ids(4, 9, cfg["vocab"])
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b[:5], "want": [4]}], "end": []}]
    for t in range(4):
        steps.append({"step": t + 1, "entries": [{"id": "a", "tokens": [a[66 + t]], "want": [0]},
                                                 {"id": "b", "tokens": [b[5 + t]], "want": [0]}],
                      "end": ["a", "b"] if t == 3 else []})
    steps.append({"step": 5, "entries": [{"id": "c", "tokens": b, "want": [8]}], "end": ["c"]})      # a slot used again
    for dtype in ("float32", "bfloat16"):
        d, cfg, W = folders(_for("odd", dtype))
        out_dir = str(tmp_path / ("out_" + dtype))
        p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype,
                            "--out", out_dir, "--max-tokens", "192"], input="".join(json.dumps(s) + "\n" for s in steps),
                           capture_output=True, text=True, timeout=900)
        assert p.returncode == 0 and "done 5" in p.stdout, p.stderr[-2000:]
        ra, rb = P.logits(cfg, W, a), P.logits(cfg, W, b)
        got = [np.fromfile(os.path.join(out_dir, "0.f32"), dtype="<f4").reshape(3, cfg["vocab"])]
        want = [ra[0], ra[65], rb[4]]
        for t in range(4):
            got.append(np.fromfile(os.path.join(out_dir, f"{t + 1}.f32"), dtype="<f4").reshape(2, cfg["vocab"]))
            want += [ra[66 + t], rb[5 + t]]
        got.append(np.fromfile(os.path.join(out_dir, "5.f32"), dtype="<f4").reshape(1, cfg["vocab"]))
        want.append(rb[8])
        agree(np.concatenate(got), np.stack(want), dtype, 8, dtype)
