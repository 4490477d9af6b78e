"""Vusalix on the GPU against the plain implementation (tests/plain_vusalix.py): the kernels of the stream's copies
and of the router alone, every mixer and the routed feed-forward as one-layer models, keys made to stand out at
the edges of windows and pages, then whole models from small configurations with random weights: prompts,
token-by-token decoding, portions, batches of unequal requests, slots used again, long decoding, greedy
generation, trace replay."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT, close_enough, has_gpu
from vusalix_configs import CONFIGS, _attention, _delta, _latent, _layer, _moe

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


# ---------------------------------------------------------------------------------------
# the copies of the stream
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("S,T,width", [(1, 5, 48), (2, 37, 100), (3, 64, 64), (5, 130, 257), (8, 3, 1024), (4, 9, 2048), (2, 3, 4100),
                                       (3, 7, 130)])
def test_a_pass_over_the_copies_writes_and_reads(S, T, width, out_dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(S * 100 + T)
    x = torch.randn(T, width, generator=g)
    xs = torch.empty(S, T, width, device=DEV)
    ops.streams_fill(x.to(DEV), xs)
    assert torch.equal(xs.cpu(), x[None].expand(S, T, width))
    xs = torch.randn(S, T, width, generator=g).to(DEV)
    mix, b, a = torch.randn(S, S, generator=g), torch.randn(S, generator=g), torch.randn(S, generator=g)
    w = 1 + 0.2 * torch.randn(width, generator=g)
    y = torch.randn(T, width, generator=g)
    eps = 1e-5
    old = xs.double().cpu()
    new = torch.einsum("sr,stw->rtw", mix.double(), old) + b.double()[:, None, None] * y.double()[None]
    u = torch.einsum("s,stw->tw", a.double(), new)
    ref = u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps) * w.double()
    # write, and the next sublayer's read in the same pass
    out = torch.empty(T, width, dtype=out_dtype, device=DEV)
    yd = y.to(DEV)
    ops.streams_pass(xs, write=(mix.to(DEV), b.to(DEV), yd), read=(a.to(DEV), w.to(DEV), eps), out=out)
    assert rel_err(xs, new) < 1e-6 and float(yd.abs().max()) == 0.0          # y is cleared for the next sublayer
    assert rel_err(out, ref) < (1e-5 if out_dtype == torch.float32 else 2 ** -7)
    # a read alone, of chosen rows, with the plain sum and no norm: what the model's end does
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32, device=DEV)
    total = torch.empty(3, width, device=DEV)
    ops.streams_pass(xs, read=(None, None, 0.0), out=total, rows=rows)
    assert rel_err(total, new.sum(0)[rows.long().cpu()]) < 1e-6
    # a write alone
    xs2 = old.float().to(DEV)
    ops.streams_pass(xs2, write=(mix.to(DEV), b.to(DEV), y.to(DEV)))
    assert rel_err(xs2, new) < 1e-6


# ---------------------------------------------------------------------------------------
# the router
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("ne,ni,groups,top", [(6, 2, (4, 2), 3), (20, 4, (2, 1), 5), (5, 0, None, 2), (3, 1, None, 1),
                                              (12, 4, (4, 3), 3), (8, 0, (8, 2), 2), (60, 4, (8, 3), 6)])
def test_the_router_chooses_by_corrected_scores_within_the_kept_groups_and_weights_by_the_plain_ones(ne, ni, groups, top):
    """The correction is larger than the scores and partly negative, so that choice scores are negative too: an
    output outside the kept groups must count as minus infinity, not as 0."""
    import plain_vusalix as P
    ops = _ops()
    n_out, T = ne + ni, 200
    g = torch.Generator().manual_seed(ne)
    z = (torch.randn(T, n_out, generator=g) * 2).float()
    corr = (torch.randn(n_out, generator=g) * 0.3 - 0.4).float()
    f = {"router": {"experts": ne, "identity": ni, "top": top}}
    if groups:
        f["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    ref_idx, ref_w = P.route(z.double(), {"r.router": torch.eye(n_out, dtype=torch.float64), "r.correction": corr.double()}, f, "r.")
    idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, device=DEV)
    counts = torch.zeros(ne, dtype=torch.int32, device=DEV)
    ops.route(z.to(DEV), corr.to(DEV), ne, top, groups[0] if groups else 1, groups[1] if groups else 1, idx, wts, counts)
    idx, wts = idx.cpu().long(), wts.cpu().double()
    for t in range(T):
        got = dict(zip(idx[t].tolist(), wts[t].tolist()))
        want = dict(zip(ref_idx[t].tolist(), ref_w[t].tolist()))
        assert set(got) == set(want), (t, got, want)
        assert all(abs(got[e] - want[e]) < 1e-6 for e in want), (t, got, want)
    assert counts.cpu().tolist() == torch.bincount(ref_idx[ref_idx < ne].flatten(), minlength=ne).tolist()
    # a step of few tokens: routing, plan and places in one launch agree with the three kernels
    Ts, tile = min(T, ops.ROUTE_SMALL_TOKENS), 16
    zs = z[:Ts].contiguous().to(DEV)
    i3, w3 = torch.empty(Ts, top, dtype=torch.int32, device=DEV), torch.empty(Ts, top, device=DEV)
    ws = torch.zeros(3 * ne + 4, dtype=torch.int32, device=DEV)
    max_tiles = Ts * top + ne
    t3, rp3, sr3 = (torch.full((max_tiles, 4), -7, dtype=torch.int32, device=DEV), torch.empty(Ts, top, dtype=torch.int32, device=DEV),
                    torch.full((Ts * top,), -7, dtype=torch.int32, device=DEV))
    ops.route(zs, corr.to(DEV), ne, top, groups[0] if groups else 1, groups[1] if groups else 1, i3, w3, ws[:ne])
    ops.route_plan(ws[:ne], ws[ne:2 * ne], ws[2 * ne:3 * ne], t3, ws[3 * ne:3 * ne + 1], ne, tile)
    ops.route_scatter(i3, ws[2 * ne:3 * ne], ws[ne:2 * ne], rp3, sr3, ne)
    i1, w1 = torch.empty_like(i3), torch.empty_like(w3)
    t1, rp1, sr1, n1 = torch.full_like(t3, -7), torch.empty_like(rp3), torch.full_like(sr3, -7), torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.route_small(zs, corr.to(DEV), ne, top, groups[0] if groups else 1, groups[1] if groups else 1, i1, w1, t1, n1, rp1, sr1, tile)
    n = int(n1.item())
    assert torch.equal(i1, i3) and torch.equal(w1, w3) and n == int(ws[3 * ne].item()) and torch.equal(t1[:n, :3], t3[:n, :3])
    # places within an expert's segment are handed out in any order: the same tokens, and every choice at a row of its expert
    seg = {}
    for e, r0, k in t1[:n, :3].cpu().tolist():
        lo, hi = seg.get(e, (r0, r0))
        seg[e] = (min(lo, r0), max(hi, r0 + k))
    rp, sr, ii = rp1.cpu(), sr1.cpu(), i1.cpu()
    for t in range(Ts):
        for k in range(top):
            e, p = int(ii[t, k]), int(rp[t, k])
            if e >= ne:
                assert p == -1
            else:
                assert seg[e][0] <= p < seg[e][1] and int(sr[p]) == t
    live = rp[rp >= 0]
    assert live.numel() == len(set(live.tolist())) == int((ii < ne).sum())
    # the same logits handed over as three K slices whose sum they are
    coarse = (z * 4).round() / 4
    rest = z - coarse
    parts = torch.stack([coarse, rest, torch.zeros_like(z)]).contiguous()        # (both sums are exact)
    assert torch.equal(parts[0] + parts[1] + parts[2], z)
    idx2, wts2 = torch.empty_like(idx, dtype=torch.int32, device=DEV), torch.empty(T, top, device=DEV)
    counts.zero_()
    ops.route(parts.to(DEV), corr.to(DEV), ne, top, groups[0] if groups else 1, groups[1] if groups else 1, idx2, wts2, counts)
    assert torch.equal(idx2.cpu().long(), idx) and torch.equal(wts2.cpu().double(), wts)


@pytest.mark.parametrize("y_dtype,h_dtype", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                             (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("T,width,top", [(1, 30, 1), (7, 64, 3), (33, 100, 2), (5, 4104, 4), (3, 1030, 5)])
def test_the_weighted_sum_of_the_chosen_rows_with_identity_choices(T, width, top, y_dtype, h_dtype):
    """Widths that are and are not a multiple of 4 (four columns a thread, or one); a choice without a row hands the
    token's own input on."""
    ops = _ops()
    g = torch.Generator().manual_seed(T * 7 + top)
    rows = T * top
    y = torch.randn(rows + 2, width, generator=g).to(y_dtype)
    h = torch.randn(T, width, generator=g).to(h_dtype)
    res = torch.randn(T, width, generator=g)
    wts = torch.rand(T, top, generator=g)
    row_pos = torch.randperm(rows + 2, generator=g)[:rows].reshape(T, top).to(torch.int32)
    row_pos[torch.rand(T, top, generator=g) < 0.3] = -1
    want = res.double().clone()
    for t in range(T):
        for k in range(top):
            src = h[t] if row_pos[t, k] < 0 else y[row_pos[t, k]]
            want[t] += wts[t, k].double() * src.double()
    out = res.to(DEV)
    ops.route_combine(y.to(DEV), h.to(DEV), row_pos.to(DEV), wts.to(DEV), out)
    assert rel_err(out, want) < 1e-6


# ---------------------------------------------------------------------------------------
# products of many small matrices on the tensor cores
# ---------------------------------------------------------------------------------------
class _Rt:
    def __init__(self):
        self.status = torch.zeros(4, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("tile", [16, 64, 128])
def test_grouped_product_over_sorted_rows_on_the_tensor_cores(tile):
    """Experts with no rows, with a few, with more than a tile and with exactly a tile; N no multiple of 128, K no
    multiple of 64; the gate product from two halves of one stacked matrix, and the plain product into float32."""
    from ultima_b200.kernels import gemm_tc
    from ultima_b200.parts.routed import RoutePlan
    ops = _ops()
    counts = [0, 3, 130, tile, 17, 0, 1]
    E, N, K = len(counts), 192, 136
    rows = sum(counts)
    g = torch.Generator().manual_seed(tile)
    a = (torch.randn(rows + 5, K, generator=g)).to(torch.bfloat16).to(DEV)
    a[rows:] = float("nan")                                     # rows of no expert: they must reach no result
    w = (torch.randn(E, 2 * N, K, generator=g) * 0.2).to(torch.bfloat16).to(DEV)
    max_tiles = -(-rows // tile) + E
    tiles = torch.zeros(max_tiles + 3, 4, dtype=torch.int32, device=DEV)
    ws = torch.zeros(3 * E + 1, dtype=torch.int32, device=DEV)
    ws[:E] = torch.tensor(counts, dtype=torch.int32)
    ops.route_plan(ws[:E], ws[E:2 * E], ws[2 * E:3 * E], tiles, ws[3 * E:], E, tile)
    plan = RoutePlan(tiles, ws[3 * E:], None, max_tiles + 3, rows, gather=False, tile=tile)
    expert = torch.repeat_interleave(torch.arange(E), torch.tensor(counts))
    ad, wd = a[:rows].double().cpu(), w.double().cpu()
    gate = torch.einsum("rk,rnk->rn", ad, wd[expert, :N])
    up = torch.einsum("rk,rnk->rn", ad, wd[expert, N:])
    rt = _Rt()
    out = torch.full((rows + 5, N), 7.0, dtype=torch.bfloat16, device=DEV)
    assert gemm_tc.accepts_grouped(a, w[:, :N], out, ops.EPI_SWIGLU, w[:, N:])
    gemm_tc.grouped(a, w[:, :N], out, plan, ops.EPI_SWIGLU, w[:, N:], rt)
    assert rel_err(out[:rows], gate * torch.sigmoid(gate) * up) < 2 ** -7
    assert bool((out[rows:] == 7.0).all()) and rt.status.tolist() == [0, 0, 0, 0]
    out32 = torch.full((rows + 5, N), 7.0, device=DEV)
    gemm_tc.grouped(a, w[:, N:], out32, plan, ops.EPI_STORE, None, rt)
    assert rel_err(out32[:rows], up) < 1e-5 and bool((out32[rows:] == 7.0).all())
    if tile <= ops.ROUTE_TILE:                                  # against the CUDA-core product of the same tiles
        simt = torch.empty(rows, N, device=DEV)
        ops.gemm_grouped(a, w[:, N:], simt, tiles, ws[3 * E:], None, max_tiles + 3)
        assert rel_err(out32[:rows], simt) < 1e-5


@pytest.mark.parametrize("T", [1, 37, 300])
def test_one_small_matrix_a_head_on_the_tensor_cores(T):
    """Inputs and outputs that are column ranges of wider rows, K no multiple of 64."""
    from ultima_b200.kernels import gemm_tc
    B, K, N = 3, 40, 72
    g = torch.Generator().manual_seed(T)
    wide_a = torch.randn(T, B, K + 24, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(B, N, K, generator=g) * 0.3).to(torch.bfloat16).to(DEV)
    a = wide_a[:, :, :K]
    ref = torch.einsum("tbk,bnk->tbn", a.double().cpu(), w.double().cpu())
    for dtype, tol in ((torch.bfloat16, 2 ** -7), (torch.float32, 1e-5)):
        wide_o = torch.full((T, B, N + 8), 3.0, dtype=dtype, device=DEV)
        out = wide_o[:, :, 8:]
        assert gemm_tc.accepts_batched(a, w, out)
        gemm_tc.batched(a, w, out, _Rt())
        assert rel_err(out, ref) < tol and bool((wide_o[:, :, :8] == 3.0).all())


# ---------------------------------------------------------------------------------------
# models of one layer: every mixer and the routed feed-forward alone
# ---------------------------------------------------------------------------------------
def _model(layers, vocab=97, width=64, eps=1e-5, streams=None):
    d = {"architecture": "Vusalix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams:
        d["streams"] = streams
    return d


_TINY = _delta(2, 1, 8, 8, 2)
_YARN = {"factor": 6.0, "original": 48, "fast": 8.0, "slow": 1.5}
ONE_LAYER = {
    "attention_capped": _model([_layer("attention", _attention(6, 2, 16, 24, 0.4, 50, 10, softcap=3.0, mask=45))]),
    "attention_no_cap_no_window": _model([_layer("attention", _attention(2, 2, 40, 8, 0.3, 300, 9))], width=72),
    "attention_one_head": _model([_layer("attention", _attention(1, 1, 64, 64, 0.2, 20, 4, softcap=50.0, mask=1))], streams=2),
    # a table by distance too large for the prompt kernel's shared memory (8 heads a group, 901 distances): read in place
    "attention_wide_table": _model([_layer("attention", _attention(8, 1, 16, 16, 0.3, 900, 24, softcap=6.0))]),
    "latent_rescaled": _model([_layer("latent_attention", _latent(3, 24, 16, 40, 48, 0.2, 500.0, _YARN, mask=33))]),
    "latent_plain": _model([_layer("latent_attention", _latent(5, 8, 4, 8, 12, 0.5, 10000.0))], width=40, streams=3),
    "delta_shared_keys": _model([_layer("delta", _delta(6, 2, 16, 24, 4))]),
    "delta_one_tap": _model([_layer("delta", _delta(1, 1, 40, 72, 1))], width=56, streams=2),
    "routed_groups": _model([_layer("delta", _TINY, _moe(10, 3, 24, identity=2, groups=(3, 2), shared=40))]),
    "routed_plain": _model([_layer("delta", _TINY, _moe(7, 7, 16))], width=48),
    "routed_identity_mostly": _model([_layer("delta", _TINY, _moe(1, 2, 32, identity=5, groups=(6, 4)))], streams=2),
}


def _sharpen(W, amp=2.5):
    """Random weights scaled so that attention weights are far from uniform, sinks weigh something, decays differ
    from head to head and the router's scores are far from equal."""
    out = {}
    for n, t in W.items():
        leaf = n.split(".")[-1]
        if ".mix." in n and t.dim() == 2 and leaf in ("q", "k", "dkv", "uk"):
            t = t * amp
        if leaf == "sink":
            t = t * 2 + 1.5
        if leaf == "rel":
            t = t * 2
        out[n] = t.to(torch.bfloat16)
    return out


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    import plain_vusalix as P
    import ultima_b200 as u
    from ultima_b200.weights.safetensors_io import write_safetensors
    base = tmp_path_factory.mktemp("vusalix")
    made = {}

    def get(name, raw=None, change=None):
        if name not in made:
            d = str(base / name.replace("/", "_"))
            plain_name = name.split("/")[0]
            raw = copy.deepcopy(raw or CONFIGS.get(plain_name) or ONE_LAYER[plain_name])
            if name.endswith("/all_chosen"):
                for L in raw["layers"]:
                    if L.get("mlp"):
                        r = L["mlp"]["router"]
                        r["top"] = r["experts"] + r.get("identity", 0)
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
    """The model's folder for a run in ``dtype``.  In bfloat16 a router's near tie between two outputs may go either
    way, and one other choice reaches every later position through states and keys; so the bfloat16 runs of whole
    models use the same models with routers that choose every output (the weights still differ from token to token).
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
    import plain_vusalix as P
    d, cfg, W = folders(name)
    eng = _engine(d, dtype, poison_cache=True)
    n = 140
    ids = _ids(len(name), n, cfg["vocab"])
    layers = []
    with torch.no_grad():
        ref = P.forward(cfg, W, ids, torch.float64, layers).numpy()
    taps = []
    eng.model.tap = lambda i, x: taps.append(x.detach().double().cpu())
    got = _whole(eng, ids)
    eng.model.tap = None
    assert len(taps) == len(layers) == 1
    if dtype == "float32":
        assert rel_err(taps[0], layers[0]) < 2e-5, name           # the stream (the sum of its copies) behind the layer
    agree(got, ref, dtype, 2, (name, "prompt"))
    agree(_prompt_then_single_tokens(eng, ids, 3), ref, dtype, 2, (name, "single tokens"))


# ---------------------------------------------------------------------------------------
# one key made to stand out: it is seen exactly where the mask says so
# ---------------------------------------------------------------------------------------
ASKER, MARKED = 5, 11


def _stand_out(cfg, W):
    """Layer 0's queries of token ASKER are turned towards the keys of token MARKED (a rank-one change of W_q a head),
    so that this one score lies far above the others, and MARKED's values are made large."""
    import plain_vusalix as P
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    h = {t: P.rms_norm(W["embed"][t], W["l0.norm1"], eps) for t in (ASKER, MARKED)}
    towards = h[ASKER] / (h[ASKER] @ h[ASKER])
    H, d = m["heads"], m["dim"]
    q = W["l0.mix.q"].clone()
    if cfg["layers"][0]["type"] == "attention":
        k = (W["l0.mix.k"] @ h[MARKED]).view(m["kv_heads"], d)
        for a in range(H):
            kh = k[a // (H // m["kv_heads"])]
            q[a * d:(a + 1) * d] += torch.outer(kh / kh.norm() ** 2 * (9.0 / m["scale"]), towards)
        W["l0.mix.v"] = W["l0.mix.v"] + torch.outer(torch.ones(W["l0.mix.v"].shape[0], dtype=torch.float64) * 4.0, h[MARKED] / (h[MARKED] @ h[MARKED]))
    else:
        rank, r = m["kv_rank"], m["rot_dim"]
        c = P.rms_norm((W["l0.mix.dkv"] @ h[MARKED])[:rank], W["l0.mix.dkv.norm"], eps)
        k = (W["l0.mix.uk"] @ c).view(H, d)
        for a in range(H):
            q[a * (d + r):a * (d + r) + d] += torch.outer(k[a] / k[a].norm() ** 2 * (9.0 / m["scale"]), towards)
        W["l0.mix.uv"] = W["l0.mix.uv"] + torch.outer(torch.ones(W["l0.mix.uv"].shape[0], dtype=torch.float64) * 0.5, c / (c @ c))
    W["l0.mix.q"] = q
    return W


MARKED_MODELS = {
    "marked_attention": (_model([_layer("attention", _attention(4, 2, 32, 16, 0.2, 100, 12, softcap=15.0, mask=70)),
                                 _layer("delta", _delta(2, 2, 16, 16, 3))]), 70),
    "marked_attention_page_window": (_model([_layer("attention", _attention(2, 1, 16, 32, 0.3, 40, 6, mask=64))]), 64),
    "marked_attention_no_window": (_model([_layer("attention", _attention(3, 3, 16, 16, 0.25, 64, 8, softcap=12.0))]), None),
    "marked_latent": (_model([_layer("latent_attention", _latent(4, 16, 16, 24, 32, 0.17, 10000.0, _YARN, mask=50)),
                              _layer("delta", _delta(2, 2, 16, 16, 3))]), 50),
    "marked_latent_no_window": (_model([_layer("latent_attention", _latent(2, 24, 8, 16, 40, 0.2, 300.0))]), None),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(MARKED_MODELS))
def test_a_key_just_inside_and_just_outside_the_window_at_page_borders_and_far_away(folders, name, dtype):
    import plain_vusalix as P
    raw, window = MARKED_MODELS[name]
    d, cfg, W = folders(name, raw, _stand_out)
    eng = _engine(d, dtype, poison_cache=True)
    cases = []                                                   # (place of the marked key, place of the asking token)
    if window is None:
        cases = [(0, 1), (3, 420), (63, 64), (64, 300), (0, 449)]
    else:
        for m in (0, 1, 63, 64, 127, 200):
            cases += [(m, m + window - 1), (m, m + window), (m, m + 1), (m, m + window + 1)]
    for m, p in cases:
        ids = _ids(m * 1000 + p, p + 1, cfg["vocab"], avoid=(ASKER, MARKED))
        ids[m], ids[p] = MARKED, ASKER
        ref = P.logits(cfg, W, ids)[p]
        seen = window is None or p - m < window
        without = list(ids)
        without[m] = ids[m + 1] if m + 1 < p else ids[m - 1]
        bound = close_enough(ref[None], ref[None], dtype, 2)[1]
        moved = float(np.abs(P.logits(cfg, W, without)[p] - ref).max())
        assert moved > 0.06 or not seen, (name, m, p, moved)      # the test's weights do show the key: several times the bound
        got = _whole(eng, ids, [p])[0]                             # the asking token in a prompt
        err = float(np.abs(got - ref).max())
        assert err <= bound, (name, dtype, m, p, "prompt", err, bound)
        cut = max(1, p - 3)                                         # and decoded alone, three tokens behind the prompt
        got = _prompt_then_single_tokens(eng, ids, cut, want_from=cut - 1)[-1]
        err = float(np.abs(got - ref).max())
        assert err <= bound, (name, dtype, m, p, "decoded", err, bound)


def test_the_sink_takes_weight_and_the_state_keeps_an_early_input(folders):
    """Two faults that random weights would hide: a sink that is left out (here it outweighs the keys), and a
    recurrent state that is lost (here the decay is close to one, so the first tokens still count after hundreds)."""
    import plain_vusalix as P

    def heavy_sink(cfg, W):
        W["l0.mix.sink"] = W["l0.mix.sink"] * 0 + torch.tensor([6.0, -3.0, 4.0], dtype=torch.float64)
        return W

    def slow_decay(cfg, W):
        W["l0.mix.A_log"] = W["l0.mix.A_log"] * 0 - 9.0
        W["l0.mix.b"] = W["l0.mix.b"] * 0.2              # weak writes: the state is not soon overwritten
        return W
    raw = _model([_layer("attention", _attention(3, 1, 16, 16, 0.25, 64, 8, mask=30))])
    d, cfg, W = folders("heavy_sink", raw, heavy_sink)
    ids = _ids(1, 100, cfg["vocab"])
    ref = P.logits(cfg, W, ids)
    no_sink = P.logits(cfg, {**W, "l0.mix.sink": W["l0.mix.sink"] - 50.0}, ids)
    assert np.abs(no_sink - ref).max() > 0.05 * np.abs(ref).max()
    for dtype in ("float32", "bfloat16"):
        agree(_whole(_engine(d, dtype), ids), ref, dtype, 2, ("sink", dtype))
    raw = _model([_layer("delta", _delta(2, 1, 16, 24, 3))])
    d, cfg, W = folders("slow_decay", raw, slow_decay)
    ids = _ids(2, 400, cfg["vocab"])
    ref = P.logits(cfg, W, ids)
    other = P.logits(cfg, W, _ids(3, 4, cfg["vocab"]) + ids[4:])
    assert np.abs(other[-1] - ref[-1]).max() > 1e-3           # the first four tokens still count at the end (the 32-bit run shows it)
    for dtype in ("float32", "bfloat16"):
        eng = _engine(d, dtype)
        agree(_whole(eng, ids), ref, dtype, 2, ("state", dtype, "prompt"))
        agree(_prompt_then_single_tokens(eng, ids, 150)[-200:], ref[-200:], dtype, 2, ("state", dtype, "decoded"))


# ---------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_a_prompt_in_one_step_every_position_and_every_layer(folders, name, dtype):
    import plain_vusalix as P
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
    import plain_vusalix as P
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
    # and with a windowed layer's ring sized for passes shorter and longer than the windows
    for wp in (24, 2048):
        eng2 = _engine(d, "float32", window_pass=wp, poison_cache=True)
        agree(_whole(eng2, ids), ref, "float32", 4, (name, "window_pass", wp))
        agree(_prompt_then_single_tokens(eng2, ids, 97), ref, "float32", 4, (name, "window_pass then tokens", wp))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_unequal_requests_together_then_decoded_with_slots_used_again(folders, name, dtype):
    import plain_vusalix as P
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
    import plain_vusalix as P
    d, cfg, W = folders(_for(name, dtype))
    eng = _engine(d, dtype)
    ids = _ids(5, 210, cfg["vocab"])
    ref = P.logits(cfg, W, ids)
    agree(_prompt_then_single_tokens(eng, ids, 4), ref, dtype, 2 * len(cfg["layers"]), (name, dtype))


def test_greedy_generation_through_the_loop(folders):
    import plain_vusalix as P
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
    import plain_vusalix as P
    d, cfg, W = folders("odd")
    listed = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "ultima"), "archinfo", d], capture_output=True,
                            text=True, timeout=300)
    assert listed.returncode == 0 and "l0.mix.dkv.norm" in listed.stdout and "all " in listed.stdout, listed.stderr[-1500:]
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
