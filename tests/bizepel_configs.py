"""Small Bizepel configurations for the tests.  They differ from one another in every size and option: order of layers,
widths (one not a multiple of 8), heads and groups, key and value sizes (equal and unequal, multiples of 16 and not),
rotated parts (the whole head, a part, none), windows that end on and off a page's border or are absent, with and
without kept first positions, convolutions of 1 to 5 taps or none, value mixing over two, three or no layers, state
sizes, ranks that are and are not multiples of 8, routers with and without groups and shared experts, top 1 to 4,
layers without feed-forward, with and without the input convolution, the per-layer token input and the logit scale."""


def _attention(heads, kv_heads, dim, vdim, scale, conv=None, rot=None, mask=None, v_mix=False):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if conv is not None:
        m["conv"] = conv
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    if mask is not None:
        m["mask"] = {"size": mask[0], "keep_first": mask[1]}
    if v_mix:
        m["v_mix"] = True
    return m


def _mamba(inner, state, dt_rank, conv):
    return {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}


def _delta(heads, dim, rank):
    # the rank stands in no key of the design; a configuration of this package carries it for random models
    return {"heads": heads, "dim": dim, "decay_rank": rank}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, scale=None, groups=None, shared=None):
    router = {"experts": experts, "top": top}
    if scale is not None:
        router["scale"] = scale
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    f = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        f["shared"] = {"ff": shared}
    return f


def _layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def _model(layers, vocab=97, width=64, eps=1e-5, taps=3, side=8, logit_scale=1.5):
    d = {"architecture": "Bizepel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if taps:
        d["canon"] = {"taps": taps}
    if side:
        d["token_side"] = {"dim": side}
    if logit_scale is not None:
        d["logit_scale"] = logit_scale
    return d


MIXED = _model([
    _layer("general_delta", _delta(3, 16, 5), _moe(6, 2, 24, scale=1.7, groups=(3, 2), shared=40)),
    _layer("attention", _attention(4, 2, 32, 16, 0.2, conv=3, rot=(10000.0, 16), mask=(40, 6), v_mix=True), _dense(96)),
    _layer("mamba1", _mamba(96, 10, 6, 4), _moe(5, 3, 32, shared=24)),
    _layer("attention", _attention(2, 1, 24, 32, 0.25, conv=2, rot=(500.0, 24), mask=(70, 3), v_mix=True), _moe(8, 2, 16, scale=2.5, groups=(2, 1))),
    _layer("attention", _attention(4, 4, 16, 8, 0.3, conv=5, rot=(100.0, 8), v_mix=True)),
], vocab=300, width=64, taps=3, side=8, logit_scale=1.5)

ODD = _model([
    _layer("mamba1", _mamba(70, 3, 1, 2), _dense(50)),
    _layer("attention", _attention(3, 3, 20, 20, 0.22, mask=(33, 0)), _moe(4, 1, 36, scale=0.5)),
    _layer("general_delta", _delta(2, 36, 8), _moe(3, 3, 50, groups=(3, 3), shared=20)),
    _layer("attention", _attention(2, 1, 12, 28, 0.3, conv=1, rot=(300.0, 12), mask=(64, 64))),
], vocab=257, width=100, eps=3e-6, taps=2, side=5, logit_scale=None)

WIDE = _model([
    _layer("attention", _attention(8, 2, 64, 64, 0.125, conv=4, rot=(10000.0, 32), mask=(64, 4), v_mix=True), _moe(8, 2, 64, scale=2.0, groups=(4, 2), shared=128)),
    _layer("general_delta", _delta(2, 64, 16), _dense(256)),
    _layer("attention", _attention(2, 2, 128, 128, 0.09, conv=4, rot=(10000.0, 128), mask=(130, 20)), _moe(12, 4, 64, groups=(4, 3))),
    _layer("mamba1", _mamba(256, 16, 8, 4), _moe(20, 5, 64, scale=2.25, groups=(4, 2), shared=64)),
    _layer("attention", _attention(4, 2, 64, 64, 0.125, conv=4, rot=(10000.0, 64), mask=(100, 1), v_mix=True), _dense(256)),
], vocab=384, width=128, eps=1e-6, taps=4, side=16, logit_scale=0.75)

# no input convolution, no token input, no logit scale, a layer without feed-forward first
PLAIN = _model([
    _layer("attention", _attention(3, 1, 24, 40, 0.2, rot=(777.0, 8))),
    _layer("mamba1", _mamba(48, 24, 16, 3), _dense(64)),
    _layer("general_delta", _delta(6, 8, 3)),
], vocab=130, width=48, taps=0, side=0, logit_scale=None)

CONFIGS = {"mixed": MIXED, "odd": ODD, "wide": WIDE, "plain": PLAIN}
