"""Small Vusalix configurations for the tests.  They differ from one another in every size and option: order of
layers, widths (one not a multiple of 8), copies of the stream (none, 1, 3, 4), heads and groups, key and value sizes
(multiples of 16 and not), windows that end on and off a page's border or are absent, with and without a score cap,
even and odd bucket counts, latent sizes whose key row is and is not one the tensor-core kernels take, with and
without frequency rescaling, taps, experts with and without groups, identity experts, a shared expert, top 1 to 3,
and a layer without feed-forward."""


def _attention(heads, kv_heads, dim, vdim, scale, bias_max, buckets, softcap=None, mask=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": bias_max, "buckets": buckets}
    if softcap is not None:
        m["softcap"] = softcap
    if mask is not None:
        m["mask"] = {"size": mask}
    return m


def _latent(heads, dim, rot_dim, vdim, kv_rank, scale, base, scaling=None, mask=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = scaling
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot}
    if mask is not None:
        m["mask"] = {"size": mask}
    return m


def _delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def _moe(experts, top, ff, identity=None, groups=None, shared=None):
    router = {"experts": experts, "top": top}
    if identity is not None:
        router["identity"] = identity
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    f = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        f["shared"] = {"ff": shared}
    return f


def _layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


_YARN_A = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}
_YARN_B = {"factor": 2.5, "original": 200, "fast": 40.0, "slow": 0.5}

MIXED = {"architecture": "Vusalix", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "streams": 3, "layers": [
    _layer("delta", _delta(4, 2, 24, 40, 3), _moe(6, 3, 32, identity=2, groups=(4, 2), shared=48)),
    _layer("attention", _attention(4, 2, 32, 16, 0.2, 100, 12, softcap=15.0, mask=40), _moe(6, 3, 32, identity=2, groups=(4, 2), shared=48)),
    _layer("latent_attention", _latent(4, 16, 16, 24, 32, 0.17, 10000.0, _YARN_A, mask=50), _moe(4, 2, 24, identity=4, groups=(2, 1))),
    _layer("attention", _attention(6, 3, 16, 32, 0.3, 60, 8, softcap=5.0, mask=70)),
    _layer("delta", _delta(3, 3, 16, 32, 2)),
]}

ODD = {"architecture": "Vusalix", "vocab": 257, "width": 100, "norm": {"eps": 3e-6}, "streams": 1, "layers": [
    _layer("latent_attention", _latent(3, 20, 12, 28, 40, 0.2, 300.0), _moe(5, 2, 36)),
    _layer("attention", _attention(3, 3, 20, 20, 0.22, 30, 7), _moe(5, 1, 36, identity=1)),
    _layer("delta", _delta(2, 1, 72, 33, 5), _moe(3, 3, 50, shared=20)),
    _layer("latent_attention", _latent(2, 24, 8, 12, 24, 0.25, 5000.0, _YARN_B, mask=64)),
]}

WIDE = {"architecture": "Vusalix", "vocab": 384, "width": 128, "norm": {"eps": 1e-6}, "streams": 4, "layers": [
    _layer("attention", _attention(8, 2, 64, 64, 0.125, 128, 32, softcap=30.0, mask=64), _moe(8, 2, 64, groups=(2, 1), shared=128)),
    _layer("latent_attention", _latent(8, 64, 64, 64, 64, 0.09, 1000.0, _YARN_B, mask=100), _moe(8, 2, 64, groups=(2, 1), shared=128)),
    _layer("delta", _delta(4, 2, 64, 64, 4), _moe(12, 3, 64, identity=4, groups=(4, 3))),
    _layer("attention", _attention(2, 2, 128, 128, 0.09, 500, 16, mask=130), _moe(4, 1, 128)),
    _layer("latent_attention", _latent(4, 48, 16, 48, 48, 0.12, 1000.0), _moe(4, 1, 128)),
]}

# one stream, plain residual sums: no 'streams' key
PLAIN = {"architecture": "Vusalix", "vocab": 130, "width": 48, "norm": {"eps": 1e-5}, "layers": [
    _layer("attention", _attention(3, 1, 24, 40, 0.2, 20, 6, softcap=8.0, mask=33), _moe(3, 2, 40, identity=1)),
    _layer("delta", _delta(6, 3, 16, 12, 3)),
    _layer("latent_attention", _latent(2, 8, 8, 16, 24, 0.3, 777.0, mask=20), _moe(2, 1, 64, shared=32)),
]}

CONFIGS = {"mixed": MIXED, "odd": ODD, "wide": WIDE, "plain": PLAIN}
