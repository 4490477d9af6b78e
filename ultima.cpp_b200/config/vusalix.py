"""Vusalix: the typed configuration, read from the design's own config.json keys.

    architecture  "Vusalix"
    vocab, width  sizes of the embedding table
    norm.eps      the eps of every RMS norm of the model
    streams       copies of the residual stream (hyper-connections); absent: one stream and plain residual sums
    layers        a list; each entry has
        type      "attention", "latent_attention" or "delta"
        mixer     the mixer's sizes and constants (below)
        mlp       null, or {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "identity",
                  "groups": {"count", "keep"}}, "shared": {"ff"}}
    attention mixer:         heads, kv_heads, dim, vdim, scale, softcap, bias_max, mask.size
    latent_attention mixer:  heads, dim, rot_dim, vdim, kv_rank, scale, mask.size,
                             rot {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}}
    delta mixer:             heads, kv_heads, dim, vdim, conv (taps)

The number of rows of an attention layer's table of distance biases stands in no key: it is the shape
of the stored tensor (``with_tensor_shapes``); a configuration written by this package carries it as
``buckets`` so that a random model can be made from it.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional

from .base import ConfigError

ATTENTION, LATENT, DELTA = "attention", "latent_attention", "delta"


def _int(d: dict, key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: {where}'{key}' must be an integer, got {v!r}")
    if v < minimum:
        raise ConfigError(f"config.json: {where}'{key}' must be >= {minimum}, got {v}")
    return v


def _num(d: dict, key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}'{key}' must be a number, got {v!r}")
    return float(v)


def _window(m: dict, where: str) -> Optional[int]:
    mask = m.get("mask")
    if mask is None:
        return None
    if not isinstance(mask, dict):
        raise ConfigError(f"config.json: {where}mask must be an object with 'size'")
    return _int(mask, "size", where + "mask.")


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    bias_max: float
    window: Optional[int]
    buckets: Optional[int] = None            # rows of the bias table; from the tensor's shape when the file has no key


@dataclass(frozen=True)
class YarnScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    scaling: Optional[YarnScaling]
    window: Optional[int]


@dataclass(frozen=True)
class DeltaMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class RoutedConfig:
    experts: int
    top: int
    identity: int
    ff: int
    groups: Optional[tuple] = None           # (count, keep)
    shared_ff: Optional[int] = None


@dataclass(frozen=True)
class VusalixLayer:
    kind: str
    mixer: object
    mlp: Optional[RoutedConfig]


def _read_mixer(kind, m: dict, where: str):
    if kind == ATTENTION:
        heads, kv_heads = _int(m, "heads", where), _int(m, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}heads must be a multiple of kv_heads")
        cap = m.get("softcap")
        buckets = m.get("buckets")
        return AttentionMixer(heads, kv_heads, _int(m, "dim", where), _int(m, "vdim", where), _num(m, "scale", where),
                              None if cap is None else _num(m, "softcap", where), _num(m, "bias_max", where),
                              _window(m, where), None if buckets is None else _int(m, "buckets", where, 2))
    if kind == LATENT:
        rot = m.get("rot")
        if not isinstance(rot, dict):
            raise ConfigError(f"config.json: {where}rot must be an object with 'base' and 'dims'")
        rot_dim = _int(m, "rot_dim", where, 2)
        dims = _int(rot, "dims", where + "rot.", 2)
        if dims % 2 or dims > rot_dim:
            raise ConfigError(f"config.json: {where}rot.dims must be even and at most rot_dim")
        sc = rot.get("scaling")
        if sc is not None:
            sc = YarnScaling(*(_num(sc, k, where + "rot.scaling.") for k in ("factor", "original", "fast", "slow")))
            if sc.factor <= 0:
                raise ConfigError(f"config.json: {where}rot.scaling.factor must be positive")
        return LatentMixer(_int(m, "heads", where), _int(m, "dim", where), rot_dim, _int(m, "vdim", where),
                           _int(m, "kv_rank", where), _num(m, "scale", where), _num(rot, "base", where + "rot."), dims, sc,
                           _window(m, where))
    if kind == DELTA:
        heads, kv_heads = _int(m, "heads", where), _int(m, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}heads must be a multiple of kv_heads")
        return DeltaMixer(heads, kv_heads, _int(m, "dim", where), _int(m, "vdim", where), _int(m, "conv", where))
    raise ConfigError(f"config.json: {where[:-6]}type must be '{ATTENTION}', '{LATENT}' or '{DELTA}', got {kind!r}")


def _read_mlp(f, where: str) -> Optional[RoutedConfig]:
    if f is None:
        return None
    if not isinstance(f, dict) or f.get("kind") != "moe":
        raise ConfigError(f"config.json: {where}kind must be 'moe', got {f.get('kind') if isinstance(f, dict) else f!r}")
    r, e = f.get("router"), f.get("expert")
    if not isinstance(r, dict) or not isinstance(e, dict):
        raise ConfigError(f"config.json: {where}router and {where}expert must be objects")
    experts, top = _int(r, "experts", where + "router."), _int(r, "top", where + "router.")
    identity = _int(r, "identity", where + "router.", 0) if r.get("identity") is not None else 0
    groups = None
    if r.get("groups") is not None:
        g = r["groups"]
        groups = (_int(g, "count", where + "router.groups."), _int(g, "keep", where + "router.groups."))
        if (experts + identity) % groups[0] or groups[1] > groups[0]:
            raise ConfigError(f"config.json: {where}router.groups: the router's outputs must divide into 'count' equal "
                              f"groups, of which 'keep' are kept")
        if groups[1] * ((experts + identity) // groups[0]) < top:
            raise ConfigError(f"config.json: {where}router: the kept groups hold fewer experts than 'top'")
    if top > experts + identity:
        raise ConfigError(f"config.json: {where}router.top is more than the router has outputs")
    shared = f.get("shared")
    return RoutedConfig(experts, top, identity, _int(e, "ff", where + "expert."), groups,
                        None if shared is None else _int(shared, "ff", where + "shared."))


@dataclass(frozen=True)
class VusalixConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple
    streams: Optional[int] = None
    max_position_embeddings: int = 131072
    torch_dtype: str = "bfloat16"
    eos_token_id: tuple = ()
    architecture: str = "Vusalix"
    model_type: str = "vusalix"

    # ---- reading ---------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: dict) -> "VusalixConfig":
        vocab, width = _int(d, "vocab", ""), _int(d, "width", "")
        norm = d.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        eps = _num(norm, "eps", "norm.")
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(L, dict) or not isinstance(L.get("mixer"), dict):
                raise ConfigError(f"config.json: {where}mixer must be an object")
            layers.append(VusalixLayer(L.get("type"), _read_mixer(L.get("type"), L["mixer"], where + "mixer."),
                                       _read_mlp(L.get("mlp"), where + "mlp.")))
        eos = d.get("eos_token_id")
        eos = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        streams = _int(d, "streams", "") if d.get("streams") is not None else None
        return cls(vocab=vocab, width=width, eps=eps, layers=tuple(layers), streams=streams,
                   max_position_embeddings=int(d.get("max_positions", 131072)),
                   torch_dtype=str(d.get("torch_dtype", "bfloat16")), eos_token_id=eos)

    # ---- sizes that only the tensors give ------------------------------------------------------
    @property
    def needs_tensor_shapes(self) -> bool:
        return any(L.kind == ATTENTION and L.mixer.buckets is None for L in self.layers)

    def with_tensor_shapes(self, shapes: dict) -> "VusalixConfig":
        """The configuration with the bias tables' row counts read from the stored tensors' shapes
        (``shapes``: stored name -> shape)."""
        layers = []
        for i, L in enumerate(self.layers):
            m = L.mixer
            if L.kind == ATTENTION and m.buckets is None:
                name = f"l{i}.mix.rel"
                if name not in shapes or len(shapes[name]) != 2:
                    raise ConfigError(f"the model's files hold no table '{name}' to take the layer's bias buckets from")
                m = replace(m, buckets=int(shapes[name][0]))
            layers.append(VusalixLayer(L.kind, m, L.mlp))
        return replace(self, layers=tuple(layers))

    # ---- writing ---------------------------------------------------------------------------
    def to_dict(self) -> dict:
        out = []
        for L in self.layers:
            m = L.mixer
            if L.kind == ATTENTION:
                d = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                     "bias_max": m.bias_max}
                if m.softcap is not None:
                    d["softcap"] = m.softcap
                if m.buckets is not None:
                    d["buckets"] = m.buckets
            elif L.kind == LATENT:
                d = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank,
                     "scale": m.scale, "rot": {"base": m.rot_base, "dims": m.rot_dims}}
                if m.scaling is not None:
                    d["rot"]["scaling"] = {"factor": m.scaling.factor, "original": m.scaling.original,
                                           "fast": m.scaling.fast, "slow": m.scaling.slow}
            else:
                d = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.conv}
            if L.kind != DELTA and m.window is not None:
                d["mask"] = {"size": m.window}
            mlp = None
            if L.mlp is not None:
                f = L.mlp
                router = {"experts": f.experts, "top": f.top, "identity": f.identity}
                if f.groups is not None:
                    router["groups"] = {"count": f.groups[0], "keep": f.groups[1]}
                mlp = {"kind": "moe", "expert": {"ff": f.ff}, "router": router}
                if f.shared_ff is not None:
                    mlp["shared"] = {"ff": f.shared_ff}
            out.append({"type": L.kind, "mixer": d, "mlp": mlp})
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "layers": out, "max_positions": self.max_position_embeddings, "torch_dtype": self.torch_dtype}
        if self.streams is not None:
            d["streams"] = self.streams
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d
