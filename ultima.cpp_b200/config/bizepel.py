"""Bizepel: the typed configuration, read from the design's own config.json keys.

    architecture  "Bizepel"
    vocab, width  sizes of the embedding table
    norm.eps      the eps of every norm of the model
    canon.taps    taps of the causal convolution that every sublayer's input passes (absent: none)
    token_side.dim   columns a layer takes of the second embedding table (absent: no per-layer token input)
    logit_scale   a constant on the logits (absent: 1)
    layers        a list; each entry has
        type      "attention", "mamba1" or "general_delta"
        mixer     the mixer's sizes and constants (below)
        mlp       null, {"kind": "dense", "ff"} or {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "scale",
                  "groups": {"count", "keep"}}, "shared": {"ff"}}
    attention mixer:      heads, kv_heads, dim, vdim, scale, conv (taps), rot {"base", "dims"}, mask {"size", "keep_first"},
                          v_mix
    mamba1 mixer:         inner, state, dt_rank, conv (taps)
    general_delta mixer:  heads, dim

The inner size of a general_delta layer's low-rank decay product stands in no key: it is the shape of the stored
tensor (``with_tensor_shapes``); a configuration written by this package carries it as ``decay_rank`` so that a random
model can be made from it.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional

from .base import ConfigError

ATTENTION, MAMBA1, GENERAL_DELTA = "attention", "mamba1", "general_delta"


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


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int                                # taps; 0: no convolution behind the projections
    rot_base: Optional[float]
    rot_dims: Optional[int]
    window: Optional[int]
    keep_first: int
    v_mix: bool


@dataclass(frozen=True)
class Mamba1Mixer:
    inner: int
    state: int
    dt_rank: int
    conv: int


@dataclass(frozen=True)
class GeneralDeltaMixer:
    heads: int
    dim: int
    decay_rank: Optional[int] = None         # from the tensor's shape when the file has no key


@dataclass(frozen=True)
class DenseConfig:
    ff: int


@dataclass(frozen=True)
class RoutedConfig:
    experts: int
    top: int
    ff: int
    scale: float = 1.0
    groups: Optional[tuple] = None           # (count, keep)
    shared_ff: Optional[int] = None


@dataclass(frozen=True)
class BizepelLayer:
    kind: str
    mixer: object
    mlp: object                              # None, DenseConfig or RoutedConfig


def _read_mixer(kind, m: dict, where: str):
    if kind == ATTENTION:
        heads, kv_heads = _int(m, "heads", where), _int(m, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}heads must be a multiple of kv_heads")
        dim = _int(m, "dim", where)
        rot, base, dims = m.get("rot"), None, None
        if rot is not None:
            if not isinstance(rot, dict):
                raise ConfigError(f"config.json: {where}rot must be an object with 'base' and 'dims'")
            base, dims = _num(rot, "base", where + "rot."), _int(rot, "dims", where + "rot.", 2)
            if dims % 2 or dims > dim:
                raise ConfigError(f"config.json: {where}rot.dims must be even and at most dim")
        mask, window, keep = m.get("mask"), None, 0
        if mask is not None:
            if not isinstance(mask, dict):
                raise ConfigError(f"config.json: {where}mask must be an object with 'size'")
            window = _int(mask, "size", where + "mask.")
            keep = _int(mask, "keep_first", where + "mask.", 0) if mask.get("keep_first") is not None else 0
        conv = _int(m, "conv", where, 0) if m.get("conv") is not None else 0
        if conv > 16:
            raise ConfigError(f"config.json: {where}conv: at most 16 taps")
        return AttentionMixer(heads, kv_heads, dim, _int(m, "vdim", where), _num(m, "scale", where), conv, base, dims, window,
                              keep, bool(m.get("v_mix", False)))
    if kind == MAMBA1:
        conv = _int(m, "conv", where)
        if conv > 16:
            raise ConfigError(f"config.json: {where}conv: at most 16 taps")
        return Mamba1Mixer(_int(m, "inner", where), _int(m, "state", where), _int(m, "dt_rank", where), conv)
    if kind == GENERAL_DELTA:
        rank = m.get("decay_rank")
        return GeneralDeltaMixer(_int(m, "heads", where), _int(m, "dim", where),
                                 None if rank is None else _int(m, "decay_rank", where))
    raise ConfigError(f"config.json: {where[:-6]}type must be '{ATTENTION}', '{MAMBA1}' or '{GENERAL_DELTA}', got {kind!r}")


def _read_mlp(f, where: str):
    if f is None:
        return None
    if not isinstance(f, dict) or f.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"config.json: {where}kind must be 'dense' or 'moe', got {f.get('kind') if isinstance(f, dict) else f!r}")
    if f["kind"] == "dense":
        return DenseConfig(_int(f, "ff", where))
    r, e = f.get("router"), f.get("expert")
    if not isinstance(r, dict) or not isinstance(e, dict):
        raise ConfigError(f"config.json: {where}router and {where}expert must be objects")
    experts, top = _int(r, "experts", where + "router."), _int(r, "top", where + "router.")
    if top > experts:
        raise ConfigError(f"config.json: {where}router.top is more than the router has experts")
    groups = None
    if r.get("groups") is not None:
        g = r["groups"]
        if not isinstance(g, dict):
            raise ConfigError(f"config.json: {where}router.groups must be an object with 'count' and 'keep'")
        groups = (_int(g, "count", where + "router.groups."), _int(g, "keep", where + "router.groups."))
        if experts % groups[0] or groups[1] > groups[0]:
            raise ConfigError(f"config.json: {where}router.groups: the experts must divide into 'count' equal groups, of "
                              f"which 'keep' are kept")
        if groups[1] * (experts // groups[0]) < top:
            raise ConfigError(f"config.json: {where}router: the kept groups hold fewer experts than 'top'")
    shared = f.get("shared")
    if shared is not None and not isinstance(shared, dict):
        raise ConfigError(f"config.json: {where}shared must be an object with 'ff'")
    return RoutedConfig(experts, top, _int(e, "ff", where + "expert."),
                        _num(r, "scale", where + "router.") if r.get("scale") is not None else 1.0, groups,
                        None if shared is None else _int(shared, "ff", where + "shared."))


@dataclass(frozen=True)
class BizepelConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple
    canon_taps: int = 0
    side_dim: int = 0
    logit_scale: float = 1.0
    max_position_embeddings: int = 131072
    torch_dtype: str = "bfloat16"
    eos_token_id: tuple = ()
    architecture: str = "Bizepel"
    model_type: str = "bizepel"

    # ---- reading ---------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: dict) -> "BizepelConfig":
        vocab, width = _int(d, "vocab", ""), _int(d, "width", "")
        norm = d.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        eps = _num(norm, "eps", "norm.")
        taps = 0
        if d.get("canon") is not None:
            if not isinstance(d["canon"], dict):
                raise ConfigError("config.json: 'canon' must be an object with 'taps'")
            taps = _int(d["canon"], "taps", "canon.")
            if taps > 16:
                raise ConfigError("config.json: canon.taps: at most 16 taps")
        side = 0
        if d.get("token_side") is not None:
            if not isinstance(d["token_side"], dict):
                raise ConfigError("config.json: 'token_side' must be an object with 'dim'")
            side = _int(d["token_side"], "dim", "token_side.")
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(L, dict) or not isinstance(L.get("mixer"), dict):
                raise ConfigError(f"config.json: {where}mixer must be an object")
            layers.append(BizepelLayer(L.get("type"), _read_mixer(L.get("type"), L["mixer"], where + "mixer."),
                                       _read_mlp(L.get("mlp"), where + "mlp.")))
        widths = {L.mixer.kv_heads * L.mixer.vdim for L in layers if L.kind == ATTENTION and L.mixer.v_mix}
        if len(widths) > 1:
            raise ConfigError("config.json: layers that mix values (v_mix) must have value rows of one width "
                              "(kv_heads * vdim)")
        eos = d.get("eos_token_id")
        eos = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(vocab=vocab, width=width, eps=eps, layers=tuple(layers), canon_taps=taps, side_dim=side,
                   logit_scale=_num(d, "logit_scale", "") if d.get("logit_scale") is not None else 1.0,
                   max_position_embeddings=int(d.get("max_positions", 131072)),
                   torch_dtype=str(d.get("torch_dtype", "bfloat16")), eos_token_id=eos)

    # ---- sizes that only the tensors give ------------------------------------------------------
    @property
    def needs_tensor_shapes(self) -> bool:
        return any(L.kind == GENERAL_DELTA and L.mixer.decay_rank is None for L in self.layers)

    def with_tensor_shapes(self, shapes: dict) -> "BizepelConfig":
        """The configuration with the decay products' inner sizes read from the stored tensors' shapes
        (``shapes``: stored name -> shape)."""
        layers = []
        for i, L in enumerate(self.layers):
            m = L.mixer
            if L.kind == GENERAL_DELTA and m.decay_rank is None:
                name = f"l{i}.mix.w1"
                if name not in shapes or len(shapes[name]) != 2:
                    raise ConfigError(f"the model's files hold no matrix '{name}' to take the layer's decay rank from")
                m = replace(m, decay_rank=int(shapes[name][0]))
            layers.append(BizepelLayer(L.kind, m, L.mlp))
        return replace(self, layers=tuple(layers))

    # ---- writing ---------------------------------------------------------------------------
    def to_dict(self) -> dict:
        out = []
        for L in self.layers:
            m = L.mixer
            if L.kind == ATTENTION:
                d = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
                if m.conv:
                    d["conv"] = m.conv
                if m.rot_dims is not None:
                    d["rot"] = {"base": m.rot_base, "dims": m.rot_dims}
                if m.window is not None:
                    d["mask"] = {"size": m.window, "keep_first": m.keep_first}
                if m.v_mix:
                    d["v_mix"] = True
            elif L.kind == MAMBA1:
                d = {"inner": m.inner, "state": m.state, "dt_rank": m.dt_rank, "conv": m.conv}
            else:
                d = {"heads": m.heads, "dim": m.dim}
                if m.decay_rank is not None:
                    d["decay_rank"] = m.decay_rank
            f = L.mlp
            if f is None:
                mlp = None
            elif isinstance(f, DenseConfig):
                mlp = {"kind": "dense", "ff": f.ff}
            else:
                router = {"experts": f.experts, "top": f.top, "scale": f.scale}
                if f.groups is not None:
                    router["groups"] = {"count": f.groups[0], "keep": f.groups[1]}
                mlp = {"kind": "moe", "expert": {"ff": f.ff}, "router": router}
                if f.shared_ff is not None:
                    mlp["shared"] = {"ff": f.shared_ff}
            out.append({"type": L.kind, "mixer": d, "mlp": mlp})
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "layers": out, "logit_scale": self.logit_scale, "max_positions": self.max_position_embeddings,
             "torch_dtype": self.torch_dtype}
        if self.canon_taps:
            d["canon"] = {"taps": self.canon_taps}
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d
