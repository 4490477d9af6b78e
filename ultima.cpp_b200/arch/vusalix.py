"""Vusalix as data: layers of three kinds in the order the configuration lists them, over a residual stream kept in
several copies; the tensor names of its files.

A layer is pre-norm, x += mixer(norm1(x)); x += feed_forward(norm2(x)), but the stream exists in ``streams`` copies
that every sublayer reads and writes through small learned tables (arrangement ``hyper_pre_norm``, connection
``hyper``; without ``streams`` the plain ``pre_norm``).  The mixer is attention with a score cap, a learned bias by
distance in buckets, a window and a learned sink (part ``attention`` with ``softcap``, ``distance_buckets``, ``window``,
``learned_sink``), latent attention (part ``latent_attention``) or the gated delta rule with one decay a head and a
SiLU output gate (part ``gated_delta`` with ``decay="head"``, ``gate="silu"``).  The feed-forward is ``routed_experts``.
"""
from __future__ import annotations

from ..config.base import ArchitectureEntry, register_architecture
from ..config.vusalix import ATTENTION, DELTA, LATENT, VusalixConfig
from ..parts.base import ModelSpec, Run, layer, part

_NAMES = {"mixer": "mix.", "feed_forward": "mlp.", "mixer_norm": "norm1.", "feed_forward_norm": "norm2.",
          "mixer_connection": "hc1.", "feed_forward_connection": "hc2."}

# part's own tensor name -> the name below the role's prefix in the files
_ATTENTION_NAMES = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o", "rel": "rel",
                    "sink": "sink"}
_LATENT_NAMES = {"q_proj.weight": "q", "kv_down.weight": "dkv", "kv_norm.weight": "dkv.norm", "k_up.weight": "uk",
                 "v_up.weight": "uv", "o_proj.weight": "o"}
_DELTA_NAMES = {"q_proj.weight": "q", "q_conv.weight": "q.conv", "k_proj.weight": "k", "k_conv.weight": "k.conv",
                "v_proj.weight": "v", "v_conv.weight": "v.conv", "b_proj.weight": "b", "a_log": "A_log",
                "o_norm.weight": "norm", "a_proj.weight": "a", "dt_bias": "dt_bias", "gate_proj.weight": "g",
                "o_proj.weight": "o"}
_DENSE_NAMES = {"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"}


def build_spec(cfg: VusalixConfig, max_positions: int | None = None) -> ModelSpec:
    if cfg.needs_tensor_shapes:
        raise ValueError("Vusalix: the number of distance buckets is not known; read the configuration with config_from_dir "
                         "(which takes it from the bias table's shape) or give 'buckets'")
    max_pos = int(max_positions or cfg.max_position_embeddings)
    norm = part("rms", width=cfg.width, eps=cfg.eps)
    S = cfg.streams
    layers, runs = [], []
    renames = [("embed.weight", "embed"), ("final.norm.weight", "final.norm"), ("head.weight", "head")]
    for i, L in enumerate(cfg.layers):
        m, pre = L.mixer, f"l{i}."
        if L.kind == ATTENTION:
            mixer = part("attention", width=cfg.width, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, qk_norm=False,
                         eps=cfg.eps, position=None, window=m.window, scale=m.scale, v_head_dim=m.vdim, softcap=m.softcap,
                         distance_buckets=(m.buckets, m.bias_max), learned_sink=True)
            names = _ATTENTION_NAMES
        elif L.kind == LATENT:
            sc = m.scaling
            mixer = part("latent_attention", width=cfg.width, n_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim,
                         v_head_dim=m.vdim, rank=m.kv_rank, scale=m.scale, eps=cfg.eps, theta=m.rot_base, rotary_dim=m.rot_dims,
                         max_positions=max_pos, window=m.window,
                         yarn=None if sc is None else (sc.factor, sc.original, sc.fast, sc.slow))
            names = _LATENT_NAMES
        elif L.kind == DELTA:
            mixer = part("gated_delta", width=cfg.width, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim,
                         v_head_dim=m.vdim, conv=m.conv, eps=cfg.eps, decay="head", gate="silu")
            names = _DELTA_NAMES
        else:
            raise ValueError(f"Vusalix: unknown layer type {L.kind!r}")
        renames += [(f"{pre}mix.{a}", f"{pre}mix.{b}") for a, b in names.items()]
        renames.append((f"{pre}norm1.weight", f"{pre}norm1"))
        roles = {"mixer_norm": norm, "mixer": mixer}
        if S:
            roles["mixer_connection"] = part("hyper", streams=S)
        if L.mlp is not None:
            f = L.mlp
            roles["feed_forward_norm"] = norm
            roles["feed_forward"] = part("routed_experts", width=cfg.width, inner=f.ff, n_experts=f.experts, top=f.top,
                                         n_identity=f.identity, groups=f.groups, shared_inner=f.shared_ff)
            if S:
                roles["feed_forward_connection"] = part("hyper", streams=S)
            renames.append((f"{pre}norm2.weight", f"{pre}norm2"))
            renames.append((f"{pre}mlp.router.weight", f"{pre}mlp.router"))
            for e in range(f.experts):
                renames += [(f"{pre}mlp.experts.{e}.{a}", f"{pre}mlp.e{e}.{b}") for a, b in _DENSE_NAMES.items()]
            if f.shared_ff is not None:
                renames += [(f"{pre}mlp.shared.{a}", f"{pre}mlp.shared.{b}") for a, b in _DENSE_NAMES.items()]
            kind = "hyper_pre_norm" if S else "pre_norm"
        else:
            kind = "hyper_pre_norm_mixer_only" if S else "pre_norm_mixer_only"
        layers.append(layer(part(kind), prefix=pre, names=tuple((r, _NAMES[r]) for r in roles), **roles))
        runs.append(Run(i))
    return ModelSpec(
        width=cfg.width, vocab_size=cfg.vocab, max_positions=max_pos,
        embedding=part("token_table", vocab_size=cfg.vocab, width=cfg.width), embedding_name="embed.",
        layers=tuple(layers), runs=tuple(runs), final_norm=norm, final_norm_name="final.norm.",
        head=part("linear", vocab_size=cfg.vocab, width=cfg.width, tied=False), head_name="head.",
        stop_token_ids=tuple(cfg.eos_token_id), renames=tuple(renames), streams=int(S or 0))


register_architecture(ArchitectureEntry(
    name="Vusalix", model_type="vusalix", supported=True,
    notes="Vusalix: capped attention with a learned bias by distance and a sink, latent attention and gated delta-rule "
          "layers over a residual stream in several copies, routed feed-forwards",
    config_cls=VusalixConfig, build_spec=build_spec))
