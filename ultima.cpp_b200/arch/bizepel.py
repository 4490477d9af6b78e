"""Bizepel as data: layers of three kinds in the order the configuration lists them; the tensor names of its files.

A layer is pre-norm with layer norms (a weight, no bias): each sublayer reads norm(x) through a causal convolution over
time that is added to its own input, and its result is multiplied channel by channel by a learned vector before the
sum; behind the feed-forward the stream takes a per-layer input made from a second embedding of the token
(arrangement ``pre_norm_filtered`` with ``causal_conv_residual``, ``layer_scale`` and ``token_side``).  The mixer is
attention with biases, short convolutions on q, k and v, per-head q/k norm, a rotation of neighbouring columns, a window
with kept first positions and values blended with the first such layer's (part ``attention``), the selective scan
(``selective_scan``) or the generalised delta rule (``general_delta``).  The feed-forward is dense with the exact GELU
(``plain_mlp``) or routed with sigmoid scores, groups scored by their two best, renormalised weights and
squared-rectifier experts (``routed_experts``).  The embedding's rows pass a layer norm; the logits come from the
embedding table and are multiplied by a constant, which stands on the final norm's weight.
"""
from __future__ import annotations

from ..config.base import ArchitectureEntry, register_architecture
from ..config.bizepel import ATTENTION, GENERAL_DELTA, MAMBA1, BizepelConfig, DenseConfig
from ..parts.base import ModelSpec, Run, layer, part

_NAMES = {"mixer_norm": "norm1.", "mixer_filter": "canon1.", "mixer": "mix.", "mixer_gate": "ls1.",
          "feed_forward_norm": "norm2.", "feed_forward_filter": "canon2.", "feed_forward": "mlp.",
          "feed_forward_gate": "ls2.", "tail": "side."}

# part's own tensor name -> the name below the role's prefix in the files
_ATTENTION_NAMES = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
                    "q_proj.bias": "q.b", "k_proj.bias": "k.b", "v_proj.bias": "v.b", "q_norm.weight": "q.norm",
                    "k_norm.weight": "k.norm", "q_conv.weight": "q.conv", "k_conv.weight": "k.conv", "v_conv.weight": "v.conv",
                    "vmix": "vmix"}
_MAMBA_NAMES = {"in_proj.weight": "in", "conv.weight": "conv", "conv.bias": "conv.b", "x_proj.weight": "x",
                "dt_proj.weight": "dt", "dt_bias": "dt.b", "a_log": "A_log", "d_skip": "D", "o_proj.weight": "o"}
_DELTA_NAMES = {"r_proj.weight": "r", "k_proj.weight": "k", "v_proj.weight": "v", "gate_proj.weight": "g",
                "a_proj.weight": "a", "a_bias": "a.b", "w_down.weight": "w1", "w_up.weight": "w2", "w_bias": "w0",
                "o_norm.weight": "norm", "o_proj.weight": "o"}
_PLAIN_NAMES = {"up_proj.weight": "up", "down_proj.weight": "down"}


def build_spec(cfg: BizepelConfig, max_positions: int | None = None) -> ModelSpec:
    if cfg.needs_tensor_shapes:
        raise ValueError("Bizepel: the inner size of a general_delta layer's decay product is not known; read the configuration "
                         "with config_from_dir (which takes it from the stored matrix's shape) or give 'decay_rank'")
    max_pos = int(max_positions or cfg.max_position_embeddings)
    W, eps = cfg.width, cfg.eps
    norm = part("layer", width=W, eps=eps)
    layers, runs = [], []
    renames = [("embed.weight", "embed"), ("embed.norm.weight", "embed.norm"), ("final.norm.weight", "final.norm")]
    mixes_values = False
    optional = []
    n_layers = len(cfg.layers)
    for i, L in enumerate(cfg.layers):
        m, pre = L.mixer, f"l{i}."
        if L.kind == ATTENTION:
            position = None
            if m.rot_dims is not None:
                position = part("rotary_interleaved", head_dim=m.dim, theta=m.rot_base, max_positions=max_pos, rotary_dim=m.rot_dims)
            mix = None
            if m.v_mix:
                mix = "blend" if mixes_values else "source"
                mixes_values = True
            mixer = part("attention", width=W, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, qk_norm=True, eps=eps,
                         position=position, window=m.window, keep_first=m.keep_first if m.window is not None else 0,
                         scale=m.scale, v_head_dim=m.vdim, in_bias=True, conv=m.conv, value_mix=mix)
            names = _ATTENTION_NAMES
            if mix is None:
                optional.append(f"{pre}mix.vmix")            # a file may carry the number for a layer that blends nothing
        elif L.kind == MAMBA1:
            mixer = part("selective_scan", width=W, inner=m.inner, state=m.state, dt_rank=m.dt_rank, conv=m.conv)
            names = _MAMBA_NAMES
        elif L.kind == GENERAL_DELTA:
            mixer = part("general_delta", width=W, n_heads=m.heads, head_dim=m.dim, decay_rank=m.decay_rank, eps=eps)
            names = _DELTA_NAMES
        else:
            raise ValueError(f"Bizepel: unknown layer type {L.kind!r}")
        renames += [(f"{pre}mix.{a}", f"{pre}mix.{b}") for a, b in names.items()]
        renames += [(f"{pre}norm1.weight", f"{pre}norm1"), (f"{pre}canon1.weight", f"{pre}canon1"), (f"{pre}ls1.scale", f"{pre}ls1"),
                    (f"{pre}side.embed", "side.embed")]
        flt = part("causal_conv_residual", width=W, taps=cfg.canon_taps) if cfg.canon_taps else part("none")
        tail = part("token_side", width=W, vocab_size=cfg.vocab, dim=cfg.side_dim, index=i, tables=n_layers, eps=eps) \
            if cfg.side_dim else part("none")
        roles = {"mixer_norm": norm, "mixer_filter": flt, "mixer": mixer, "mixer_gate": part("layer_scale", width=W)}
        f = L.mlp
        if f is not None:
            if isinstance(f, DenseConfig):
                ff = part("plain_mlp", width=W, inner=f.ff, activation="gelu_erf")
                renames += [(f"{pre}mlp.{a}", f"{pre}mlp.{b}") for a, b in _PLAIN_NAMES.items()]
            else:
                ff = part("routed_experts", width=W, inner=f.ff, n_experts=f.experts, top=f.top, groups=f.groups,
                          shared_inner=f.shared_ff, score="sigmoid", group_score="top2_sum", normalise=True,
                          weight_scale=f.scale, expert="relu_squared")
                renames.append((f"{pre}mlp.router.weight", f"{pre}mlp.router"))
                for e in range(f.experts):
                    renames += [(f"{pre}mlp.experts.{e}.{a}", f"{pre}mlp.e{e}.{b}") for a, b in _PLAIN_NAMES.items()]
                if f.shared_ff is not None:
                    renames += [(f"{pre}mlp.shared.{a}", f"{pre}mlp.shared.{b}") for a, b in _PLAIN_NAMES.items()]
            roles.update(feed_forward_norm=norm, feed_forward_filter=flt, feed_forward=ff,
                         feed_forward_gate=part("layer_scale", width=W))
            renames += [(f"{pre}norm2.weight", f"{pre}norm2"), (f"{pre}canon2.weight", f"{pre}canon2"),
                        (f"{pre}ls2.scale", f"{pre}ls2")]
            kind = "pre_norm_filtered"
        else:
            kind = "pre_norm_filtered_mixer_only"
            optional += [f"{pre}norm2", f"{pre}canon2", f"{pre}ls2"]      # a file may carry them for a layer without feed-forward
        roles["tail"] = tail
        layers.append(layer(part(kind), prefix=pre, names=tuple((r, _NAMES[r]) for r in roles), **roles))
        runs.append(Run(i))
    return ModelSpec(
        width=W, vocab_size=cfg.vocab, max_positions=max_pos,
        embedding=part("token_table", vocab_size=cfg.vocab, width=W, norm="layer", eps=eps), embedding_name="embed.",
        layers=tuple(layers), runs=tuple(runs),
        final_norm=part("layer", width=W, eps=eps, scale=cfg.logit_scale), final_norm_name="final.norm.",
        head=part("linear", vocab_size=cfg.vocab, width=W, tied=True), head_name="head.",
        stop_token_ids=tuple(cfg.eos_token_id), renames=tuple(renames), optional_tensors=tuple(optional))


register_architecture(ArchitectureEntry(
    name="Bizepel", model_type="bizepel", supported=True,
    notes="Bizepel: attention with short convolutions and blended values, the selective scan and the generalised delta rule "
          "behind input convolutions and layer scales, dense and routed feed-forwards, a per-layer token input",
    config_cls=BizepelConfig, build_spec=build_spec))
