"""A plain, slow implementation of the Vusalix design: one function for each mechanism, with
whole-sequence matrices or token by token, on the CPU.  It shares no code with the package: it takes
config.json's dictionary and a dictionary of tensors by their stored names.

``dt`` is the type everything is computed in (float64 for an oracle).  Nothing here keeps a cache: a
sequence is always run whole.
"""
from __future__ import annotations

import math

import torch


def rms_norm(x, w, eps):
    """x * w / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


# ---------------------------------------------------------------------------------------
# masks and the softmax
# ---------------------------------------------------------------------------------------
def visible(T, window):
    """[T, T] bool: query i sees key j when 0 <= i - j < window (no window: every j <= i)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & (i - j < window)
    return seen


def softmax_with_sink(scores, seen, sink=None):
    """Weights over the visible keys; ``sink`` [H]: the denominator has one more term exp(sink_h), which
    brings no value.  scores [H, T, T]."""
    s = scores.masked_fill(~seen[None], -math.inf)
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink[:, None, None] - m)
    return e / den


# ---------------------------------------------------------------------------------------
# attention with a score cap, a learned bias by distance and a sink
# ---------------------------------------------------------------------------------------
def distance_bucket(n: int, B: int, D: float) -> int:
    """Distances below B/2 have a bucket each; the others share the rest in equal steps of ln(distance) up to D."""
    half = B // 2
    if n < half:
        return n
    return min(B - 1, half + int(math.floor(math.log(n / half) / math.log(D / half) * (B - half))))


def capped_biased_attention(h, W, m, pre):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[pre + "q"].T).view(T, H, d).transpose(0, 1)
    k = (h @ W[pre + "k"].T).view(T, G, d).transpose(0, 1).repeat_interleave(H // G, dim=0)
    v = (h @ W[pre + "v"].T).view(T, G, dv).transpose(0, 1).repeat_interleave(H // G, dim=0)
    s = q @ k.transpose(1, 2) * m["scale"]
    cap = m.get("softcap")
    if cap:
        s = cap * torch.tanh(s / cap)
    rel = W[pre + "rel"]
    B = rel.shape[0]
    bucket = torch.tensor([[distance_bucket(i - j, B, m["bias_max"]) if j <= i else 0 for j in range(T)] for i in range(T)])
    s = s + rel[bucket].permute(2, 0, 1)
    window = m["mask"]["size"] if m.get("mask") else None
    p = softmax_with_sink(s, visible(T, window), W[pre + "sink"])
    o = (p @ v).transpose(0, 1).reshape(T, H * dv)
    return o @ W[pre + "o"].T


# ---------------------------------------------------------------------------------------
# latent attention: keys and values from one small vector a position, one rotated key part for all heads
# ---------------------------------------------------------------------------------------
def rotary_frequencies(rot, dt=torch.float64):
    dims, base = rot["dims"], rot["base"]
    i = torch.arange(dims // 2, dtype=dt)
    f = torch.tensor(base, dtype=dt) ** (-2.0 * i / dims)
    amp = 1.0
    sc = rot.get("scaling")
    if sc:
        def where(t):
            return dims * math.log(sc["original"] / (2 * math.pi * t)) / (2 * math.log(base))
        lo = max(math.floor(where(sc["fast"])), 0)
        hi = min(math.ceil(where(sc["slow"])), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
        f = f / sc["factor"] * ramp + f * (1 - ramp)
        amp = 0.1 * math.log(sc["factor"]) + 1.0
    return f, amp


def rotate_neighbours(x, positions, rot):
    """x [T, ..., dims]: the pair (2i, 2i + 1) turns by positions * f_i; cos and sin carry the amplitude."""
    f, amp = rotary_frequencies(rot, x.dtype)
    a = positions.to(x.dtype)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [f.numel()]
    c, s = (torch.cos(a) * amp).view(shape), (torch.sin(a) * amp).view(shape)
    u, v = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = u * c - v * s
    out[..., 1::2] = v * c + u * s
    return out


def latent_attention(h, W, m, eps, pre):
    T = h.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (h @ W[pre + "q"].T).view(T, H, d + r)
    q_plain, q_rot = q[..., :d], rotate_neighbours(q[..., d:], pos, m["rot"])
    low = h @ W[pre + "dkv"].T
    c = rms_norm(low[:, :rank], W[pre + "dkv.norm"], eps)
    k_rot = rotate_neighbours(low[:, rank:], pos, m["rot"])                 # [T, r], the same for every head
    k_plain = (c @ W[pre + "uk"].T).view(T, H, d)
    v = (c @ W[pre + "uv"].T).view(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    window = m["mask"]["size"] if m.get("mask") else None
    p = softmax_with_sink(s, visible(T, window))
    o = torch.einsum("hij,jhe->ihe", p, v).reshape(T, H * dv)
    return o @ W[pre + "o"].T


# ---------------------------------------------------------------------------------------
# the gated delta rule
# ---------------------------------------------------------------------------------------
def short_conv_silu(x, taps):
    """x [T, C]; taps [C, n], the last column on the current token, zeros before the start; then silu."""
    T, C = x.shape
    n = taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, C, dtype=x.dtype), x], 0)
    y = torch.zeros_like(x)
    for j in range(n):
        y = y + padded[j: j + T] * taps[:, j]
    return silu(y)


def delta_rule_scan(q, k, v, beta, g):
    """q, k [T, H, D], v [T, H, E], beta, g [T, H].  S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, H, D = q.shape
    E = v.shape[2]
    S = torch.zeros(H, D, E, dtype=q.dtype)
    out = torch.zeros(T, H, E, dtype=q.dtype)
    for t in range(T):
        S = g[t][:, None, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hde,hd->he", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hde,hd->he", S, q[t])
    return out


def delta_mixer(h, W, m, eps, pre):
    T = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv_silu(h @ W[pre + "q"].T, W[pre + "q.conv"]).view(T, G, D)
    k = short_conv_silu(h @ W[pre + "k"].T, W[pre + "k.conv"]).view(T, G, D)
    v = short_conv_silu(h @ W[pre + "v"].T, W[pre + "v.conv"]).view(T, H, E)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q = q.repeat_interleave(H // G, dim=1)
    k = k.repeat_interleave(H // G, dim=1)
    beta = torch.sigmoid(h @ W[pre + "b"].T)
    g = torch.exp(-torch.exp(W[pre + "A_log"]) * softplus(h @ W[pre + "a"].T + W[pre + "dt_bias"]))
    o = delta_rule_scan(q, k, v, beta, g)
    o = rms_norm(o, W[pre + "norm"], eps) * silu(h @ W[pre + "g"].T).view(T, H, E)
    return o.reshape(T, H * E) @ W[pre + "o"].T


# ---------------------------------------------------------------------------------------
# the routed feed-forward
# ---------------------------------------------------------------------------------------
def gated_expert(h, W, pre):
    return (silu(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


def route(h, W, f, pre):
    """For every token the chosen router outputs and their weights: [T, top] each."""
    r = f["router"]
    n = r["experts"] + r.get("identity", 0)
    s = torch.softmax(h @ W[pre + "router"].T, dim=-1)
    choice = s + W[pre + "correction"]
    groups = r.get("groups")
    if groups:
        size = n // groups["count"]
        best = choice.view(-1, groups["count"], size).max(-1).values
        keep = torch.topk(best, groups["keep"], dim=-1).indices
        allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, keep, True).repeat_interleave(size, dim=1)
        choice = choice.masked_fill(~allowed, -math.inf)
    idx = torch.topk(choice, r["top"], dim=-1).indices
    return idx, torch.gather(s, 1, idx)


def routed_feed_forward(h, W, f, pre):
    r = f["router"]
    idx, w = route(h, W, f, pre)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(idx[t].tolist(), w[t]):
            if e >= r["experts"]:
                out[t] += a * h[t]                      # an identity expert hands its input on
            else:
                out[t] += a * gated_expert(h[t:t + 1], W, f"{pre}e{e}.")[0]
    if f.get("shared"):
        out = out + gated_expert(h, W, pre + "shared.")
    return out


# ---------------------------------------------------------------------------------------
# the layer: several copies of the stream, read and written through small learned tables
# ---------------------------------------------------------------------------------------
def connected(xs, W, pre, norm_w, eps, sublayer):
    """xs [s, T, width].  u = sum_s in[s] x_s; y = sublayer(norm(u)); x_t <- sum_s mix[s, t] x_s + out[t] y."""
    u = torch.einsum("s,stw->tw", W[pre + "in"], xs)
    y = sublayer(rms_norm(u, norm_w, eps))
    return torch.einsum("sr,stw->rtw", W[pre + "mix"], xs) + W[pre + "out"][:, None, None] * y[None]


def mixer_of(L, W, eps, pre):
    kind, m = L["type"], L["mixer"]
    if kind == "attention":
        return lambda h: capped_biased_attention(h, W, m, pre)
    if kind == "latent_attention":
        return lambda h: latent_attention(h, W, m, eps, pre)
    if kind == "delta":
        return lambda h: delta_mixer(h, W, m, eps, pre)
    raise ValueError(kind)


def forward(cfg, W, tokens, dt=torch.float64, layers_out=None):
    """Logits [T, vocab] of one sequence; ``layers_out``: a list that receives the residual stream (the sum of
    its copies) after every layer."""
    W = {n: (t.to(dt) if t.is_floating_point() else t) for n, t in W.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    streams = cfg.get("streams")
    xs = x[None].repeat(streams or 1, 1, 1)
    for i, L in enumerate(cfg["layers"]):
        mixer = mixer_of(L, W, eps, f"l{i}.mix.")
        ff = (lambda h, i=i, L=L: routed_feed_forward(h, W, L["mlp"], f"l{i}.mlp.")) if L.get("mlp") else None
        if streams:
            xs = connected(xs, W, f"l{i}.hc1.", W[f"l{i}.norm1"], eps, mixer)
            if ff is not None:
                xs = connected(xs, W, f"l{i}.hc2.", W[f"l{i}.norm2"], eps, ff)
        else:
            xs = xs + mixer(rms_norm(xs[0], W[f"l{i}.norm1"], eps))[None]
            if ff is not None:
                xs = xs + ff(rms_norm(xs[0], W[f"l{i}.norm2"], eps))[None]
        if layers_out is not None:
            layers_out.append(xs.sum(0).clone())
    return rms_norm(xs.sum(0), W["final.norm"], eps) @ W["head"].T


def read_folder(model_dir: str):
    """(config.json's dictionary, stored name -> float64 tensor) read with nothing but the file format."""
    import json
    import os
    import struct

    import numpy as np
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    header.pop("__metadata__", None)
    W = {}
    for name, e in header.items():
        raw = data[e["data_offsets"][0]:e["data_offsets"][1]]
        if e["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif e["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4")
        else:
            raise ValueError(f"plain reader: dtype {e['dtype']} of {name}")
        W[name] = torch.from_numpy(a.astype(np.float64).reshape(e["shape"]))
    return cfg, W


def logits(cfg, W, tokens):
    """float64 numpy [T, vocab]."""
    with torch.no_grad():
        return forward(cfg, W, tokens, torch.float64).numpy()
