"""A plain, slow implementation of the Bizepel design: one function for each mechanism, whole sequences on the
CPU, token loops where the design has a recurrence.  It shares no code with the package: it takes config.json's
dictionary and a dictionary of tensors by their stored names, already in the type everything is computed in
(float64 for an oracle).  Nothing here keeps a cache: a sequence is always run whole.
"""
from __future__ import annotations

import math

import torch


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w over the last axis, the variance about the mean; no bias."""
    m = x.mean(-1, keepdim=True)
    d = x - m
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    return 0.5 * z * (1 + torch.erf(z / math.sqrt(2)))


def causal_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), nothing before the start."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += w[:, j] * u[:T - back]
    return y


# ---------------------------------------------------------------------------------------
# attention: biases, short convolutions, q/k norm, rotation of neighbours, window with kept first tokens, value mixing
# ---------------------------------------------------------------------------------------
def rotate_neighbours(x, rot):
    """x [T, heads, dim]: pairs (2i, 2i + 1) of the first rot.dims columns turn by position * base^(-2i/dims)."""
    T, dims = x.shape[0], rot["dims"]
    i = torch.arange(dims // 2, dtype=x.dtype)
    f = torch.tensor(rot["base"], dtype=x.dtype) ** (-2.0 * i / dims)
    a = torch.arange(T, dtype=x.dtype)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def visible(T, mask):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if mask:
        seen = seen & ((i - j < mask["size"]) | (j < mask.get("keep_first", 0)))
    return seen


def attention(h, W, m, eps, pre, v_first=None):
    """Returns (output, the values of this layer after the convolution and before any mixing)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ W[pre + "q"].T + W[pre + "q.b"]
    k = h @ W[pre + "k"].T + W[pre + "k.b"]
    v = h @ W[pre + "v"].T + W[pre + "v.b"]
    if m.get("conv"):
        q, k, v = causal_conv(q, W[pre + "q.conv"]), causal_conv(k, W[pre + "k.conv"]), causal_conv(v, W[pre + "v.conv"])
    own_v = v
    if v_first is not None:
        lam = W[pre + "vmix"]
        v = (1 - lam) * v + lam * v_first
    q = rms_norm(q.view(T, H, d), W[pre + "q.norm"], eps)
    k = rms_norm(k.view(T, G, d), W[pre + "k.norm"], eps)
    if m.get("rot"):
        q, k = rotate_neighbours(q, m["rot"]), rotate_neighbours(k, m["rot"])
    q = q.transpose(0, 1)
    k = k.transpose(0, 1).repeat_interleave(H // G, dim=0)
    vv = v.view(T, G, dv).transpose(0, 1).repeat_interleave(H // G, dim=0)
    s = q @ k.transpose(1, 2) * m["scale"]
    s = s.masked_fill(~visible(T, m.get("mask"))[None], -math.inf)
    p = torch.softmax(s, dim=-1)
    o = (p @ vv).transpose(0, 1).reshape(T, H * dv)
    return o @ W[pre + "o"].T, own_v


# ---------------------------------------------------------------------------------------
# the selective scan (first Mamba form): a decay for every channel and state element
# ---------------------------------------------------------------------------------------
def mamba1(h, W, m, pre):
    T = h.shape[0]
    inner, N, R = m["inner"], m["state"], m["dt_rank"]
    xz = h @ W[pre + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, W[pre + "conv"]) + W[pre + "conv.b"])
    p = x @ W[pre + "x"].T
    dt, B, C = p[:, :R], p[:, R:R + N], p[:, R + N:R + 2 * N]
    dt = softplus(dt @ W[pre + "dt"].T + W[pre + "dt.b"])
    A = -torch.exp(W[pre + "A_log"])
    S = torch.zeros(inner, N, dtype=h.dtype)
    y = torch.empty(T, inner, dtype=h.dtype)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + W[pre + "D"] * x[t]
    return (y * silu(z)) @ W[pre + "o"].T


# ---------------------------------------------------------------------------------------
# the generalised delta rule: a decay and a removal rate for every key channel
# ---------------------------------------------------------------------------------------
def general_delta(h, W, m, eps, pre):
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    r = (h @ W[pre + "r"].T).view(T, H, D)
    k = (h @ W[pre + "k"].T).view(T, H, D)
    v = (h @ W[pre + "v"].T).view(T, H, D)
    w = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ W[pre + "w1"].T) @ W[pre + "w2"].T + W[pre + "w0"])).view(T, H, D)
    a = torch.sigmoid(h @ W[pre + "a"].T + W[pre + "a.b"]).view(T, H, D)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    S = torch.zeros(H, D, D, dtype=h.dtype)
    o = torch.empty(T, H, D, dtype=h.dtype)
    for t in range(T):
        uS = torch.einsum("hd,hde->he", u[t], S)
        S = w[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hde,hd->he", S, r[t])
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps)
    o = o.reshape(T, H * D) * W[pre + "norm"] * torch.sigmoid(h @ W[pre + "g"].T)
    return o @ W[pre + "o"].T


# ---------------------------------------------------------------------------------------
# feed-forwards
# ---------------------------------------------------------------------------------------
def dense_ff(h, W, pre):
    return gelu_erf(h @ W[pre + "up"].T) @ W[pre + "down"].T


def expert(h, W, pre):
    return torch.relu(h @ W[pre + "up"].T) ** 2 @ W[pre + "down"].T


def route(h, W, f, pre):
    """(indices [T, top], weights [T, top]) of the chosen experts."""
    r = f["router"]
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ W[pre + "router"].T)
    choice = s + W[pre + "correction"]
    g = r.get("groups")
    if g:
        per = E // g["count"]
        grouped = choice.view(-1, g["count"], per)
        score = grouped.topk(min(2, per), dim=-1).values.sum(-1)
        keep = score.topk(g["keep"], dim=-1).indices
        allowed = torch.zeros_like(score, dtype=torch.bool).scatter_(1, keep, True)
        choice = choice.masked_fill(~allowed.repeat_interleave(per, dim=1), -math.inf)
    idx = choice.topk(top, dim=-1).indices
    wts = s.gather(1, idx)
    wts = wts / (wts.sum(-1, keepdim=True) + 1e-20) * r.get("scale", 1.0)
    return idx, wts


def moe_ff(h, W, f, pre):
    idx, wts = route(h, W, f, pre)
    out = torch.zeros(h.shape[0], W[pre + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for c in range(idx.shape[1]):
            out[t] += wts[t, c] * expert(h[t:t + 1], W, f"{pre}e{int(idx[t, c])}.")[0]
    if f.get("shared"):
        out = out + expert(h, W, pre + "shared.")
    return out


def feed_forward(h, W, f, pre):
    return dense_ff(h, W, pre) if f["kind"] == "dense" else moe_ff(h, W, f, pre)


# ---------------------------------------------------------------------------------------
# a layer and the model
# ---------------------------------------------------------------------------------------
def side_input(x, tokens, W, cfg, i, pre):
    dim, eps = cfg["token_side"]["dim"], cfg["norm"]["eps"]
    e = W["side.embed"][tokens][:, i * dim:(i + 1) * dim]
    g = gelu_tanh(x @ W[pre + "side.gate"].T) * e
    y = g @ W[pre + "side.proj"].T
    return x + rms_norm(y, W[pre + "side.norm"], eps)


def forward(cfg, W, tokens, dt=torch.float64, taps=None):
    """Logits [T, vocab] of one whole sequence; ``taps`` (a list) receives the stream behind every layer."""
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    W = {n: (t.to(dt) if t.is_floating_point() else t) for n, t in W.items()}
    x = layer_norm(W["embed"][tokens], W["embed.norm"], eps)
    v_first = None
    for i, L in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h = layer_norm(x, W[pre + "norm1"], eps)
        if cfg.get("canon"):
            h = h + causal_conv(h, W[pre + "canon1"])
        m = L["mixer"]
        if L["type"] == "attention":
            y, own_v = attention(h, W, m, eps, pre + "mix.", v_first if m.get("v_mix") else None)
            if m.get("v_mix") and v_first is None:
                v_first = own_v
        elif L["type"] == "mamba1":
            y = mamba1(h, W, m, pre + "mix.")
        elif L["type"] == "general_delta":
            y = general_delta(h, W, m, eps, pre + "mix.")
        else:
            raise ValueError(L["type"])
        x = x + y * W[pre + "ls1"]
        if L.get("mlp"):
            h = layer_norm(x, W[pre + "norm2"], eps)
            if cfg.get("canon"):
                h = h + causal_conv(h, W[pre + "canon2"])
            x = x + feed_forward(h, W, L["mlp"], pre + "mlp.") * W[pre + "ls2"]
        if cfg.get("token_side"):
            x = side_input(x, tokens, W, cfg, i, pre)
        if taps is not None:
            taps.append(x.clone())
    x = layer_norm(x, W["final.norm"], eps)
    return x @ W["embed"].T * cfg.get("logit_scale", 1.0)


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
