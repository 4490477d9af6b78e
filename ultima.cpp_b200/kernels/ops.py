"""Python entry points of the CUDA kernels.  Each takes torch tensors on the GPU, checks
what the kernel assumes, and launches on torch's current stream.  There is no other
implementation behind them: on a machine without the GPU or the compiler they raise.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

import numpy as np
import torch

from . import build

F32, BF16 = 0, 1
EPI_STORE, EPI_ADD, EPI_SWIGLU, EPI_SWIGLU_IL = 0, 1, 2, 3
MAX_HEAD_DIM = 256          # the largest head size the attention and q/k preparation kernels take


class KernelError(RuntimeError):
    pass


_sm_counts: dict = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (the current one by default), asked of the device once.
    Slice counts, K splits and the choice between kernels follow it."""
    if device is None:
        n = _sm_counts.get(None)
        if n is not None:
            return n
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: the number of multiprocessors cannot be asked")
    idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    n = _sm_counts.get(idx)
    if n is None:
        n = _sm_counts[idx] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
    if device is None:
        _sm_counts[None] = n            # (one process drives one GPU: the current device does not change)
    return n


def _code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _ptr(t):
    return 0 if t is None else t.data_ptr()


# The current stream's handle is asked for at every launch: through the raw accessor that torch's own
# extensions use (a few hundred nanoseconds) where it exists, not through the Stream object (microseconds).
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    if _raw_stream is None or _raw_device is None:
        return torch.cuda.current_stream().cuda_stream
    return _raw_stream(_raw_device())


def _check(rc: int, what: str) -> None:
    if rc == 0:
        return
    if rc == -1:
        raise KernelError(f"{what}: an argument is outside what the kernel takes")
    if rc == -2:
        raise KernelError(f"{what}: this combination of element types is not built")
    raise KernelError(f"{what}: CUDA error {rc} at launch")


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels run on CUDA tensors only; there is no CPU path")


_sigs_done = set()


def _lib(source: str, defines=()):
    lib = build.load(source, tuple(defines))
    key = (source, tuple(defines))
    if key not in _sigs_done:
        _declare(lib, source)
        _sigs_done.add(key)
    return lib


def _declare(lib, source: str) -> None:
    P, I, L, F, U = c_void_p, c_int, c_longlong, c_float, c_ulonglong
    sigs = {
        "basic.cu": {
            "ub_embed": [P, I, P, P, I, I, I, P, P],
            "ub_rmsnorm": [P, P, P, P, I, I, I, F, P],
            "ub_qk_prepare": [P, I, I, L, P, I, L, P, P, P, P, P, P, P, P, I, P, I, I, I, I, I, I, I, F, I, I, I, P, P, L, P],
            "ub_rotate_pairs": [P, I, L, I, I, I, P, P, P, I, I, P],
            "ub_kv_write": [P, P, I, L, P, P, P, P, I, P, I, I, I, I, I, I, P],
            "ub_silu_mul": [P, I, I, L, P, I, I, I, P],
            "ub_rmsnorm_add": [P, P, P, P, I, I, I, F, I, P],
            "ub_glu_clamped": [P, I, P, I, I, I, F, F, F, P],
            "ub_head_gate": [P, I, L, P, L, I, I, I, P],
            "ub_convert": [P, I, P, I, L, P],
            "ub_add_into": [P, P, I, L, P],
            "ub_fill_normal": [P, I, L, U, F, F, P],
            "ub_embed_pairs": [P, P, I, P, P, P, P, P, P, I, I, I, F, I, L, L, P, P],
            "ub_gated_add": [P, L, I, L, P, P, P, I, I, I, P],
            "ub_add_rows": [P, P, P, I, I, P],
            "ub_elem_gate": [P, I, L, P, L, I, I, F, P],
        },
        "gemm_simt.cu": {"ub_gemm_simt": [P, I, P, P, I, P, I, I, I, I, L, L, L, I, P],
                         "ub_gemm_simt_batched": [P, I, P, I, P, I, I, I, I, L, L, L, I, L, L, L, P],
                         "ub_gemm_simt_grouped": [P, I, P, P, I, P, I, I, I, L, L, L, L, P, P, P, I, I, P]},
        "streams.cu": {"ub_streams_fill": [P, P, I, I, I, P],
                       "ub_streams_pass": [P, L, I, P, P, P, P, I, P, P, P, I, I, I, F, P]},
        "routed.cu": {"ub_route": [P, L, I, L, P, I, I, I, I, I, I, P, P, P, I, F, P],
                      "ub_route_plan": [P, P, P, P, P, I, I, P],
                      "ub_route_scatter": [P, P, P, P, P, I, I, I, P],
                      "ub_route_small": [P, L, I, L, P, I, I, I, I, I, I, P, P, P, P, P, P, I, I, F, P],
                      "ub_route_combine": [P, I, P, I, P, P, P, I, I, I, P],
                      "ub_route_gather": [P, P, P, I, I, L, P]},
        "latent.cu": {"ub_latent_place": [P, I, L, I, L, I, I, P, P, I, P, P, P, I, P, P, P, I, P, I, I, I, I, I, I, I, I, F, P]},
        "attn_simple.cu": {"ub_attn_simple": [P, L, I, P, P, I, P, L, P, P, P, I, I, I, I, I, I, I, I, F, I, I, P, L, I, P, I, I, F, F, P, I, P, I, P],
                           "ub_qkv_place_rows": [P, I, L, I, L, I, I, I, P, I, L, P, P, I, P, P, I, I, P, P, P, P, I, P, I, I, I, I, I,
                                                 I, I, I, F, I, I, P, P],
                           "ub_qkv_place": [P, I, L, I, L, I, I, I, P, I, L, P, P, P, P, I, P, P, P, P, I, P, I, I, I, I, I,
                                            I, I, I, F, I, P, P]},
        "delta.cu": {"ub_delta_prepare": [P, L, I, L, P, P, P, I, P, P, P, P, P, P, P, P, P, P, P, I, F, F, P],
                     "ub_conv_state_update": [P, L, I, L, P, P, P, I, I, I, P],
                     "ub_delta_scan": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, P, P, P],
                     "ub_delta_finish": [P, P, L, I, L, I, P, P, I, I, I, I, F, I, P],
                     "ub_gdelta_prepare": [P, L, I, L, I, I, I, I, P, P, P, P, P, P, P, P, P, I, I, I, F, F, P]},
        "ssm.cu": {"ub_ssm_prepare": [P, L, I, L, P, P, P, P, I, P, P, P, P, P, P, P, P, I, P],
                   "ub_ssm_conv_state_update": [P, L, I, L, P, P, P, P, I, P],
                   "ub_ssm_scan": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, P],
                   "ub_ssm_finish": [P, P, L, I, L, P, P, P, I, I, I, F, F, P],
                   "ub_mamba1_scan": [P, I, P, P, P, L, I, I, P, P, P, L, I, L, P, I, P, P, P, I, I, I, I, P],
                   "ub_mamba1_scan_staged": [P, I, P, P, P, L, I, I, P, P, P, L, I, L, P, I, P, P, P, I, I, I, I, P, P]},
        "rowwise.cu": {"ub_layernorm": [P, P, P, I, P, I, I, F, P],
                       "ub_scale_add_norm": [P, P, P, I, P, F, P, I, I, I, I, P],
                       "ub_causal_conv": [P, I, L, I, L, I, P, P, P, I, P, P, P, P, I, L, I, I, I, I, I, I, I, I, P, P, P, P],
                       "ub_causal_conv_state": [P, I, L, I, L, I, P, P, P, P, I, I, I, P],
                       "ub_take_cols": [P, L, I, L, I, I, I, P, I, L, I, I, P],
                       "ub_unary": [P, I, P, I, L, I, P],
                       "ub_side_gate": [P, L, P, I, L, I, P, I, P, I, L, I, I, I, P]},
        "sampling.cu": {"ub_sample": [P, L, P, I, I, P, P, P, P, P, U, P, P, I, P], "ub_sample_params_size": []},
    }.get(source, {})
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = c_int


# ---------------------------------------------------------------------------------------
def embed(table, ids, out, status):
    """out[t, :] = table[ids[t], :] as float32; a bad id raises ``status`` (int32[1])."""
    _need_cuda(table, ids, out, status)
    T, width = out.shape
    assert out.dtype == torch.float32 and ids.dtype == torch.int32 and out.is_contiguous()
    assert table.is_contiguous() and table.shape[1] == width
    _check(_lib("basic.cu").ub_embed(_ptr(table), _code(table), _ptr(ids), _ptr(out), T, width,
                                     table.shape[0], _ptr(status), _stream()), "embed")


def embed_pairs(table, pairs, ids, batch, last, out, status, scale, buckets, mul_prev, mul_cur):
    """out[t, :] = scale * table[ids[t], :] + pairs[row, :], row = (previous token * mul_prev + ids[t] * mul_cur) mod
    buckets, or ``buckets`` for a sequence's first token.  ``last`` (int32 [slots]): the token before the step's first
    one, plus one (zero: none); the kernel moves it on to the step's last token."""
    _need_cuda(table, pairs, ids, out, status, last)
    T, width = out.shape
    assert out.dtype == torch.float32 and ids.dtype == torch.int32 and out.is_contiguous() and last.dtype == torch.int32
    assert table.is_contiguous() and pairs.is_contiguous() and table.shape[1] == width and pairs.shape == (buckets + 1, width)
    assert table.dtype == pairs.dtype and last.is_contiguous()
    _check(_lib("basic.cu").ub_embed_pairs(_ptr(table), _ptr(pairs), _code(table), _ptr(ids), _ptr(batch.tok_seq),
                                           _ptr(batch.seq_start), _ptr(batch.seq_slot), _ptr(last), _ptr(out), T, width,
                                           table.shape[0], float(scale), int(buckets), int(mul_prev), int(mul_cur),
                                           _ptr(status), _stream()), "embed_pairs")


def gated_add(g, bias, y, x, clear_y=False):
    """x += sigmoid(g + bias) * y; x, y float32 [T, width]; g float32 [T, width] or [parts, T, width] (summed), rows of
    any stride (a column range of a wider product); ``clear_y`` zeroes y behind the read."""
    _need_cuda(g, bias, y, x)
    T, width = x.shape
    assert x.dtype == y.dtype == g.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous() and y.shape == x.shape
    if g.dim() == 3:
        n_parts, part_stride, ldg = g.shape[0], g.stride(0), g.stride(1)
        assert g.shape[1:] == x.shape and g.stride(2) == 1
    else:
        n_parts, part_stride, ldg = 1, 0, g.stride(0)
        assert g.shape == x.shape and g.stride(1) == 1
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == width and bias.is_contiguous())
    _check(_lib("basic.cu").ub_gated_add(_ptr(g), ldg, n_parts, part_stride, _ptr(bias), _ptr(y), _ptr(x), T, width,
                                         1 if clear_y else 0, _stream()), "gated_add")


def add_rows(x, a=None, v=None):
    """x += a + v: ``a`` a float32 matrix of x's shape, ``v`` one float32 row added to every row."""
    _need_cuda(x, a, v)
    T, width = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous()
    assert a is None or (a.dtype == torch.float32 and a.shape == x.shape and a.is_contiguous())
    assert v is None or (v.dtype == torch.float32 and v.numel() == width and v.is_contiguous())
    _check(_lib("basic.cu").ub_add_rows(_ptr(x), _ptr(a), _ptr(v), T, width, _stream()), "add_rows")


def elem_gate(o, gate, scale=1.0):
    """o[t, c] *= scale * sigmoid(gate[t, c]) in place; gate float32 [T, cols] (any row stride)."""
    _need_cuda(o, gate)
    T, cols = o.shape
    assert o.stride(1) == 1 and gate.dtype == torch.float32 and gate.shape == (T, cols) and gate.stride(1) == 1
    _check(_lib("basic.cu").ub_elem_gate(_ptr(o), _code(o), o.stride(0), _ptr(gate), gate.stride(0), T, cols, float(scale),
                                         _stream()), "elem_gate")


def rmsnorm(x, weight, out, eps, rows=None):
    """out[r, :] = x[rows[r] or r, :] * weight / sqrt(mean(x^2) + eps); x float32."""
    _need_cuda(x, weight, out, rows)
    assert x.dtype == torch.float32 and weight.dtype == torch.float32
    assert x.is_contiguous() and out.is_contiguous() and weight.is_contiguous()
    n, width = out.shape
    assert x.shape[1] == width and weight.numel() == width
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.numel() == n
    _check(_lib("basic.cu").ub_rmsnorm(_ptr(x), _ptr(rows), _ptr(weight), _ptr(out), _code(out), n,
                                       width, float(eps), _stream()), "rmsnorm")


def qk_prepare(qkv, q_weight, k_weight, cos, sin, tok_pos, tok_seq, k_cache, v_cache, table,
               ring, page, n_heads, n_kv_heads, head_dim, eps, write_kv=True, q_out=None,
               rotary_dim=None, interleaved=False, kv_out=None):
    """Per-head norm and rotation of q and k, and the write of k, v into the cache.

    qkv: [T, (heads + 2 kv heads) * head size], or [parts, T, ...] whose sum over parts it is
    (slices of K of the projection).  q goes to ``q_out`` ([T, heads * head size], any row stride),
    or back into qkv's q columns when q_out is None (one part only).  cos, sin: [positions,
    rotary_dim / 2]; the first ``rotary_dim`` columns of a head (default: all) are rotated, in pairs
    (j, j + rotary_dim / 2) or, ``interleaved``, (2j, 2j + 1).  ``kv_out`` = (k, v), each
    [T, kv heads * head size] with q_out's element type and one row stride: keys and values go
    there instead of into the cache (see ``kv_write``)."""
    _need_cuda(qkv, k_cache, v_cache, table)
    width = (n_heads + 2 * n_kv_heads) * head_dim
    if qkv.dim() == 3:
        n_parts, T = qkv.shape[0], qkv.shape[1]
        part_stride = qkv.stride(0)
        assert qkv.shape[2] == width and qkv.stride(1) == width and qkv.stride(2) == 1
        assert q_out is not None
    else:
        n_parts, T, part_stride = 1, qkv.shape[0], 0
        assert qkv.is_contiguous() and qkv.shape[1] == width
    if q_out is None:
        q_out = qkv
    assert q_out.stride(1) == 1 and q_out.shape[0] == T
    assert table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
    for v in (q_weight, k_weight, cos, sin):
        assert v is None or (v.dtype == torch.float32 and v.is_contiguous())
    rd = int(rotary_dim) if rotary_dim is not None else head_dim
    if cos is not None:
        if rd % 2 or not (2 <= rd <= head_dim):
            raise KernelError(f"qk_prepare: rotary size {rd} must be even and at most the head size {head_dim}")
        assert cos.shape[1] == rd // 2 and sin.shape == cos.shape
    k_out = v_out = None
    kv_stride = 0
    if kv_out is not None:
        k_out, v_out = kv_out
        assert k_out.dtype == q_out.dtype == v_out.dtype and k_out.stride(1) == 1 and v_out.stride(1) == 1
        assert k_out.stride(0) == v_out.stride(0) and k_out.shape == v_out.shape == (T, n_kv_heads * head_dim)
        kv_stride = k_out.stride(0)
    _check(_lib("basic.cu").ub_qk_prepare(
        _ptr(qkv), _code(qkv), n_parts, part_stride, _ptr(q_out), _code(q_out), q_out.stride(0),
        _ptr(q_weight), _ptr(k_weight), _ptr(cos), _ptr(sin), _ptr(tok_pos),
        _ptr(tok_seq), _ptr(k_cache), _ptr(v_cache), _code(k_cache), _ptr(table), table.shape[1],
        ring, page, T, n_heads, n_kv_heads, head_dim, float(eps), 1 if write_kv else 0,
        rd, 1 if interleaved else 0, _ptr(k_out), _ptr(v_out), kv_stride, _stream()),
        "qk_prepare")


def rotate_pairs(x, cos, sin, tok_pos, rotary_dim=None, interleaved=False):
    """Rotate, in place, pairs of the first ``rotary_dim`` columns of every head of x [T, heads,
    head size] (heads side by side in a row, any row stride) by the angles of each token's position."""
    _need_cuda(x, cos, sin, tok_pos)
    T, n_heads, hd = x.shape
    assert x.stride(2) == 1 and x.stride(1) == hd and cos.dtype == torch.float32 and cos.is_contiguous()
    rd = int(rotary_dim) if rotary_dim is not None else hd
    assert cos.shape[1] == rd // 2 and sin.shape == cos.shape and tok_pos.dtype == torch.int32
    _check(_lib("basic.cu").ub_rotate_pairs(_ptr(x), _code(x), x.stride(0), T, n_heads, hd, _ptr(cos), _ptr(sin),
                                            _ptr(tok_pos), rd, 1 if interleaved else 0, _stream()), "rotate_pairs")


def kv_write(k, v, tok_pos, tok_seq, k_cache, v_cache, table, ring, page, n_kv_heads, head_dim):
    """k, v [T, kv heads * head size] (one row stride) into the paged cache at each token's position."""
    _need_cuda(k, v, k_cache, v_cache, table)
    T = k.shape[0]
    assert k.shape == v.shape == (T, n_kv_heads * head_dim) and k.stride(1) == 1 and v.stride(1) == 1
    assert k.stride(0) == v.stride(0) and k.dtype == v.dtype
    assert table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
    _check(_lib("basic.cu").ub_kv_write(_ptr(k), _ptr(v), _code(k), k.stride(0), _ptr(tok_pos), _ptr(tok_seq), _ptr(k_cache),
                                        _ptr(v_cache), _code(k_cache), _ptr(table), table.shape[1], ring, page, T,
                                        n_kv_heads, head_dim, _stream()), "kv_write")


def silu_mul(gate_up, out):
    """out[t, f] = silu(g[t, f]) * g[t, F + f], g being gate_up ([T, 2F]) or the sum over the first
    axis of gate_up ([parts, T, 2F])."""
    _need_cuda(gate_up, out)
    T, F = out.shape
    if gate_up.dim() == 3:
        n_parts, part_stride = gate_up.shape[0], gate_up.stride(0)
        assert gate_up.shape[1:] == (T, 2 * F) and gate_up.stride(1) == 2 * F and gate_up.stride(2) == 1
    else:
        n_parts, part_stride = 1, 0
        assert gate_up.shape == (T, 2 * F) and gate_up.is_contiguous()
    assert out.is_contiguous()
    _check(_lib("basic.cu").ub_silu_mul(_ptr(gate_up), _code(gate_up), n_parts, part_stride, _ptr(out),
                                        _code(out), T, F, _stream()), "silu_mul")


def rmsnorm_add(y, weight, x, eps, h=None, clear_y=False):
    """x += y * weight / sqrt(mean(y^2) + eps), row by row (x, y float32).  ``h``: the new x in h's type,
    for the next reader; ``clear_y``: y is zeroed behind the read."""
    _need_cuda(y, weight, x, h)
    n, width = x.shape
    assert x.dtype == y.dtype == weight.dtype == torch.float32 and y.shape == x.shape and weight.numel() == width
    assert x.is_contiguous() and y.is_contiguous() and (h is None or (h.is_contiguous() and h.shape == x.shape))
    _check(_lib("basic.cu").ub_rmsnorm_add(_ptr(y), _ptr(weight), _ptr(x), _ptr(h), _code(h) if h is not None else F32,
                                           n, width, float(eps), 1 if clear_y else 0, _stream()), "rmsnorm_add")


def glu_clamped(gate_up, out, limit, alpha, shift):
    """out = g' * sigmoid(alpha g') * (u' + shift) with g' = min(g, limit), u' = clamp(u, -limit, limit);
    gate_up [T, 2F] holds g and u side by side."""
    _need_cuda(gate_up, out)
    T, F = out.shape
    assert gate_up.shape == (T, 2 * F) and gate_up.is_contiguous() and out.is_contiguous()
    _check(_lib("basic.cu").ub_glu_clamped(_ptr(gate_up), _code(gate_up), _ptr(out), _code(out), T, F, float(limit),
                                           float(alpha), float(shift), _stream()), "glu_clamped")


def head_gate(o, gate, n_heads, head_dim):
    """o[t, h, :] *= sigmoid(gate[t, h]) in place; gate float32 [T, heads] (any row stride)."""
    _need_cuda(o, gate)
    T = o.shape[0]
    assert o.stride(1) == 1 and o.shape[1] == n_heads * head_dim and gate.dtype == torch.float32
    assert gate.shape == (T, n_heads) and gate.stride(1) == 1
    _check(_lib("basic.cu").ub_head_gate(_ptr(o), _code(o), o.stride(0), _ptr(gate), gate.stride(0), T, n_heads, head_dim,
                                         _stream()), "head_gate")


def convert(src, dst):
    _need_cuda(src, dst)
    assert src.numel() == dst.numel() and src.is_contiguous() and dst.is_contiguous()
    _check(_lib("basic.cu").ub_convert(_ptr(src), _code(src), _ptr(dst), _code(dst), src.numel(),
                                       _stream()), "convert")


def add_into(acc, src):
    _need_cuda(acc, src)
    assert acc.dtype == torch.float32 and acc.numel() == src.numel()
    assert acc.is_contiguous() and src.is_contiguous()
    _check(_lib("basic.cu").ub_add_into(_ptr(acc), _ptr(src), _code(src), acc.numel(), _stream()),
           "add_into")


def fill_normal(out, seed: int, shift: float, std: float):
    _need_cuda(out)
    assert out.is_contiguous()
    _check(_lib("basic.cu").ub_fill_normal(_ptr(out), _code(out), out.numel(), seed & (2**64 - 1),
                                           float(shift), float(std), _stream()), "fill_normal")


def gemm_simt(a, w, out, epilogue=EPI_STORE, w2=None):
    """out[t, n] (=, +=) sum_k a[t, k] w[n, k] on the CUDA cores with float32 FMA;
    EPI_SWIGLU: out = silu(a w^T) * (a w2^T)."""
    _need_cuda(a, w, out, w2)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    if w2 is not None:
        assert w2.shape == w.shape and w2.dtype == w.dtype and w2.stride() == w.stride()
    _check(_lib("gemm_simt.cu").ub_gemm_simt(
        _ptr(a), _code(a), _ptr(w), _ptr(w2), _code(w), _ptr(out), _code(out), M, N, K,
        a.stride(0), w.stride(0), out.stride(0), epilogue, _stream()), "gemm_simt")


def attn_simple(q, k_cache, v_cache, out, tok_pos, tok_seq, table, ring, page, n_heads,
                n_kv_heads, head_dim, window, scale, v_head_dim=None, block=None, gate=None, keep_first=0, slopes=None,
                sink=False, out_scale=1.0, softcap=None, dist_bias=None, sink_vals=None, v_row=None):
    """Attention of every token of the step over its sequence's cached keys and values.  ``v_head_dim``:
    the values' head size where it differs; ``block``: positions are masked in blocks of this many,
    counted from the sequence's start; ``gate`` float32 [T, heads] or [T, heads * value size]: the output
    times its sigmoid, head by head or element by element; ``keep_first``: positions that stay visible
    behind the window; ``slopes`` float32 [heads]: slope * distance is taken off a score; ``sink``: one
    more term exp(0) in the softmax's sum (``sink_vals`` float32 [heads]: exp(sink_vals[h]) instead);
    ``out_scale`` multiplies the output; ``softcap``: a scaled score s becomes softcap * tanh(s / softcap);
    ``dist_bias`` float32 [distances, heads]: the row of min(distance, rows - 1) is added to the score behind the
    cap; ``v_row``: the width of a row of ``v_cache`` where it is more than the values' head size (values that
    are the leading columns of the key rows)."""
    _need_cuda(q, k_cache, v_cache, out, table, gate, slopes, dist_bias, sink_vals)
    assert dist_bias is None or (dist_bias.dtype == torch.float32 and dist_bias.is_contiguous() and dist_bias.dim() == 2
                                 and dist_bias.shape[1] == n_heads)
    assert sink_vals is None or (sink_vals.dtype == torch.float32 and sink_vals.is_contiguous() and sink_vals.numel() == n_heads)
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype
    assert table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
    gate_wide = 0
    if gate is not None:
        assert gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape[0] == T
        gate_wide = 0 if gate.shape[1] == n_heads and (v_head_dim or head_dim) != 1 else 1
        assert gate.shape[1] == (n_heads * int(v_head_dim or head_dim) if gate_wide else n_heads)
    assert slopes is None or (slopes.dtype == torch.float32 and slopes.numel() == n_heads and slopes.is_contiguous())
    _check(_lib("attn_simple.cu").ub_attn_simple(
        _ptr(q), q.stride(0), _code(q), _ptr(k_cache), _ptr(v_cache), _code(k_cache), _ptr(out),
        out.stride(0), _ptr(tok_pos), _ptr(tok_seq), _ptr(table), table.shape[1], ring, page, T,
        n_heads, n_kv_heads, head_dim, int(window or 0), float(scale), int(v_head_dim or head_dim), int(block or 0),
        _ptr(gate), gate.stride(0) if gate is not None else 0, int(keep_first or 0), _ptr(slopes),
        1 if (sink or sink_vals is not None) else 0, gate_wide, float(out_scale), float(softcap or 0.0), _ptr(dist_bias),
        dist_bias.shape[0] if dist_bias is not None else 0, _ptr(sink_vals), int(v_row or 0), _stream()), "attn_simple")


def qkv_place(x, q_off, k_off, v_off, q_out, q_weight, k_weight, cos, sin, rotary_dim, tok_pos, tok_seq, k_cache,
              v_cache, table, ring, page, n_heads, n_kv_heads, head_dim, v_head_dim, eps, g_off=None, gate_out=None):
    """Queries normed and rotated into ``q_out`` [T, heads * head size]; keys (normed, rotated) and values into the
    paged cache.  x: projection rows [T, N] or [parts, T, N] (summed), with the query heads from column q_off, the
    key heads from k_off and the value heads from v_off; k_off None: queries only.  ``gate_out`` (float32
    [T, heads], contiguous) receives the ``heads`` columns from ``g_off`` on (summed over the parts)."""
    _need_cuda(x, q_out, k_cache, v_cache, table)
    if x.dim() == 3:
        n_parts, T, part_stride, ldx = x.shape[0], x.shape[1], x.stride(0), x.stride(1)
        assert x.stride(2) == 1
    else:
        n_parts, T, part_stride, ldx = 1, x.shape[0], 0, x.stride(0)
        assert x.stride(1) == 1
    assert q_out.stride(1) == 1 and q_out.shape == (T, n_heads * head_dim)
    assert table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
    for v in (q_weight, k_weight, cos, sin):
        assert v is None or (v.dtype == torch.float32 and v.is_contiguous())
    rd = int(rotary_dim or 0)
    if cos is not None:
        assert cos.shape[1] == rd // 2 and sin.shape == cos.shape
    if gate_out is not None:
        assert gate_out.dtype == torch.float32 and gate_out.is_contiguous() and gate_out.shape == (T, n_heads)
        assert g_off is not None
    _check(_lib("attn_simple.cu").ub_qkv_place(
        _ptr(x), _code(x), ldx, n_parts, part_stride, int(q_off), -1 if k_off is None else int(k_off),
        -1 if v_off is None else int(v_off), _ptr(q_out), _code(q_out), q_out.stride(0), _ptr(q_weight), _ptr(k_weight),
        _ptr(cos), _ptr(sin), rd, _ptr(tok_pos), _ptr(tok_seq), _ptr(k_cache), _ptr(v_cache), _code(k_cache), _ptr(table),
        table.shape[1], ring, page, T, n_heads, n_kv_heads, head_dim, int(v_head_dim), float(eps), int(g_off or 0),
        _ptr(gate_out), _stream()), "qkv_place")


def qkv_place_rows(x, q_off, k_off, v_off, q_out, q_weight, k_weight, norm_whole, cos, sin, rotary_dim, interleaved, tok_pos,
                   tok_seq, k_cache, v_cache, table, ring, page, n_heads, n_kv_heads, head_dim, v_head_dim, eps, g_off=None,
                   gate_out=None):
    """``qkv_place`` with one block a token: the norm may run over all query heads (and all key heads) at once
    (``norm_whole``; weights [heads * head size]), the rotation may pair neighbouring columns (``interleaved``), and
    the values may be any columns of the row (``v_off`` = ``k_off``: the keys before norm and rotation).
    ``gate_out`` (float32 [T, any width], contiguous) receives that many columns from ``g_off`` on."""
    _need_cuda(x, q_out, k_cache, v_cache, table)
    if x.dim() == 3:
        n_parts, T, part_stride, ldx = x.shape[0], x.shape[1], x.stride(0), x.stride(1)
        assert x.stride(2) == 1
    else:
        n_parts, T, part_stride, ldx = 1, x.shape[0], 0, x.stride(0)
        assert x.stride(1) == 1
    assert q_out.stride(1) == 1 and q_out.shape == (T, n_heads * head_dim)
    assert table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
    for v, n in ((q_weight, n_heads), (k_weight, n_kv_heads)):
        assert v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == (n * head_dim if norm_whole else head_dim))
    rd = int(rotary_dim or 0)
    if cos is not None:
        assert cos.dtype == torch.float32 and cos.is_contiguous() and cos.shape[1] == rd // 2 and sin.shape == cos.shape
    g_width = 0
    if gate_out is not None:
        assert gate_out.dtype == torch.float32 and gate_out.is_contiguous() and gate_out.shape[0] == T and g_off is not None
        g_width = gate_out.shape[1]
    _check(_lib("attn_simple.cu").ub_qkv_place_rows(
        _ptr(x), _code(x), ldx, n_parts, part_stride, int(q_off), -1 if k_off is None else int(k_off),
        -1 if v_off is None else int(v_off), _ptr(q_out), _code(q_out), q_out.stride(0), _ptr(q_weight), _ptr(k_weight),
        1 if norm_whole else 0, _ptr(cos), _ptr(sin), rd, 1 if interleaved else 0, _ptr(tok_pos), _ptr(tok_seq), _ptr(k_cache),
        _ptr(v_cache), _code(k_cache), _ptr(table), table.shape[1], ring, page, T, n_heads, n_kv_heads, head_dim,
        int(v_head_dim), float(eps), int(g_off or 0), g_width, _ptr(gate_out), _stream()), "qkv_place_rows")


# ---------------------------------------------------------------------------------------
# several copies of the residual stream (csrc/streams.cu)
def streams_fill(x, xs):
    """Every copy xs[s] (float32 [S, T, width]) becomes x (float32 [T, width])."""
    _need_cuda(x, xs)
    assert x.dtype == xs.dtype == torch.float32 and x.is_contiguous() and xs.is_contiguous() and xs.shape[1:] == x.shape
    _check(_lib("streams.cu").ub_streams_fill(_ptr(x), _ptr(xs), x.shape[0], x.shape[1], xs.shape[0], _stream()), "streams_fill")


def streams_pass(xs, write=None, read=None, out=None, rows=None):
    """One pass over the copies xs (float32 [S, T, width]), row by row.  ``write`` = (mix [S, S] indexed [from, to],
    b [S], y [T, width]): xs'[t] = sum_s mix[s, t] xs[s] + b[t] y, and y is cleared.  ``read`` = (a [S] or None for the
    plain sum, norm weight [width] or None for no norm, eps): ``out`` [T or len(rows), width] receives
    norm(sum_s a[s] xs[s]) of the (new) copies; ``rows`` (int32) picks the rows that are read (no write then)."""
    _need_cuda(xs, out, rows)
    S, T, width = xs.shape
    assert xs.dtype == torch.float32 and xs.is_contiguous()
    mix = b = y = a = w = None
    eps = 0.0
    if write is not None:
        mix, b, y = write
        for t, n in ((mix, S * S), (b, S)):
            assert t.dtype == torch.float32 and t.is_contiguous() and t.numel() == n
        assert y.dtype == torch.float32 and y.is_contiguous() and y.shape == (T, width) and rows is None
    n_rows = T
    if read is not None:
        a, w, eps = read
        assert a is None or (a.dtype == torch.float32 and a.is_contiguous() and a.numel() == S)
        assert w is None or (w.dtype == torch.float32 and w.is_contiguous() and w.numel() == width)
        n_rows = T if rows is None else rows.numel()
        assert out is not None and out.is_contiguous() and out.shape == (n_rows, width)
        assert rows is None or rows.dtype == torch.int32
    _check(_lib("streams.cu").ub_streams_pass(_ptr(xs), xs.stride(0), S, _ptr(mix), _ptr(b), _ptr(y), _ptr(a),
                                              1 if read is not None else 0, _ptr(w), _ptr(rows), _ptr(out),
                                              _code(out) if out is not None else F32, n_rows, width, float(eps), _stream()),
           "streams_pass")


# ---------------------------------------------------------------------------------------
# products of many small matrices (csrc/gemm_simt.cu)
def gemm_batched(a, w, out):
    """out[:, b, :] = a[:, b, :] @ w[b].T for every b: a [T, B, K], w [B, N, K] contiguous, out [T, B, N]; a and out
    may be column ranges of wider rows (any row and batch stride, last stride 1).  CUDA cores, float32 sums in k order."""
    _need_cuda(a, w, out)
    T, B, K = a.shape
    N = w.shape[1]
    assert w.shape == (B, N, K) and w.is_contiguous() and out.shape == (T, B, N) and a.stride(2) == 1 and out.stride(2) == 1
    _check(_lib("gemm_simt.cu").ub_gemm_simt_batched(_ptr(a), _code(a), _ptr(w), _code(w), _ptr(out), _code(out), T, N, K,
                                                     a.stride(0), K, out.stride(0), B, a.stride(1), N * K, out.stride(1),
                                                     _stream()), "gemm_batched")


def gemm_grouped(a, w, out, tiles, n_tiles, src_rows, max_tiles, epilogue=EPI_STORE, w2=None):
    """Sorted rows against the matrix their tile names: out[p, :] = a[src_rows[p] (or p), :] @ w[e].T; w [E, N, K]
    contiguous; EPI_SWIGLU: out = silu(a w[e]^T) * (a w2[e]^T), w2 a view with w's strides.  ``tiles`` int32
    [max_tiles, 4] (matrix, first row, rows, -) and ``n_tiles`` int32 [1] on the device (csrc/routed.cu makes them)."""
    _need_cuda(a, w, out, tiles, n_tiles, src_rows)
    E, N, K = w.shape
    assert w.stride(2) == 1 and w.stride(1) >= K and a.stride(1) == 1 and out.stride(1) == 1 and out.shape[1] == N and a.shape[1] == K
    assert tiles.dtype == torch.int32 and tiles.is_contiguous() and tiles.numel() >= 4 * max_tiles
    if w2 is not None:
        assert w2.shape == w.shape and w2.stride() == w.stride() and w2.dtype == w.dtype
    _check(_lib("gemm_simt.cu").ub_gemm_simt_grouped(_ptr(a), _code(a), _ptr(w), _ptr(w2), _code(w), _ptr(out), _code(out), N, K,
                                                     a.stride(0), w.stride(1), out.stride(0), w.stride(0), _ptr(tiles),
                                                     _ptr(n_tiles), _ptr(src_rows), int(max_tiles), epilogue, _stream()),
           "gemm_grouped")


# ---------------------------------------------------------------------------------------
# the routed feed-forward (csrc/routed.cu)
ROUTE_TILE = 64          # sorted rows a tile of the grouped products


ROUTE_SIGMOID, ROUTE_GROUP_TOP2, ROUTE_NORMALISE = 1, 2, 4      # bits of a router's ``mode`` (csrc/routed.cu)


def route(z, correction, n_experts, top, n_groups, keep, idx, wts, counts, mode=0, wscale=1.0):
    """z float32 [T, outputs] router logits (or [parts, T, outputs], summed in that order) -> idx int32 [T, top], wts
    float32 [T, top]; counts int32 [n_experts] += rows.  ``mode``: ROUTE_* bits; ``wscale`` multiplies the weights."""
    _need_cuda(z, correction, idx, wts, counts)
    T, ldz, n_parts, part_stride = _parts_of(z)
    n_out = z.shape[-1]
    assert z.dtype == torch.float32 and z.stride(-1) == 1 and idx.dtype == torch.int32 and wts.dtype == torch.float32
    assert idx.is_contiguous() and wts.is_contiguous() and idx.shape == wts.shape == (T, top) and counts.dtype == torch.int32
    assert correction is None or (correction.dtype == torch.float32 and correction.is_contiguous() and correction.numel() == n_out)
    _check(_lib("routed.cu").ub_route(_ptr(z), ldz, n_parts, part_stride, _ptr(correction), T, n_out, n_experts, top, n_groups, keep,
                                      _ptr(idx), _ptr(wts), _ptr(counts), int(mode), float(wscale), _stream()), "route")


ROUTE_SMALL_TOKENS = 16      # steps of at most this many tokens (a warp each): route, plan and scatter as one launch (csrc/routed.cu)


def route_small(z, correction, n_experts, top, n_groups, keep, idx, wts, tiles, n_tiles, row_pos, src_rows, tile, mode=0,
                wscale=1.0):
    """``route``, ``route_plan`` and ``route_scatter`` of a step of at most ROUTE_SMALL_TOKENS tokens in one launch of one
    block; the counters of the separate kernels are not used."""
    _need_cuda(z, correction, idx, wts, tiles, n_tiles, row_pos, src_rows)
    T, ldz, n_parts, part_stride = _parts_of(z)
    n_out = z.shape[-1]
    assert T <= ROUTE_SMALL_TOKENS and z.dtype == torch.float32 and z.stride(-1) == 1
    assert idx.dtype == torch.int32 and wts.dtype == torch.float32 and idx.is_contiguous() and wts.is_contiguous()
    assert idx.shape == wts.shape == (T, top) and row_pos.dtype == src_rows.dtype == torch.int32
    assert row_pos.is_contiguous() and row_pos.numel() == T * top and src_rows.numel() >= T * top
    assert tiles.dtype == torch.int32 and tiles.is_contiguous() and n_tiles.dtype == torch.int32
    assert correction is None or (correction.dtype == torch.float32 and correction.is_contiguous() and correction.numel() == n_out)
    _check(_lib("routed.cu").ub_route_small(_ptr(z), ldz, n_parts, part_stride, _ptr(correction), T, n_out, n_experts, top,
                                            n_groups, keep, _ptr(idx), _ptr(wts), _ptr(tiles), _ptr(n_tiles), _ptr(row_pos),
                                            _ptr(src_rows), tile, int(mode), float(wscale), _stream()), "route_small")


def route_plan(counts, cursor, seg_start, tiles, n_tiles, n_experts, tile=ROUTE_TILE):
    _need_cuda(counts, cursor, seg_start, tiles, n_tiles)
    for t in (counts, cursor, seg_start, tiles, n_tiles):
        assert t.dtype == torch.int32 and t.is_contiguous()
    _check(_lib("routed.cu").ub_route_plan(_ptr(counts), _ptr(cursor), _ptr(seg_start), _ptr(tiles), _ptr(n_tiles), n_experts,
                                           tile, _stream()), "route_plan")


def route_scatter(idx, seg_start, cursor, row_pos, src_rows, n_experts):
    _need_cuda(idx, seg_start, cursor, row_pos, src_rows)
    T, top = idx.shape
    assert row_pos.dtype == src_rows.dtype == torch.int32 and row_pos.numel() == T * top and src_rows.numel() >= T * top
    _check(_lib("routed.cu").ub_route_scatter(_ptr(idx), _ptr(seg_start), _ptr(cursor), _ptr(row_pos), _ptr(src_rows), T, top,
                                              n_experts, _stream()), "route_scatter")


def route_gather(h, row_pos, out):
    """out[row_pos[t, k]] = h[t] for every choice that has a row (row_pos >= 0): the tokens' rows in the sorted order."""
    _need_cuda(h, row_pos, out)
    T, top = row_pos.shape
    assert h.is_contiguous() and out.is_contiguous() and h.dtype == out.dtype and h.shape[0] == T and out.shape[1] == h.shape[1]
    assert row_pos.dtype == torch.int32 and row_pos.is_contiguous()
    _check(_lib("routed.cu").ub_route_gather(_ptr(h), _ptr(row_pos), _ptr(out), T, top, h.shape[1] * h.element_size(), _stream()),
           "route_gather")


def route_combine(y, h, row_pos, wts, residual):
    """residual[t] += sum_k wts[t, k] * (y[row_pos[t, k]] or, where row_pos is -1, h[t])."""
    _need_cuda(y, h, row_pos, wts, residual)
    T, width = residual.shape
    assert residual.dtype == torch.float32 and residual.is_contiguous() and h.is_contiguous() and h.shape == (T, width)
    assert y.is_contiguous() and y.shape[1] == width
    _check(_lib("routed.cu").ub_route_combine(_ptr(y), _code(y), _ptr(h), _code(h), _ptr(row_pos), _ptr(wts), _ptr(residual),
                                              T, width, wts.shape[1], _stream()), "route_combine")


# ---------------------------------------------------------------------------------------
# latent attention (csrc/latent.cu)
def latent_place(x, q_off, c_off, q_plain, q_lat, c_weight, cos, sin, rotary_dim, tok_pos, tok_seq, k_cache, table, ring, page,
                 n_heads, dim, rot, rank, eps):
    """From projection rows x ([T, N] or [parts, T, N], summed): the heads' unrotated query parts into q_plain
    [T, heads, dim], their rotated parts into q_lat[:, :, rank:] ([T, heads, rank + rot]), and the position's cache row
    [normed latent | rotated key part]."""
    _need_cuda(x, q_plain, q_lat, k_cache, table)
    T, ldx, n_parts, part_stride = _parts_of(x)
    assert q_plain.is_contiguous() and q_lat.is_contiguous() and q_plain.dtype == q_lat.dtype
    assert q_plain.shape == (T, n_heads, dim) and q_lat.shape == (T, n_heads, rank + rot)
    assert c_weight.dtype == torch.float32 and c_weight.is_contiguous() and c_weight.numel() == rank
    assert table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
    if cos is not None:
        assert cos.dtype == torch.float32 and cos.is_contiguous() and cos.shape[1] == rotary_dim // 2 and sin.shape == cos.shape
    _check(_lib("latent.cu").ub_latent_place(
        _ptr(x), _code(x), ldx, n_parts, part_stride, int(q_off), int(c_off), _ptr(q_plain), _ptr(q_lat), _code(q_lat),
        _ptr(c_weight), _ptr(cos), _ptr(sin), int(rotary_dim or 0), _ptr(tok_pos), _ptr(tok_seq), _ptr(k_cache), _code(k_cache),
        _ptr(table), table.shape[1], ring, page, T, n_heads, dim, rot, rank, float(eps), _stream()), "latent_place")


# ---------------------------------------------------------------------------------------
# the state-space mixer (csrc/ssm.cu)
def ssm_shape(H, P, N, G, taps, offs):
    """The shape record the state-space kernels read: sizes and the first columns of z, x, B, C and dt in a
    projection row."""
    vals = [H, P, N, G, taps] + [int(o) for o in offs]
    return (c_int * len(vals))(*vals)


def ssm_prepare(p, shape, conv_w, conv_b, conv_state, dt_bias, a_log, batch, xbc, dtv, dec, update_state=False):
    """p: the projection [z | x | B | C | dt] in float32.  Fills xbc (the convolution's channels after bias and SiLU),
    dtv (step sizes) and dec (decays).  ``update_state`` (every sequence brings one token): the convolution's state
    moves on in this kernel."""
    _need_cuda(p, conv_w, conv_state, xbc, dtv, dec)
    assert p.dtype == torch.float32
    T, ldp, n_parts, part_stride = _parts_of(p)
    for t in (conv_w, conv_b, conv_state, dt_bias, a_log, xbc, dtv, dec):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous())
    if update_state:
        assert batch.n_seqs == T
    _check(_lib("ssm.cu").ub_ssm_prepare(_ptr(p), ldp, n_parts, part_stride, shape, _ptr(conv_w), _ptr(conv_b), _ptr(conv_state),
                                         1 if update_state else 0, _ptr(dt_bias), _ptr(a_log), _ptr(batch.tok_seq),
                                         _ptr(batch.seq_start), _ptr(batch.seq_slot), _ptr(xbc), _ptr(dtv), _ptr(dec), T,
                                         _stream()), "ssm_prepare")


def ssm_conv_state_update(p, shape, conv_state, batch):
    _need_cuda(p, conv_state)
    assert p.dtype == torch.float32 and conv_state.dtype == torch.float32 and conv_state.is_contiguous()
    _, ldp, n_parts, part_stride = _parts_of(p)
    _check(_lib("ssm.cu").ub_ssm_conv_state_update(_ptr(p), ldp, n_parts, part_stride, shape, _ptr(conv_state),
                                                   _ptr(batch.seq_start), _ptr(batch.seq_slot), batch.n_seqs, _stream()),
           "ssm_conv_state_update")


def ssm_scan(xbc, dtv, dec, d_skip, y, state, batch, H, P, N, G):
    _need_cuda(xbc, dtv, dec, d_skip, y, state)
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (H, N, P)
    for t in (xbc, dtv, dec, d_skip, y):
        assert t.dtype == torch.float32 and t.is_contiguous()
    _check(_lib("ssm.cu").ub_ssm_scan(_ptr(xbc), _ptr(dtv), _ptr(dec), _ptr(d_skip), _ptr(y), _ptr(state), _ptr(batch.seq_start),
                                      _ptr(batch.seq_slot), batch.n_seqs, xbc.shape[0], H, P, N, G, sm_count(), _stream()), "ssm_scan")


def ssm_finish(y, p, shape, weight, out, n_groups, eps, scale=1.0):
    """out = v / rms(v) * weight * scale in ``n_groups`` equal parts of a row, v = y * silu(z), z from the projection."""
    _need_cuda(y, p, weight, out)
    assert y.dtype == torch.float32 and y.is_contiguous() and out.is_contiguous() and out.shape == y.shape
    assert weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() == y.shape[1]
    _, ldp, n_parts, part_stride = _parts_of(p)
    _check(_lib("ssm.cu").ub_ssm_finish(_ptr(y), _ptr(p), ldp, n_parts, part_stride, shape, _ptr(weight), _ptr(out), _code(out),
                                        y.shape[0], int(n_groups), float(eps), float(scale), _stream()), "ssm_finish")


# ---------------------------------------------------------------------------------------
# the gated delta-rule mixer (csrc/delta.cu)
def delta_shape(H, G, D, E, taps, offs, a_off=-1):
    """The shape record the delta kernels read: sizes and the first columns of q, k, v and the write
    strength in a projection row; ``a_off`` >= 0: one decay a head, its sums in the row's columns from there on."""
    from ctypes import c_int as _ci
    vals = [H, G, D, E, taps] + [int(o) for o in offs] + [int(a_off)]
    return (_ci * len(vals))(*vals)


def _parts_of(p):
    """(rows, row stride, parts, part stride) of projections [T, N] or [parts, T, N] (summed over parts)."""
    if p.dim() == 3:
        assert p.stride(2) == 1
        return p.shape[1], p.stride(1), p.shape[0], p.stride(0)
    assert p.stride(1) == 1
    return p.shape[0], p.stride(0), 1, 0


def delta_prepare(p, shape, conv_w, conv_state, decay_pre, dt_bias, a_log, batch, qn, kn, vc, beta, dec, unit_eps, q_scale,
                  update_state=False):
    """p: the projections [q | k | v | write strength] in float32; decay_pre [T, heads * key size]: the decay's
    sums before the bias.  Fills qn, kn (unit vectors), vc, beta and dec.  ``update_state`` (every sequence brings
    one token): the convolution's state moves on in this kernel, and ``conv_state_update`` is not needed."""
    _need_cuda(p, conv_w, conv_state, decay_pre, qn, kn, vc, beta, dec)
    assert p.dtype == torch.float32
    T, ldp, n_parts, part_stride = _parts_of(p)
    for t in (conv_w, conv_state, decay_pre, dt_bias, a_log, qn, kn, vc, beta, dec):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous())
    assert decay_pre is not None or shape[9] >= 0, "one decay a head reads its sums from the projection row"
    if update_state:
        assert batch.n_seqs == T, "the state moves on in this kernel only when every sequence brings one token"
    _check(_lib("delta.cu").ub_delta_prepare(
        _ptr(p), ldp, n_parts, part_stride, shape, _ptr(conv_w), _ptr(conv_state), 1 if update_state else 0,
        _ptr(decay_pre), _ptr(dt_bias),
        _ptr(a_log), _ptr(batch.tok_seq), _ptr(batch.seq_start), _ptr(batch.seq_slot), _ptr(qn), _ptr(kn), _ptr(vc),
        _ptr(beta), _ptr(dec), T, float(unit_eps), float(q_scale), _stream()), "delta_prepare")


def conv_state_update(p, conv_state, batch, n_channels, taps):
    _need_cuda(p, conv_state)
    assert p.dtype == torch.float32 and conv_state.dtype == torch.float32 and conv_state.is_contiguous()
    _, ldp, n_parts, part_stride = _parts_of(p)
    _check(_lib("delta.cu").ub_conv_state_update(_ptr(p), ldp, n_parts, part_stride, _ptr(conv_state),
                                                 _ptr(batch.seq_start), _ptr(batch.seq_slot), batch.n_seqs, n_channels,
                                                 taps, _stream()), "conv_state_update")


def delta_scan(qn, kn, vc, beta, dec, out, state, batch, H, G, D, E, rem=None, kraw=None):
    """``rem`` and ``kraw`` (both or neither, float32 of the keys' shape): the generalised rule, S[d, :] = dec[d] S[d, :]
    - rem[d] (S^T kn) + kraw[d] v with both terms reading the old state; ``beta`` is then not read."""
    _need_cuda(qn, kn, vc, beta, dec, out, state, rem, kraw)
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (H, D, E)
    assert (rem is None) == (kraw is None)
    for t in (rem, kraw):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.shape == kn.shape)
    _check(_lib("delta.cu").ub_delta_scan(_ptr(qn), _ptr(kn), _ptr(vc), _ptr(beta), _ptr(dec), _ptr(out), _ptr(state),
                                          _ptr(batch.seq_start), _ptr(batch.seq_slot), batch.n_seqs, qn.shape[0], H, G, D, E, sm_count(),
                                          _ptr(rem), _ptr(kraw), _stream()),
           "delta_scan")


def gdelta_prepare(p, offs, a_bias, wpre, w0, rn, un, kraw, rem, dec, vc, H, D, unit_eps, decay_scale):
    """The generalised delta rule's operands from the projection row p (float32 [T, N] or [parts, T, N]; ``offs`` the first
    columns of r, k, v and the removal rate's sums) and the decay's sums ``wpre`` [T, H * D]: see csrc/delta.cu."""
    _need_cuda(p, a_bias, wpre, w0, rn, un, kraw, rem, dec, vc)
    assert p.dtype == torch.float32
    T, ldp, n_parts, part_stride = _parts_of(p)
    for t in (a_bias, wpre, w0, rn, un, kraw, rem, dec, vc):
        assert t.dtype == torch.float32 and t.is_contiguous()
    _check(_lib("delta.cu").ub_gdelta_prepare(_ptr(p), ldp, n_parts, part_stride, int(offs[0]), int(offs[1]), int(offs[2]),
                                              int(offs[3]), _ptr(a_bias), _ptr(wpre), _ptr(w0), _ptr(rn), _ptr(un), _ptr(kraw),
                                              _ptr(rem), _ptr(dec), _ptr(vc), T, H, D, float(unit_eps), float(decay_scale),
                                              _stream()), "gdelta_prepare")


def delta_finish(o, gate_pre, weight, out, H, E, eps, silu_gate=False):
    """out = o / rms(o) * weight * sigmoid(gate_pre) (``silu_gate``: * silu(gate_pre)), head by head; o float32
    [T, H * E]; gate_pre float32 [T, H * E] or [parts, T, H * E] (summed), rows of any stride.  ``weight``: [E], shared
    by the heads, or [H * E], a weight for every head."""
    _need_cuda(o, gate_pre, weight, out)
    assert o.dtype == torch.float32 and o.is_contiguous() and out.is_contiguous()
    assert gate_pre.dtype == torch.float32 and gate_pre.shape[-2:] == o.shape
    _, ldz, n_parts, part_stride = _parts_of(gate_pre)
    _check(_lib("delta.cu").ub_delta_finish(_ptr(o), _ptr(gate_pre), ldz, n_parts, part_stride, 1 if silu_gate else 0,
                                            _ptr(weight), _ptr(out), _code(out), o.shape[0], H, E, float(eps),
                                            1 if (weight.numel() == H * E and H > 1) else 0, _stream()),
           "delta_finish")


# ---------------------------------------------------------------------------------------
# ---------------------------------------------------------------------------------------
# row-wise kernels of a stream with scaled sublayers and input convolutions (csrc/rowwise.cu)
def layernorm(x, weight, out, eps, rows=None):
    """out = (x - mean) / sqrt(var + eps) * weight row by row (no bias); x float32 [T, width]; ``rows`` int32: only these."""
    _need_cuda(x, weight, out, rows)
    width = x.shape[1]
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and out.shape[1] == width
    assert weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() == width
    n = x.shape[0] if rows is None else rows.numel()
    assert out.shape[0] == n
    _check(_lib("rowwise.cu").ub_layernorm(_ptr(x), _ptr(weight), _ptr(out), _code(out), _ptr(rows), n, width, float(eps),
                                           _stream()), "layernorm")


NEXT_NONE, NEXT_PLAIN, NEXT_RMS, NEXT_LAYER = 0, 1, 2, 3


def scale_add_norm(y, scale, x, mode=NEXT_NONE, norm_weight=None, eps=0.0, out=None, clear_y=True):
    """x += scale * y (``scale`` float32 [width] or None for 1), y cleared; ``out`` receives what the next sublayer reads:
    the new x as it is (NEXT_PLAIN), its RMS norm (NEXT_RMS) or its layer norm (NEXT_LAYER) times ``norm_weight``."""
    _need_cuda(y, scale, x, norm_weight, out)
    T, width = x.shape
    assert x.dtype == y.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous() and y.shape == x.shape
    for v in (scale, norm_weight):
        assert v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == width)
    assert out is None or (out.is_contiguous() and tuple(out.shape) == (T, width))
    _check(_lib("rowwise.cu").ub_scale_add_norm(_ptr(y), _ptr(scale), _ptr(x), int(mode), _ptr(norm_weight), float(eps), _ptr(out),
                                                _code(out) if out is not None else F32, T, width, 1 if clear_y else 0, _stream()),
           "scale_add_norm")


def _conv_in(x, col_off, n_cols):
    if x.dim() == 3:
        assert x.stride(2) == 1 and col_off + n_cols <= x.shape[2]
        return x.shape[1], x.stride(1), x.shape[0], x.stride(0)
    assert x.stride(1) == 1 and col_off + n_cols <= x.shape[1]
    return x.shape[0], x.stride(0), 1, 0


def causal_conv(x, w, state, batch, out, col_off=0, bias=None, add_input=False, silu=False, mix=None, out_bias=None,
                update_state=False):
    """A short causal convolution over time on ``C = out.shape[1]`` channels of x (columns from ``col_off`` on; x [T, N] or
    [parts, T, N], summed; ``bias`` [C] is added to every input first): out_t = sum_j w[:, j] u_(t - taps + 1 + j), with the
    inputs of before the step from ``state`` float32 [slots, taps - 1, C] and zeros before a sequence's start.  ``w`` None:
    no convolution (out = u).  ``add_input``: out = u + conv(u).  ``out_bias`` [C]: added to the result (a bias of the
    convolution, which the state does not hold).  ``silu``: through SiLU.  ``mix`` = (mode, lo, hi, lam,
    shared): the channels lo .. hi - 1 go out to ``shared`` float32 [T, hi - lo] (mode 1) or become (1 - lam) * own +
    lam * shared (mode 2; lam a float32 scalar on the device).  The state is moved on by ``causal_conv_state``, or here with
    ``update_state`` when every sequence brings ONE token (a channel's state then has one reader)."""
    _need_cuda(x, w, state, out, bias, out_bias)
    assert out_bias is None or (out_bias.dtype == torch.float32 and out_bias.is_contiguous() and out_bias.numel() == out.shape[1])
    C = out.shape[1]
    T, ldx, n_parts, part_stride = _conv_in(x, col_off, C)
    taps = 0 if w is None else w.shape[1]
    assert out.shape[0] == T and out.stride(1) == 1
    assert w is None or (w.dtype == torch.float32 and w.is_contiguous() and w.shape[0] == C)
    assert bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == C)
    if taps > 1:
        assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (taps - 1, C)
    if update_state:
        assert batch.n_seqs == T, "the state moves on in this kernel only when every sequence brings one token"
    mode, lo, hi, lam, shared = mix if mix is not None else (0, 0, 0, None, None)
    if mode:
        _need_cuda(lam, shared)
        assert shared.dtype == torch.float32 and shared.is_contiguous() and tuple(shared.shape) == (T, hi - lo)
        assert lam is None or (lam.dtype == torch.float32 and lam.numel() == 1)
    _check(_lib("rowwise.cu").ub_causal_conv(
        _ptr(x), _code(x), ldx, n_parts, part_stride, int(col_off), _ptr(bias), _ptr(w), _ptr(state) if taps > 1 else 0,
        1 if (update_state and taps > 1) else 0, _ptr(batch.tok_seq), _ptr(batch.seq_start), _ptr(batch.seq_slot), _ptr(out), _code(out), out.stride(0), T, C, taps,
        1 if add_input else 0, 1 if silu else 0, int(mode), int(lo), int(hi), _ptr(lam), _ptr(shared), _ptr(out_bias),
        _stream()), "causal_conv")


def causal_conv_state(x, state, batch, col_off=0, bias=None):
    """The last taps - 1 inputs of (state ++ the step's inputs) become the state; x, col_off and bias as ``causal_conv`` got them."""
    _need_cuda(x, state, bias)
    K, C = state.shape[1], state.shape[2]
    _, ldx, n_parts, part_stride = _conv_in(x, col_off, C)
    assert state.dtype == torch.float32 and state.is_contiguous()
    _check(_lib("rowwise.cu").ub_causal_conv_state(_ptr(x), _code(x), ldx, n_parts, part_stride, int(col_off), _ptr(bias),
                                                   _ptr(state), _ptr(batch.seq_start), _ptr(batch.seq_slot), batch.n_seqs, C,
                                                   K + 1, _stream()), "causal_conv_state")


def take_cols(x, col_off, n, out, tanh=False):
    """out[:, :n] = x[:, col_off : col_off + n] (x float32 [T, N] or [parts, T, N], summed), through tanh if asked; the
    columns of ``out`` from n on are zeroed (an operand padded to an aligned width)."""
    _need_cuda(x, out)
    assert x.dtype == torch.float32 and out.stride(1) == 1 and n <= out.shape[1]
    T, ldx, n_parts, part_stride = _conv_in(x, col_off, n)
    assert out.shape[0] == T
    _check(_lib("rowwise.cu").ub_take_cols(_ptr(x), ldx, n_parts, part_stride, int(col_off), int(n), 1 if tanh else 0, _ptr(out),
                                           _code(out), out.stride(0), out.shape[1], T, _stream()), "take_cols")


UNARY_GELU_ERF, UNARY_RELU_SQUARED = 1, 2


def unary(x, out, kind):
    _need_cuda(x, out)
    assert x.is_contiguous() and out.is_contiguous() and x.shape == out.shape
    _check(_lib("rowwise.cu").ub_unary(_ptr(x), _code(x), _ptr(out), _code(out), x.numel(), int(kind), _stream()), "unary")


def side_gate(s, table, col0, ids, out, dim):
    """out[t, j] = gelu_tanh(s[t, j]) * table[ids[t], col0 + j] for j < dim, zero beyond; s float32 [T, >= dim]."""
    _need_cuda(s, table, ids, out)
    assert s.dtype == torch.float32 and s.stride(1) == 1 and table.stride(1) == 1 and out.stride(1) == 1
    assert ids.dtype == torch.int32 and col0 + dim <= table.shape[1] and dim <= out.shape[1] and dim <= s.shape[1]
    _check(_lib("rowwise.cu").ub_side_gate(_ptr(s), s.stride(0), _ptr(table), _code(table), table.stride(0), int(col0), _ptr(ids),
                                           table.shape[0], _ptr(out), _code(out), out.stride(0), int(dim), out.shape[1],
                                           s.shape[0], _stream()), "side_gate")


def mamba1_scan(x, dtp, dt_bias, bc, b_off, c_off, A, d_skip, z, out, state, batch, N, work=None):
    """The selective scan with a decay for every (channel, state element); see csrc/ssm.cu.  x, out [T, inner] in the
    activation type; dtp float32 [T, inner] (the step size's sums before the bias); bc float32 [T, >= c_off + N] with the B
    row from column b_off and the C row from c_off; A float32 [inner, N] (negative); z float32 [T, M] or [parts, T, M] whose
    first ``inner`` columns are the gate's sums; state float32 [slots, inner, N].  ``work`` (float32 [2, T, inner]): the
    three-kernel form for steps of many tokens a sequence, which takes what depends on one (token, channel) alone out of the
    chain from token to token; ``dtp`` is then overwritten with the step sizes."""
    _need_cuda(x, dtp, dt_bias, bc, A, d_skip, z, out, state)
    T, inner = x.shape
    assert x.is_contiguous() and out.is_contiguous() and out.shape == x.shape and x.dtype == out.dtype
    for t in (dtp, dt_bias, A, d_skip, state):
        assert t.dtype == torch.float32 and t.is_contiguous()
    assert bc.dtype == torch.float32 and bc.stride(1) == 1 and z.dtype == torch.float32
    assert tuple(state.shape[1:]) == (inner, N) and tuple(A.shape) == (inner, N) and tuple(dtp.shape) == (T, inner)
    _, ldz, z_parts, z_stride = _conv_in(z, 0, inner)
    if work is not None:
        _need_cuda(work)
        assert work.dtype == torch.float32 and work.is_contiguous() and work.numel() >= 2 * T * inner
        _check(_lib("ssm.cu").ub_mamba1_scan_staged(
            _ptr(x), _code(x), _ptr(dtp), _ptr(dt_bias), _ptr(bc), bc.stride(0), int(b_off), int(c_off), _ptr(A), _ptr(d_skip),
            _ptr(z), ldz, z_parts, z_stride, _ptr(out), _code(out), _ptr(state), _ptr(batch.seq_start), _ptr(batch.seq_slot),
            batch.n_seqs, T, inner, int(N), _ptr(work), _stream()), "mamba1_scan_staged")
        return
    _check(_lib("ssm.cu").ub_mamba1_scan(_ptr(x), _code(x), _ptr(dtp), _ptr(dt_bias), _ptr(bc), bc.stride(0), int(b_off), int(c_off),
                                         _ptr(A), _ptr(d_skip), _ptr(z), ldz, z_parts, z_stride, _ptr(out), _code(out), _ptr(state),
                                         _ptr(batch.seq_start), _ptr(batch.seq_slot), batch.n_seqs, T, inner, int(N), _stream()),
           "mamba1_scan")


SAMPLE_DTYPE = np.dtype([
    ("temperature", "<f4"), ("top_p", "<f4"), ("min_p", "<f4"), ("rep_penalty", "<f4"),
    ("freq_penalty", "<f4"), ("presence_penalty", "<f4"), ("dry_multiplier", "<f4"),
    ("dry_base", "<f4"), ("top_k", "<i4"), ("repeat_last_n", "<i4"), ("dry_last_n", "<i4"),
    ("dry_allowed_len", "<i4"), ("n_recent", "<i4"), ("recent_offset", "<i4"), ("n_bias", "<i4"),
    ("bias_offset", "<i4"), ("seed", "<u8"), ("counter", "<u8")])


def sample(logits, work, params_dev, recent, bias_ids, bias_vals, out_ids, counter_add: int = 0,
           hist=None, hist_len=None):
    """One token id for each row of float32 ``logits``; ``params_dev`` holds one record of
    SAMPLE_DTYPE a row (as bytes on the device); ``counter_add`` is added to every row's counter.
    ``hist`` [rings, capacity] int32 and ``hist_len`` [rings] int32: rings of recent tokens that stay on
    the device; a row whose record has n_recent < 0 reads ring ``recent_offset`` and appends its token."""
    _need_cuda(logits, work, params_dev, out_ids)
    lib = _lib("sampling.cu")
    assert lib.ub_sample_params_size() == SAMPLE_DTYPE.itemsize
    n, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert work is None or (work.dtype == torch.float32 and work.is_contiguous() and work.numel() >= n * V)
    assert out_ids.dtype == torch.int32 and out_ids.numel() >= n
    cap = 0
    if hist is not None:
        assert hist.dtype == torch.int32 and hist.dim() == 2 and hist.is_contiguous()
        assert hist_len is not None and hist_len.dtype == torch.int32 and hist_len.numel() >= hist.shape[0]
        cap = hist.shape[1]
    _check(lib.ub_sample(_ptr(logits), logits.stride(0), _ptr(work), n, V, _ptr(params_dev),
                         _ptr(recent), _ptr(bias_ids), _ptr(bias_vals), _ptr(out_ids), int(counter_add),
                         _ptr(hist), _ptr(hist_len), cap, _stream()),
           "sample")
