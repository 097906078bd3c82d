"""The Lomopel decoder written out plainly: one function per mechanism, whole sequences, token by
token where the mechanism is a recurrence, in whatever floating type the tensors have (the tests
use float64). Nothing here is shared with the engine: no kernel, no part, no cache.

Notation. x [T, width] is a sequence of T tokens at positions 0 .. T-1. A linear weight W is stored
[out, in] and applied as x W^T. rms(z) = z / sqrt(mean(z^2) + eps) over the last axis. `t` is the
dictionary of tensors by name, `p` the prefix of a mixer's tensors, `m` the mixer's configuration.
"""
from __future__ import annotations

import math

import torch


# ----------------------------------------------------------------------------------- small pieces
def rms(z: torch.Tensor, eps: float) -> torch.Tensor:
    return z / torch.sqrt((z * z).mean(-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight lies around zero: the factor is 1 + w."""
    return rms(x, eps) * (1.0 + w)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_partial(z: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """z [T, heads, d], token i at position i: of every head the first `dims` features are rotated,
    feature i with feature i + dims/2, by position * base^(-2i/dims); the others stay."""
    T = z.shape[0]
    half = dims // 2
    freq = base ** (-2.0 * torch.arange(half, dtype=z.dtype) / dims)
    ang = torch.arange(T, dtype=z.dtype)[:, None, None] * freq
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = z[..., :half], z[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, z[..., dims:]], dim=-1)


def query_temperature(T: int, coef: float, every: int, dtype) -> torch.Tensor:
    """The factor on q at positions 0 .. T-1: 1 + coef * ln(floor((p + 1) / every) + 1)."""
    p = torch.arange(T)
    return 1.0 + coef * torch.log((torch.div(p + 1, every, rounding_mode="floor") + 1).to(dtype))


def softmax_rows(scores: torch.Tensor, visible: torch.Tensor, sink=None) -> torch.Tensor:
    """scores [heads, T, T], visible [T, T] bool. Weights over the visible keys; with `sink` [heads]
    the denominator also holds exp(sink) once: a key with no value."""
    scores = scores.masked_fill(~visible, -math.inf)
    top = scores.max(-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, sink[:, None, None])
    e = torch.exp(scores - top)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink[:, None, None] - top)
    return e / den


def attend(q, k, v, scale, visible, sink=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head a uses key/value head a // (H / G)."""
    H, G = q.shape[1], k.shape[1]
    kk = k.repeat_interleave(H // G, dim=1)
    vv = v.repeat_interleave(H // G, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, kk) * scale
    w = softmax_rows(scores, visible, sink)
    return torch.einsum("hij,jhd->ihd", w, vv)


# ----------------------------------------------------------------------------------- mixers
def sink_attention(h, t, p, m, v_first=None):
    """Causal attention over all earlier tokens with biased projections, no rotation, a query factor
    that grows with the position, a sink in the softmax, and (where `v_first` is given) values mixed
    with those of the first such layer. Returns (result, the values as they are cached)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ t[p + "q"].T + t[p + "q.b"]).reshape(T, H, d)
    k = (h @ t[p + "k"].T + t[p + "k.b"]).reshape(T, G, d)
    v = (h @ t[p + "v"].T + t[p + "v.b"]).reshape(T, G, dv)
    qt = m.get("q_temp")
    if qt:
        q = q * query_temperature(T, qt["coef"], qt["every"], h.dtype)[:, None, None]
    if v_first is not None:
        lam = t[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    i = torch.arange(T)
    visible = i[None, :] <= i[:, None]
    o = attend(q, k, v, m["scale"], visible, t[p + "sink"])
    return o.reshape(T, H * dv) @ t[p + "o"].T + t[p + "o.b"], v


def window_attention(h, t, p, m, eps):
    """Attention over the last `mask.size` tokens (itself included; all earlier ones without `mask`): rotary positions on part of each
    head, then q and k divided by their root mean square per head, ordinary softmax, and a sigmoid
    gate from the same input on the heads' results before the output projection."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ t[p + "q"].T).reshape(T, H, d)
    k = (h @ t[p + "k"].T).reshape(T, G, d)
    v = (h @ t[p + "v"].T).reshape(T, G, dv)
    rot = m.get("rot")
    if rot:
        q, k = rotate_partial(q, rot["dims"], rot["base"]), rotate_partial(k, rot["dims"], rot["base"])
    q, k = rms(q, eps), rms(k, eps)
    i = torch.arange(T)
    dist = i[:, None] - i[None, :]
    visible = dist >= 0
    if m.get("mask"):
        visible = visible & (dist < m["mask"]["size"])
    o = attend(q, k, v, m["scale"], visible).reshape(T, H * dv)
    return (o * torch.sigmoid(h @ t[p + "g"].T)) @ t[p + "o"].T


def causal_conv_silu(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [T, C], w [C, taps] with the last column the current token's; zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    return y * torch.sigmoid(y)


def gated_delta(h, t, p, m, eps):
    """Gated delta rule. Per value head a state S [dim, vdim], zero at the start; for every token
        S <- g * S (g per key channel);  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv_silu(h @ t[p + "q"].T, t[p + "q.conv"]).reshape(T, G, d)
    k = causal_conv_silu(h @ t[p + "k"].T, t[p + "k.conv"]).reshape(T, G, d)
    v = causal_conv_silu(h @ t[p + "v"].T, t[p + "v.conv"]).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q, k = q.repeat_interleave(H // G, dim=1), k.repeat_interleave(H // G, dim=1)
    beta = torch.sigmoid(h @ t[p + "b"].T)                                     # [T, H]
    step = torch.nn.functional.softplus((h @ t[p + "a1"].T) @ t[p + "a2"].T + t[p + "dt_bias"]).reshape(T, H, d)
    g = torch.exp(-torch.exp(t[p + "A_log"])[None, :, None] * step)            # [T, H, d]
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for i in range(T):
        S = g[i][:, :, None] * S
        u = beta[i][:, None] * (v[i] - torch.einsum("hkv,hk->hv", S, k[i]))
        S = S + k[i][:, :, None] * u[:, None, :]
        o[i] = torch.einsum("hkv,hk->hv", S, q[i])
    gate = torch.sigmoid((h @ t[p + "g1"].T) @ t[p + "g2"].T).reshape(T, H, dv)
    o = rms(o, eps) * t[p + "norm"] * gate
    return o.reshape(T, H * dv) @ t[p + "o"].T


def feed_forward(h, t, p):
    return (gelu_tanh(h @ t[p + "gate"].T) * (h @ t[p + "up"].T)) @ t[p + "down"].T


# ----------------------------------------------------------------------------------- the model
def forward(cfg: dict, tensors: dict, tokens, dtype=torch.float64, layers_out=None):
    """Logits [T, vocab] of one sequence. `layers_out`, a list, receives the residual after every layer."""
    t = {n: (x.to(dtype) if x.is_floating_point() else x) for n, x in tensors.items()}
    eps = cfg["norm"]["eps"]
    x = t["embed"][torch.tensor(list(tokens), dtype=torch.long)] * cfg["embedding"]["scale"]
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = offset_norm(x, t[p + "norm1"], eps)
        m = layer["mixer"]
        if layer["type"] == "attention":
            y, v = sink_attention(h, t, p + "mix.", m, v_first if m.get("v_mix") else None)
            if m.get("v_mix") and v_first is None:
                v_first = v
        elif layer["type"] == "parallel":
            y = (m["left_scale"] * window_attention(h, t, p + "mix.left.", m["left"], eps)
                 + m["right_scale"] * gated_delta(h, t, p + "mix.right.", m["right"], eps))
        else:
            raise ValueError(layer["type"])
        x = x + y * t[p + "ls1"]
        if layer.get("mlp"):
            x = x + feed_forward(offset_norm(x, t[p + "norm2"], eps), t, p + "mlp.") * t[p + "ls2"]
        if layers_out is not None:
            layers_out.append(x.clone())
    return offset_norm(x, t["final.norm"], eps) @ t["head"].T
