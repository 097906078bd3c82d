"""The Rotepel decoder written out plainly: one function per mechanism, whole sequences, token by
token where the mechanism is a recurrence, in whatever floating type the tensors have (the tests
use float64). Nothing here is shared with the engine: no kernel, no part, no cache.

Notation. x [T, width] is a sequence of T tokens. A linear weight W is stored [out, in] and
applied as x W^T. rms(z) = z / sqrt(mean(z^2) + eps) over the last axis.
"""
from __future__ import annotations

import math

import torch


# ----------------------------------------------------------------------------------- norms
def rms(z: torch.Tensor, eps: float) -> torch.Tensor:
    return z / torch.sqrt((z * z).mean(-1, keepdim=True) + eps)


def group_rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, groups: int) -> torch.Tensor:
    """The width is cut into `groups` equal consecutive parts; each part is divided by its own
    root mean square; the whole is multiplied by w."""
    T, n = x.shape
    parts = x.reshape(T, groups, n // groups)
    return rms(parts, eps).reshape(T, n) * w


# ----------------------------------------------------------------------------------- rotation
def rotate(z: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """z [T, heads, d]: the first `dims` features of every head are rotated, feature i with feature
    i + dims/2, by the angle position * base^(-2i/dims); the rest pass unchanged."""
    half = dims // 2
    i = torch.arange(half, dtype=z.dtype)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(z.dtype)[:, None, None] * freq
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = z[..., :half], z[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, z[..., dims:]], dim=-1)


# ----------------------------------------------------------------------------------- mixers
def general_delta(h, t, p, heads, dim, eps):
    """Generalized delta rule. Per head a state S [dim (key), dim (value)], zero at the start:
        S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T,   o_t = S_t^T r_t
    with u_t the key scaled to unit length, w_t a decay and a_t a removal rate per key channel."""
    T = h.shape[0]
    r = (h @ t[p + "r"].T).reshape(T, heads, dim)
    k = (h @ t[p + "k"].T).reshape(T, heads, dim)
    v = (h @ t[p + "v"].T).reshape(T, heads, dim)
    lora = torch.tanh(h @ t[p + "w1"].T) @ t[p + "w2"].T + t[p + "w0"]
    w = torch.exp(-math.exp(-0.5) * torch.sigmoid(lora)).reshape(T, heads, dim)
    a = torch.sigmoid(h @ t[p + "a"].T + t[p + "a.b"]).reshape(T, heads, dim)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    S = torch.zeros(heads, dim, dim, dtype=h.dtype)
    o = torch.zeros(T, heads, dim, dtype=h.dtype)
    for i in range(T):
        uS = torch.einsum("hk,hkv->hv", u[i], S)
        S = w[i][:, :, None] * S - (a[i] * u[i])[:, :, None] * uS[:, None, :] + k[i][:, :, None] * v[i][:, None, :]
        o[i] = torch.einsum("hkv,hk->hv", S, r[i])
    o = rms(o, eps).reshape(T, heads * dim) * t[p + "norm"]
    o = o * torch.sigmoid(h @ t[p + "g"].T)
    return o @ t[p + "o"].T


def retention(h, t, p, positions, heads, dim, vdim, decay, rot_dims, rot_base, eps):
    """Linear attention with a fixed decay per head, no softmax and no denominator:
        S_t = decay_h S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,   k scaled by dim^-1/2 after rotation."""
    T = h.shape[0]
    q = rotate((h @ t[p + "q"].T).reshape(T, heads, dim), positions, rot_dims, rot_base)
    k = rotate((h @ t[p + "k"].T).reshape(T, heads, dim), positions, rot_dims, rot_base) * dim ** -0.5
    v = (h @ t[p + "v"].T).reshape(T, heads, vdim)
    S = torch.zeros(heads, dim, vdim, dtype=h.dtype)
    o = torch.zeros(T, heads, vdim, dtype=h.dtype)
    d = torch.tensor(decay, dtype=h.dtype)[:, None, None]
    for i in range(T):
        S = d * S + k[i][:, :, None] * v[i][:, None, :]
        o[i] = torch.einsum("hkv,hk->hv", S, q[i])
    o = rms(o, eps).reshape(T, heads * vdim)
    g = h @ t[p + "g"].T
    return (o * (g * torch.sigmoid(g))) @ t[p + "o"].T


def latent_attention(h, t, p, positions, heads, dim, rot_dim, vdim, kv_rank, scale, rot_base, eps):
    """Attention whose keys and values are made from one small latent vector per token plus one
    rotated key part that all heads share; causal, ordinary softmax."""
    T = h.shape[0]
    q = (h @ t[p + "q"].T).reshape(T, heads, dim + rot_dim)
    q_plain, q_rot = q[..., :dim], rotate(q[..., dim:], positions, rot_dim, rot_base)
    down = h @ t[p + "dkv"].T
    c = rms(down[:, :kv_rank], eps) * t[p + "dkv.norm"]
    k_rot = rotate(down[:, None, kv_rank:], positions, rot_dim, rot_base)[:, 0]
    k_plain = (c @ t[p + "uk"].T).reshape(T, heads, dim)
    v = (c @ t[p + "uv"].T).reshape(T, heads, vdim)
    score = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * scale
    causal = torch.ones(T, T, dtype=torch.bool).tril()
    score = score.masked_fill(~causal, float("-inf"))
    out = torch.einsum("hij,jhd->ihd", torch.softmax(score, -1), v).reshape(T, heads * vdim)
    return out @ t[p + "o"].T


def mixer(kind, h, t, p, positions, m, eps):
    if kind == "general_delta":
        return general_delta(h, t, p, m["heads"], m["dim"], eps)
    if kind == "retention":
        return retention(h, t, p, positions, m["heads"], m["dim"], m["vdim"], m["decay"], m["rot"]["dims"], m["rot"]["base"], eps)
    if kind == "latent_attention":
        return latent_attention(h, t, p, positions, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["scale"],
                                m["rot"]["base"], eps)
    raise ValueError(kind)


# ----------------------------------------------------------------------------------- feed-forward
def dense_feed_forward(h, t, p):
    g = h @ t[p + "gate"].T
    return ((g * torch.sigmoid(g)) * (h @ t[p + "up"].T)) @ t[p + "down"].T


# ----------------------------------------------------------------------------------- streams
def hyper_sublayer(streams, t, p, fn):
    """streams [s, T, width]. The sublayer reads u = sum_s in[s] x_s; every new stream is a mix of
    the old ones plus its own share of the sublayer's output: x_t' = sum_s mix[s, t] x_s + out[t] y."""
    u = torch.einsum("s,stw->tw", t[p + "in"], streams)
    y = fn(u)
    return torch.einsum("sr,stw->rtw", t[p + "mix"], streams) + t[p + "out"][:, None, None] * y[None]


# ----------------------------------------------------------------------------------- the model
def run_order(cfg):
    """Layer numbers in the order they run: layers start .. stop-1 `times` times in a row."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg, t, tokens, dtype=torch.float64, layer_sums=None):
    """Logits [T, vocab] of a whole sequence. `layer_sums`, a list, receives the residual stream
    (the sum of the streams) after every layer run."""
    t = {k: v.to(dtype) for k, v in t.items()}
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    T = len(tokens)
    positions = torch.arange(T)
    x = group_rms_norm(t["embed"][torch.tensor(tokens)], t["embed.norm"], eps, groups)
    s = cfg.get("streams")
    streams = x[None].repeat(s if s else 1, 1, 1)
    for i in run_order(cfg):
        layer, p = cfg["layers"][i], f"l{i}."

        def mix(u):
            return mixer(layer["type"], group_rms_norm(u, t[p + "norm1"], eps, groups), t, p + "mix.", positions, layer["mixer"], eps)

        def ff(u):
            return dense_feed_forward(group_rms_norm(u, t[p + "norm2"], eps, groups), t, p + "mlp.")
        if s:
            streams = hyper_sublayer(streams, t, p + "hc1.", mix)
            if layer.get("mlp"):
                streams = hyper_sublayer(streams, t, p + "hc2.", ff)
        else:
            streams = streams + mix(streams[0])[None]
            if layer.get("mlp"):
                streams = streams + ff(streams[0])[None]
        if layer_sums is not None:
            layer_sums.append(streams.sum(0))
    x = group_rms_norm(streams.sum(0), t["final.norm"], eps, groups)
    return x @ t["head"].T
