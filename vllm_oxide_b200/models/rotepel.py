"""The Rotepel decoder as a list of parts.

embedding -> the model's norm -> `streams` copies; then the layers in run order (a range of them
may run several times in a row with the same weights, each pass with a cache or state of its own:
the run order names a layer several times and every call gets its own cache number and state
tensor); then the sum of the streams -> the model's norm -> the head. Every norm is the RMS norm in
groups (`StreamNorm`); a layer is a `StreamBlock` around one of three mixers (`GeneralDelta`,
`Retention`, `LatentAttention`) and an optional dense SwiGLU feed-forward.

Tensor names are the checkpoint's own: `embed`, `embed.norm`, `final.norm`, `head`, and per layer i
`l<i>.norm1|norm2`, `l<i>.mix.*`, `l<i>.mlp.gate|up|down`, `l<i>.hc1|hc2.in|out|mix`.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.registry import Architecture, register_architecture
from ..config.rotepel_config import NAME, RotepelConfig
from ..parts import Embedding, LayerCall, LMHead, ModelSpec, SwiGLU
from ..parts.latent_attention import LatentAttention
from ..parts.linear import to_compute
from ..parts.recurrent import GeneralDelta, Retention
from ..parts.streams import StreamBlock, StreamCoefficients, StreamEmbedding, StreamNorm
from ..weights.loader import TensorSpec, WeightSet


def rotepel_manifest(cfg: RotepelConfig) -> Dict[str, TensorSpec]:
    w = cfg.width
    m = {"embed": TensorSpec((cfg.vocab, w)), "embed.norm": TensorSpec((w,), init="ones")}
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m[p + "norm1"] = TensorSpec((w,), init="ones")
        x = p + "mix."
        if layer.type == "general_delta":
            hd = layer.heads * layer.dim
            rank = layer.decay_rank if layer.decay_rank is not None else -1
            for n in ("r", "k", "v", "g", "a"):
                m[x + n] = TensorSpec((hd, w))
            m[x + "a.b"] = TensorSpec((hd,))
            m[x + "w1"] = TensorSpec((rank, w))
            m[x + "w2"] = TensorSpec((hd, rank))
            m[x + "w0"] = TensorSpec((hd,))
            m[x + "norm"] = TensorSpec((hd,), init="ones")
            m[x + "o"] = TensorSpec((w, hd))
        elif layer.type == "retention":
            hk, hv = layer.heads * layer.dim, layer.heads * layer.vdim
            m[x + "q"] = TensorSpec((hk, w))
            m[x + "k"] = TensorSpec((hk, w))
            m[x + "v"] = TensorSpec((hv, w))
            m[x + "g"] = TensorSpec((hv, w))
            m[x + "o"] = TensorSpec((w, hv))
        else:
            H, L = layer.heads, layer.kv_rank
            m[x + "q"] = TensorSpec((H * (layer.dim + layer.rot_dim), w))
            m[x + "dkv"] = TensorSpec((L + layer.rot_dim, w))
            m[x + "dkv.norm"] = TensorSpec((L,), init="ones")
            m[x + "uk"] = TensorSpec((H * layer.dim, L))
            m[x + "uv"] = TensorSpec((H * layer.vdim, L))
            m[x + "o"] = TensorSpec((w, H * layer.vdim))
        subs = ["hc1"]
        if layer.ff:
            m[p + "norm2"] = TensorSpec((w,), init="ones")
            m[p + "mlp.gate"] = TensorSpec((layer.ff, w))
            m[p + "mlp.up"] = TensorSpec((layer.ff, w))
            m[p + "mlp.down"] = TensorSpec((w, layer.ff))
            subs.append("hc2")
        if cfg.streams is not None:
            for hc in subs:
                m[p + hc + ".in"] = TensorSpec((cfg.streams,), init="ones")
                m[p + hc + ".out"] = TensorSpec((cfg.streams,), init="ones")
                m[p + hc + ".mix"] = TensorSpec((cfg.streams, cfg.streams), init="identity")
    m["final.norm"] = TensorSpec((w,), init="ones")
    m["head"] = TensorSpec((cfg.vocab, w))
    return m


def _mixer(layer, weights: WeightSet, x: str, eps: float, dt, dev):
    t = weights.take
    if layer.type == "general_delta":
        return GeneralDelta(t(x + "r"), t(x + "k"), t(x + "v"), t(x + "a"), t(x + "a.b"), t(x + "g"), t(x + "w1"), t(x + "w2"),
                            t(x + "w0"), t(x + "norm"), t(x + "o"), layer.heads, layer.dim, eps, dt, dev)
    if layer.type == "retention":
        return Retention(t(x + "q"), t(x + "k"), t(x + "v"), t(x + "g"), t(x + "o"), layer.heads, layer.dim, layer.vdim, layer.decay,
                         layer.rot_dims, layer.rot_base, eps, dt, dev)
    return LatentAttention(t(x + "q"), t(x + "dkv"), t(x + "dkv.norm"), t(x + "uk"), t(x + "uv"), t(x + "o"), layer.heads, layer.dim,
                           layer.rot_dim, layer.vdim, layer.kv_rank, layer.scale, layer.rot_base, eps, dt, dev)


def build_rotepel(cfg: RotepelConfig, weights: WeightSet, ctx) -> ModelSpec:
    dt, dev = ctx.dtype, ctx.device
    eps, groups = cfg.norm_eps, cfg.norm_groups
    S = cfg.streams if cfg.streams is not None else 1

    def coefficients(p):
        if cfg.streams is None:
            return StreamCoefficients.plain(dev)
        return StreamCoefficients.make(weights.take(p + ".in"), weights.take(p + ".out"), weights.take(p + ".mix"), dev)

    embedding = StreamEmbedding(Embedding(weights.take("embed"), dt, dev),
                                StreamNorm(weights.take("embed.norm"), eps, groups, streams=1, copies=S, out_dtype=torch.float32, device=dev))
    blocks = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        c1 = coefficients(p + "hc1")
        norm1 = StreamNorm(weights.take(p + "norm1"), eps, groups, S, read=c1.read, device=dev)
        mixer = _mixer(layer, weights, p + "mix.", eps, dt, dev)
        if layer.ff:
            c2 = coefficients(p + "hc2")
            norm2 = StreamNorm(weights.take(p + "norm2"), eps, groups, S, read=c2.read, device=dev)
            ff = SwiGLU(weights.take(p + "mlp.gate"), weights.take(p + "mlp.up"), weights.take(p + "mlp.down"), dt, dev)
            blocks.append(StreamBlock(norm1, mixer, c1, norm2, ff, c2))
        else:
            blocks.append(StreamBlock(norm1, mixer, c1))
    # every call of the run order has a cache number of its own (and, by its place, a state of its own)
    schedule = [LayerCall(layer=i, cache=n if blocks[i].mixer.cache_spec() is not None else None, write=True)
                for n, i in enumerate(cfg.run_order())]
    final_norm = StreamNorm(weights.take("final.norm"), eps, groups, S, read=None, device=dev)
    head = LMHead(to_compute(weights.take("head"), dt, dev))
    weights.finish()
    wbytes = sum(blocks[c.layer].weight_bytes() for c in schedule) + final_norm.weight_bytes() + head.weight_bytes()
    return ModelSpec(embedding=embedding, blocks=blocks, schedule=schedule, final_norm=final_norm, lm_head=head,
                     hidden_size=cfg.width, vocab_size=cfg.vocab, max_position=None, eos_token_ids=cfg.eos_token_ids,
                     weight_bytes=wbytes, residual_streams=S)


ROTEPEL = Architecture(name=NAME, config_cls=RotepelConfig, manifest=rotepel_manifest, build=build_rotepel)
register_architecture(ROTEPEL, replace=True)
