"""The Lomopel decoder as a list of parts.

embedding times a constant; then the layers in order, each a pre-norm `Block` whose norms keep their
weights around zero (factor 1 + w), whose two results are scaled per feature before they are added
(`ls1`, `ls2`) and whose feed-forward (gated, the tanh form of gelu) may be absent; then the model's
norm and the head. A layer of type `attention` mixes with `SoftmaxAttention` (biases, query factor,
sink, values mixed with the first such layer's); a layer of type `parallel` with a `ParallelMixer` of
a windowed `SoftmaxAttention` (partial rotary positions, unit-RMS q and k, output gate) beside a
`GatedDelta`.

Tensor names are the checkpoint's own: `embed`, `final.norm`, `head`, and per layer i `l<i>.norm1|norm2`,
`l<i>.ls1|ls2`, `l<i>.mlp.gate|up|down`, `l<i>.mix.*` (`q k v o` with `.b` biases, `vmix`, `sink`; or
`left.q|k|v|g|o` and `right.q|k|v` with `.conv`, `right.b|A_log|a1|a2|dt_bias|g1|g2|norm|o`).
"""
from __future__ import annotations

from typing import Dict

from ..config.lomopel_config import NAME, LomopelConfig
from ..config.registry import Architecture, register_architecture
from ..parts import Block, Embedding, LayerCall, LMHead, ModelSpec, RMSNorm, SwiGLU
from ..parts.flex_attention import SoftmaxAttention
from ..parts.linear import to_compute
from ..parts.parallel import ParallelMixer
from ..parts.recurrent import GatedDelta
from ..weights.loader import TensorSpec, WeightSet

V_FIRST = "v_first"      # the step buffer in which the first mixing layer leaves its values


def lomopel_manifest(cfg: LomopelConfig) -> Dict[str, TensorSpec]:
    w = cfg.width
    m = {"embed": TensorSpec((cfg.vocab, w))}
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m[p + "norm1"] = TensorSpec((w,))
        m[p + "ls1"] = TensorSpec((w,), init="ones")
        x = p + "mix."
        if layer.type == "attention":
            a = layer.attention
            nq, nk, nv = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
            m[x + "q"], m[x + "q.b"] = TensorSpec((nq, w)), TensorSpec((nq,))
            m[x + "k"], m[x + "k.b"] = TensorSpec((nk, w)), TensorSpec((nk,))
            m[x + "v"], m[x + "v.b"] = TensorSpec((nv, w)), TensorSpec((nv,))
            m[x + "vmix"] = TensorSpec((), optional=not a.v_mix)
            m[x + "sink"] = TensorSpec((a.heads,))
            m[x + "o"], m[x + "o.b"] = TensorSpec((w, a.heads * a.vdim)), TensorSpec((w,))
        else:
            a, r = layer.left, layer.right
            y = x + "left."
            m[y + "q"] = TensorSpec((a.heads * a.dim, w))
            m[y + "k"] = TensorSpec((a.kv_heads * a.dim, w))
            m[y + "v"] = TensorSpec((a.kv_heads * a.vdim, w))
            m[y + "g"] = TensorSpec((a.heads * a.vdim, w))
            m[y + "o"] = TensorSpec((w, a.heads * a.vdim))
            y = x + "right."
            gk, hk, hv = r.kv_heads * r.dim, r.heads * r.dim, r.heads * r.vdim
            ra = r.decay_rank if r.decay_rank is not None else -1
            rg = r.gate_rank if r.gate_rank is not None else -1
            for n, rows in (("q", gk), ("k", gk), ("v", hv)):
                m[y + n] = TensorSpec((rows, w))
                m[y + n + ".conv"] = TensorSpec((rows, r.conv))
            m[y + "b"] = TensorSpec((r.heads, w))
            m[y + "A_log"] = TensorSpec((r.heads,))
            m[y + "norm"] = TensorSpec((r.vdim,), init="ones")
            m[y + "a1"], m[y + "a2"] = TensorSpec((ra, w)), TensorSpec((hk, ra))
            m[y + "dt_bias"] = TensorSpec((hk,))
            m[y + "g1"], m[y + "g2"] = TensorSpec((rg, w)), TensorSpec((hv, rg))
            m[y + "o"] = TensorSpec((w, hv))
        if layer.ff:
            m[p + "norm2"] = TensorSpec((w,))
            m[p + "ls2"] = TensorSpec((w,), init="ones")
            m[p + "mlp.gate"] = TensorSpec((layer.ff, w))
            m[p + "mlp.up"] = TensorSpec((layer.ff, w))
            m[p + "mlp.down"] = TensorSpec((w, layer.ff))
        else:
            m[p + "norm2"] = TensorSpec((w,), optional=True)
            m[p + "ls2"] = TensorSpec((w,), optional=True)
    m["final.norm"] = TensorSpec((w,))
    m["head"] = TensorSpec((cfg.vocab, w))
    return m


def _attention(a, t, x: str, value_mix, dt, dev) -> SoftmaxAttention:
    return SoftmaxAttention(t(x + "q"), t(x + "k"), t(x + "v"), t(x + "o"), a.heads, a.kv_heads, a.dim, a.vdim, a.scale,
                            bias_q=t(x + "q.b"), bias_k=t(x + "k.b"), bias_v=t(x + "v.b"), bias_o=t(x + "o.b"), window=a.window,
                            rot_dims=a.rot_dims, rot_base=a.rot_base or 10000.0, q_temp=a.q_temp, sink=t(x + "sink"),
                            value_mix=value_mix, mix_weight=t(x + "vmix") if value_mix == "mix" else None, shared_name=V_FIRST,
                            dtype=dt, device=dev)


def build_lomopel(cfg: LomopelConfig, weights: WeightSet, ctx) -> ModelSpec:
    dt, dev = ctx.dtype, ctx.device
    eps, t = cfg.norm_eps, weights.take
    mixing = [i for i, x in enumerate(cfg.layers) if x.type == "attention" and x.attention.v_mix]
    embedding = Embedding(t("embed"), dt, dev, scale=cfg.embedding_scale)
    blocks, schedule, buffers = [], [], {}
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        x = p + "mix."
        if layer.type == "attention":
            # the first mixing layer leaves its values for the others; alone, it has nobody to leave them to
            mode = None if i not in mixing or len(mixing) < 2 else ("first" if i == mixing[0] else "mix")
            mixer = _attention(layer.attention, t, x, mode, dt, dev)
            if mode != "mix":
                weights.skip(x + "vmix")
            if mode is not None:
                buffers[V_FIRST] = (layer.attention.kv_heads * layer.attention.vdim, None)
        else:
            a, r = layer.left, layer.right
            y = x + "left."
            left = SoftmaxAttention(t(y + "q"), t(y + "k"), t(y + "v"), t(y + "o"), a.heads, a.kv_heads, a.dim, a.vdim, a.scale,
                                    window=a.window, rot_dims=a.rot_dims, rot_base=a.rot_base or 10000.0, unit_rms_eps=eps,
                                    gate_weight=t(y + "g"), dtype=dt, device=dev)
            y = x + "right."
            right = GatedDelta(t(y + "q"), t(y + "k"), t(y + "v"), t(y + "q.conv"), t(y + "k.conv"), t(y + "v.conv"), t(y + "b"),
                               t(y + "A_log"), t(y + "a1"), t(y + "a2"), t(y + "dt_bias"), t(y + "g1"), t(y + "g2"), t(y + "norm"),
                               t(y + "o"), r.heads, r.kv_heads, r.dim, r.vdim, eps, dt, dev)
            mixer = ParallelMixer(left, right, layer.left_scale, layer.right_scale)
        norm1 = RMSNorm(t(p + "norm1"), eps, dev, unit_offset=True)
        if layer.ff:
            ff = SwiGLU(t(p + "mlp.gate"), t(p + "mlp.up"), t(p + "mlp.down"), dt, dev, activation="gelu_tanh")
            blocks.append(Block(norm1, mixer, RMSNorm(t(p + "norm2"), eps, dev, unit_offset=True), ff, mixer_scale=t(p + "ls1"),
                                ff_scale=t(p + "ls2")))
        else:
            weights.skip(p + "norm2")
            weights.skip(p + "ls2")
            blocks.append(Block(norm1, mixer, None, None, mixer_scale=t(p + "ls1")))
        schedule.append(LayerCall(layer=i, cache=i, write=True))
    final_norm = RMSNorm(t("final.norm"), eps, dev, unit_offset=True)
    head = LMHead(to_compute(t("head"), dt, dev))
    weights.finish()
    wbytes = sum(b.weight_bytes() for b in blocks) + final_norm.weight_bytes() + head.weight_bytes()
    return ModelSpec(embedding=embedding, blocks=blocks, schedule=schedule, final_norm=final_norm, lm_head=head,
                     hidden_size=cfg.width, vocab_size=cfg.vocab, max_position=None, eos_token_ids=cfg.eos_token_ids,
                     weight_bytes=wbytes, step_buffers=buffers)


LOMOPEL = Architecture(name=NAME, config_cls=LomopelConfig, manifest=lomopel_manifest, build=build_lomopel)
register_architecture(LOMOPEL, replace=True)
