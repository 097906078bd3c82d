"""Softmax attention with options, over a paged cache whose keys and values have sizes of their own.

Per step: one fused projection [q | k | v (| gate)] (with its biases, if the design has them), one
preparation kernel (rotary positions on the first `rot_dims` features of each head, q and k divided
by their root mean square, the query factor, value mixing, the cache write), attention of every row
over its request's pages, the output projection. What a design may switch on, each with its constants
as parameters:

* `dim` / `vdim`     key and value sizes of a head (the cache holds two tensors of different widths);
* `bias_*`           biases of the q, k, v and output projections;
* `window`           a query sees itself and the window - 1 tokens before it (pages behind are given back);
* `rot_dims`, `rot_base`   partial rotary positions, feature i paired with i + rot_dims / 2;
* `unit_rms_eps`     q and k divided by sqrt(mean(x^2) + eps) per head, after the rotation, no weight;
* `q_temp`           (coef, every): q times 1 + coef * ln(floor((pos + 1) / every) + 1);
* `sink`             one number per head whose exponential joins the softmax's denominator (no key, no value);
* `gate_weight`      the heads' results times sigmoid(W_g x) before the output projection;
* `value_mix`        "first": this layer's values of the step's tokens are left in `ctx.shared[shared_name]`;
                     "mix": v <- (1 - lambda) v + lambda * those values, before v is cached.

A mixer that runs beside another one in one layer offers its halves separately: `w_in` / `b_in`,
`core(proj, ...)` (everything between the two projections, writing into a column range of a wider
buffer) and `w_o` / `b_o`.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import kernels
from .base import CacheSpec, LayerCache, Mixer, PagedTensorSpec, StepContext, aligned
from .linear import to_compute
from .rotary import rotary_inv_freq


class SoftmaxAttention(Mixer):
    def __init__(self, wq: torch.Tensor, wk: torch.Tensor, wv: torch.Tensor, wo: torch.Tensor, heads: int, kv_heads: int, dim: int,
                 vdim: int, scale: float, *, bias_q=None, bias_k=None, bias_v=None, bias_o=None, window: int = 0, rot_dims: int = 0,
                 rot_base: float = 10000.0, unit_rms_eps: Optional[float] = None, q_temp: Optional[Tuple[float, int]] = None,
                 sink: Optional[torch.Tensor] = None, gate_weight: Optional[torch.Tensor] = None, value_mix: Optional[str] = None,
                 mix_weight: Optional[torch.Tensor] = None, shared_name: str = "v_first", dtype=torch.bfloat16, device="cuda"):
        self.H, self.G, self.D, self.DV = int(heads), int(kv_heads), int(dim), int(vdim)
        if self.H % self.G:
            raise ValueError(f"{self.H} heads are not a multiple of {self.G} kv heads")
        if self.D > 256 or self.DV > 256:
            raise ValueError(f"head sizes {self.D} / {self.DV} are beyond 256")
        hidden = wq.shape[1]
        nq, nk, nv = self.H * self.D, self.G * self.D, self.G * self.DV
        self.n_pre = self.H * self.DV
        if wq.shape != (nq, hidden) or wk.shape != (nk, hidden) or wv.shape != (nv, hidden) or wo.shape != (hidden, self.n_pre):
            raise ValueError(f"projection shapes {list(wq.shape)} / {list(wk.shape)} / {list(wv.shape)} / {list(wo.shape)} do not fit "
                             f"{self.H} heads on {self.G} of {self.D} / {self.DV} over a width of {hidden}")
        mats = [wq, wk, wv]
        self.gated = gate_weight is not None
        if self.gated:
            if gate_weight.shape != (self.n_pre, hidden):
                raise ValueError(f"gate projection {list(gate_weight.shape)} does not fit {self.n_pre} x {hidden}")
            mats.append(gate_weight)
        self.w_in = to_compute(torch.cat(mats, dim=0), dtype, device)
        self.q_off, self.k_off, self.v_off, self.g_off = 0, nq, nq + nk, nq + nk + nv
        biases = (bias_q, bias_k, bias_v)
        self.b_in = None
        if any(b is not None for b in biases):
            parts = []
            for b, n in zip(biases, (nq, nk, nv)):
                if b is not None and b.shape != (n,):
                    raise ValueError(f"a bias of {list(b.shape)} does not fit {n}")
                parts.append(b.float() if b is not None else torch.zeros(n))
            if self.gated:
                parts.append(torch.zeros(self.n_pre))
            self.b_in = to_compute(torch.cat([p.to("cpu") for p in parts]), dtype, device)
        self.w_o = to_compute(wo, dtype, device)
        if bias_o is not None and bias_o.shape != (hidden,):
            raise ValueError(f"output bias {list(bias_o.shape)} does not fit {hidden}")
        self.b_o = to_compute(bias_o, dtype, device) if bias_o is not None else None
        self.window = int(window) if window else 0
        self.scale = float(scale)
        self.rot = int(rot_dims)
        if self.rot % 2 or not 0 <= self.rot <= self.D:
            raise ValueError(f"{self.rot} rotated features do not fit a head of {self.D}")
        self.inv_freq = torch.from_numpy(rotary_inv_freq(self.rot, rot_base).copy()).to(device) if self.rot else None
        self.unit_rms = unit_rms_eps is not None
        self.eps = float(unit_rms_eps) if self.unit_rms else 0.0
        self.q_temp = (float(q_temp[0]), int(q_temp[1])) if q_temp else None
        f32 = dict(device=device, dtype=torch.float32)
        if sink is not None and sink.shape != (self.H,):
            raise ValueError(f"sink {list(sink.shape)} does not fit {self.H} heads")
        self.sink = sink.to(**f32).contiguous() if sink is not None else None
        if value_mix not in (None, "first", "mix"):
            raise ValueError(f"value_mix {value_mix!r} is not known (first or mix)")
        self.v_mode = {None: 0, "first": 1, "mix": 2}[value_mix]
        if self.v_mode == 2 and (mix_weight is None or mix_weight.numel() != 1):
            raise ValueError("value mixing needs its weight, one number")
        self.mix_weight = mix_weight.to(**f32).reshape(1).contiguous() if self.v_mode == 2 else None
        self.shared_name = shared_name
        self.hidden, self.dtype = hidden, dtype

    # ------------------------------------------------------------------ what the runtime asks
    def cache_spec(self) -> Optional[CacheSpec]:
        return CacheSpec(kind="window" if self.window else "full", window=self.window,
                         tensors=(PagedTensorSpec(self.G, self.D), PagedTensorSpec(self.G, self.DV)))

    def shared_buffer(self) -> Optional[Tuple[str, int]]:
        """(name, columns) of the step buffer this mixer writes or reads, or None."""
        return (self.shared_name, self.G * self.DV) if self.v_mode else None

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size()

    def core_workspace_bytes(self, rows: int) -> int:
        return aligned(rows * self.H * self.D * self.w_in.element_size())

    def workspace_bytes(self, rows: int) -> int:
        es = self.w_in.element_size()
        return aligned(rows * self.w_in.shape[0] * es) + aligned(rows * self.n_pre * es) + self.core_workspace_bytes(rows)

    def kernel_modules(self, dtype, max_rows):
        return ("gemm_f32", "attention_flex") if dtype == torch.float32 else ("gemm_sm100", "attention_flex")

    # ------------------------------------------------------------------ the step
    def core(self, proj: torch.Tensor, ctx: StepContext, cache: Optional[LayerCache], state, pre_out: torch.Tensor,
             out_scale: float = 1.0) -> None:
        """proj [T, >= w_in rows] -> pre_out [T, n_pre]: everything between the two projections."""
        if cache is None:
            raise ValueError("attention needs a cache")
        T = proj.shape[0]
        kc, vc = cache.tensors[0], cache.tensors[1]
        q = ctx.alloc((T, self.H * self.D))
        v_first = ctx.shared.get(self.shared_name) if self.v_mode else None
        if self.v_mode and v_first is None:
            raise ValueError(f"the step has no buffer {self.shared_name!r} for the values that layers mix")
        kernels.flex_prep(proj, self.q_off, self.k_off, self.v_off, ctx.positions, ctx.slot_mapping[cache.group] if cache.write else None,
                          self.inv_freq, self.rot, self.unit_rms, self.eps, self.q_temp, self.mix_weight, v_first, self.v_mode, q, kc, vc,
                          self.H, self.G, self.D, self.DV)
        gate = proj[:, self.g_off:self.g_off + self.n_pre] if self.gated else None
        kernels.flex_attention(q, pre_out, kc, vc, ctx.block_tables[cache.group], ctx.row_seq, ctx.positions, self.H, self.G, self.D,
                               self.DV, self.scale, self.window, self.sink, gate, out_scale)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[LayerCache], state=None, out=None) -> torch.Tensor:
        T = x.shape[0]
        proj = ctx.alloc((T, self.w_in.shape[0]))
        kernels.linear(x, self.w_in, proj, self.b_in)
        pre = ctx.alloc((T, self.n_pre))
        self.core(proj, ctx, cache, state, pre)
        out = out if out is not None else ctx.alloc((T, self.hidden))
        kernels.linear(pre, self.w_o, out, self.b_o)
        return out
