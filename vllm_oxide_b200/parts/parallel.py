"""Two mixers side by side in one layer: both read the same input, and the layer's result is
    left_scale * left(x) + right_scale * right(x).
Each half offers `w_in` (its fused input projection, with `b_in`), `core(proj, ctx, cache, state, pre_out,
out_scale)` (everything between its projections) and `w_o` (with `b_o`). The two input projections become
ONE product over [W_in_left; W_in_right], the two output projections ONE product over
[W_o_left | W_o_right] applied to the halves' results side by side, each already times its scale: the
weighted sum happens inside the product's float32 accumulation. At most one half may keep pages; the
per-request state is the two halves' states one after the other.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import CacheSpec, LayerCache, Mixer, StepContext, aligned


def _states(m) -> tuple:
    ss = m.state_spec()
    return () if ss is None else (tuple(ss) if isinstance(ss, (tuple, list)) else (ss,))


class ParallelMixer(Mixer):
    def __init__(self, left: Mixer, right: Mixer, left_scale: float = 1.0, right_scale: float = 1.0):
        for m in (left, right):
            for need in ("w_in", "w_o", "core", "n_pre"):
                if not hasattr(m, need):
                    raise ValueError(f"{type(m).__name__} does not offer its halves separately ('{need}' is missing)")
        if left.cache_spec() is not None and right.cache_spec() is not None:
            raise ValueError("only one of two mixers side by side may keep pages")
        if left.w_in.shape[1] != right.w_in.shape[1] or left.w_in.dtype != right.w_in.dtype:
            raise ValueError("the two mixers read inputs of different widths or types")
        self.left, self.right = left, right
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        self.n_left_in = left.w_in.shape[0]
        self.w_in = torch.cat([left.w_in, right.w_in], dim=0).contiguous()
        self.w_o = torch.cat([left.w_o, right.w_o], dim=1).contiguous()
        self.hidden = self.w_o.shape[0]
        dt, dev = self.w_in.dtype, self.w_in.device
        bl, br = getattr(left, "b_in", None), getattr(right, "b_in", None)
        self.b_in = None
        if bl is not None or br is not None:
            self.b_in = torch.cat([bl if bl is not None else torch.zeros(left.w_in.shape[0], dtype=dt, device=dev),
                                   br if br is not None else torch.zeros(right.w_in.shape[0], dtype=dt, device=dev)]).contiguous()
        ol, orr = getattr(left, "b_o", None), getattr(right, "b_o", None)
        self.b_o = None
        if ol is not None or orr is not None:
            total = torch.zeros(self.hidden, dtype=torch.float32, device=dev)
            if ol is not None:
                total += self.left_scale * ol.float()
            if orr is not None:
                total += self.right_scale * orr.float()
            self.b_o = total.to(dt).contiguous()
        self.n_left_state = len(_states(left))
        # the halves' own matrices are not needed any more: the fused ones are what a step reads
        for m in (left, right):
            m.w_in = m.w_in[:0]
            m.w_o = m.w_o[:, :0]

    def cache_spec(self) -> Optional[CacheSpec]:
        return self.left.cache_spec() or self.right.cache_spec()

    def state_spec(self):
        both = _states(self.left) + _states(self.right)
        return both or None

    def shared_buffer(self):
        return getattr(self.left, "shared_buffer", lambda: None)() or getattr(self.right, "shared_buffer", lambda: None)()

    def weight_bytes(self) -> int:
        extra = sum(getattr(m, "w_low").numel() for m in (self.left, self.right) if hasattr(m, "w_low"))
        return (self.w_in.numel() + self.w_o.numel() + extra) * self.w_in.element_size()

    def workspace_bytes(self, rows: int) -> int:
        es = self.w_in.element_size()
        return (aligned(rows * self.w_in.shape[0] * es) + aligned(rows * self.w_o.shape[1] * es)
                + max(self.left.core_workspace_bytes(rows), self.right.core_workspace_bytes(rows)))

    def kernel_modules(self, dtype, max_rows):
        return tuple(self.left.kernel_modules(dtype, max_rows)) + tuple(self.right.kernel_modules(dtype, max_rows))

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[LayerCache], state, out=None) -> torch.Tensor:
        T = x.shape[0]
        proj = ctx.alloc((T, self.w_in.shape[0]))
        kernels.linear(x, self.w_in, proj, self.b_in)
        pre = ctx.alloc((T, self.w_o.shape[1]))
        st = () if state is None else (tuple(state) if isinstance(state, (tuple, list)) else (state,))
        ls, rs = st[:self.n_left_state], st[self.n_left_state:]
        nl = self.left.n_pre
        with ctx.workspace.scope():
            self.left.core(proj[:, :self.n_left_in], ctx, cache if self.left.cache_spec() is not None else None, ls or None,
                           pre[:, :nl], self.left_scale)
        with ctx.workspace.scope():
            self.right.core(proj[:, self.n_left_in:], ctx, cache if self.right.cache_spec() is not None else None, rs or None,
                            pre[:, nl:], self.right_scale)
        out = out if out is not None else ctx.alloc((T, self.hidden))
        kernels.linear(pre, self.w_o, out, self.b_o)
        return out
