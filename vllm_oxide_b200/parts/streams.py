"""A residual kept in several streams (hyper-connections), the RMS norm in groups that reads it,
and the layer arranged around both.

Instead of one residual x there are S streams x_1 .. x_S, all equal to the embedding's output at
the start. A sublayer (mixer or feed-forward) with coefficients `in` [S], `out` [S], `mix` [S, S]:
    u = sum_s in[s] x_s;   y = sublayer(norm(u));   x_t <- sum_s mix[s, t] x_s + out[t] y  (all t at once).
The model's output is read from the sum of the streams. S = 1 with all coefficients 1 is the plain
pre-norm residual layer, and `StreamCoefficients.plain` makes exactly that.

As in `Block`, a sublayer's output is not written into the residual when it is produced: it is
handed on as a `PendingWrite` and the kernel that reads the streams next (the next norm, or the
model's final norm) does the write first, in the same pass over the row.

The norm (`StreamNorm`): the vector is cut into `groups` equal consecutive parts, each divided by
its own sqrt(mean(part^2) + eps), the whole multiplied by the weight; `groups` = 1 is RMSNorm.
The streams, the coefficients and all sums are float32.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import kernels
from .base import FeedForward, LayerCache, Mixer, Norm, StepContext, aligned


@dataclass
class StreamCoefficients:
    """One sublayer's coefficients, float32 on the device: `read` [S], `write` [S], `mix` [S, S] ([from, to])."""
    read: torch.Tensor
    write: torch.Tensor
    mix: torch.Tensor

    @classmethod
    def make(cls, read, write, mix, device) -> "StreamCoefficients":
        def f(t):
            return t.to(device=device, dtype=torch.float32).contiguous()
        read, write, mix = f(read), f(write), f(mix)
        s = read.numel()
        if read.dim() != 1 or write.shape != (s,) or mix.shape != (s, s):
            raise ValueError(f"stream coefficients do not fit one another: in {list(read.shape)}, out {list(write.shape)}, mix {list(mix.shape)}")
        return cls(read, write, mix)

    @classmethod
    def plain(cls, device) -> "StreamCoefficients":
        """One stream, x <- x + y: the ordinary residual sum."""
        one = torch.ones(1)
        return cls.make(one, one, one.view(1, 1), device)


@dataclass
class PendingWrite:
    """A sublayer's output that is still to be written into the streams."""
    y: torch.Tensor             # [rows, width], activations' type
    coef: StreamCoefficients


class StreamNorm(Norm):
    """Reads S streams through `read` coefficients (None: their sum) and normalises in groups.
    `copies` > 1 writes the result that many times side by side (the embedding's output filling
    all streams); `out_dtype` None means the activations' type."""

    def __init__(self, weight: torch.Tensor, eps: float, groups: int, streams: int, read: Optional[torch.Tensor] = None,
                 copies: int = 1, out_dtype: Optional[torch.dtype] = None, device="cuda"):
        if weight.dim() != 1 or weight.shape[0] % groups != 0:
            raise ValueError(f"a norm weight of {list(weight.shape)} cannot be cut into {groups} groups")
        self.weight = weight.to(device=device, dtype=torch.float32).contiguous()
        self.eps, self.groups, self.streams, self.copies = float(eps), int(groups), int(streams), int(copies)
        self.width = weight.shape[0]
        self.read = read
        self.out_dtype = out_dtype

    def weight_bytes(self) -> int:
        return self.weight.numel() * 4

    def workspace_bytes(self, rows: int, act_bytes: int) -> int:
        return aligned(rows * self.copies * self.width * (4 if self.out_dtype == torch.float32 else act_bytes))

    def kernel_modules(self, dtype, max_rows):
        return ("streams",)

    def forward(self, resid: torch.Tensor, pending: Optional[PendingWrite], ctx: StepContext,
                rows: Optional[torch.Tensor] = None, num_rows: Optional[int] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """resid float32 [T, streams * width]. With `rows` only those rows are normalised and the
        pending write is applied to what is read, not stored."""
        T = resid.shape[0]
        n = T if rows is None else (num_rows if num_rows is not None else rows.numel())
        if out is None:
            out = ctx.alloc((n, self.copies * self.width), self.out_dtype or ctx.dtype)
        y = pending.y if pending is not None else None
        c = pending.coef if pending is not None else None
        kernels.stream_norm(resid.view(T, self.streams, self.width), y, c.mix if c else None, c.write if c else None, self.read,
                            self.weight, self.groups, self.eps, out, rows[:n] if rows is not None else None)
        return out


class StreamEmbedding:
    """Token embedding, then the model's norm, then the result copied into every stream."""

    def __init__(self, embedding, norm: StreamNorm):
        self.embedding, self.norm = embedding, norm
        self.table, self.vocab, self.hidden = embedding.table, embedding.vocab, embedding.hidden
        self.err_flag = embedding.err_flag

    def kernel_modules(self, dtype, max_rows):
        return tuple(self.embedding.kernel_modules(dtype, max_rows)) + tuple(self.norm.kernel_modules(dtype, max_rows))

    def scratch_bytes(self, rows: int) -> int:
        """What `forward` takes from the workspace beside the residual itself."""
        return aligned(rows * self.hidden * 4)

    def forward(self, ctx: StepContext) -> torch.Tensor:
        resid = ctx.alloc((ctx.rows, self.norm.copies * self.hidden), torch.float32)
        with ctx.workspace.scope():
            raw = self.embedding.forward(ctx)                      # float32 [rows, hidden]: one stream
            self.norm.forward(raw, None, ctx, out=resid)
        return resid


class StreamBlock:
    """norm -> mixer -> write, norm -> feed-forward -> write, over a residual in streams. A layer
    without a feed-forward has `norm2`, `feed_forward`, `coef2` None."""

    def __init__(self, norm1: StreamNorm, mixer: Mixer, coef1: StreamCoefficients, norm2: Optional[StreamNorm] = None,
                 feed_forward: Optional[FeedForward] = None, coef2: Optional[StreamCoefficients] = None):
        if (norm2 is None) != (feed_forward is None) or (norm2 is None) != (coef2 is None):
            raise ValueError("a feed-forward needs its norm and its stream coefficients, and the other way round")
        self.norm1, self.mixer, self.coef1 = norm1, mixer, coef1
        self.norm2, self.feed_forward, self.coef2 = norm2, feed_forward, coef2

    def _parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None]

    def weight_bytes(self) -> int:
        return sum(getattr(p, "weight_bytes", lambda: 0)() for p in self._parts())

    def workspace_bytes(self, rows: int, hidden: int, act_bytes: int) -> int:
        mixed = aligned(rows * hidden * act_bytes)
        first = self.norm1.workspace_bytes(rows, act_bytes) + self.mixer.workspace_bytes(rows)
        if self.feed_forward is None:
            return first
        return mixed + max(first, self.norm2.workspace_bytes(rows, act_bytes) + self.feed_forward.workspace_bytes(rows))

    def kernel_modules(self, dtype, max_rows):
        mods = []
        for p in self._parts():
            mods += list(getattr(p, "kernel_modules", lambda d, r: ())(dtype, max_rows))
        return tuple(mods)

    def can_fold(self) -> bool:
        return False

    def forward(self, resid: torch.Tensor, pending: Optional[PendingWrite], ctx: StepContext, cache: Optional[LayerCache],
                state: Optional[torch.Tensor], out: torch.Tensor) -> PendingWrite:
        """`pending`: the write the previous layer left to do. The last sublayer's output goes to
        `out` (which outlives this layer's scratch) and is returned as the next pending write."""
        ws = ctx.workspace

        def mix_into(dst):
            with ws.scope():
                normed = self.norm1.forward(resid, pending, ctx)
                m = self.mixer.forward(normed, ctx, cache, state, out=dst)
                if m.data_ptr() != dst.data_ptr():
                    dst.copy_(m)
        if self.feed_forward is None:
            mix_into(out)
            return PendingWrite(out, self.coef1)
        with ws.scope():
            mixed = ctx.alloc(out.shape, out.dtype)
            mix_into(mixed)
            normed2 = self.norm2.forward(resid, PendingWrite(mixed, self.coef1), ctx)
            ff = self.feed_forward.forward(normed2, ctx, out=out)
            if ff.data_ptr() != out.data_ptr():
                out.copy_(ff)
        return PendingWrite(out, self.coef2)
