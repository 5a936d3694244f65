"""One float residual stream with a norm before AND after every sublayer ("sandwich" norms).

    x <- x + post(mixer(pre(x)));   x <- x + post'(feed_forward(pre'(x)))        (feed_forward None: the first line only)

All four norms are vector-weight RMSNorms.  The stream is float on both paths and lives in one workspace buffer
[tokens, width]; it is never rounded to 16 bits.  One kernel (`kernels.residual_norm_step`) takes the output of the
sublayer before through its post-norm into the stream and forms the input of the next sublayer by its pre-norm, so a
sublayer costs one pass over the stream, as the fused add+norm does for a bfloat16 stream.  Between blocks the
convention of the other blocks holds: `(hidden, residual)` = (output of the last sublayer, not yet in the stream; the
stream), and the norm that the pending output still has to pass travels in `ctx.pending_norm`.

The same norm kind serves as a plan's embedding norm (`open_stream`: the embedded tokens become the pending output of
"nothing", their norm is the stream's first value) and as its last norm.  A run with `ExecStep.reinject` gets the
embedding norm's output, which the first kernel of the step kept in `ctx.embedding_out`, added to the stream in the
same pass that enters its first sublayer.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Block, Norm, PartSpec, build_part, register_part


class StreamRMSNorm(Norm):
    """x / sqrt(mean(x^2) + eps) * w on a float residual stream, fused with the stream's update."""
    graph_safe = True

    def __init__(self, size: int, eps: float, weight_name: str, **_):
        self.size, self.eps, self.weight_name = int(size), float(eps), weight_name
        self.weight = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.weight_name, (self.size,), "norm")]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].contiguous()

    def open_stream(self, hidden, ctx, keep: bool = False):
        ctx.pending_norm = self
        ctx.embedding_out = ctx.ws.get("embedding_out", hidden.shape[0], self.size, torch.float32) if keep else None
        ctx.stream_keep = ctx.embedding_out
        return hidden, None

    def enter(self, hidden, stream, ctx, name: str, rows=None, n_rows=None):
        """The pending output `hidden` goes through its norm into `stream` (None: the stream begins with it), what a run
        adds back is added, and this norm of the result is returned with the stream."""
        pending = getattr(ctx, "pending_norm", None)
        if pending is not None and pending.eps != self.eps:
            raise ValueError("the norms around one residual stream share one eps")
        T = hidden.shape[0] if hidden is not None else stream.shape[0]
        dtype = hidden.dtype if hidden is not None else ctx.ws.dtype
        init = stream is None
        if init:
            stream = ctx.ws.get("residual_stream", T, self.size, torch.float32)
        inject = ctx.embedding_out if getattr(ctx, "reinject", False) and rows is None else None
        keep = getattr(ctx, "stream_keep", None) if rows is None else None
        out = ctx.ws.get(name, T if rows is None else n_rows, self.size, dtype)
        kernels.residual_norm_step(stream, self.eps, ctx.err, y=hidden, w_post=pending.weight if pending is not None else None,
                                   inject=inject, keep=keep, w_pre=self.weight, out=out, rows=rows, n_out=n_rows, init=init)
        if rows is None:
            ctx.pending_norm = ctx.stream_keep = None
            ctx.reinject = False
        return out, stream

    def forward(self, x, residual, ctx, rows=None, n_rows=None, name="normed"):
        """As a model's last norm: norm(stream after the pending write of `x`), on the wanted rows."""
        return self.enter(x, residual, ctx, name, rows=rows, n_rows=n_rows)


class SandwichBlock(Block):
    def __init__(self, mixer: PartSpec, feed_forward: Optional[PartSpec], pre_mixer_norm: PartSpec, post_mixer_norm: PartSpec,
                 pre_ff_norm: Optional[PartSpec], post_ff_norm: Optional[PartSpec], size: int, **common):
        self.size = int(size)
        self.pre_mixer_norm = build_part("norm", pre_mixer_norm, **common)
        self.mixer = build_part("mixer", mixer, **common)
        self.post_mixer_norm = build_part("norm", post_mixer_norm, **common)
        self.feed_forward = build_part("feed_forward", feed_forward, **common) if feed_forward is not None else None
        self.pre_ff_norm = build_part("norm", pre_ff_norm, **common) if feed_forward is not None else None
        self.post_ff_norm = build_part("norm", post_ff_norm, **common) if feed_forward is not None else None
        self._parts = [p for p in (self.pre_mixer_norm, self.mixer, self.post_mixer_norm, self.pre_ff_norm, self.feed_forward,
                                   self.post_ff_norm) if p is not None]
        for n in (self.pre_mixer_norm, self.post_mixer_norm, self.pre_ff_norm, self.post_ff_norm):
            if n is not None and not isinstance(n, StreamRMSNorm):
                raise ValueError("the sandwich block fuses its norms into the stream's kernel: they must be of kind 'rmsnorm_stream'")
        self.input_norm = self.pre_mixer_norm
        self.graph_safe = all(p.graph_safe for p in self._parts)

    def parts(self):
        return list(self._parts)

    def tensor_specs(self) -> List[TensorSpec]:
        return [s for p in self._parts for s in p.tensor_specs()]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self._parts:
            p.load({s.name: tensors[s.name] for s in p.tensor_specs()})

    def forward(self, hidden, residual, ctx, cache, state, write_cache=True):
        normed, stream = self.pre_mixer_norm.enter(hidden, residual, ctx, "normed")
        y = self.mixer.forward(normed, ctx, cache, state, write_cache)
        ctx.pending_norm = self.post_mixer_norm
        if self.feed_forward is not None:
            normed, stream = self.pre_ff_norm.enter(y, stream, ctx, "normed_ff")
            y = self.feed_forward.forward(normed, ctx)
            ctx.pending_norm = self.post_ff_norm
        return y, stream


def stream_value(hidden, stream, ctx) -> torch.Tensor:
    """The residual stream [tokens, width] (float, a new tensor) after the pending write of `hidden`: what the next
    sublayer's norm would see.  For inspection; no step of the engine needs it."""
    x = stream.clone()
    pending = getattr(ctx, "pending_norm", None)
    if hidden is not None:
        kernels.residual_norm_step(x, pending.eps if pending is not None else 0.0, ctx.err, y=hidden,
                                   w_post=pending.weight if pending is not None else None)
    return x


register_part("norm", "rmsnorm_stream", StreamRMSNorm)
register_part("block", "sandwich", SandwichBlock)
