"""Several residual streams a token ("hyper-connections"), and the norm with a single gain that goes with them.

A token carries S residual streams x_1..x_S instead of one; each begins as a copy of the embedded token.  A sublayer
(the mixer, or the feed-forward) reads one combination of them and writes into all of them:

    u = sum_s a_s x_s;   y = sublayer(norm(u));   x'_t = sum_s B[s][t] x_s + b_t y      (B indexed [from][to])

with learned a [S], b [S], B [S, S] per sublayer.  The streams are float on both paths (the residual sum is never rounded
to 16 bits) and live in one workspace buffer [tokens, S * width].  One kernel (`kernels.stream_step`) does the update
after a sublayer together with the combination and the norm before the next one, so a sublayer costs one pass over the
streams, as the fused add+norm does for a single stream.  Between blocks the convention of the other blocks holds:
`(hidden, residual)` = (output of the last sublayer, not yet written into the streams; the streams), and the coefficients
that the pending write needs travel in `ctx.stream_pending`.

`streams=1` without coefficient tensors (`coefficients=False`) is the plain pre-norm residual, kept in float.

`GainRMSNorm` is x / sqrt(mean(x^2) + eps) * g with ONE learned number g; it is taken of the sum of the streams
(after the pending write), which is what the model's last norm sees.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Block, Norm, PartSpec, build_part, register_part


class GainRMSNorm(Norm):
    graph_safe = True

    def __init__(self, size: int, eps: float, weight_name: str, streams: int = 1, **_):
        self.size, self.eps, self.weight_name, self.streams = size, float(eps), weight_name, int(streams)
        self.weight = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.weight_name, (), "norm")]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].reshape(1).contiguous()

    def forward(self, x, residual, ctx, rows=None, n_rows=None, name="normed"):
        """norm(sum of the streams) for the streams in `residual`, after the write of `x` that is still pending (x None:
        none is).  `residual` None: `x` [tokens, size] is the only stream there is."""
        if residual is None:
            streams = ctx.ws.get("streams", x.shape[0], self.streams * self.size, torch.float32)
            y = ctx.ws.get(name, x.shape[0] if rows is None else n_rows, self.size, x.dtype)
            kernels.stream_step(streams, self.streams, self.size, self.eps, ctx.err, init=x, gain=self.weight, normed=y,
                                rows=rows, n_out=n_rows)
            return y, streams
        mix, out_w = getattr(ctx, "stream_pending", None) or (None, None)
        dtype = x.dtype if x is not None else ctx.ws.dtype
        y = ctx.ws.get(name, residual.shape[0] if rows is None else n_rows, self.size, dtype)
        kernels.stream_step(residual, self.streams, self.size, self.eps, ctx.err, y=x, mix=mix, out_w=out_w,
                            gain=self.weight, normed=y, rows=rows, n_out=n_rows)
        if rows is None:
            ctx.stream_pending = None
            return y, residual
        return y, residual


class _Sublayer:
    """The coefficients of one sublayer and its norm."""

    def __init__(self, norm: Norm, prefix: Optional[str], streams: int):
        self.norm, self.prefix, self.S = norm, prefix, streams
        self.a = self.b = self.B = None

    def tensor_specs(self) -> List[TensorSpec]:
        if self.prefix is None:
            return []
        S = self.S
        return [TensorSpec(self.prefix + "in", (S,), "coefficient", init="mean"),
                TensorSpec(self.prefix + "out", (S,), "coefficient", init="one"),
                TensorSpec(self.prefix + "mix", (S, S), "coefficient", init="identity")]

    def load(self, tensors) -> None:
        if self.prefix is not None:
            self.a = tensors[self.prefix + "in"].contiguous()
            self.b = tensors[self.prefix + "out"].contiguous()
            self.B = tensors[self.prefix + "mix"].contiguous()


class StreamsBlock(Block):
    """norm -> mixer -> (norm -> feed-forward) over S residual streams; `feed_forward` None: the mixer is the whole layer."""

    def __init__(self, mixer: PartSpec, feed_forward: Optional[PartSpec], input_norm: PartSpec,
                 post_mixer_norm: Optional[PartSpec], streams: int, size: int, mixer_coefficients: Optional[str] = None,
                 feed_forward_coefficients: Optional[str] = None, **common):
        self.S, self.size = int(streams), int(size)
        if not 1 <= self.S <= 16:
            raise ValueError(f"the stream kernels take 1 to 16 residual streams, not {self.S}")
        if (mixer_coefficients is None or (feed_forward is not None and feed_forward_coefficients is None)) and self.S != 1:
            raise ValueError("several residual streams need their coefficient tensors")
        self.input_norm = build_part("norm", input_norm, **common)
        self.mixer = build_part("mixer", mixer, **common)
        self.feed_forward = build_part("feed_forward", feed_forward, **common) if feed_forward is not None else None
        self.post_mixer_norm = build_part("norm", post_mixer_norm, **common) if feed_forward is not None else None
        for n in (self.input_norm, self.post_mixer_norm):
            if n is not None and not isinstance(n, GainRMSNorm):
                raise ValueError("the streams block fuses its norms into the stream kernel: they must be of kind 'rmsnorm_gain'")
        self.sub1 = _Sublayer(self.input_norm, mixer_coefficients, self.S)
        self.sub2 = _Sublayer(self.post_mixer_norm, feed_forward_coefficients, self.S) if feed_forward is not None else None
        self._parts = [p for p in (self.input_norm, self.mixer, self.post_mixer_norm, self.feed_forward) if p is not None]
        self.graph_safe = all(p.graph_safe for p in self._parts)

    def parts(self):
        return list(self._parts)

    def device_tensors(self):
        own = [t for s in (self.sub1, self.sub2) if s is not None for t in (s.a, s.b, s.B) if t is not None]
        return own + [t for p in self._parts for t in p.device_tensors()]

    def tensor_specs(self) -> List[TensorSpec]:
        specs = [s for p in self._parts for s in p.tensor_specs()]
        for sub in (self.sub1, self.sub2):
            if sub is not None:
                specs += sub.tensor_specs()
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self._parts:
            p.load({s.name: tensors[s.name] for s in p.tensor_specs()})
        for sub in (self.sub1, self.sub2):
            if sub is not None:
                sub.load(tensors)

    def _enter(self, sub: _Sublayer, hidden, streams, ctx, name: str):
        """Writes the pending output into the streams (or starts them from the embedded tokens) and returns what `sub`
        reads: norm(sum_s a_s x_s)."""
        T = hidden.shape[0]
        normed = ctx.ws.get(name, T, self.size, hidden.dtype)
        if streams is None:
            streams = ctx.ws.get("streams", T, self.S * self.size, torch.float32)
            kernels.stream_step(streams, self.S, self.size, sub.norm.eps, ctx.err, init=hidden, in_w=sub.a,
                                gain=sub.norm.weight, normed=normed)
        else:
            mix, out_w = getattr(ctx, "stream_pending", None) or (None, None)
            kernels.stream_step(streams, self.S, self.size, sub.norm.eps, ctx.err, y=hidden, mix=mix, out_w=out_w,
                                in_w=sub.a, gain=sub.norm.weight, normed=normed)
        ctx.stream_pending = None
        return normed, streams

    def forward(self, hidden, residual, ctx, cache, state, write_cache=True):
        normed, streams = self._enter(self.sub1, hidden, residual, ctx, "normed")
        y = self.mixer.forward(normed, ctx, cache, state, write_cache)
        ctx.stream_pending = (self.sub1.B, self.sub1.b)
        if self.feed_forward is not None:
            normed, streams = self._enter(self.sub2, y, streams, ctx, "normed_ff")
            y = self.feed_forward.forward(normed, ctx)
            ctx.stream_pending = (self.sub2.B, self.sub2.b)
        return y, streams


def stream_sums(hidden, streams, ctx, num_streams: int, width: int) -> torch.Tensor:
    """The sum of the streams [tokens, width] (float, a new tensor) after the pending write of `hidden`: what a model
    with one stream would call its residual stream.  For inspection; no step of the engine needs it."""
    x = streams.clone()
    mix, out_w = getattr(ctx, "stream_pending", None) or (None, None)
    if hidden is not None:
        kernels.stream_step(x, num_streams, width, 0.0, ctx.err, y=hidden, mix=mix, out_w=out_w)
    sums = torch.empty((x.shape[0], width), dtype=torch.float32, device=x.device)
    kernels.stream_sum(x, sums, num_streams, width)
    return sums


register_part("norm", "rmsnorm_gain", GainRMSNorm)
register_part("block", "streams", StreamsBlock)
