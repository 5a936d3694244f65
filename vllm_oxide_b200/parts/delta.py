"""The gated delta rule as a token mixer: a matrix state per head instead of pages.

With `heads` value heads of size vdim and `kv_heads` query/key heads of size dim (value head h reads query/key head
h / (heads / kv_heads)), and x the mixer's input:

    q, k, v = SiLU(conv(W_q x)), SiLU(conv(W_k x)), SiLU(conv(W_v x))      short causal convolutions over time, one filter
                                                                           a channel (<tensor>.conv [channels, taps], the
                                                                           last tap is the current token's)
    q, k    = unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q also times dim^(-1/2)
    beta    = sigmoid(W_b x),   g = exp(-exp(A_log) * softplus(W_a x + dt_bias))        one of each per value head
    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q                      per head, S [dim, vdim]
    out     = W_o [ RMSNorm_vdim(o) * norm * SiLU(W_g x) ]                               norm: one weight for all heads

All seven projections are one product.  The state of a request, [heads, dim, vdim] floats followed by the last taps - 1
inputs of every convolution channel, lives in the cache manager's state slots (float; zeroed when a slot is assigned).
Unit vectors, beta, the decay, the recurrence and the norm are float on both paths (csrc/kernels/delta.cu).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Mixer, StateSpec, register_part
from .linear import linear


SHORT_PORTIONS = 8      # up to this many tokens a request, the convolution and its state are one kernel


class GatedDelta(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, taps: int, eps: float,
                 prefix: str, dtype=None, device=None, **_):
        self.H, self.nh, self.kvh, self.dk, self.dv = int(hidden_size), int(num_heads), int(num_kv_heads), int(dim), int(vdim)
        self.taps, self.eps, self.prefix = int(taps), float(eps), prefix
        if self.nh % self.kvh:
            raise ValueError(f"heads {self.nh} is not a multiple of kv_heads {self.kvh}")
        if self.dk > 256:
            raise ValueError(f"the delta-rule scan keeps a column of the state in registers: dim up to 256, not {self.dk}")
        if not 1 <= self.taps <= 9:
            raise ValueError(f"the short convolution takes 1 to 9 taps, not {self.taps}")
        self.channels = 2 * self.kvh * self.dk + self.nh * self.dv           # q | k | v: what the convolutions see
        self.gate_off = self.channels                                        # then the output gate, beta, the decay
        self.b_off = self.gate_off + self.nh * self.dv
        self.a_off = self.b_off + self.nh
        self.width = (self.a_off + self.nh + 7) // 8 * 8                     # rows stay 16-byte aligned
        self.matrix_floats = self.nh * self.dk * self.dv
        self.w_in = self.wo = self.conv_w = self.A_log = self.dt_bias = self.norm_weight = None

    def tensor_specs(self) -> List[TensorSpec]:
        p, H, qk, vd = self.prefix, self.H, self.kvh * self.dk, self.nh * self.dv
        conv = lambda name, c: TensorSpec(p + name + ".conv", (c, self.taps), "coefficient", self.taps, init="normal")
        return [TensorSpec(p + "q", (qk, H), "matrix", H), conv("q", qk), TensorSpec(p + "k", (qk, H), "matrix", H), conv("k", qk),
                TensorSpec(p + "v", (vd, H), "matrix", H), conv("v", vd), TensorSpec(p + "b", (self.nh, H), "matrix", H),
                TensorSpec(p + "A_log", (self.nh,), "coefficient", init="normal"), TensorSpec(p + "norm", (self.dv,), "norm"),
                TensorSpec(p + "a", (self.nh, H), "matrix", H), TensorSpec(p + "dt_bias", (self.nh,), "coefficient", init="normal"),
                TensorSpec(p + "g", (vd, H), "matrix", H), TensorSpec(p + "o", (H, vd), "matrix", vd)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        p = self.prefix
        rows = [tensors[p + n] for n in ("q", "k", "v", "g", "b", "a")]
        rows.append(rows[0].new_zeros((self.width - self.a_off - self.nh, self.H)))
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.conv_w = torch.cat([tensors[p + n + ".conv"] for n in ("q", "k", "v")], dim=0).contiguous()
        self.A_log, self.dt_bias = tensors[p + "A_log"].contiguous(), tensors[p + "dt_bias"].contiguous()
        self.norm_weight, self.wo = tensors[p + "norm"].contiguous(), tensors[p + "o"].contiguous()

    def state_spec(self) -> StateSpec:
        return StateSpec((self.matrix_floats + (self.taps - 1) * self.channels,), torch.float32)

    def forward(self, x, ctx, cache, state, write_cache: bool = True):
        T, B = x.shape[0], ctx.launch_requests
        proj = linear(x, self.w_in, ctx.ws.get("delta_in", T, self.width, x.dtype), ctx)
        qkv = ctx.ws.get("delta_qkv", T, self.channels, torch.float32)
        if ctx.max_q <= SHORT_PORTIONS:
            # short portions (decoding): a thread a (request, channel) does the filter and leaves the slot's inputs, one launch
            kernels.short_conv_step(proj, self.channels, self.conv_w, state, self.matrix_floats, ctx.cu_q, ctx.state_slots,
                                    qkv, B, ctx.err)
        else:
            kernels.short_conv_silu(proj, self.channels, self.conv_w, state, self.matrix_floats, ctx.token_req, ctx.cu_q,
                                    ctx.state_slots, qkv, T, ctx.err)
            kernels.short_conv_state(proj, self.channels, self.taps, state, self.matrix_floats, ctx.cu_q, ctx.state_slots, B)
        raw = ctx.ws.get("delta_raw", T, self.nh * self.dv, torch.float32)
        kernels.delta_scan(qkv, proj, self.b_off, self.a_off, self.A_log, self.dt_bias, state, ctx.cu_q, ctx.state_slots, raw,
                           B, self.nh, self.kvh, self.dk, self.dv, ctx.err)
        out = ctx.ws.get("delta_out", T, self.nh * self.dv, x.dtype)
        kernels.delta_out_norm(raw, proj[:, self.gate_off:], self.norm_weight, out, T, self.nh, self.dv, self.eps)
        return linear(out, self.wo, ctx.ws.get("mixer_proj", T, self.H, x.dtype), ctx)


register_part("mixer", "gated_delta", GatedDelta)
