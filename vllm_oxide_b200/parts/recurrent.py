"""Recurrent token mixers: a fixed-size state per request instead of pages.

Both keep their state in float in the cache manager's state slots (`state_spec()`), carried from step to step;
a request's slot is zeroed when it is assigned.  Projections are the package's usual products (merged where several
read the same input); gates, decays and the recurrence itself are float inside one scan kernel a mixer.

`MinGRU`: both gates are functions of the current token alone, never of the state.  z = sigmoid(Wz h + bz), u = Wx h + bx, candidate = u + 1/2 where
u >= 0 and sigmoid(u) below, s_t = (1 - z) s_{t-1} + z * candidate (element by element, `width` channels), output
Wo (s_t * silu(Wg h)).  (The recurrence of Feng, Tung, Ahmed, Bengio and Hajimirsadeghi, "Were RNNs All We Needed?".)

`HGRN2`: a matrix-valued state per head with one gate for two jobs: f keeps, 1 - f writes.  Per head q = silu(Wq h) [dim],
v = Wv h [vdim], f = l + (1 - l) sigmoid(Wf h + bf) [dim] with a learned lower bound l; the state M [dim, vdim] goes
M_t = diag(f_t) M_{t-1} + (1 - f_t) v_t^T, o_t = M_t^T q_t; o is RMS-normed over vdim (a weight shared by the heads),
heads are concatenated and projected by Wo.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Mixer, StateSpec, register_part
from .linear import linear


class MinGRU(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, width: int, prefix: str, dtype=None, device=None, **_):
        self.H, self.W, self.prefix = int(hidden_size), int(width), prefix
        self.wzxg = self.wo = self.bz = self.bx = None

    def tensor_specs(self) -> List[TensorSpec]:
        p, H, W = self.prefix, self.H, self.W
        return [TensorSpec(p + "z", (W, H), "matrix", H), TensorSpec(p + "z.b", (W,), "bias"),
                TensorSpec(p + "x", (W, H), "matrix", H), TensorSpec(p + "x.b", (W,), "bias"),
                TensorSpec(p + "g", (W, H), "matrix", H), TensorSpec(p + "o", (H, W), "matrix", W)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        p = self.prefix
        # rows of z, then the candidate, then the output gate: one product for the three
        self.wzxg = torch.cat([tensors[p + "z"], tensors[p + "x"], tensors[p + "g"]], dim=0).contiguous()
        self.bz, self.bx = tensors[p + "z.b"].contiguous(), tensors[p + "x.b"].contiguous()
        self.wo = tensors[p + "o"].contiguous()

    def state_spec(self) -> StateSpec:
        return StateSpec((self.W,), torch.float32)

    def forward(self, x, ctx, cache, state, write_cache: bool = True):
        T = x.shape[0]
        zxg = linear(x, self.wzxg, ctx.ws.get("mingru_zxg", T, 3 * self.W, x.dtype), ctx)
        gated = ctx.ws.get("mingru_out", T, self.W, x.dtype)
        kernels.mingru_scan(zxg, self.bz, self.bx, state, ctx.cu_q, ctx.state_slots, gated, ctx.launch_requests, ctx.err,
                            chunks=kernels.scan_chunks(T, ctx.launch_requests))
        return linear(gated, self.wo, ctx.ws.get("mixer_proj", T, self.H, x.dtype), ctx)


class HGRN2(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, dim: int, vdim: int, eps: float, prefix: str, dtype=None,
                 device=None, **_):
        self.H, self.nh, self.dk, self.dv, self.eps, self.prefix = int(hidden_size), int(num_heads), int(dim), int(vdim), float(eps), prefix
        if self.dk > 256:
            raise ValueError(f"the HGRN2 scan keeps a column of the state in registers: dim up to 256, not {self.dk}")
        self.wqfv = self.wo = self.bf = self.lower = self.norm_weight = None

    def tensor_specs(self) -> List[TensorSpec]:
        p, H, qd, vd = self.prefix, self.H, self.nh * self.dk, self.nh * self.dv
        return [TensorSpec(p + "q", (qd, H), "matrix", H), TensorSpec(p + "f", (qd, H), "matrix", H),
                TensorSpec(p + "f.b", (qd,), "bias"), TensorSpec(p + "lower", (qd,), "coefficient", init="fraction"),
                TensorSpec(p + "v", (vd, H), "matrix", H), TensorSpec(p + "norm", (self.dv,), "norm"),
                TensorSpec(p + "o", (H, vd), "matrix", vd)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        p = self.prefix
        self.wqfv = torch.cat([tensors[p + "q"], tensors[p + "f"], tensors[p + "v"]], dim=0).contiguous()
        self.bf, self.lower = tensors[p + "f.b"].contiguous(), tensors[p + "lower"].contiguous()
        self.norm_weight, self.wo = tensors[p + "norm"].contiguous(), tensors[p + "o"].contiguous()

    def state_spec(self) -> StateSpec:
        return StateSpec((self.nh, self.dk, self.dv), torch.float32)

    def forward(self, x, ctx, cache, state, write_cache: bool = True):
        T = x.shape[0]
        width = self.nh * (2 * self.dk + self.dv)
        qfv = linear(x, self.wqfv, ctx.ws.get("hgrn2_qfv", T, width, x.dtype), ctx)
        out = ctx.ws.get("hgrn2_out", T, self.nh * self.dv, x.dtype)
        # decoding: one block a (request, head), norm included; portions: a head's columns over several blocks
        fuse = kernels.hgrn2_can_fuse(self.dk, self.dv) and T <= 16 * ctx.launch_requests
        raw = None if fuse else ctx.ws.get("hgrn2_raw", T, self.nh * self.dv, torch.float32)
        # longer portions are also cut along the tokens (the mean portion decides, as for every scan)
        B = ctx.launch_requests
        chunks = 1 if fuse else min(kernels.scan_chunks(T, B), 16)
        scratch = None if chunks == 1 else ctx.ws.get_flat("hgrn2_ranges", B * chunks * self.nh * self.dk * (self.dv + 1),
                                                           torch.float32)
        kernels.hgrn2_scan(qfv, self.bf, self.lower, self.norm_weight, state, ctx.cu_q, ctx.state_slots, out,
                           B, self.nh, self.dk, self.dv, self.eps, ctx.err, raw=raw, chunks=chunks, scratch=scratch)
        return linear(out, self.wo, ctx.ws.get("mixer_proj", T, self.H, x.dtype), ctx)


register_part("mixer", "mingru", MinGRU)
register_part("mixer", "hgrn2", HGRN2)
