"""The mechanisms of Kesozen one by one: each part is built alone, given a cache of its own and stepped in portions, and
compared with its plain form (tests/plain/kesozen_plain.py).  Where random numbers would hide a fault the inputs are made
to show it: one key made so large that a query sees almost nothing else, placed at the first position and at page
borders; scores pushed far below zero, where the sink takes nearly all the weight; decays that forget slowly, so that the
first tokens still count hundreds of tokens later; corrections that turn the router's choice over."""
import math

import numpy as np
import pytest
import torch

from helpers import DEV, Alone, assert_close, held, in_portions, load, make_context, rand
from plain import kesozen_plain as P

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


# ---------------------------------------------------------------- the stream and its norms
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("D", [64, 50, 33, 344, 4096, 8200])
def test_residual_norm_step(D, dt):
    from vllm_oxide_b200 import kernels
    n, eps = 7, 1e-5
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    x, y, e = rand((n, D), 1, 3.0), held(rand((n, D), 2, 0.7), dt), rand((n, D), 3)
    wa, wb = 1.0 + 0.1 * rand((D,), 4), 1.0 + 0.1 * rand((D,), 5)
    f32 = lambda t: t.float().to(DEV).contiguous()
    # the whole chain: stream += norm(y) * wa + inject; out = norm(stream) * wb
    stream, out, keep = f32(x), torch.empty((n, D), dtype=dt, device=DEV), torch.empty((n, D), dtype=torch.float32, device=DEV)
    kernels.residual_norm_step(stream, eps, err, y=y.to(dt).to(DEV), w_post=f32(wa), inject=f32(e), keep=keep, w_pre=f32(wb), out=out)
    want = x.float().double() + P.rms_norm(y, wa.float().double(), eps) + e.float().double()
    assert_close(stream, want, torch.float32, "the stream")
    assert torch.equal(keep, stream)
    assert_close(out, P.rms_norm(want, wb.float().double(), eps), dt, "the next sublayer's input")
    # the start of a stream: what was there does not count
    stream2 = torch.full((n, D), 7.0, dtype=torch.float32, device=DEV)
    kernels.residual_norm_step(stream2, eps, err, y=y.to(dt).to(DEV), w_post=f32(wa), w_pre=f32(wb), out=out, init=True)
    assert_close(stream2, P.rms_norm(y, wa.float().double(), eps), torch.float32, "a stream that begins")
    # chosen rows only: nothing is stored
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    before, picked = stream.clone(), torch.empty((3, D), dtype=dt, device=DEV)
    kernels.residual_norm_step(stream, eps, err, y=y.to(dt).to(DEV), w_post=f32(wa), w_pre=f32(wb), out=picked, rows=rows, n_out=3)
    assert torch.equal(before, stream)
    want2 = want + P.rms_norm(y, wa.float().double(), eps)
    assert_close(picked, P.rms_norm(want2, wb.float().double(), eps)[[5, 0, 5]], dt, "rows")
    assert int(err.item()) == 0


# ---------------------------------------------------------------- attention whose keys are its values
def attention_part(dt, H, nh, kvh, hd, scale, rot):
    from vllm_oxide_b200.parts import PartSpec, build_part
    positions = {}
    if rot and rot["dims"]:
        positions["r"] = build_part("position", PartSpec("rope", dict(head_dim=hd, rotary_dim=rot["dims"], max_position=1 << 30,
                                                                     theta=rot["base"], interleaved=False, table=False)), device=DEV)
    part = build_part("mixer", PartSpec("attention_shared_kv", dict(hidden_size=H, num_heads=nh, num_kv_heads=kvh, head_dim=hd,
                                                                    scale=scale, position="r" if positions else None, prefix="m.")),
                      positions=positions, dtype=dt, device=DEV)
    w = {"m.q": rand((nh * hd, H), 1, H ** -0.5), "m.k": rand((kvh * hd, H), 2, H ** -0.5), "m.g": rand((nh, H), 3, H ** -0.5),
         "m.o": rand((H, nh * hd), 4, (nh * hd) ** -0.5)}
    load(part, w, dt)
    m = dict(heads=nh, kv_heads=kvh, dim=hd, vdim=hd, scale=scale, rot=rot or dict(dims=0, base=1.0))
    return part, {k: held(v, dt) for k, v in w.items()}, m


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("case", ["part of the head rotated", "one key head", "whole head rotated, 128 wide", "nothing rotated",
                                  "as many key heads as heads", "scores far below the sink", "a head of 20", "a head of 40"])
def test_shared_kv_attention_alone_with_loud_keys(case, dt):
    bs = 16
    if case == "part of the head rotated":
        H, spec = 40, (6, 2, 48, 0.2, dict(dims=16, base=1000.0))
    elif case == "one key head":
        H, spec, bs = 64, (4, 1, 64, 0.11, dict(dims=32, base=10000.0)), 64
    elif case == "whole head rotated, 128 wide":
        H, spec = 64, (2, 2, 128, 0.07, dict(dims=128, base=50000.0))
    elif case == "nothing rotated":
        H, spec = 48, (3, 3, 16, 0.3, None)
    elif case == "as many key heads as heads":
        H, spec = 32, (5, 5, 32, 0.25, dict(dims=2, base=100.0))
    elif case == "a head of 20":               # no 16-byte loads, the plain kernel in both precisions
        H, spec = 40, (3, 1, 20, 0.3, dict(dims=6, base=50.0))
    elif case == "a head of 40":
        H, spec = 48, (4, 2, 40, 0.2, dict(dims=40, base=1000.0))
    else:
        H, spec = 40, (4, 2, 32, -3.0, dict(dims=8, base=300.0))    # a negative scale: the loud keys' own scores are far below 0
    part, w, m = attention_part(dt, H, *spec)
    n = 210
    x = rand((n, H), 33)
    for j in (0, 15, 16, 31, 100):              # the first token, both sides of page borders, one in the middle
        x[j] *= 4.0
    x = held(x, dt)
    want = P.sink_attention(x, w, "m.", m, 1e-6, torch.float64)
    # the plain form itself: with every gate at one half the rows differ
    no_gate = dict(w, **{"m.g": torch.zeros_like(w["m.g"])})
    assert (P.sink_attention(x, no_gate, "m.", m, 1e-6, torch.float64) - want).abs().max() > 0.02 * want.abs().max()
    tol = 1e-4 if dt == torch.float32 else 0.08      # scores of loud tokens run to tens: the rounding of a query or key shows
    alone = Alone([part], dt, block_size=bs, pages=max(8, 4 * (n // bs + 1)), slots=3)
    for cuts, what in (([n], "whole"), ([n - 120] + [1] * 120, "decoded"), ([2, 5, 1, 30, 3], "portions"), ([bs], "pages"), ([1], "alone")):
        assert_close(in_portions(alone, 7, x, cuts), want, dt, f"{case}: {what}", tol)
    other = held(rand((150, H), 34), dt)
    o_want = P.sink_attention(other, w, "m.", m, 1e-6, torch.float64)
    a = alone.step([(1, x[:90]), (2, other[:149])])[0]
    b = alone.step([(2, other[149:]), (1, x[90:])], end=[1, 2])[0]
    assert_close(torch.cat([a[:90], b[1:]]), want, dt, f"{case}: beside another request", tol)
    assert_close(torch.cat([a[90:], b[:1]]), o_want, dt, f"{case}: the other request", tol)


def test_the_sink_takes_the_weight_that_low_scores_leave():
    """Tokens that are nearly alike and queries that point away from the keys: every score is far below zero, the sink
    takes nearly all the weight and the output is nearly nothing, where a softmax without the sink would still return a
    full average of the values."""
    dt = torch.float32
    part, w, m = attention_part(dt, 32, 2, 1, 16, 1.0, None)
    x = held(rand((1, 32), 5).repeat(40, 1) * 0.5 + 0.02 * rand((40, 32), 6), dt)
    w["m.q"] = -2.0 * w["m.k"].repeat(2, 1)
    w["m.g"] = w["m.g"] * 0.0 + 1.0
    load(part, w, dt)
    want = P.sink_attention(x, w, "m.", m, 1e-6, torch.float64)
    values = x @ w["m.k"].T
    assert want.abs().max() < 0.1 * (values @ w["m.o"][:, :16].T).abs().max()
    got = in_portions(Alone([part], dt), 0, x, [17, 1, 1, 21])
    assert_close(got, want, dt, "low scores", 1e-4)


# ---------------------------------------------------------------- the gated delta rule
def delta_part(dt, H, nh, kvh, dk, dv, taps, eps, slow=True):
    from vllm_oxide_b200.parts import PartSpec, build_part
    part = build_part("mixer", PartSpec("gated_delta", dict(hidden_size=H, num_heads=nh, num_kv_heads=kvh, dim=dk, vdim=dv, taps=taps,
                                                            eps=eps, prefix="m.")), positions={}, dtype=dt, device=DEV)
    A_log = rand((nh,), 8)
    if slow:
        A_log[::2] = -6.0          # every other head forgets almost nothing: the first tokens' writes are still there at the end
    w = {"m.q": rand((kvh * dk, H), 1, H ** -0.5), "m.k": rand((kvh * dk, H), 2, H ** -0.5), "m.v": rand((nh * dv, H), 3, H ** -0.5),
         "m.q.conv": rand((kvh * dk, taps), 4, taps ** -0.5), "m.k.conv": rand((kvh * dk, taps), 5, taps ** -0.5),
         "m.v.conv": rand((nh * dv, taps), 6, taps ** -0.5), "m.b": rand((nh, H), 7, H ** -0.5), "m.A_log": A_log,
         "m.norm": 1.0 + 0.1 * rand((dv,), 9), "m.a": rand((nh, H), 10, H ** -0.5), "m.dt_bias": rand((nh,), 11),
         "m.g": rand((nh * dv, H), 12, H ** -0.5), "m.o": rand((H, nh * dv), 13, (nh * dv) ** -0.5)}
    load(part, w, dt)
    floats = ("m.q.conv", "m.k.conv", "m.v.conv", "m.A_log", "m.norm", "m.dt_bias")
    wh = {k: (v.float().double() if k in floats else held(v, dt)) for k, v in w.items()}
    return part, wh, dict(heads=nh, kv_heads=kvh, dim=dk, vdim=dv, conv=taps)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("H,nh,kvh,dk,dv,taps", [(48, 3, 3, 16, 24, 4), (64, 4, 2, 64, 40, 3), (32, 2, 1, 128, 32, 2), (40, 6, 2, 20, 8, 5),
                                                 (32, 1, 1, 256, 16, 1), (32, 2, 2, 200, 130, 4), (64, 2, 2, 32, 64, 9)])
def test_gated_delta_alone(H, nh, kvh, dk, dv, taps, dt):
    eps = 1e-5
    part, w, m = delta_part(dt, H, nh, kvh, dk, dv, taps, eps)
    n = 200
    x = held(rand((n, H), 20), dt)
    want = P.delta_mixer(x, w, "m.", m, eps, torch.float64)
    # the plain form itself remembers: started 120 tokens late, the last output is another
    assert (P.delta_mixer(x[120:], w, "m.", m, eps, torch.float64)[-1] - want[-1]).abs().max() > 0.01 * want.abs().max()
    alone = Alone([part], dt, slots=2)
    tol = 1e-4 if dt == torch.float32 else 0.05
    assert_close(in_portions(alone, 0, x, [n]), want, dt, "whole", tol)
    assert_close(in_portions(alone, 1, x, [n - 40] + [1] * 40), want, dt, "decoded", tol)
    assert_close(in_portions(alone, 0, x, [2, 9, 1, 8, 30]), want, dt, "portions", tol)
    assert_close(in_portions(alone, 1, x, [1, 2]), want, dt, "portions shorter than the filters", tol)
    y = held(rand((90, H), 21), dt)
    out = alone.step([(5, y[:60]), (6, x[:31])])[0]
    out2 = alone.step([(6, x[31:32]), (5, y[60:])], end=[5, 6])[0]
    assert_close(torch.cat([out[:60], out2[1:]]), P.delta_mixer(y, w, "m.", m, eps, torch.float64), dt, "beside another request", tol)
    assert_close(torch.cat([out[60:], out2[:1]]), want[:32], dt, "the other request", tol)
    # a slot that is used again starts from zero, filters included
    assert_close(in_portions(alone, 9, y, [3, 87]), P.delta_mixer(y, w, "m.", m, eps, torch.float64), dt, "a slot used again", tol)


# ---------------------------------------------------------------- feed-forwards
def ff_context(n, dt):
    from vllm_oxide_b200.cache.paged_cache import PagedCache
    from vllm_oxide_b200.parts.base import CacheSpec
    cache = PagedCache([CacheSpec(1, 16)], [None], dt, DEV, 16, 64, 1)
    assert cache.manager.add_request(0) and cache.manager.ensure(0, 0, n)
    return make_context(cache.manager, [(0, 0, [0] * n, [])], dt)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("H,I", [(64, 128), (50, 33), (344, 1000)])
def test_relu_squared_mlp(H, I, dt):
    from vllm_oxide_b200.parts import PartSpec, build_part
    part = build_part("feed_forward", PartSpec("relu2_mlp", dict(hidden_size=H, intermediate_size=I, prefix="f.")), positions={}, dtype=dt, device=DEV)
    w = {"f.up": rand((I, H), 1, H ** -0.5), "f.down": rand((H, I), 2, I ** -0.5)}
    load(part, w, dt)
    for n in (1, 5, 40):
        x = held(rand((n, H), 3 + n), dt)
        got = part.forward(x.to(dt).to(DEV), ff_context(n, dt))
        assert_close(got, P.dense_ff(x, {k: held(v, dt) for k, v in w.items()}, "f.", torch.float64), dt, f"{n} tokens")


@pytest.mark.parametrize("E,top,count,keep", [(16, 4, 2, 1), (12, 3, 1, 1), (8, 1, 4, 2), (30, 6, 5, 3), (6, 6, 3, 3), (64, 8, 8, 4), (5, 2, 5, 2)])
def test_the_router_alone(E, top, count, keep):
    """Corrections as large as the scores (and negative): the choice goes by score + correction, the weights by the score."""
    from vllm_oxide_b200 import kernels
    H, n = 48, 300
    x = rand((n, H), 1)
    w = {"f.router": (rand((E, H), 2, 2.0 * H ** -0.5)).float().double(), "f.correction": (rand((E,), 3, 0.3) - 0.2).float().double()}
    r = dict(experts=E, top=top, groups=dict(count=count, keep=keep))
    idx, weight = P.route(x.float().double(), w, "f.", r, torch.float64)
    ids = torch.empty((n, top), dtype=torch.int32, device=DEV)
    wts = torch.empty((n, top), dtype=torch.float32, device=DEV)
    kernels.moe_route(x.float().to(DEV), w["f.router"].float().to(DEV), w["f.correction"].float().to(DEV), ids, wts, n, top, count, keep)
    assert torch.equal(ids.cpu().long(), idx), "the chosen experts, in order"
    assert (wts.cpu().double() - weight).abs().max() < 1e-6
    plain_choice = torch.softmax(x.float().double() @ w["f.router"].T, -1).topk(top).indices
    assert not torch.equal(plain_choice, idx), "the corrections and groups change the choice in this test"
    assert top == E or abs(float(weight.sum(-1).mean()) - 1.0) > 0.05, "the weights are not renormalised"


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("H,I,E,top,count,keep", [(64, 32, 8, 2, 2, 1), (50, 33, 5, 5, 1, 1), (128, 96, 16, 4, 4, 2), (64, 200, 3, 1, 3, 2),
                                                  (200, 264, 6, 2, 3, 2)])
def test_routed_experts(H, I, E, top, count, keep, dt):
    from vllm_oxide_b200.parts import PartSpec, build_part
    part = build_part("feed_forward", PartSpec("routed_experts", dict(hidden_size=H, expert_size=I, experts=E, top=top, groups=count,
                                                                      keep=keep, prefix="f.")), positions={}, dtype=dt, device=DEV)
    w = {"f.router": rand((E, H), 2, 2.0 * H ** -0.5), "f.correction": rand((E,), 3, 0.2)}
    for e in range(E):
        w[f"f.e{e}.up"] = rand((I, H), 10 + e, H ** -0.5)
        w[f"f.e{e}.down"] = rand((H, I), 50 + e, I ** -0.5)
    load(part, w, dt)
    wh = {k: (v.float().double() if k in ("f.router", "f.correction") else held(v, dt)) for k, v in w.items()}
    mlp = dict(kind="moe", expert=dict(ff=I), router=dict(experts=E, top=top, groups=dict(count=count, keep=keep)))
    # from 256 (token, choice) pairs on, bfloat16 takes the tensor-core product of the experts: widths that end inside its
    # tiles of 128 rows and its slices of 64 columns, experts with one row and experts with hundreds
    for n in (1, 3, 70, 200) + ((700,) if H == 200 else ()):
        x = held(rand((n, H), 3 + n), dt)
        got = part.forward(x.to(dt).to(DEV), ff_context(n, dt))
        assert_close(got, P.moe_ff(x, wh, "f.", mlp, torch.float64), dt, f"{n} tokens")
    # a token's output does not depend on its neighbours in the batch
    x = held(rand((90, H), 99), dt).to(dt).to(DEV)
    whole = part.forward(x, ff_context(90, dt)).clone()
    alone = torch.cat([part.forward(x[i:i + 1].contiguous(), ff_context(1, dt)).clone() for i in (0, 17, 89)])
    if dt == torch.float32:
        assert torch.equal(whole[[0, 17, 89]], alone)
    else:
        assert_close(alone, whole[[0, 17, 89]], dt, "alone against in a batch")
