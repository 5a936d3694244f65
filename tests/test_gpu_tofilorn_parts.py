"""The mechanisms of Tofilorn one by one: each part is built alone, given a cache of its own and stepped in portions,
and compared with its plain form (tests/plain/tofilorn_plain.py).  Where random numbers would hide a fault the inputs
are made to show it: gates that forget slowly, so that the first tokens still count hundreds of tokens later; one key
made so large that a query sees almost nothing else, placed just inside and just outside a window and at page borders."""
import math

import numpy as np
import pytest
import torch

from helpers import DEV, Alone, assert_close, held, in_portions, load, rand, tolerance
from plain import tofilorn_plain as P

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


# ---------------------------------------------------------------- residual streams
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("S,D", [(1, 64), (3, 50), (4, 256), (5, 33), (6, 64), (8, 128), (16, 96)])
def test_stream_step(S, D, dt):
    from vllm_oxide_b200 import kernels
    n, eps = 7, 1e-5
    X = rand((S, n, D), 1)
    y, a, b, B = rand((n, D), 2), rand((S,), 3), rand((S,), 4), rand((S, S), 5)
    gain = torch.tensor([1.3], dtype=torch.float64)
    y_held = held(y, dt)
    new = torch.einsum("st,snd->tnd", B, X.float().double()) + b[:, None, None] * y_held[None]
    normed = P.gain_norm(torch.einsum("s,snd->nd", a.float().double(), new), gain.float().double(), eps)
    f32 = lambda t: t.float().to(DEV).contiguous()
    streams = f32(X.permute(1, 0, 2).reshape(n, S * D))
    out = torch.empty((n, D), dtype=dt, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.stream_step(streams, S, D, eps, err, y=y.to(dt).to(DEV), mix=f32(B), out_w=f32(b), in_w=f32(a), gain=f32(gain), normed=out)
    assert_close(streams.reshape(n, S, D).permute(1, 0, 2), new, torch.float32, "new streams", 1e-5)
    assert_close(out, normed, dt, "combination and norm", 1e-5 if dt == torch.float32 else 0.01)
    # rows (one of them twice): the same numbers without touching the streams; here on top of a second pending write
    before = streams.clone()
    rows = torch.tensor([4, 0, 4], dtype=torch.int32, device=DEV)
    picked = torch.empty((3, D), dtype=dt, device=DEV)
    kernels.stream_step(streams, S, D, eps, err, y=y.to(dt).to(DEV), mix=f32(B), out_w=f32(b), gain=f32(gain), normed=picked,
                        rows=rows, n_out=3)
    assert torch.equal(before, streams)
    again = torch.einsum("st,snd->tnd", B.float().double(), new.float().double()) + b.float().double()[:, None, None] * y_held[None]
    assert_close(picked, P.gain_norm(again.sum(0), gain.float().double(), eps)[[4, 0, 4]], dt, "rows", 1e-4 if dt == torch.float32 else 0.01)
    # the start: every stream is the embedded token
    kernels.stream_step(streams, S, D, eps, err, init=y.to(dt).to(DEV), in_w=f32(a), gain=f32(gain), normed=out)
    assert_close(streams.reshape(n, S, D)[:, S - 1], y_held, torch.float32, "start", 1e-7)
    assert_close(out, P.gain_norm(a.float().double().sum() * y_held, gain.float().double(), eps), dt, "start, normed",
                 1e-5 if dt == torch.float32 else 0.01)
    assert int(err.item()) == 0


# ---------------------------------------------------------------- rotation frequencies (no device needed, but cheap here)
@pytest.mark.parametrize("rot", [dict(dims=16, base=50000.0), dict(dims=8, base=1000.0, scaling=dict(factor=4.0, original=32, fast=8.0, slow=1.0)),
                                 dict(dims=64, base=10000.0, scaling=dict(factor=40.0, original=4096, fast=32.0, slow=1.0)),
                                 dict(dims=6, base=77.0, scaling=dict(factor=1.5, original=10, fast=1.0, slow=1.0))])
def test_stretched_frequencies(rot):
    from vllm_oxide_b200.parts.rope import scaled_frequencies
    w, amp = scaled_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    want, want_amp = P.rotation_frequencies(rot, torch.float64)
    assert w.dtype == torch.float32 and abs(amp - want_amp) < 1e-12
    assert ((w.double() - want).abs() / want).max() < 1e-6


# ---------------------------------------------------------------- minGRU
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("H,W", [(48, 40), (64, 192)])
def test_mingru_alone(H, W, dt):
    from vllm_oxide_b200.parts import PartSpec, build_part
    part = build_part("mixer", PartSpec("mingru", dict(hidden_size=H, width=W, prefix="m.")), positions={}, dtype=dt, device=DEV)
    w = {"m.z": rand((W, H), 1, H ** -0.5), "m.x": rand((W, H), 2, H ** -0.5), "m.g": rand((W, H), 3, H ** -0.5),
         "m.o": rand((H, W), 4, W ** -0.5), "m.z.b": rand((W,), 5) - 5.0, "m.x.b": rand((W,), 6)}
    # z is near 1/150 with the bias of -5: a state forgets over hundreds of tokens, so the first ones still count at the end
    load(part, w, dt)
    wh = {k: held(v, dt) for k, v in w.items()}
    n = 300
    x = [held(rand((n, H), 10 + r), dt) for r in range(2)]
    want = [P.mingru(xi, wh, "m.") for xi in x]
    # without what the first 200 tokens left in the state the last row is another one
    assert ((P.mingru(x[0][200:], wh, "m.")[-1] - want[0][-1]).abs().max() > 0.05 * want[0].abs().max())
    alone = Alone([part], dt, slots=2)
    assert_close(in_portions(alone, 0, x[0], [n]), want[0], dt, "whole")
    assert_close(in_portions(alone, 0, x[0], [n - 50] + [1] * 50), want[0], dt, "decoded")
    assert_close(in_portions(alone, 0, x[0], [2, 1, 33, 7]), want[0], dt, "portions")
    # two requests side by side, unequal portions, in slots that the runs above have used
    got = {0: [], 1: []}
    at = {0: 0, 1: 0}
    sizes = {0: [64, 1, 1, 30], 1: [3, 50, 1]}
    k = 0
    while at[0] < n or at[1] < n:
        portions = []
        for r in (1, 0):
            if at[r] < n:
                c = min(sizes[r][k % len(sizes[r])], n - at[r])
                portions.append((r, x[r][at[r]:at[r] + c]))
                at[r] += c
        out = alone.step(portions, end=[r for r, _ in portions if at[r] == n])[0]
        o = 0
        for r, rows in portions:
            got[r].append(out[o:o + rows.shape[0]])
            o += rows.shape[0]
        k += 1
    for r in (0, 1):
        assert_close(torch.cat(got[r]), want[r], dt, f"request {r} beside the other")


# ---------------------------------------------------------------- HGRN2
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("H,nh,dk,dv", [(48, 3, 16, 24), (64, 1, 64, 160), (32, 2, 128, 32), (40, 2, 20, 8), (32, 1, 256, 16), (32, 2, 200, 40)])
def test_hgrn2_alone(H, nh, dk, dv, dt):
    from vllm_oxide_b200.parts import PartSpec, build_part
    eps = 1e-5
    part = build_part("mixer", PartSpec("hgrn2", dict(hidden_size=H, num_heads=nh, dim=dk, vdim=dv, eps=eps, prefix="m.")),
                      positions={}, dtype=dt, device=DEV)
    lower = torch.sigmoid(rand((nh * dk,), 7))
    lower[::2] = 0.995        # every other channel forgets almost nothing: what the first tokens wrote is still there at the end
    w = {"m.q": rand((nh * dk, H), 1, H ** -0.5), "m.f": rand((nh * dk, H), 2, H ** -0.5), "m.v": rand((nh * dv, H), 3, H ** -0.5),
         "m.o": rand((H, nh * dv), 4, (nh * dv) ** -0.5), "m.f.b": rand((nh * dk,), 5), "m.lower": lower,
         "m.norm": 1.0 + 0.1 * rand((dv,), 6)}
    load(part, w, dt)
    wh = {k: (v.float().double() if k in ("m.lower", "m.norm") else held(v, dt)) for k, v in w.items()}
    m = dict(heads=nh, dim=dk, vdim=dv)
    n = 200
    x = held(rand((n, H), 20), dt)
    want = P.hgrn2(x, wh, "m.", m, eps)
    assert (P.hgrn2(x[120:], wh, "m.", m, eps)[-1] - want[-1]).abs().max() > 0.01 * want.abs().max()
    alone = Alone([part], dt, slots=2)
    tol = None if dt == torch.float32 else 0.05
    assert_close(in_portions(alone, 0, x, [n]), want, dt, "whole", tol)
    assert_close(in_portions(alone, 1, x, [n - 40] + [1] * 40), want, dt, "decoded", tol)
    assert_close(in_portions(alone, 0, x, [2, 9, 1, 8, 30]), want, dt, "portions", tol)
    y = held(rand((90, H), 21), dt)
    out = alone.step([(5, y[:60]), (6, x[:31])])[0]
    out2 = alone.step([(6, x[31:32]), (5, y[60:])], end=[5, 6])[0]
    assert_close(torch.cat([out[:60], out2[1:]]), P.hgrn2(y, wh, "m.", m, eps), dt, "beside another request", tol)
    assert_close(torch.cat([out[60:], out2[:1]]), want[:32], dt, "the other request", tol)


# ---------------------------------------------------------------- latent attention
def latent_parts(dt, H, nh, dk, dr, dv, qr, kr, scale, rot, window, reader=None):
    from vllm_oxide_b200.parts import PartSpec, build_part
    positions = {"r": build_part("position", PartSpec("rope", dict(head_dim=dr, rotary_dim=rot["dims"], max_position=1 << 30,
                                                                    theta=rot["base"], interleaved=True, scaling=rot.get("scaling"),
                                                                    table=False)), device=DEV)}
    eps = 1e-6

    def make(prefix, nh, dk, dv, qr, scale, window, borrow, cache_window):
        part = build_part("mixer", PartSpec("latent_attention", dict(
            hidden_size=H, num_heads=nh, dim=dk, rot_dim=dr, vdim=dv, q_rank=qr, kv_rank=kr, scale=scale, eps=eps, window=window,
            cache_window=cache_window, position="r", prefix=prefix, borrow=borrow)), positions=positions, dtype=dt, device=DEV)
        s = 100 if prefix == "a." else 200
        w = {prefix + "dq": rand((qr, H), s + 1, H ** -0.5), prefix + "dq.norm": 1.0 + 0.1 * rand((qr,), s + 2),
             prefix + "uq": rand((nh * (dk + dr), qr), s + 3, qr ** -0.5), prefix + "uk": rand((nh * dk, kr), s + 4, kr ** -0.5),
             prefix + "uv": rand((nh * dv, kr), s + 5, kr ** -0.5), prefix + "o": rand((H, nh * dv), s + 6, (nh * dv) ** -0.5)}
        if not borrow:
            w.update({prefix + "dkv": rand((kr + dr, H), s + 7, H ** -0.5), prefix + "dkv.norm": 1.0 + 0.1 * rand((kr,), s + 8)})
        load(part, w, dt)
        m = dict(heads=nh, dim=dk, rot_dim=dr, vdim=dv, q_rank=qr, kv_rank=kr, scale=scale, rot=rot, mask={"size": window or 1 << 30})
        return part, {k: (v.float().double() if k.endswith("norm") else held(v, dt)) for k, v in w.items()}, m, eps
    keep = max(window, reader["window"]) if reader and window and reader["window"] else (window if not reader else 0)
    own = make("a.", nh, dk, dv, qr, scale, window, False, keep)
    if reader is None:
        return [own]
    return [own, make("b.", reader["nh"], reader["dk"], reader["dv"], reader["qr"], reader["scale"], reader["window"], True, keep)]


def plain_latent(spec, x, kept=None):
    part, w, m, eps = spec
    pos = torch.arange(x.shape[0])
    if kept is None:
        kept = P.latent_keys(x, w, part.prefix, m, eps, pos)
    return P.latent_attention(x, w, part.prefix, m, eps, pos, kept), kept


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("case", ["odd sizes", "a window of one page, cache row of 64", "no window, wide latent", "rotated part wider than rotated dims",
                                  "more heads than the tensor-core kernels take at once"])
def test_latent_attention_alone_with_one_loud_key(case, dt):
    """One token's shared key part is made 60 times larger than the others: for about half of the (query, head) pairs its
    score then drowns all others, so a query that sees it by mistake, or misses it, gives another row altogether."""
    bs = 16
    if case == "odd sizes":
        H, W = 40, 19
        specs = latent_parts(dt, H, 3, 24, 8, 40, 48, 36, 0.2, dict(dims=8, base=1000.0, scaling=dict(factor=4.0, original=32, fast=8.0, slow=1.0)), W,
                             reader=dict(nh=2, dk=16, dv=24, qr=32, scale=0.3, window=33))
    elif case == "a window of one page, cache row of 64":
        H, W, bs = 64, 64, 64
        specs = latent_parts(dt, H, 4, 32, 16, 48, 64, 48, 0.15, dict(dims=16, base=10000.0), W)
    elif case == "no window, wide latent":
        H, W = 64, 0
        specs = latent_parts(dt, H, 2, 64, 32, 64, 128, 96, 0.1, dict(dims=32, base=500.0, scaling=dict(factor=8.0, original=64, fast=4.0, slow=2.0)), None)
    elif case == "more heads than the tensor-core kernels take at once":
        H, W = 64, 40         # 21 heads: a group of 16 and a group of 5 in bfloat16, all at once in 32-bit
        specs = latent_parts(dt, H, 21, 16, 8, 16, 32, 24, 0.25, dict(dims=8, base=300.0), W)
    else:
        H, W = 32, 7
        specs = latent_parts(dt, H, 1, 32, 16, 16, 16, 24, 0.2, dict(dims=8, base=100.0), W)
    n = 210
    x = rand((n, H), 33)
    loud = [0, 15, 16, 31, 100]                  # the first token, both sides of page borders, one in the middle
    for j in loud:
        x[j] *= 60.0
    x = held(x, dt)
    want, kept = plain_latent(specs[0], x)
    wants = [want] + ([plain_latent(specs[1], x, kept)[0]] if len(specs) > 1 else [])
    if W:      # the plain form itself: with a window one token longer, the first query past the loud key gives another row
        part0, w0, m0, eps0 = specs[0]
        longer = plain_latent((part0, w0, dict(m0, mask={"size": W + 1}), eps0), x)[0]
        assert (longer[100 + W] - want[100 + W]).abs().max() > 0.02 * want.abs().max()
    # scores of the loud key run to hundreds: the rounding of a query or a key shows more than among random scores
    tol = 1e-4 if dt == torch.float32 else 0.1
    parts = [s[0] for s in specs]
    plane_of = [0, 0] if len(specs) > 1 else None

    def run(cuts, rid):
        alone_rows, at, k = [[] for _ in parts], 0, 0
        while at < n:
            c = min(cuts[k % len(cuts)], n - at)
            k += 1
            outs = alone.step([(rid, x[at:at + c])], end=[rid] if at + c == n else [], plane_of=plane_of)
            for i, o in enumerate(outs):
                alone_rows[i].append(o)
            at += c
        return [torch.cat(r) for r in alone_rows]
    alone = Alone(parts, dt, block_size=bs, pages=max(8, 4 * (n // bs + 1)), slots=3)
    for cuts, what in (([n], "whole"), ([n - 120] + [1] * 120, "decoded"), ([2, 5, 1, 30, 3], "portions"), ([bs], "pages"), ([1], "alone")):
        for got, wnt, i in zip(run(cuts, 7), wants, range(2)):
            assert_close(got, wnt, dt, f"{case}: {what}, layer {i}", tol)
    # beside another request whose portion is longer, with pages that the runs above have given back
    other = held(rand((150, H), 34), dt)
    o_want = plain_latent(specs[0], other)[0]
    a = alone.step([(1, x[:90]), (2, other[:149])], plane_of=plane_of)[0]
    b = alone.step([(2, other[149:]), (1, x[90:])], end=[1, 2], plane_of=plane_of)[0]
    assert_close(torch.cat([a[:90], b[1:]]), wants[0], dt, f"{case}: beside another request", tol)
    assert_close(torch.cat([a[90:], b[:1]]), o_want, dt, f"{case}: the other request", tol)
