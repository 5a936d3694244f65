"""Plain, slow Kesozen forward pass: whole sequences, no cache, one function per mechanism.

The oracle for the engine's Kesozen model.  It shares no code with the package: it reads a model folder with
its own few lines (or takes a dict of tensors), works on one whole sequence at a time and keeps nothing between
calls.  Every function works in the dtype `dt` it is given (float64 for an oracle); nothing is rounded below `dt`.

Notation: n tokens, D the model width.  A layer is  x += post1(mixer(pre1(x)));  x += post2(ff(pre2(x)))  with four
vector-weight RMS norms; the mixer is `attention` (keys double as values, a sink in the softmax, a gate per head) or
`delta` (a gated delta rule over a matrix state, behind short convolutions); the feed-forward is dense or a mixture
of experts, both with the squared relu.  A stretch of layers may run several times with the same weights.
"""
import json
import math
import struct

import torch

_ST = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
       "I32": torch.int32, "I64": torch.int64}


def read_folder(path):
    with open(f"{path}/config.json") as f:
        cfg = json.load(f)
    with open(f"{path}/model.safetensors", "rb") as f:
        blob = f.read()
    (n,) = struct.unpack("<Q", blob[:8])
    head = json.loads(blob[8:8 + n])
    out = {}
    for name, meta in head.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        t = torch.frombuffer(bytearray(blob[8 + n + a:8 + n + b]), dtype=_ST[meta["dtype"]])
        out[name] = t.reshape(meta["shape"]).clone()
    return cfg, out


# ---------------------------------------------------------------- small functions
def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(x):
    return x / (1.0 + torch.exp(-x))


def softplus(x):
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def relu_squared(x):
    return torch.clamp(x, min=0.0) ** 2


# ---------------------------------------------------------------- rotation
def rotate_front(x, rot, positions):
    """x [n, heads, dim]: the first rot.dims elements of every head turn, element i with element i + dims/2, by the
    angle position * base^(-2i/dims); the rest pass."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = torch.as_tensor(base, dtype=x.dtype) ** (-2.0 * i / dims)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------- mixers
def sink_attention(h, w, p, m, eps, dt):
    """Causal attention whose values are the keys as projected (before the rotation), whose softmax has a silent extra
    entry of score 0 (weights exp(s) / (1 + sum exp(s))), and whose heads are each scaled by a sigmoid gate."""
    n = h.shape[0]
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = (h @ w[p + "q"].to(dt).T).reshape(n, H, d)
    k = (h @ w[p + "k"].to(dt).T).reshape(n, G, d)
    gate = torch.sigmoid(h @ w[p + "g"].to(dt).T)                      # [n, H]
    v = k
    pos = torch.arange(n)
    q, kr = rotate_front(q, m["rot"], pos), rotate_front(k, m["rot"], pos)
    out = torch.zeros(n, H, d, dtype=dt)
    causal = pos[None, :] <= pos[:, None]
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ kr[:, g].T) * float(m["scale"])
        s = torch.where(causal, s, torch.full_like(s, -math.inf))
        top = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
        e = torch.exp(s - top)
        prob = e / (torch.exp(-top) + e.sum(-1, keepdim=True))
        out[:, head] = (prob @ v[:, g]) * gate[:, head:head + 1]
    return out.reshape(n, H * d) @ w[p + "o"].to(dt).T


def short_conv(x, taps_w):
    """x [n, C], taps_w [C, taps]: y_t = sum_j taps_w[:, j] * x_{t - (taps - 1) + j}, zeros before the start."""
    n, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + padded[j:j + n] * taps_w[:, j][None, :]
    return y


def delta_rule(q, k, v, beta, decay):
    """One head.  q, k [n, d], v [n, e], beta, decay [n].  S <- decay S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    n, d = q.shape
    S = torch.zeros(d, v.shape[1], dtype=q.dtype)
    out = torch.zeros_like(v)
    for t in range(n):
        S = decay[t] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def delta_mixer(h, w, p, m, eps, dt):
    n = h.shape[0]
    H, G, d, e = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    lin = lambda name: h @ w[p + name].to(dt).T
    q = silu(short_conv(lin("q"), w[p + "q.conv"].to(dt))).reshape(n, G, d)
    k = silu(short_conv(lin("k"), w[p + "k.conv"].to(dt))).reshape(n, G, d)
    v = silu(short_conv(lin("v"), w[p + "v.conv"].to(dt))).reshape(n, H, e)
    unit = lambda x: x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)
    q, k = unit(q) * d ** -0.5, unit(k)
    beta = torch.sigmoid(lin("b"))                                                            # [n, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"].to(dt)) * softplus(lin("a") + w[p + "dt_bias"].to(dt)))   # [n, H]
    out_gate = silu(lin("g")).reshape(n, H, e)
    o = torch.zeros(n, H, e, dtype=dt)
    for head in range(H):
        g = head // (H // G)
        o[:, head] = delta_rule(q[:, g], k[:, g], v[:, head], beta[:, head], decay[:, head])
    o = rms_norm(o, w[p + "norm"].to(dt), eps) * out_gate
    return o.reshape(n, H * e) @ w[p + "o"].to(dt).T


# ---------------------------------------------------------------- feed-forwards
def dense_ff(h, w, p, dt):
    return relu_squared(h @ w[p + "up"].to(dt).T) @ w[p + "down"].to(dt).T


def route(h, w, p, r, dt, margins=None):
    """(chosen experts [n, top], their weights [n, top]).  Scores are a softmax over all experts; the choice is by score
    plus a correction, among the experts of the `keep` groups whose best choice score is largest; the weights are the
    plain scores of the chosen, as they are.  `margins` (a list): a tensor [n] is appended, how far each token's choice
    was from falling otherwise: the gap between the last group or expert taken and the first one left, as a share of
    the two's plain scores times the spread of the token's logits."""
    E, top = int(r["experts"]), int(r["top"])
    groups = r.get("groups") or {"count": 1, "keep": 1}
    count, keep = int(groups["count"]), int(groups["keep"])
    z = h @ w[p + "router"].to(dt).T
    s = torch.softmax(z, dim=-1)
    choice = choice_all = s + w[p + "correction"].to(dt)
    best = choice.reshape(-1, count, E // count).max(-1).values                     # [n, count]
    kept = torch.zeros_like(best, dtype=torch.bool)
    kept.scatter_(1, best.topk(keep, dim=-1).indices, True)
    allowed = kept[:, :, None].expand(-1, -1, E // count).reshape(-1, E)
    choice = torch.where(allowed, choice, torch.full_like(choice, -math.inf))
    idx = choice.topk(top, dim=-1).indices
    if margins is not None:
        # rounding moves a logit by a share of the logits' size, and a score by that times itself: the gap is measured
        # against the two scores on either side of it times the spread of the token's logits
        n = h.shape[0]
        ratio = torch.full((n,), math.inf, dtype=dt)
        spread = z.std(-1) if E > 1 else torch.ones(n, dtype=dt)
        if keep < count:
            per = E // count
            first = choice_all.reshape(n, count, per).argmax(-1) + torch.arange(count) * per       # each group's best expert
            order = best.argsort(-1, descending=True)
            a, b = order[:, keep - 1:keep], order[:, keep:keep + 1]
            gap = (best.gather(1, a) - best.gather(1, b))[:, 0]
            ratio = torch.minimum(ratio, gap / ((s.gather(1, first.gather(1, a)) + s.gather(1, first.gather(1, b)))[:, 0] * spread))
        if top < (E // count) * keep:
            order = choice.argsort(-1, descending=True)
            a, b = order[:, top - 1:top], order[:, top:top + 1]
            gap = (choice.gather(1, a) - choice.gather(1, b))[:, 0]
            ratio = torch.minimum(ratio, gap / ((s.gather(1, a) + s.gather(1, b))[:, 0] * spread))
        margins.append(ratio)
    return idx, s.gather(1, idx)


def moe_ff(h, w, p, mlp, dt, margins=None):
    idx, weight = route(h, w, p, mlp["router"], dt, margins)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            y = relu_squared(h[t] @ w[f"{p}e{e}.up"].to(dt).T) @ w[f"{p}e{e}.down"].to(dt).T
            out[t] = out[t] + weight[t, j] * y
    return out


# ---------------------------------------------------------------- the model
def layer_runs(cfg):
    """The layers in the order they run: a stretch start..stop-1 may repeat; (layer, first of a later pass)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, False) for i in range(a)]
    for rep in range(times):
        runs += [(i, rep > 0 and i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n)]


def forward(cfg, w, tokens, dt=torch.float64, return_layers=False, margins=None, noise=None):
    """Logits [n, vocab] for one whole sequence; with `return_layers` also the residual stream after every layer run.
    `margins` (a list): every run of a routed feed-forward appends its tokens' margins (see `route`).  `noise` (a
    function of a tensor): applied to what every sublayer reads and returns, e.g. a rounding to 16 bits, to see how far
    rounding alone moves a row."""
    eps = float(cfg["norm"]["eps"])
    noise = noise or (lambda t: t)
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = rms_norm(w["embed"].to(dt)[ids], w["embed.norm"].to(dt), eps)
    embedded = x
    after = []
    for i, again in layer_runs(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        if again:
            x = x + embedded
        h = noise(rms_norm(x, w[p + "norm1"].to(dt), eps))
        mix = sink_attention if layer["type"] == "attention" else delta_mixer
        x = x + rms_norm(noise(mix(h, w, p + "mix.", layer["mixer"], eps, dt)), w[p + "norm1b"].to(dt), eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = noise(rms_norm(x, w[p + "norm2"].to(dt), eps))
            y = dense_ff(h, w, p + "mlp.", dt) if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp, dt, margins)
            x = x + rms_norm(noise(y), w[p + "norm2b"].to(dt), eps)
        after.append(x)
    logits = noise(rms_norm(x, w["final.norm"].to(dt), eps)) @ w["head"].to(dt).T
    return (logits, torch.stack(after)) if return_layers else logits
