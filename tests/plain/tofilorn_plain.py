"""Plain, slow Tofilorn forward pass: whole sequences, no cache, one function per mechanism.

The oracle for the engine's Tofilorn model.  It shares no code with the package: it reads a model
folder with its own few lines (or takes a dict of tensors), works on one whole sequence at a time and
keeps nothing between calls.  Every function works in the dtype `dt` it is given (float64 for an oracle,
float32 to see what 32-bit rounding does); nothing is rounded below `dt`.

Notation: n tokens, D the model width, S residual streams.  A layer has a token mixer (one of
`mingru`, `latent_attention`, `hgrn2`) and may have a gated feed-forward.  Matrices are [out, in].
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


# ---------------------------------------------------------------- norms
def gain_norm(x, gain, eps):
    """x / sqrt(mean(x^2) + eps) * gain over the last axis; `gain` is one number or a vector."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain


# ---------------------------------------------------------------- rotation
def rotation_frequencies(rot, dt):
    """(frequencies [dims/2], amplitude) of a rotary encoding with an optional long-context correction.

    Base frequencies w_i = base^(-2i/dims).  With `scaling` = {factor, original, fast, slow}: the
    index at which a wave makes t turns over `original` positions is
        d(t) = dims * ln(original / (2 pi t)) / (2 ln base);
    between lo = max(floor(d(fast)), 0) and hi = min(ceil(d(slow)), dims - 1) a ramp r_i goes from 0 to 1
    (clamped, its width at least 0.001); w_i <- w_i / factor * r_i + w_i * (1 - r_i), and cos and sin are both
    multiplied by amplitude = 0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=dt)
    w = torch.as_tensor(base, dtype=dt) ** (-2.0 * i / dims)
    amp = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def index_of(turns):
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(index_of(float(sc["fast"]))), 0)
        hi = min(math.ceil(index_of(float(sc["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        w = w / factor * ramp + w * (1.0 - ramp)
        amp = 0.1 * math.log(factor) + 1.0
    return w, amp


def rotate_pairs(x, pos, w, amp):
    """x [..., n, d]: among the first 2 len(w) elements, neighbours (2i, 2i+1) are turned by the angle pos * w_i and
    scaled by amp; what lies behind them passes unchanged."""
    ang = pos.to(w.dtype)[:, None] * w[None, :]
    c, s = torch.cos(ang) * amp, torch.sin(ang) * amp
    m = 2 * w.shape[0]
    a, b = x[..., 0:m:2], x[..., 1:m:2]
    out = x.clone()
    out[..., 0:m:2] = a * c - b * s
    out[..., 1:m:2] = b * c + a * s
    return out


# ---------------------------------------------------------------- mixers
def mingru(h, W, p):
    """Gated recurrence whose gates see the current token only.  z = sigmoid(Wz h + bz); u = Wx h + bx;
    candidate = u + 1/2 where u >= 0, sigmoid(u) below; s_t = (1 - z) s_{t-1} + z * candidate, s_0 = 0;
    output Wo (s_t * silu(Wg h))."""
    z = torch.sigmoid(h @ W[p + "z"].T + W[p + "z.b"])
    u = h @ W[p + "x"].T + W[p + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    g = h @ W[p + "g"].T
    s = torch.zeros_like(z[0])
    rows = []
    for t in range(h.shape[0]):
        s = (1.0 - z[t]) * s + z[t] * cand[t]
        rows.append(s)
    return (torch.stack(rows) * torch.nn.functional.silu(g)) @ W[p + "o"].T


def hgrn2(h, W, p, m, eps):
    """Linear attention whose forget gate is also its input gate.  Per head: q = silu(Wq h) [dim], v = Wv h [vdim],
    f = l + (1 - l) sigmoid(Wf h + bf) [dim] with the lower bound l; the matrix state M [dim, vdim] goes
    M_t = diag(f_t) M_{t-1} + (1 - f_t) v_t^T, M_0 = 0; o_t = M_t^T q_t, normalised over vdim with a weight shared by
    the heads; heads side by side, then Wo."""
    nh, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    n = h.shape[0]
    q = torch.nn.functional.silu(h @ W[p + "q"].T).reshape(n, nh, dk)
    v = (h @ W[p + "v"].T).reshape(n, nh, dv)
    low = W[p + "lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ W[p + "f"].T + W[p + "f.b"])).reshape(n, nh, dk)
    M = torch.zeros(nh, dk, dv, dtype=h.dtype)
    out = []
    for t in range(n):
        M = f[t][:, :, None] * M + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hkv,hk->hv", M, q[t]))
    o = gain_norm(torch.stack(out), W[p + "norm"], eps)
    return o.reshape(n, nh * dv) @ W[p + "o"].T


def latent_keys(h, W, p, m, eps, pos):
    """What a latent-attention layer keeps of a token: the normalised latent c [kv_rank] and one rotated key part
    [rot_dim] that all heads share."""
    r = int(m["kv_rank"])
    d = h @ W[p + "dkv"].T
    c = gain_norm(d[:, :r], W[p + "dkv.norm"], eps)
    w, amp = rotation_frequencies(m["rot"], h.dtype)
    return c, rotate_pairs(d[:, r:], pos, w, amp)


def latent_attention(h, W, p, m, eps, pos, kept):
    """Attention with keys and values expanded per head from a shared latent.  Queries: cq = norm(Wdq h), q = Wuq cq,
    per head [dim plain | rot_dim rotated].  Per head: plain key Wuk c, value Wuv c; score = (q_plain . k_plain +
    q_rot . k_rot) * scale; position i sees j with 0 <= i - j (< window, if there is one); softmax; Wo on the heads side by side.
    `kept` = (c, k_rot) of this layer or of the layer it borrows from."""
    nh, dk, dr, dv = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"])
    n = h.shape[0]
    cq = gain_norm(h @ W[p + "dq"].T, W[p + "dq.norm"], eps)
    q = (cq @ W[p + "uq"].T).reshape(n, nh, dk + dr)
    w, amp = rotation_frequencies(m["rot"], h.dtype)
    q_rot = rotate_pairs(q[:, :, dk:].transpose(0, 1), pos, w, amp).transpose(0, 1)
    c, k_rot = kept
    k = (c @ W[p + "uk"].T).reshape(n, nh, dk)
    v = (c @ W[p + "uv"].T).reshape(n, nh, dv)
    score = (torch.einsum("ihd,jhd->hij", q[:, :, :dk], k) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * float(m["scale"])
    dist = pos[:, None] - pos[None, :]
    seen = dist >= 0
    if m.get("mask"):
        seen &= dist < int(m["mask"]["size"])
    score = score.masked_fill(~seen[None], float("-inf"))
    o = torch.einsum("hij,jhd->ihd", torch.softmax(score, -1), v)
    return o.reshape(n, nh * dv) @ W[p + "o"].T


def gated_ff(h, W, p):
    return (torch.nn.functional.silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


# ---------------------------------------------------------------- residual streams
def stream_sublayer(X, W, hc, gain, eps, fn):
    """X [S, n, D].  u = sum_s a_s X_s; y = fn(norm(u)); X'_t = sum_s B[s, t] X_s + b_t y  (a = hc.in, b = hc.out,
    B = hc.mix indexed [from, to]); the right-hand side uses the streams as they were before the sublayer."""
    u = torch.einsum("s,snd->nd", W[hc + "in"], X)
    y = fn(gain_norm(u, gain, eps))
    return torch.einsum("st,snd->tnd", W[hc + "mix"], X) + W[hc + "out"][:, None, None] * y[None]


def forward(cfg, weights, tokens, dt=torch.float64):
    """(logits [n, vocab], stream sums after every layer [layers, n, D]) of one sequence."""
    W = {k: (v.to(dt) if v.dtype.is_floating_point else v) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    S = int(cfg.get("streams", 1))
    n = len(tokens)
    pos = torch.arange(n)
    x = W["embed"][torch.as_tensor(tokens)]
    X = x[None].repeat(S, 1, 1)
    kept, sums = {}, []
    for i, layer in enumerate(cfg["layers"]):
        L, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        p = L + "mix."
        if kind == "mingru":
            fn = lambda h: mingru(h, W, p)
        elif kind == "hgrn2":
            fn = lambda h: hgrn2(h, W, p, m, eps)
        elif kind == "latent_attention":
            def fn(h):
                if m.get("kv_from") is None:
                    kept[i] = latent_keys(h, W, p, m, eps, pos)
                    return latent_attention(h, W, p, m, eps, pos, kept[i])
                return latent_attention(h, W, p, m, eps, pos, kept[int(m["kv_from"])])
        else:
            raise ValueError(kind)
        subs = [(L + "hc1.", W[L + "norm1"], fn)]
        if layer.get("mlp") is not None:
            subs.append((L + "hc2.", W[L + "norm2"], lambda h: gated_ff(h, W, L + "mlp.")))
        for hc, gain, f in subs:
            if "streams" in cfg:
                X = stream_sublayer(X, W, hc, gain, eps, f)
            else:
                X = X + f(gain_norm(X[0], gain, eps))[None]
        sums.append(X.sum(0))
    logits = gain_norm(X.sum(0), W["final.norm"], eps) @ W["head"].T
    return logits, torch.stack(sums)
