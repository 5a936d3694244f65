"""Tofilorn: config.json -> plan.

The layers come one by one from the configuration, each a `streams` block (several float residual streams with
learned mixing, parts/streams.py) around one of three mixers: `mingru` and `hgrn2` (parts/recurrent.py, state in slots)
and `latent_attention` (parts/latent_attention.py, one latent row a token in windowed pages, rotation with stretched
frequencies computed from the position), and an optional gated feed-forward (the stock `swiglu`).  Norms have one
learned gain.  Tensors are named l<i>.norm1, l<i>.mix.<name>, l<i>.mlp.<name>, l<i>.hc<q>.in|out|mix, embed,
final.norm, head.

Cache planes are numbered like the layers.  A latent-attention layer with `kv_from: j` has no keys of its own: its
run reads plane j (`write_cache=False`), and plane j keeps the largest window among its readers and itself.
"""
from __future__ import annotations

from ..config.model_config import TofilornConfig
from ..parts.base import PartSpec
from .plan import ExecStep, ModelPlan

NO_POSITION_LIMIT = 1 << 30     # angles are computed from the position: nothing but int32 bounds it


def tofilorn_plan(cfg: TofilornConfig) -> ModelPlan:
    D, S = cfg.width, cfg.streams
    window = lambda m: int(m["mask"]["size"]) if m.get("mask") else 0
    # the window that every plane must keep: its own layer's and its readers' (0: all keys)
    keep = {}
    for i, layer in enumerate(cfg.layers):
        if layer.type == "latent_attention":
            j = layer.mixer.get("kv_from")
            j = i if j is None else int(j)
            w = window(layer.mixer)
            keep[j] = w if j not in keep else (0 if 0 in (w, keep[j]) else max(w, keep[j]))
    layers, order, positions = [], [], {}
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        plane, writes = i, True
        if layer.type == "mingru":
            mixer = PartSpec("mingru", dict(hidden_size=D, width=int(m["width"]), prefix=p + "mix."))
        elif layer.type == "hgrn2":
            mixer = PartSpec("hgrn2", dict(hidden_size=D, num_heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                                           eps=cfg.eps, prefix=p + "mix."))
        else:
            rot = m["rot"]
            positions[p + "rot"] = PartSpec("rope", dict(head_dim=int(m["rot_dim"]), rotary_dim=int(rot["dims"]),
                                                         max_position=NO_POSITION_LIMIT, theta=float(rot["base"]),
                                                         interleaved=True, scaling=rot.get("scaling"), table=False))
            src = m.get("kv_from")
            if src is not None:
                plane, writes = int(src), False
            mixer = PartSpec("latent_attention", dict(
                hidden_size=D, num_heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=int(m["rot_dim"]), vdim=int(m["vdim"]),
                q_rank=int(m["q_rank"]), kv_rank=int(m["kv_rank"]), scale=float(m["scale"]), eps=cfg.eps,
                window=window(m) or None, cache_window=keep[plane], position=p + "rot", prefix=p + "mix.", borrow=not writes))
        ff = None
        if layer.ff is not None:
            ff = PartSpec("swiglu", dict(hidden_size=D, intermediate_size=layer.ff, prefix=p + "mlp.",
                                         names=("gate", "up", "down")))
        gain = lambda name: PartSpec("rmsnorm_gain", dict(size=D, eps=cfg.eps, weight_name=name, streams=S or 1))
        layers.append(PartSpec("streams", dict(
            mixer=mixer, feed_forward=ff, input_norm=gain(p + "norm1"), post_mixer_norm=gain(p + "norm2") if ff else None,
            streams=S or 1, size=D, mixer_coefficients=p + "hc1." if S else None,
            feed_forward_coefficients=p + "hc2." if S and ff else None)))
        order.append(ExecStep(i, plane, writes))
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=D, vocab_size=cfg.vocab, max_position=NO_POSITION_LIMIT,
        embedding_name="embed", lm_head_name="head",
        final_norm=PartSpec("rmsnorm_gain", dict(size=D, eps=cfg.eps, weight_name="final.norm", streams=S or 1)),
        positions=positions, layers=layers, order=order, eos_token_id=None, default_dtype=cfg.torch_dtype)
