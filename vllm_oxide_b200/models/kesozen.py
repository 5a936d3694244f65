"""Kesozen: config.json -> plan.

The layers come one by one from the configuration, each a `sandwich` block (one float residual stream, a norm before
and after each sublayer, parts/sandwich.py) around one of two mixers: `attention_shared_kv` (parts/attention.py: the
keys double as values, a sink in the softmax, a gate per head, the front of each head rotated by angles computed from
the position) and `gated_delta` (parts/delta.py: a matrix state per head behind short convolutions, state in slots);
the feed-forward is `relu2_mlp`, `routed_experts` (parts/moe.py) or absent.  The embedded tokens pass a norm of their own
before the first layer.  Tensors are named embed, embed.norm, l<i>.norm1|norm1b|norm2|norm2b, l<i>.mix.<name>,
l<i>.mlp.<name>, final.norm, head.

`loop` = {start, stop, times}: layers start..stop-1 run `times` times in a row with the same weights.  Every run of a
layer is an `ExecStep` with a cache plane (or state) of its own, numbered in running order; the first run of every pass
but the first has `reinject`: the normed embedding is added to the stream right before it.
"""
from __future__ import annotations

from ..config.model_config import KesozenConfig
from ..parts.base import PartSpec
from .plan import ExecStep, ModelPlan

NO_POSITION_LIMIT = 1 << 30     # angles are computed from the position: nothing but int32 bounds it


def kesozen_plan(cfg: KesozenConfig) -> ModelPlan:
    D = cfg.width
    norm = lambda name: PartSpec("rmsnorm_stream", dict(size=D, eps=cfg.eps, weight_name=name))
    layers, positions = [], {}
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if layer.type == "attention":
            rot, position = m.get("rot"), None
            if rot and int(rot["dims"]) > 0:
                position = p + "rot"
                positions[position] = PartSpec("rope", dict(head_dim=int(m["dim"]), rotary_dim=int(rot["dims"]),
                                                            max_position=NO_POSITION_LIMIT, theta=float(rot["base"]),
                                                            interleaved=False, table=False))
            mixer = PartSpec("attention_shared_kv", dict(hidden_size=D, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]),
                                                         head_dim=int(m["dim"]), scale=float(m["scale"]), sink=True, gate=True,
                                                         position=position, prefix=p + "mix."))
        else:
            mixer = PartSpec("gated_delta", dict(hidden_size=D, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]),
                                                 dim=int(m["dim"]), vdim=int(m["vdim"]), taps=int(m["conv"]), eps=cfg.eps,
                                                 prefix=p + "mix."))
        ff, mlp = None, layer.mlp
        if mlp is not None and mlp["kind"] == "dense":
            ff = PartSpec("relu2_mlp", dict(hidden_size=D, intermediate_size=int(mlp["ff"]), prefix=p + "mlp."))
        elif mlp is not None:
            r = mlp["router"]
            g = r.get("groups") or {"count": 1, "keep": 1}
            ff = PartSpec("routed_experts", dict(hidden_size=D, expert_size=int(mlp["expert"]["ff"]), experts=int(r["experts"]),
                                                 top=int(r["top"]), groups=int(g["count"]), keep=int(g["keep"]), prefix=p + "mlp."))
        layers.append(PartSpec("sandwich", dict(
            mixer=mixer, feed_forward=ff, pre_mixer_norm=norm(p + "norm1"), post_mixer_norm=norm(p + "norm1b"),
            pre_ff_norm=norm(p + "norm2") if ff else None, post_ff_norm=norm(p + "norm2b") if ff else None, size=D)))
    order = [ExecStep(layer, plane, True, reinject=again) for plane, (layer, again) in enumerate(cfg.runs())]
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=D, vocab_size=cfg.vocab, max_position=NO_POSITION_LIMIT,
        embedding_name="embed", lm_head_name="head", final_norm=norm("final.norm"), positions=positions, layers=layers,
        order=order, eos_token_id=None, default_dtype=cfg.torch_dtype, embedding_norm=norm("embed.norm"))
