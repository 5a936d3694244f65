"""Kesozen without a GPU: configuration, plan, random folders, and closed forms of the plain mechanisms."""
import math

import pytest
import torch

from plain import kesozen_plain as P


def _cfg(**kw):
    base = {"architecture": "Kesozen", "vocab": 60, "width": 48, "norm": {"eps": 1e-6}, "layers": [
        {"type": "delta", "mixer": dict(heads=2, kv_heads=1, dim=8, vdim=12, conv=3), "mlp": {"kind": "dense", "ff": 40}},
        {"type": "attention", "mixer": dict(heads=4, kv_heads=2, dim=16, vdim=16, scale=0.3, rot=dict(dims=8, base=100.0)),
         "mlp": {"kind": "moe", "expert": {"ff": 10}, "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}}}},
        {"type": "attention", "mixer": dict(heads=1, kv_heads=1, dim=32, vdim=32, scale=0.1, rot=dict(dims=32, base=10.0)), "mlp": None}]}
    base.update(kw)
    return base


def test_the_plan_runs_a_stretch_again_with_planes_of_its_own():
    from vllm_oxide_b200.models.registry import resolve
    cfg, plan = resolve(_cfg(loop={"start": 1, "stop": 3, "times": 3}))
    assert [(s.layer, s.plane, s.reinject) for s in plan.order] == [
        (0, 0, False), (1, 1, False), (2, 2, False), (1, 3, True), (2, 4, False), (1, 5, True), (2, 6, False)]
    assert all(s.write_cache for s in plan.order) and plan.num_planes() == 7
    assert plan.embedding_norm is not None and plan.embedding_norm.params["weight_name"] == "embed.norm"
    _, plan = resolve(_cfg())
    assert [(s.layer, s.reinject) for s in plan.order] == [(0, False), (1, False), (2, False)]
    _, plan = resolve(_cfg(loop={"start": 0, "stop": 0, "times": 4}))
    assert [s.layer for s in plan.order] == [0, 1, 2]
    assert [i for i, _ in P.layer_runs(_cfg(loop={"start": 1, "stop": 3, "times": 3}))] == [s.layer for s in resolve(_cfg(loop={"start": 1, "stop": 3, "times": 3}))[1].order]


def test_tensor_names_and_state_sizes():
    from vllm_oxide_b200.models.causal_lm import CausalLM
    from vllm_oxide_b200.models.registry import resolve
    _, plan = resolve(_cfg(loop={"start": 0, "stop": 1, "times": 2}))
    model = CausalLM(plan, torch.float32, "cpu")
    shapes = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert shapes["embed.norm"] == (48,) and shapes["final.norm"] == (48,) and shapes["head"] == (60, 48)
    assert shapes["l0.mix.q"] == (8, 48) and shapes["l0.mix.v.conv"] == (24, 3) and shapes["l0.mix.A_log"] == (2,)
    assert shapes["l1.mix.k"] == (32, 48) and shapes["l1.mix.g"] == (4, 48) and "l1.mix.v" not in shapes
    assert shapes["l1.mlp.e5.down"] == (48, 10) and shapes["l1.mlp.router"] == (6, 48) and shapes["l1.mlp.correction"] == (6,)
    assert "l2.norm2" not in shapes and "l2.norm1b" in shapes
    states = model.state_specs()
    assert states[0].shape == (2 * 8 * 12 + 2 * (8 + 8 + 24),) and states[1].shape == states[0].shape and states[2] is None
    specs = model.cache_specs()
    assert specs[0] is None and specs[2].kv_heads == 2 and specs[2].head_dim == 16 and specs[2].tensors == 2


@pytest.mark.parametrize("change,what", [
    (lambda c: c["layers"][1]["mixer"].update(vdim=8), "vdim"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3, kv_heads=2), "multiple"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "choices"),
    (lambda c: c.update(loop={"start": 2, "stop": 1, "times": 2}), "loop"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "kind"),
])
def test_configurations_that_cannot_be_are_refused(change, what):
    from vllm_oxide_b200.config import ConfigError
    from vllm_oxide_b200.models.registry import resolve
    cfg = _cfg()
    change(cfg)
    with pytest.raises(ConfigError, match=what):
        resolve(cfg)


def test_a_random_folder_reads_back(tmp_path):
    from vllm_oxide_b200.engine.loading import write_random_model_folder
    write_random_model_folder(str(tmp_path), _cfg(loop={"start": 0, "stop": 2, "times": 2}), 5, "fan_in", torch.float32)
    cfg, w = P.read_folder(str(tmp_path))
    assert cfg["loop"] == {"start": 0, "stop": 2, "times": 2} and cfg["layers"][1]["mlp"]["router"]["groups"] == {"count": 3, "keep": 2}
    logits, layers = P.forward(cfg, w, [1, 2, 3, 4, 5], torch.float64, return_layers=True)
    assert logits.shape == (5, 60) and layers.shape == (5, 5, 48) and torch.isfinite(logits).all()


# ---------------------------------------------------------------- closed forms of the plain mechanisms
def test_the_delta_rule_overwrites_what_a_key_held():
    """With beta = 1 and no decay, writing a second value under the same key replaces the first: reading with that key
    returns the second value alone."""
    one = torch.ones(3, dtype=torch.float64)
    k = torch.tensor([[1.0, 0.0], [1.0, 0.0], [0.0, 1.0]], dtype=torch.float64)
    v = torch.tensor([[3.0], [5.0], [7.0]], dtype=torch.float64)
    assert P.delta_rule(k, k, v, one, one).flatten().tolist() == [3.0, 5.0, 7.0]
    # a decay of one half a token; the third token writes nothing (beta 0) and reads 3 * 0.5 * 0.5
    out = P.delta_rule(k[[0, 2, 0]], k[[0, 2, 0]], v, torch.tensor([1.0, 1.0, 0.0], dtype=torch.float64), 0.5 * one)
    assert out.flatten().tolist() == [3.0, 5.0, 0.75]


def test_the_short_convolution_ends_on_the_current_token():
    x = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None]
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64)
    assert P.short_conv(x, w).flatten().tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]


def test_the_sink_holds_one_share_of_the_softmax():
    """One token, score s: the weight is e^s / (1 + e^s), so the output is that share of the value times the gate."""
    H = 4
    m = dict(heads=1, kv_heads=1, dim=2, vdim=2, scale=1.0, rot=dict(dims=0, base=1.0))
    w = {"m.q": torch.eye(2, H, dtype=torch.float64), "m.k": torch.eye(2, H, dtype=torch.float64), "m.g": torch.zeros(1, H, dtype=torch.float64),
         "m.o": torch.eye(H, 2, dtype=torch.float64)}
    h = torch.tensor([[1.0, 2.0, 0.0, 0.0]], dtype=torch.float64)
    s = 5.0
    want = 0.5 * math.exp(s) / (1.0 + math.exp(s)) * torch.tensor([1.0, 2.0, 0.0, 0.0], dtype=torch.float64)
    assert torch.allclose(P.sink_attention(h, w, "m.", m, 1e-6, torch.float64)[0], want, atol=1e-12)


def test_rotation_keeps_the_back_of_a_head_and_turns_pairs_half_a_head_apart():
    x = torch.tensor([[[1.0, 0.0, 0.0, 0.0, 9.0, 8.0]]], dtype=torch.float64)
    out = P.rotate_front(x, dict(dims=4, base=100.0), torch.tensor([3]))
    # element 0 pairs with element 2 (frequency 1), element 1 with element 3 (frequency 1/10)
    assert torch.allclose(out[0, 0], torch.tensor([math.cos(3.0), 0.0, math.sin(3.0), 0.0, 9.0, 8.0], dtype=torch.float64), atol=1e-12)
    y = torch.tensor([[[0.0, 1.0, 0.0, 0.0, 0.0, 0.0]]], dtype=torch.float64)
    out = P.rotate_front(y, dict(dims=4, base=100.0), torch.tensor([3]))
    assert torch.allclose(out[0, 0, [1, 3]], torch.tensor([math.cos(0.3), math.sin(0.3)], dtype=torch.float64), atol=1e-12)


def test_the_router_chooses_by_corrected_scores_within_the_best_groups_and_weighs_by_plain_scores():
    H = 4
    h = torch.tensor([[1.0, 0.0, 0.0, 0.0]], dtype=torch.float64)
    logits = torch.tensor([2.0, 0.0, 1.0, 1.5, -1.0, 0.5], dtype=torch.float64)
    w = {"f.router": torch.cat([logits[:, None], torch.zeros(6, H - 1, dtype=torch.float64)], 1),
         "f.correction": torch.tensor([-1.0, 0.0, 0.0, 0.0, 0.9, 0.0], dtype=torch.float64)}
    s = torch.softmax(logits, -1)
    # groups (0,1) (2,3) (4,5): best corrected scores s3 (group 1) and s4 + 0.9 (group 2) win over group 0, whose best is s1
    idx, weight = P.route(h, w, "f.", dict(experts=6, top=3, groups=dict(count=3, keep=2)), torch.float64)
    assert idx[0].tolist() == [4, 3, 2]
    assert torch.allclose(weight[0], s[[4, 3, 2]])
    # without groups expert 0 still loses to its correction
    idx, _ = P.route(h, w, "f.", dict(experts=6, top=2), torch.float64)
    assert idx[0].tolist() == [4, 3]
