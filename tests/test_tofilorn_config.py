"""Tofilorn's configuration and plan, and closed forms of its plain mechanisms (no device needed)."""
import math

import pytest
import torch

from plain import tofilorn_plain as P


def _config(**kw):
    base = {"architecture": "Tofilorn", "vocab": 50, "width": 32, "streams": 2, "norm": {"eps": 1e-5}, "layers": [
        {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 48},
         "mixer": {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 12, "q_rank": 16, "kv_rank": 10, "scale": 0.3, "mask": {"size": 9},
                   "rot": {"dims": 4, "base": 100.0}}},
        {"type": "mingru", "mixer": {"width": 24}, "mlp": None},
        {"type": "hgrn2", "mixer": {"heads": 2, "dim": 8, "vdim": 6}, "mlp": None},
        {"type": "latent_attention", "mlp": None,
         "mixer": {"heads": 1, "dim": 4, "rot_dim": 4, "vdim": 8, "q_rank": 8, "kv_rank": 10, "scale": 0.5, "mask": {"size": 21},
                   "kv_from": 0, "rot": {"dims": 4, "base": 100.0}}}]}
    base.update(kw)
    return base


def test_plan_planes_windows_and_tensors():
    from vllm_oxide_b200.models import CausalLM, resolve
    cfg, plan = resolve(_config())
    assert plan.architecture == "Tofilorn" and plan.hidden_size == 32 and plan.vocab_size == 50
    assert [(s.layer, s.plane, s.write_cache) for s in plan.order] == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 0, False)]
    model = CausalLM(plan, torch.float32, "cpu")
    specs = model.cache_specs()
    # the plane keeps what its reader needs (21), though its own layer looks back 9; rows of 14 elements padded to 16
    assert specs[0].window == 21 and specs[0].head_dim == 16 and specs[0].tensors == 1 and specs[0].kv_heads == 1
    assert len(specs) == 3 and specs[1] is None and specs[2] is None      # the reader has no plane of its own
    states = model.state_specs()
    assert states[0] is None and states[1].shape == (24,) and states[2].shape == (2, 8, 6)
    names = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert names["l0.norm1"] == () and names["final.norm"] == () and names["l0.hc2.mix"] == (2, 2) and names["l1.hc1.in"] == (2,)
    assert names["l0.mix.dkv"] == (14, 32) and "l3.mix.dkv" not in names and names["l3.mix.uk"] == (4, 10)
    assert names["l0.mlp.gate"] == (48, 32) and "l1.hc2.in" not in names and names["head"] == (50, 32)


def test_one_plain_stream_needs_no_coefficients():
    from vllm_oxide_b200.models import CausalLM, resolve
    c = _config()
    del c["streams"]
    _, plan = resolve(c)
    names = {s.name for s in CausalLM(plan, torch.float32, "cpu").tensor_specs()}
    assert not any(".hc" in n for n in names)


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="mamba"), "type"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_rank=12), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "mlp"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_bad_configurations_are_named(change, word):
    from vllm_oxide_b200.config.model_config import ConfigError
    from vllm_oxide_b200.models import resolve
    c = _config()
    change(c)
    with pytest.raises(ConfigError, match=word):
        resolve(c)


def test_random_model_folder_round_trip(tmp_path):
    """A written random folder is what the plain reader reads, with tame coefficients."""
    from vllm_oxide_b200.engine.loading import write_random_model_folder
    write_random_model_folder(str(tmp_path), _config(), 3, "fan_in", torch.float32)
    cfg, w = P.read_folder(str(tmp_path))
    assert cfg["architecture"] == "Tofilorn" and cfg["layers"][3]["mixer"]["kv_from"] == 0
    assert w["l0.norm1"].shape == () and 0 < float(w["l2.mix.lower"].min()) and float(w["l2.mix.lower"].max()) < 1
    assert (w["l0.hc1.mix"] - torch.eye(2)).abs().max() < 0.5
    logits, sums = P.forward(cfg, w, [1, 2, 3, 4, 5], torch.float64)
    assert logits.shape == (5, 50) and sums.shape == (4, 5, 32) and torch.isfinite(logits).all()


# ---------------------------------------------------------------- closed forms of the plain mechanisms
def test_plain_mingru_with_constant_gates():
    """Zero matrices leave the biases: z and the candidate are constants, and s_t = c (1 - (1 - z)^t)."""
    W, H, n = 3, 4, 6
    w = {"m.z": torch.zeros(W, H), "m.x": torch.zeros(W, H), "m.g": torch.zeros(W, H), "m.o": torch.eye(H, W),
         "m.z.b": torch.tensor([0.0, 1.0, -2.0]), "m.x.b": torch.tensor([1.0, -1.0, 0.0])}
    w = {k: v.double() for k, v in w.items()}
    w["m.g"][:, 0] = 1.0
    h = torch.zeros(n, H, dtype=torch.float64)
    h[:, 0] = 2.0          # output gate: silu(2) for every channel
    out = P.mingru(h, w, "m.")
    z = torch.sigmoid(w["m.z.b"])
    cand = torch.tensor([1.5, 1 / (1 + math.e), 0.5], dtype=torch.float64)
    t = torch.arange(1, n + 1, dtype=torch.float64)[:, None]
    want = cand * (1 - (1 - z) ** t) * (2.0 / (1 + math.exp(-2.0)))
    assert torch.allclose(out[:, :W], want, atol=1e-12)


def test_plain_hgrn2_keeps_what_the_gate_does_not_forget():
    """With the lower bound 1 the state never changes (f = 1 writes nothing): the output is the norm of zero, zero."""
    H, nh, dk, dv = 4, 1, 2, 3
    w = {"m.q": torch.ones(dk, H), "m.f": torch.zeros(dk, H), "m.f.b": torch.zeros(dk), "m.lower": torch.ones(dk),
         "m.v": torch.ones(dv, H), "m.norm": torch.ones(dv), "m.o": torch.ones(H, dv)}
    w = {k: v.double() for k, v in w.items()}
    out = P.hgrn2(torch.ones(5, H, dtype=torch.float64), w, "m.", dict(heads=nh, dim=dk, vdim=dv), 1e-5)
    assert out.abs().max() == 0
    # lower bound 0 and a zero gate matrix: f = 1/2, M_t = (1 - 2^-t) v per row, the norm takes the size away
    w["m.lower"] = torch.zeros(dk, dtype=torch.float64)
    out = P.hgrn2(torch.ones(3, H, dtype=torch.float64), w, "m.", dict(heads=nh, dim=dk, vdim=dv), 0.0)
    assert torch.allclose(out, torch.full((3, H), 3.0, dtype=torch.float64), atol=1e-12)


def test_plain_rotation_turns_and_scales():
    w, amp = P.rotation_frequencies({"dims": 4, "base": 100.0, "scaling": {"factor": math.e, "original": 8, "fast": 4.0, "slow": 1.0}}, torch.float64)
    assert abs(amp - 1.1) < 1e-12
    x = torch.tensor([[1.0, 0.0, 0.0, 2.0]], dtype=torch.float64).repeat(3, 1)
    y = P.rotate_pairs(x, torch.arange(3), w, amp)
    assert torch.allclose((y[:, :2] ** 2).sum(-1), torch.full((3,), amp ** 2, dtype=torch.float64))
    assert torch.allclose(y[1, 0], amp * torch.cos(w[0])) and torch.allclose(y[1, 2], -2 * amp * torch.sin(w[1]))


def test_plain_stream_sublayer_is_the_plain_sum_for_one_stream():
    X = torch.randn(1, 4, 8, dtype=torch.float64)
    W = {"h.in": torch.ones(1, dtype=torch.float64), "h.out": torch.ones(1, dtype=torch.float64), "h.mix": torch.ones(1, 1, dtype=torch.float64)}
    f = lambda h: 2.0 * h
    out = P.stream_sublayer(X, W, "h.", torch.tensor(1.5, dtype=torch.float64), 1e-6, f)
    assert torch.allclose(out[0], X[0] + 2.0 * P.gain_norm(X[0], 1.5, 1e-6))
