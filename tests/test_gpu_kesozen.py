"""Kesozen through the engine against the plain implementation (tests/plain/kesozen_plain.py): whole prompts, decoding
token by token, portions down to two tokens, unequal requests in one batch over pages and state slots that are used
again, long decoding across page borders, the first tokens, greedy generation through `LLM` and the replay program
itself.  The configurations are made here; they differ from each other in every size."""
import json
import os
import random
import subprocess

import numpy as np
import pytest
import torch

from conftest import ROOT
from plain import kesozen_plain as P

pytestmark = pytest.mark.gpu


def _attention(heads, kv_heads, dim, scale, rot_dims, base):
    return {"type": "attention", "mixer": dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale,
                                               rot=dict(dims=rot_dims, base=base))}


def _delta(heads, kv_heads, dim, vdim, conv):
    return {"type": "delta", "mixer": dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv)}


def _dense(layer, ff):
    return dict(layer, mlp={"kind": "dense", "ff": ff})


def _moe(layer, ff, experts, top, count=None, keep=None):
    router = {"experts": experts, "top": top}
    if count:
        router["groups"] = {"count": count, "keep": keep}
    return dict(layer, mlp={"kind": "moe", "expert": {"ff": ff}, "router": router})


def _none(layer):
    return dict(layer, mlp=None)


CONFIGS = {
    # the first two layers run three times; a layer without a feed-forward; three value heads a key head; groups of two
    "P": dict(block_size=16, config={
        "architecture": "Kesozen", "vocab": 211, "width": 96, "norm": {"eps": 1e-6}, "loop": {"start": 0, "stop": 2, "times": 3},
        "layers": [_dense(_delta(3, 3, 16, 24, 3), 160), _moe(_attention(6, 2, 48, 0.2, 16, 1000.0), 40, 8, 2, 4, 2),
                   _none(_attention(2, 2, 32, 0.3, 32, 50000.0))]}),
    # no loop; widths in multiples of 64; one key head for four; experts without groups; two delta layers in a row, the
    # second with a matrix state of 128 rows
    "Q": dict(block_size=64, config={
        "architecture": "Kesozen", "vocab": 384, "width": 128, "norm": {"eps": 1e-5},
        "layers": [_moe(_attention(4, 1, 64, 0.125, 32, 10000.0), 64, 6, 3), _none(_delta(4, 2, 64, 32, 4)),
                   _dense(_delta(2, 2, 128, 64, 2), 192), _dense(_attention(2, 2, 128, 0.09, 64, 500000.0), 128)]}),
    # one head; nothing rotated in the first layer; a filter of one tap; every expert a group of its own; the loop runs to the
    # last layer
    "R": dict(block_size=32, config={
        "architecture": "Kesozen", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "loop": {"start": 1, "stop": 3, "times": 2},
        "layers": [_moe(_attention(1, 1, 64, 0.15, 0, 100.0), 48, 5, 2, 5, 3), _dense(_delta(1, 1, 32, 16, 1), 64),
                   _moe(_delta(4, 1, 24, 40, 5), 33, 4, 1, 2, 1)]}),
}
NAMES = sorted(CONFIGS)
DTYPES = ["float32", "bfloat16"]
KEPT_FLOAT = ("norm", ".conv", "A_log", "dt_bias", "router", "correction")


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: random_folders(tmp_path_factory.mktemp(f"kesozen_{name}"), spec["config"], 31 + k)
            for k, (name, spec) in enumerate(sorted(CONFIGS.items()))}


_models, _truth = {}, {}


def tokens_for(name, n, salt=0):
    g = torch.Generator().manual_seed(6007 * (NAMES.index(name) + 1) + salt)
    return torch.randint(0, CONFIGS[name]["config"]["vocab"], (n,), generator=g).tolist()


def as_held(w, dtype):
    """The weights as the engine holds them: matrices rounded to bfloat16 on that path; norms, filters, rates, the router and
    its corrections stay float."""
    if dtype == "float32":
        return w
    return {k: (v if any(s in k for s in KEPT_FLOAT) or not v.dtype.is_floating_point else v.to(torch.bfloat16).to(v.dtype))
            for k, v in w.items()}


CLOSE_CALL = 0.05     # a router's choice that logits moved by a twentieth of their spread would turn over is not held against bfloat16


class Rows(np.ndarray):
    """Logits with, per row, whether some router's choice there was a close call (`unsure`) and how far rounding what the
    sublayers read and return to 16 bits moves the row, as a share of its spread (`moved`)."""


def to_16_bits(t):
    return t.to(torch.bfloat16).to(t.dtype)


def plain_logits(cfg, w, tokens):
    margins = []
    exact = P.forward(cfg, w, tokens, torch.float64, margins=margins).numpy()
    out = exact.view(Rows)
    out.unsure = (torch.stack(margins).min(0).values.numpy() < CLOSE_CALL) if margins else np.zeros(len(tokens), bool)
    rounded = P.forward(cfg, w, tokens, torch.float64, noise=to_16_bits).numpy()
    out.moved = np.sqrt(((rounded - exact) ** 2).mean(-1)) / exact.std(-1)
    return out


# A random router's scores lie close together.  Rounding to bfloat16 then turns a choice over every few dozen tokens, the
# other expert's output goes into keys and states that every later token reads, and a comparison row by row would mostly
# learn which expert rounding happened to favour.  So the two precisions get folders of their own, equal but for the
# routers' matrices: times five for the 32-bit runs (choices that differ from token to token, held exactly), times 0.02
# for bfloat16 (the corrections decide, nearly alike for every token; what is held there is the arithmetic in 16 bits:
# products, gathers, the attention kernels).  tests/test_gpu_kesozen_parts.py routes varied tokens in bfloat16 too, on
# inputs that both sides share.
ROUTER_FACTOR = {"float32": 5.0, "bfloat16": 0.02}


def scale_routers(folder, factor):
    from vllm_oxide_b200.weights.safetensors_io import write_safetensors
    _, w = P.read_folder(folder)
    write_safetensors(os.path.join(folder, "model.safetensors"), {k: (factor * v if k.endswith("router") else v) for k, v in w.items()})


def random_folders(folder, config, seed):
    """{dtype: folder} of one random model."""
    from vllm_oxide_b200.engine.loading import write_random_model_folder
    out = {}
    for dtype, factor in ROUTER_FACTOR.items():
        out[dtype] = os.path.join(str(folder), dtype)
        write_random_model_folder(out[dtype], config, seed, "fan_in", torch.float32)
        scale_routers(out[dtype], factor)
    return out


def truth(folders, name, tokens, dtype):
    key = (name, tuple(tokens), dtype)
    if key not in _truth:
        if (name, dtype) not in _models:
            cfg, w = P.read_folder(folders[name][dtype])
            _models[(name, dtype)] = (cfg, as_held(w, dtype))
        _truth[key] = plain_logits(*_models[(name, dtype)], tokens)
    return _truth[key]


def close(got, want, dtype, what):
    """float32: within 1e-4 of the logits' spread, row by row (rounding alone stays near 1e-6; a wrong key, gate, expert or
    state moves a row by percents).  bfloat16: within 0.1 of it (rounding at every operation gives about 0.01 to 0.03 in
    models this small), wider where the plain run itself moves when its sublayers round to 16 bits, and except for
    rows where the plain run says that a router's choice was a close call: bfloat16 may take the other expert there,
    which is another row altogether."""
    unsure, moved = getattr(want, "unsure", None), getattr(want, "moved", None)
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, what
    d = got - want
    err = np.sqrt((d ** 2).mean(-1)) / want.std(-1)
    if dtype == "float32":
        assert err.max() < 1e-4, f"{what}: row {int(err.argmax())} is {err.max():.3e} of the spread off"
        return
    sure = np.ones(len(err), bool) if unsure is None or len(unsure) != len(err) else ~unsure
    # a sublayer whose output is small against its rounding comes out of the norm behind it turned around: such a row
    # is held only as far as the plain run holds when its own sublayers round to 16 bits
    bound = 0.1 + 5.0 * moved if moved is not None and len(moved) == len(err) else np.full(len(err), 0.1)
    worst = np.where(sure, err / bound, 0.0)
    assert worst.max() < 1.0, f"{what}: row {int(worst.argmax())} is {err[worst.argmax()]:.3e} of the spread off"
    if len(err) >= 8:
        assert np.median(err) < 0.04, f"{what}: half of the rows are more than {np.median(err):.3e} of the spread off"
        assert np.median(bound) < 0.3, f"{what}: the plain run itself does not hold under rounding"


def pick(rows, which):
    out = np.asarray(rows)[which].view(Rows)
    out.unsure, out.moved = rows.unsure[which], rows.moved[which]
    return out


def runner(folders, name, dtype, max_tokens, max_live=4):
    from vllm_oxide_b200.engine.trace import TraceRunner
    return TraceRunner(folders[name][dtype], dtype, max_tokens, CONFIGS[name]["block_size"], max_live=max_live)


def feed(r, rid, tokens, cuts):
    """Feeds `tokens` in portions of the sizes `cuts` (cycled); logits at every position."""
    rows, at, k = [], 0, 0
    while at < len(tokens):
        n = min(cuts[k % len(cuts)], len(tokens) - at)
        k += 1
        end = [rid] if at + n == len(tokens) else []
        rows.append(r.step([{"id": rid, "tokens": tokens[at:at + n], "want": list(range(n))}], end))
        at += n
    return np.concatenate(rows, 0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_then_decoded_then_in_portions(folders, name, dtype):
    toks = tokens_for(name, 150)
    want = truth(folders, name, toks, dtype)
    r = runner(folders, name, dtype, 256)
    whole = feed(r, "w", toks, [len(toks)])
    close(whole, want, dtype, f"{name} {dtype} whole")
    decoded = feed(r, "d", toks, [len(toks) - 40] + [1] * 40)
    close(decoded, want, dtype, f"{name} {dtype} last 40 tokens one by one")
    for cuts in ([2], [3, 1, 17, 2, 64, 5], [CONFIGS[name]["block_size"]], [1, 2]):
        got = feed(r, "p", toks, cuts)
        close(got, want, dtype, f"{name} {dtype} portions {cuts}")
        if dtype == "float32":
            # the 32-bit kernels give an output element the same chain of operations however the tokens are cut
            assert np.abs(got - whole).max() <= 2e-6 * np.abs(whole).max(), f"{name} portions {cuts} against whole"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_token_by_token_from_the_first(folders, name, dtype):
    toks = tokens_for(name, 90, salt=5)
    r = runner(folders, name, dtype, 128)
    close(feed(r, "t", toks, [1]), truth(folders, name, toks, dtype), dtype, f"{name} {dtype} every token alone")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_first_tokens_of_a_sequence(folders, name, dtype):
    r = runner(folders, name, dtype, 64)
    for n in (1, 2, 3, 4, 6):
        toks = tokens_for(name, n, salt=40 + n)
        close(feed(r, f"f{n}", toks, [n]), truth(folders, name, toks, dtype), dtype, f"{name} {dtype} a prompt of {n}")
        close(feed(r, f"g{n}", toks, [1]), truth(folders, name, toks, dtype), dtype, f"{name} {dtype} {n} single tokens")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_requests_in_one_batch_over_pages_and_slots_used_again(folders, name, dtype):
    """Nine requests, at most three live, over a pool that holds far less than all of them: portions of some beside single
    tokens of others; a finished request's pages and state slot go to the next one, whose state must start from zero."""
    rng = random.Random(NAMES.index(name))
    bs = CONFIGS[name]["block_size"]
    lengths = [70, 1, 33, 130, 2, 64, 97, 18, 150]
    reqs = {f"q{i}": tokens_for(name, n, salt=100 + i) for i, n in enumerate(lengths)}
    live_cap = 3
    pool = sum(sorted(((n + bs - 1) // bs * bs for n in lengths), reverse=True)[:live_cap])
    r = runner(folders, name, dtype, pool, max_live=live_cap)
    waiting, live, at, got = list(reqs), [], {}, {k: [] for k in reqs}
    while waiting or live:
        while waiting and len(live) < live_cap:
            live.append(waiting.pop(0))
            at[live[-1]] = 0
        entries, end = [], []
        for rid in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue                              # left out of this step, goes on later
            left = len(reqs[rid]) - at[rid]
            n = min(left, rng.choice([1, 1, 2, 3, 7, bs, bs + 5, 40]))
            entries.append({"id": rid, "tokens": reqs[rid][at[rid]:at[rid] + n], "want": list(range(n))})
            at[rid] += n
            if at[rid] == len(reqs[rid]):
                end.append(rid)
                live.remove(rid)
        if not entries:
            continue
        out = r.step(entries, end)
        k = 0
        for e in entries:
            got[e["id"]].append(out[k:k + len(e["tokens"])])
            k += len(e["tokens"])
    assert r.manager.num_free_state_slots == live_cap
    for rid, toks in reqs.items():
        close(np.concatenate(got[rid], 0), truth(folders, name, toks, dtype), dtype, f"{name} {dtype} request {rid} in mixed batches")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_across_pages(folders, dtype):
    for name in ("P", "R"):
        toks = tokens_for(name, 330, salt=9)
        r = runner(folders, name, dtype, 384)
        close(feed(r, "l", toks, [6] + [1] * 324), truth(folders, name, toks, dtype), dtype, f"{name} {dtype} 324 decoded tokens")


def test_a_far_key_decides(tmp_path):
    """A model of one attention layer whose weights are set so that the last query's score with ONE key, hundreds of
    tokens back, towers over the rest (the key's token and the query's token appear nowhere else; one unrotated row of
    the key matrix answers the first, the same row of the query matrix the second).  With that token changed the plain
    model's last row is another one; the engine follows in every cut."""
    from vllm_oxide_b200.engine.loading import write_random_model_folder
    from vllm_oxide_b200.engine.trace import TraceRunner
    from vllm_oxide_b200.weights.safetensors_io import write_safetensors
    cfg = {"architecture": "Kesozen", "vocab": 50, "width": 64, "norm": {"eps": 1e-6},
           "layers": [_none(_attention(2, 1, 64, 0.5, 16, 10000.0))]}
    write_random_model_folder(str(tmp_path), cfg, 3, "fan_in", torch.float32)
    cfg, w = P.read_folder(str(tmp_path))
    g = torch.Generator().manual_seed(8)
    d_key, d_query = torch.nn.functional.normalize(torch.randn(2, 64, generator=g), dim=-1)
    w["embed"][45], w["embed"][46] = 8.0 * d_key, 8.0 * d_query
    w["l0.mix.k"][20], w["l0.mix.q"][20] = 3.0 * d_key, 3.0 * d_query         # row 20 lies behind the 16 rotated ones
    write_safetensors(str(tmp_path / "model.safetensors"), w)
    n, far = 700, 37
    toks = [1 + (i % 40) for i in range(n)]
    toks[far], toks[-1] = 45, 46
    want = P.forward(cfg, w, toks, torch.float64).numpy()
    moved = list(toks)
    moved[far] = 44
    gap = np.abs(P.forward(cfg, w, moved, torch.float64).numpy()[-1] - want[-1]).max()
    assert gap > 0.2 * want[-1].std(), "the plain model's last row hangs on the far token"
    for dtype in DTYPES:
        wt = P.forward(cfg, as_held(w, dtype), toks, torch.float64).numpy()
        r = TraceRunner(str(tmp_path), dtype, 1024, 64, max_live=2)
        for cuts in ([n], [n - 3, 1, 1, 1], [100, 2, 64], [far + 1, n - far - 2, 1]):
            close(feed(r, "x", toks, cuts), wt, dtype, f"far key, {dtype}, cuts {cuts}")


def plain_greedy(folders, name, prompt, new):
    toks = list(prompt)
    for _ in range(new):
        toks.append(int(truth(folders, name, toks, "float32")[-1].argmax()))
    return toks[len(prompt):]


@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_engine(folders, name):
    """`LLM.generate`: the scheduler cuts prompts to its token budget, batches them with decoding requests and preempts
    when the pool runs dry; the tokens are the plain implementation's."""
    from vllm_oxide_b200 import LLM, EngineOptions, SamplingParams
    bs = CONFIGS[name]["block_size"]
    llm = LLM(folders[name]["float32"], EngineOptions(dtype="float32", block_size=bs, num_kv_blocks=max(6, 320 // bs), max_num_seqs=3,
                                           max_num_batched_tokens=48, max_model_len=256))
    prompts = [tokens_for(name, n, salt=300 + n) for n in (5, 61, 1, 100, 17)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain_greedy(folders, name, p, 10), f"{name}: a prompt of {len(p)}"
    outs = llm.generate(prompts[:2], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain_greedy(folders, name, p, 10)[:4]


def test_bfloat16_generation_runs_from_graphs_and_agrees_where_the_plain_run_is_sure(folders):
    from vllm_oxide_b200 import LLM, EngineOptions, SamplingParams
    name = "Q"
    llm = LLM(folders[name]["bfloat16"], EngineOptions(dtype="bfloat16", block_size=64, num_kv_blocks=16, max_num_seqs=4, max_model_len=512))
    prompts = [tokens_for(name, n, salt=500 + n) for n in (9, 70, 130)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True))
    assert llm.core.graph_replays > 0
    for p, o in zip(prompts, outs):
        toks = list(p)
        for t in o.token_ids:
            row = truth(folders, name, toks, "bfloat16")[-1]
            top = np.sort(row)[-2:]
            if top[1] - top[0] < 0.1 * row.std():
                break                                  # too close to call in bfloat16: the runs may part here
            assert t == int(row.argmax())
            toks.append(t)


def test_the_replay_program(folders, tmp_path):
    name = "P"
    toks = tokens_for(name, 50, salt=77)
    other = tokens_for(name, 21, salt=78)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[30:32], "want": []}, {"id": "b", "tokens": other, "want": [20]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[32:], "want": [17]}], "end": ["a"]}]
    for dtype in DTYPES:
        out = tmp_path / dtype
        p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folders[name][dtype], "--dtype", dtype, "--out", str(out),
                            "--max-tokens", "128", "--block-size", "16"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                           capture_output=True, text=True, timeout=1200)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        want = truth(folders, name, toks, dtype)
        close(np.fromfile(out / "0.f32", "<f4").reshape(2, -1), pick(want, [0, 29]), dtype, "step 0")
        close(np.fromfile(out / "1.f32", "<f4").reshape(1, -1), pick(truth(folders, name, other, dtype), [20]), dtype, "step 1")
        close(np.fromfile(out / "2.f32", "<f4").reshape(1, -1), pick(want, [49]), dtype, "step 2")


def test_the_command_line(folders):
    name = "R"
    prompt = tokens_for(name, 9, salt=900)
    p = subprocess.run([os.path.join(ROOT, "bin", "vllm-oxide"), "-m", folders[name]["float32"], "--token-ids", " ".join(map(str, prompt)),
                        "--max-tokens", "6", "--dtype", "float32", "--ignore-eos", "--max-model-len", "128", "--block-size", "32",
                        "--num-kv-blocks", "16"], capture_output=True, text=True, timeout=1200)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(t) for t in p.stdout.split()] == plain_greedy(folders, name, prompt, 6)


def random_config(rng, kinds=None):
    """Sizes drawn at random, odd ones among them: no size of the design may rest on another, or on being a power of two.
    Attention heads are held to three widths of the tensor-core kernels, so that bfloat16 needs no further attention
    libraries, and two that only the plain kernel takes."""
    width = rng.choice([34, 50, 72, 96, 110, 136])
    if kinds is None:
        kinds = ["attention", "delta"] + [rng.choice(["attention", "delta"]) for _ in range(rng.randint(0, 3))]
        rng.shuffle(kinds)
    layers = []
    for kind in kinds:
        kv = rng.randint(1, 3)
        heads = kv * rng.randint(1, 3)
        if kind == "attention":
            dim = rng.choice([32, 64, 128, 24, 36])      # the last two: no tensor-core attention, the plain kernel in both precisions
            layer = _attention(heads, kv, dim, rng.choice([0.05, 0.2, 0.5]), 2 * rng.randint(0, dim // 2), rng.choice([100.0, 10000.0, 777.0]))
        else:
            layer = _delta(heads, kv, rng.randint(3, 70), rng.randint(3, 140), rng.randint(1, 6))
        what = rng.choice(["none", "dense", "moe", "moe"])
        if what == "dense":
            layer = _dense(layer, rng.randint(20, 150))
        elif what == "moe":
            count = rng.randint(1, 4)
            per = rng.randint(1, 4)
            keep = rng.randint(1, count)
            layer = _moe(layer, rng.randint(10, 80), count * per, rng.randint(1, per * keep), *((count, keep) if rng.random() < 0.8 else (None, None)))
            if "groups" not in layer["mlp"]["router"]:
                layer["mlp"]["router"]["top"] = rng.randint(1, count * per)
        else:
            layer = _none(layer)
        layers.append(layer)
    cfg = {"architecture": "Kesozen", "vocab": rng.randint(30, 300), "width": width, "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers}
    if rng.random() < 0.7:
        start = rng.randint(0, len(layers) - 1)
        cfg["loop"] = {"start": start, "stop": rng.randint(start, len(layers)), "times": rng.randint(1, 3)}
    return cfg


# seeds 10 and 11: a model without any paged layer, and one without any state
ONLY = {10: ["delta", "delta"], 11: ["attention", "attention", "attention"]}


@pytest.mark.parametrize("seed", range(12))
def test_random_configurations_and_cuts(seed, tmp_path):
    from vllm_oxide_b200.engine.trace import TraceRunner
    rng = random.Random(2000 + seed)
    cfg = random_config(rng, ONLY.get(seed))
    where = random_folders(tmp_path, cfg, seed)
    toks = [rng.randrange(cfg["vocab"]) for _ in range(75)]
    for dtype in DTYPES:
        _, w = P.read_folder(where[dtype])
        want = plain_logits(cfg, as_held(w, dtype), toks)
        r = TraceRunner(where[dtype], dtype, 128, rng.choice([16, 32, 64]), max_live=2)
        for cuts in ([75], [rng.randint(1, 9) for _ in range(5)], [60] + [1] * 15):
            close(feed(r, "x", toks, cuts), want, dtype, f"seed {seed} {dtype} cuts {cuts}: {json.dumps(cfg)[:300]}")
