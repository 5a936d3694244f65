"""Tofilorn through the engine against the plain implementation (tests/plain/tofilorn_plain.py): whole prompts, decoding
token by token, portions down to two tokens, unequal requests in one batch over pages and state slots that are used
again, long decoding across windows and page borders, the first tokens, greedy generation through `LLM` and the replay
program itself.  The configurations are made here; they differ from each other in every size."""
import json
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT
from plain import tofilorn_plain as P

pytestmark = pytest.mark.gpu


def _rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot, window=None, kv_from=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank, scale=scale, rot=rot)
    if window:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


CONFIGS = {
    # three streams; a borrowed plane whose reader looks further back (33) than its writer (19); a cache row of 44 elements
    # (padded to 48); stretched rotation; feed-forwards where the mixers are recurrent and none behind the second attention
    "P": dict(block_size=16, config={
        "architecture": "Tofilorn", "vocab": 211, "width": 96, "streams": 3, "norm": {"eps": 1e-6}, "layers": [
            _layer("latent_attention", _latent(3, 24, 8, 40, 48, 36, 0.2, _rot(8, 1000.0, (4.0, 32, 8.0, 1.0)), window=19), ff=160),
            _layer("hgrn2", dict(heads=3, dim=16, vdim=24), ff=128),
            _layer("mingru", dict(width=80)),
            _layer("latent_attention", _latent(2, 16, 8, 24, 32, 36, 0.3, _rot(8, 1000.0, (4.0, 32, 8.0, 1.0)), window=33, kv_from=0)),
            _layer("mingru", dict(width=128), ff=96)]}),
    # no `streams` key (one plain residual stream); widths in multiples of 64 (the weight-streaming product takes the decode
    # steps); a window of exactly one page; a layer without a window; one wide head whose norm runs in a kernel of its own
    "Q": dict(block_size=64, config={
        "architecture": "Tofilorn", "vocab": 384, "width": 128, "norm": {"eps": 1e-5}, "layers": [
            _layer("hgrn2", dict(heads=1, dim=64, vdim=160)),
            _layer("latent_attention", _latent(4, 32, 16, 48, 64, 48, 0.15, _rot(16, 10000.0), window=64), ff=192),
            _layer("mingru", dict(width=192)),
            _layer("latent_attention", _latent(2, 64, 32, 64, 128, 96, 0.1, _rot(16, 500.0, (8.0, 64, 4.0, 2.0))), ff=128)]}),
    # one stream WITH coefficients, one head, sizes that are 1 or equal where the other two differ
    "R": dict(block_size=32, config={
        "architecture": "Tofilorn", "vocab": 97, "width": 64, "streams": 1, "norm": {"eps": 1e-5}, "layers": [
            _layer("mingru", dict(width=64), ff=64),
            _layer("latent_attention", _latent(1, 64, 32, 64, 64, 96, 0.125, _rot(32, 50000.0, (2.0, 16, 32.0, 1.0)), window=7)),
            _layer("hgrn2", dict(heads=2, dim=128, vdim=32), ff=80),
            _layer("latent_attention", _latent(1, 32, 32, 16, 16, 96, 0.2, _rot(32, 50000.0, (2.0, 16, 32.0, 1.0)), window=7, kv_from=1))]}),
}
NAMES = sorted(CONFIGS)
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from vllm_oxide_b200.engine.loading import write_random_model_folder
    out = {}
    for k, (name, spec) in enumerate(sorted(CONFIGS.items())):
        folder = str(tmp_path_factory.mktemp(f"tofilorn_{name}"))
        write_random_model_folder(folder, spec["config"], 11 + k, "fan_in", torch.float32)
        out[name] = folder
    return out


_models, _truth = {}, {}


def tokens_for(name, n, salt=0):
    g = torch.Generator().manual_seed(7919 * (NAMES.index(name) + 1) + salt)
    return torch.randint(0, CONFIGS[name]["config"]["vocab"], (n,), generator=g).tolist()


def truth(folders, name, tokens, dtype):
    """Plain float64 logits at every position; for bfloat16 over the weights rounded to bfloat16, as the engine holds them."""
    key = (name, tuple(tokens), dtype)
    if key not in _truth:
        if (name, dtype) not in _models:
            cfg, w = P.read_folder(folders[name])
            if dtype == "bfloat16":
                w = {k: (v.to(torch.bfloat16).to(v.dtype) if v.dtype.is_floating_point and "hc" not in k and "lower" not in k
                         and "norm" not in k else v) for k, v in w.items()}
            _models[(name, dtype)] = (cfg, w)
        cfg, w = _models[(name, dtype)]
        _truth[key] = P.forward(cfg, w, tokens, torch.float64)[0].numpy()
    return _truth[key]


def close(got, want, dtype, what):
    """float32: within 1e-4 of the logits' spread, row by row (rounding alone stays near 1e-6; a wrong key, gate or
    coefficient moves a row by percents).  bfloat16: within 0.06 of it (rounding at every operation gives about 0.01)."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, what
    d = got - want
    err = np.sqrt((d ** 2).mean(-1)) / want.std(-1)
    bound = 1e-4 if dtype == "float32" else 0.06
    assert err.max() < bound, f"{what}: row {int(err.argmax())} is {err.max():.3e} of the spread off"


def runner(folders, name, dtype, max_tokens, max_live=4):
    from vllm_oxide_b200.engine.trace import TraceRunner
    return TraceRunner(folders[name], dtype, max_tokens, CONFIGS[name]["block_size"], max_live=max_live)


def feed(r, rid, tokens, cuts, want_all=True):
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
    for n in (1, 2, 3, 4):
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
    # every live request's tokens rounded up to pages (a layer without a window keeps them all)
    pool = sum(sorted(((n + bs - 1) // bs * bs for n in lengths), reverse=True)[:live_cap])
    r = runner(folders, name, dtype, pool, max_live=live_cap)
    waiting, live, at, got = list(reqs), [], {}, {k: [] for k in reqs}
    steps = 0
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
        steps += 1
    assert r.manager.num_free_state_slots == live_cap
    for rid, toks in reqs.items():
        close(np.concatenate(got[rid], 0), truth(folders, name, toks, dtype), dtype, f"{name} {dtype} request {rid} in mixed batches")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_past_windows_and_pages(folders, dtype):
    for name in ("P", "R"):
        toks = tokens_for(name, 330, salt=9)
        r = runner(folders, name, dtype, 384)
        close(feed(r, "l", toks, [6] + [1] * 324), truth(folders, name, toks, dtype), dtype, f"{name} {dtype} 324 decoded tokens")


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
    llm = LLM(folders[name], EngineOptions(dtype="float32", block_size=bs, num_kv_blocks=max(6, 320 // bs), max_num_seqs=3,
                                           max_num_batched_tokens=48, max_model_len=256))
    prompts = [tokens_for(name, n, salt=300 + n) for n in (5, 61, 1, 100, 17)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain_greedy(folders, name, p, 10), f"{name}: a prompt of {len(p)}"
    # the same engine again: slots and pages of the first call are in use again
    outs = llm.generate(prompts[:2], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain_greedy(folders, name, p, 10)[:4]


def test_bfloat16_generation_runs_from_graphs_and_agrees_where_the_plain_run_is_sure(folders):
    from vllm_oxide_b200 import LLM, EngineOptions, SamplingParams
    name = "Q"
    llm = LLM(folders[name], EngineOptions(dtype="bfloat16", block_size=64, num_kv_blocks=16, max_num_seqs=4, max_model_len=512))
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
        p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folders[name], "--dtype", dtype, "--out", str(out),
                            "--max-tokens", "128", "--block-size", "16"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                           capture_output=True, text=True, timeout=1200)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        want = truth(folders, name, toks, dtype)
        close(np.fromfile(out / "0.f32", "<f4").reshape(2, -1), want[[0, 29]], dtype, "step 0")
        close(np.fromfile(out / "1.f32", "<f4").reshape(1, -1), truth(folders, name, other, dtype)[[20]], dtype, "step 1")
        close(np.fromfile(out / "2.f32", "<f4").reshape(1, -1), want[[49]], dtype, "step 2")


def test_the_command_line(folders):
    name = "R"
    prompt = tokens_for(name, 9, salt=900)
    p = subprocess.run([os.path.join(ROOT, "bin", "vllm-oxide"), "-m", folders[name], "--token-ids", " ".join(map(str, prompt)),
                        "--max-tokens", "6", "--dtype", "float32", "--ignore-eos", "--max-model-len", "128", "--block-size", "32",
                        "--num-kv-blocks", "16"], capture_output=True, text=True, timeout=1200)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(t) for t in p.stdout.split()] == plain_greedy(folders, name, prompt, 6)


def random_config(rng, kinds=None):
    """Sizes drawn at random, odd ones among them: no size of the design may rest on another, or on being even or a power of two.
    Cache rows (kv_rank + rot_dim, padded to 16) are held to three widths so that bfloat16 needs no further attention libraries."""
    width = rng.choice([34, 50, 72, 96, 110, 136])
    layers, writers = [], []
    if kinds is None:
        kinds = ["mingru", "hgrn2", "latent_attention", "latent_attention"] + [rng.choice(["mingru", "hgrn2", "latent_attention"]) for _ in range(rng.randint(0, 3))]
        rng.shuffle(kinds)
    for i, kind in enumerate(kinds):
        ff = rng.choice([None, rng.randint(20, 150)])
        if kind == "mingru":
            m = dict(width=rng.randint(9, 200))
        elif kind == "hgrn2":
            m = dict(heads=rng.randint(1, 4), dim=rng.randint(3, 70), vdim=rng.randint(3, 140))
        else:
            src = rng.choice(writers) if writers and rng.random() < 0.5 else None
            if src is None:
                row = rng.choice([48, 64, 128])
                rot_dim = 2 * rng.randint(1, 8)
                kv_rank = row - rot_dim - rng.randint(0, 6)
                rot = _rot(2 * rng.randint(1, rot_dim // 2), rng.choice([100.0, 10000.0, 777.0]),
                           rng.choice([None, (rng.choice([2.0, 3.5, 16.0]), rng.choice([8, 32, 100]), rng.choice([4.0, 32.0]), rng.choice([1.0, 2.0]))]))
                writers.append(i)
            else:
                other = layers[src]["mixer"]
                rot_dim, kv_rank, rot = other["rot_dim"], other["kv_rank"], other["rot"]
            m = _latent(rng.randint(1, 7), rng.randint(2, 40), rot_dim, rng.randint(2, 50), rng.randint(5, 60), kv_rank,
                        rng.choice([0.05, 0.2, 0.5]), rot, window=rng.choice([None, 1, 2, 17, 40, 64]), kv_from=src)
        layers.append(_layer(kind, m, ff))
    cfg = {"architecture": "Tofilorn", "vocab": rng.randint(30, 300), "width": width, "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers}
    if rng.random() < 0.8:
        cfg["streams"] = rng.randint(1, 6)
    return cfg


# seeds 10 and 11: a model without any paged layer, and one without any state
ONLY = {10: ["hgrn2", "mingru", "mingru"], 11: ["latent_attention", "latent_attention", "latent_attention"]}


@pytest.mark.parametrize("seed", range(12))
def test_random_configurations_and_cuts(seed, tmp_path):
    from vllm_oxide_b200.engine.loading import write_random_model_folder
    from vllm_oxide_b200.engine.trace import TraceRunner
    rng = random.Random(1000 + seed)
    cfg = random_config(rng, ONLY.get(seed))
    write_random_model_folder(str(tmp_path), cfg, seed, "fan_in", torch.float32)
    _, w = P.read_folder(str(tmp_path))
    toks = [rng.randrange(cfg["vocab"]) for _ in range(75)]
    for dtype in DTYPES:
        wd = w if dtype == "float32" else {k: (v.to(torch.bfloat16).to(v.dtype) if v.dtype.is_floating_point and "hc" not in k
                                               and "lower" not in k and "norm" not in k else v) for k, v in w.items()}
        want = P.forward(cfg, wd, toks, torch.float64)[0].numpy()
        r = TraceRunner(str(tmp_path), dtype, 128, rng.choice([16, 32, 64]), max_live=2)
        for cuts in ([75], [rng.randint(1, 9) for _ in range(5)], [60] + [1] * 15):
            close(feed(r, "x", toks, cuts), want, dtype, f"seed {seed} {dtype} cuts {cuts}: {json.dumps(cfg)[:300]}")
