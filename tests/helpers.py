"""Test helpers: a step context built by hand, so that one part can be run alone, with pages and state slots of its own."""
import numpy as np
import torch

from vllm_oxide_b200 import host
from vllm_oxide_b200.engine.core import StepContext
from vllm_oxide_b200.parts import Workspace


def make_context(manager, entries, dtype, device="cuda:0"):
    """entries: [(request id, start, tokens, want)]; pages must have been ensured."""
    be = [host.BatchEntry(rid, start, list(toks), list(want)) for rid, start, toks, want in entries]
    T = sum(len(e.tokens) for e in be)
    R = max(1, sum(len(e.want) for e in be))
    pages = max(len(manager.block_table(e.id, g)) for e in be for g in range(manager.num_groups))
    layout = host.BatchLayout(T, len(be), R, manager.num_groups, max(pages, 1))
    buf = np.zeros(layout.total, dtype=np.int32)
    counts = host.fill_step_batch(manager, be, layout, buf)
    dev = torch.from_numpy(buf).to(device)
    err = torch.zeros(1, dtype=torch.int32, device=device)
    return StepContext(layout, dev, buf, counts, Workspace(T, device, dtype), err)


DEV = "cuda:0"


def rand(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g, dtype=torch.float64) * scale


def tolerance(dt):
    return 2e-5 if dt == torch.float32 else 0.03


def assert_close(got, want, dt, what, tol=None):
    got, want = got.double().cpu(), want.double().cpu()
    err = (got - want).abs().max().item() / max(want.abs().max().item(), 1e-30)
    assert err < (tol or tolerance(dt)), f"{what}: {err:.3e} of the largest value"


def held(t, dt):
    """A weight as the engine holds it: matrices, embeddings and biases in the model's type."""
    return t.to(dt).double()


class Alone:
    """One mixer with pages and state slots of its own."""

    def __init__(self, parts, dt, block_size=16, pages=40, slots=3):
        from vllm_oxide_b200.cache.paged_cache import PagedCache
        self.parts, self.dt = parts, dt
        self.cache = PagedCache([p.cache_spec() for p in parts], [p.state_spec() for p in parts], dt, DEV, block_size, pages, slots)
        self.m = self.cache.manager
        self.pos = {}

    def step(self, portions, end=(), plane_of=None):
        """portions: [(request, rows [n, width])]; returns every part's output, [n_total, ...] each, in the order of `parts`."""
        entries = []
        for rid, x in portions:
            if rid not in self.pos:
                assert self.m.add_request(rid)
                self.pos[rid] = 0
            assert self.m.ensure(rid, self.pos[rid], x.shape[0])
            entries.append((rid, self.pos[rid], [0] * x.shape[0], []))
        ctx = make_context(self.m, entries, self.dt)
        fresh = [int(s) for s, f in zip(ctx.host_view("state_slots"), ctx.host_view("state_fresh")) if f]
        self.cache.zero_states(fresh)
        x = torch.cat([x for _, x in portions]).to(self.dt).to(DEV).contiguous()
        outs = []
        for i, part in enumerate(self.parts):
            plane = i if plane_of is None else plane_of[i]
            outs.append(part.forward(x, ctx, self.cache.planes[plane], self.cache.states[plane], plane == i).clone())
        assert int(ctx.err.item()) == 0
        for rid, rows in portions:
            self.pos[rid] += rows.shape[0]
            self.m.advance(rid, self.pos[rid])
        for rid in end:
            self.m.free_request(rid)
            del self.pos[rid]
        return outs


def load(part, weights, dt):
    from vllm_oxide_b200.weights.loader import kept_dtype
    part.load({s.name: weights[s.name].to(kept_dtype(s.role, dt)).to(DEV) for s in part.tensor_specs()})


def in_portions(alone, rid, x, cuts, which=0):
    rows, at, k = [], 0, 0
    while at < x.shape[0]:
        n = min(cuts[k % len(cuts)], x.shape[0] - at)
        k += 1
        rows.append(alone.step([(rid, x[at:at + n])], end=[rid] if at + n == x.shape[0] else [])[which])
        at += n
    return torch.cat(rows)
