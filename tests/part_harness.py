"""What the tests of single parts share: a build context, tensors that bfloat16 holds exactly, error measures, and a
driver that feeds requests through a mixer alone, step by step, against scattered pages and state slots full of
rubbish."""

import numpy as np
import torch

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 3e-5, "bfloat16": 4e-2}
TOL_MODEL = {"float32": 5e-5, "bfloat16": 9e-2}


def _ctx(dtype, max_positions=1024):
    from kv_cache_optimization_for_llm_b200.parts import BuildContext
    dev = torch.device("cuda:0")
    return BuildContext(dtype=DT[dtype], device=dev, max_positions=max_positions,
                        status=torch.zeros(1, dtype=torch.int32, device=dev))


def _w(rng, shape, std=0.3, mean=0.0):
    """A tensor that bfloat16 holds exactly, and its float64 copy."""
    t = torch.as_tensor(mean + rng.normal(size=shape) * std, dtype=torch.float32).to(torch.bfloat16)
    return t, t.float().numpy().astype(np.float64)


def _rel(got, ref):
    return np.abs(got.detach().float().cpu().numpy().astype(np.float64) - ref).max() / np.abs(ref).max()


def _err(got, ref, dtype):
    """float32: the largest difference over the largest value.  bfloat16: root mean square of the differences
    over that of the values: a head whose read-out is small in front of its RMS norm, or a softmax between two
    close scores, turns a rounding of 1 % into 20 % at single elements, which says nothing about the kernel."""
    got = got.detach().float().cpu().numpy().astype(np.float64)
    if dtype == "float32":
        return np.abs(got - ref).max() / np.abs(ref).max()
    return np.sqrt(((got - ref) ** 2).mean()) / np.sqrt((ref ** 2).mean())


def _same(a, b, dtype):
    """float32: bit for bit (every sum follows absolute positions and the sizes only).  bfloat16: the products of
    steps with few rows and with many rows are different kernels, which round differently."""
    if dtype == "float32":
        return torch.equal(a, b)
    return _err(a, b.double().numpy(), dtype) < TOL[dtype]


class _Manager:
    """Stands in for the cache manager when a part runs alone."""

    def __init__(self, tables, slots):
        self.tables, self.slots = tables, slots

    def slot_of(self, rid):
        return self.slots[rid]

    def block_table(self, rid, g):
        return self.tables[rid]


def _make(family, kind, params, weights, ctx):
    from kv_cache_optimization_for_llm_b200.parts import lookup
    from kv_cache_optimization_for_llm_b200.weights.loader import to_compute
    cls = lookup(family, kind)
    specs = cls.weight_specs(params)
    assert set(specs) == set(weights), (sorted(specs), sorted(weights))
    dev = {}
    for role, t in weights.items():
        assert tuple(t.shape) == tuple(specs[role].shape), (role, t.shape, specs[role].shape)
        dev[role] = to_compute(t, specs[role], ctx.dtype, ctx.device)
    return cls(params, dev, ctx)


def _run_in_steps(mixer, ctx, x, steps, page=8, state_slots=3, tables=None):
    """Feeds requests through a mixer alone.  ``x``: request -> its inputs [T, H] (compute type, on the
    device); ``steps``: a list of steps, each a list of (request, number of tokens).  Pages lie
    scattered and backwards; states start full of rubbish, which a request that starts at position 0
    must not read.  Returns request -> outputs [T, H]."""
    from kv_cache_optimization_for_llm_b200.cache.specs import PagedKVBinding, SlotStateBinding, paged_part, state_part
    from kv_cache_optimization_for_llm_b200.engine.batch import BatchBuilder, StepEntry
    wish = mixer.cache_spec()
    n_req = len(x)
    pages_each = -(-max(t.shape[0] for t in x.values()) // page)
    if tables is None:
        tables = {r: [n_req * pages_each - 1 - (i * n_req + r) for i in range(pages_each)] for r in x}
    slots = {r: (r + 1) % (state_slots + 1) for r in x}
    state = None
    if state_part(wish) is not None:
        st = state_part(wish)
        state = torch.full((state_slots + 1,) + tuple(st.shape), 7.5, dtype=st.dtype, device=ctx.device)
    if paged_part(wish) is not None:
        pg = paged_part(wish)
        store = torch.full((pg.planes, n_req * pages_each + 1, pg.num_kv_heads, page, pg.head_dim), 3.0,
                           dtype=ctx.dtype, device=ctx.device)
        binding = PagedKVBinding(k=store[0], v=store[1] if pg.planes > 1 else None, group=0, page_size=page, state=state)
    else:
        binding = SlotStateBinding(state=state)
    builder = BatchBuilder(1024, 8, [64], ctx.device, ctx.status)
    at = {r: 0 for r in x}
    outs = {r: [] for r in x}
    for step in steps:
        entries = [StepEntry(r, [0] * n, at[r], ()) for r, n in step]
        batch = builder.build(entries, _Manager(tables, slots))
        mixed = len(step) > 1 and any(m == 1 for _, m in step) and any(m != 1 for _, m in step)
        order = sorted(range(len(step)), key=lambda i: (mixed and step[i][1] != 1, i))     # single tokens come first
        rows = torch.cat([x[step[i][0]][at[step[i][0]]:at[step[i][0]] + step[i][1]] for i in order]).contiguous()
        y = mixer.forward(rows, batch, binding)
        if isinstance(y, tuple):        # two mixers side by side hand on both outputs
            y = y[0].float() + y[1].float()
        t = 0
        for i in order:
            r, n = step[i]
            outs[r].append(y[t:t + n].float().cpu())
            t += n
            at[r] += n
    assert int(ctx.status.item()) == 0
    return {r: torch.cat(o) for r, o in outs.items()}
