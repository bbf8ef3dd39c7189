"""Tevanex on the GPU, against the plain model in tests/plain_tevanex.py (numpy float64): every mechanism alone, then
whole models through the engine's step function, its scheduler, the trace runner and the command line.  Weights and
configurations are made here."""

import math
import os
import tempfile

import numpy as np
import pytest
import torch

import plain_tevanex as S
import tiny_tevanex as tiny
from part_harness import DT, TOL, TOL_MODEL, _Manager, _ctx, _err, _make, _run_in_steps, _same, _w

pytestmark = pytest.mark.gpu


def _f32(a, dev="cuda"):
    return torch.as_tensor(np.asarray(a), dtype=torch.float32).to(dev).contiguous()


# --------------------------------------------------------------------------- embedding, post norm, logits

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_takes_its_factor_in_float32(dtype):
    from kv_cache_optimization_for_llm_b200.engine.batch import BatchBuilder, StepEntry
    rng = np.random.default_rng(0)
    ctx = _ctx(dtype)
    table, t64 = _w(rng, (31, 24), 0.5)
    emb = _make("embedding", "token_embedding", {"vocab_size": 31, "hidden_size": 24, "scale": 0.37}, {"table": table}, ctx)
    builder = BatchBuilder(64, 4, [8], ctx.device, ctx.status)
    toks = rng.integers(0, 31, 9).tolist()
    batch = builder.build([StepEntry(0, toks, 0, ())], _Manager({0: list(range(8))}, {0: 0}))
    x = emb.forward(batch)
    assert x.dtype == torch.float32
    # the table's numbers are bfloat16 in both precisions; times 0.37 they are not, and nothing may round them back
    assert np.abs(x.cpu().numpy() - t64[toks] * 0.37).max() < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("W,with_bias", [(40, True), (7, False), (264, True)])
def test_branch_output_is_normed_added_and_the_stream_handed_on(dtype, W, with_bias):
    """x <- x + rms_norm(y + bias) * (weight * factor): one launch, which also leaves the new stream in the compute type."""
    from kv_cache_optimization_for_llm_b200 import ops
    rng = np.random.default_rng(1)
    ctx = _ctx(dtype)
    T = 13
    weight = _w(rng, (W,), 0.3, 1.0)
    norm = _make("norm", "rmsnorm", {"size": W, "eps": 1e-5, "scale": 0.3}, {"weight": weight[0]}, ctx)
    x = rng.normal(size=(T, W)) * 3
    y, y64 = _w(rng, (T, W), 2.0)
    bias = _w(rng, (W,), 0.5) if with_bias else None
    xd = _f32(x)
    x32 = xd.cpu().numpy().astype(np.float64)
    pending = norm.as_pending(y.to(DT[dtype]).cuda(), None if bias is None else _f32(bias[1]))
    out = ops.add_norm(xd, pending, "copy", None, 0.0, DT[dtype])
    ref = x32 + 0.3 * S.rms_norm(y64 + (bias[1] if with_bias else 0.0), weight[1], 1e-5)
    assert np.abs(xd.cpu().numpy() - ref).max() < 2e-6 * np.abs(ref).max() + 1e-6
    assert out.dtype == DT[dtype] and _err(out, ref, dtype) < (1e-6 if dtype == "float32" else 5e-3)
    # nothing pending: the stream as it is
    again = ops.add_norm(xd, None, "copy", None, 0.0, DT[dtype])
    assert torch.equal(again.float(), xd.to(DT[dtype]).float())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("scale,cap", [(0.6, 7.0), (1.0, 2.0), (0.25, None)])
def test_logits_take_a_factor_and_a_cap(dtype, scale, cap):
    rng = np.random.default_rng(2)
    ctx = _ctx(dtype)
    w, w64 = _w(rng, (53, 24), 1.0)
    head = _make("head", "linear_head", {"vocab_size": 53, "hidden_size": 24, "scale": scale, "softcap": cap}, {"weight": w}, ctx)
    x, x64 = _w(rng, (5, 24), 2.0)
    got = head.forward(x.to(DT[dtype]).cuda())
    z = x64 @ w64.T * scale
    ref = S.soft_cap(z, cap) if cap else z
    assert got.dtype == torch.float32 and _err(got, ref, dtype) < (1e-5 if dtype == "float32" else 1e-2)
    if cap:
        assert np.abs(z).max() > cap >= np.abs(got.cpu().numpy()).max()


# --------------------------------------------------------------------------- rotation

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind,dims,D,scaling", [("rope", 8, 16, None), ("rope_interleaved", 10, 24, tiny.YARN),
                                                 ("rope_interleaved", 16, 16, None), ("rope", 6, 6, None),
                                                 ("rope", 2, 5, None), ("rope_interleaved", 4, 8, dict(tiny.YARN, factor=1.5))])
def test_norm_over_the_whole_projection_then_rotation_of_part_of_every_head(dtype, kind, dims, D, scaling):
    """The kernel in front of the attention alone: biases, one root mean square over all of a token's queries (and
    keys), a weight as wide, then the rotation in both layouts, with and without stretched frequencies, at positions
    far from 0; the keys and values land in scattered pages."""
    from kv_cache_optimization_for_llm_b200 import ops
    from kv_cache_optimization_for_llm_b200.engine.batch import BatchBuilder, StepEntry
    from kv_cache_optimization_for_llm_b200.models.spec import PartSpec
    rng = np.random.default_rng(3)
    ctx = _ctx(dtype, max_positions=4096)
    H, G, Dv, page = 3, 2, 7, 8
    params = {"dims": dims, "base": 300.0, "scaling": dict(scaling, rope_type="yarn") if scaling else None} \
        if kind == "rope_interleaved" else {"head_dim": D, "rotary_dim": dims, "theta": 300.0,
                                            "scaling": dict(scaling, rope_type="yarn") if scaling else None}
    pos_part = _make("position", kind, params, {}, ctx)
    cos, sin = pos_part.tables()
    T, start = 21, 1000
    src, s64 = _w(rng, (T, H * D + G * D + G * Dv), 1.0)
    bq, bk, bv = _w(rng, (H * D,), 0.5), _w(rng, (G * D,), 0.5), _w(rng, (G * Dv,), 0.5)
    qw, kw = _w(rng, (H * D,), 0.3, 1.0), _w(rng, (G * D,), 0.3, 1.0)
    pages = torch.zeros((T // page + 2 + start // page, G, page, D + Dv), dtype=DT[dtype], device="cuda")
    tables = {0: list(range(pages.shape[0] - 1))[::-1]}
    builder = BatchBuilder(64, 4, [pages.shape[0]], ctx.device, ctx.status)
    batch = builder.build([StepEntry(0, [0] * T, start, ())], _Manager(tables, {0: 0}))
    q = ops.qk_rot_append(src.to(DT[dtype]).cuda(), 0, H * D, H * D + G * D, _f32(bq[1]), _f32(bk[1]), _f32(bv[1]),
                          _f32(qw[1]), _f32(kw[1]), 1e-5, cos, sin, dims, "half" if kind == "rope" else "pairs", pages,
                          batch.block_tables[0], batch, H, G, D, Dv)
    assert int(ctx.status.item()) == 0
    f, grow = S.rotary_frequencies(dims, 300.0, scaling)
    positions = range(start, start + T)
    layout = "half" if kind == "rope" else "pairs"
    q_ref = S.rotate(S.rms_norm(s64[:, :H * D] + bq[1], qw[1], 1e-5).reshape(T, H, D), positions, dims, f, grow, layout)
    k_ref = S.rotate(S.rms_norm(s64[:, H * D:H * D + G * D] + bk[1], kw[1], 1e-5).reshape(T, G, D), positions, dims, f, grow, layout)
    v_ref = (s64[:, H * D + G * D:] + bv[1]).reshape(T, G, Dv)
    tol = 2e-5 if dtype == "float32" else 1e-2      # float32: the angle itself is a float of a thousand
    assert _err(q, q_ref.reshape(T, H * D), dtype) < tol
    rows = torch.stack([pages[tables[0][p // page], :, p % page] for p in positions])      # [T, G, D + Dv]
    assert _err(rows[:, :, :D].reshape(T, -1), k_ref.reshape(T, -1), dtype) < tol
    assert _err(rows[:, :, D:].reshape(T, -1), v_ref.reshape(T, -1), dtype) < tol
    if scaling:      # the stretched rotation is longer than 1: a query's length grows by the factor on cos and sin
        assert grow > 1.01


# --------------------------------------------------------------------------- attention

def _att_params(H, m, kind, eps=1e-5):
    from kv_cache_optimization_for_llm_b200.models.spec import PartSpec
    second = kind == "attention_2"
    rot = m.get("rot")
    position = None
    if rot and rot["dims"]:
        if second:
            sc = dict(rot["scaling"], rope_type="yarn") if rot.get("scaling") else None
            position = PartSpec("rope_interleaved", {"dims": rot["dims"], "base": rot["base"], "scaling": sc})
        else:
            position = PartSpec("rope", {"head_dim": m["dim"], "rotary_dim": rot["dims"], "theta": rot["base"], "scaling": None})
    return {"hidden_size": H, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
            "scale": m["scale"], "chunk": (m.get("mask") or {}).get("size"), "softcap": m.get("softcap") if second else None,
            "sink": not second, "gate": second, "bias": True, "qk_norm": True, "eps": eps, "position": position}


def _att_weights(rng, H, m, kind):
    Hq, G, D, Dv = (m[k] for k in ("heads", "kv_heads", "dim", "vdim"))
    wt, w64 = {}, {}
    rows = [("q", "q", (Hq * D, H), 0.3, 0), ("k", "k", (G * D, H), 0.3, 0), ("v", "v", (G * Dv, H), 0.3, 0),
            ("q_bias", "q.b", (Hq * D,), 0.5, 0), ("k_bias", "k.b", (G * D,), 0.5, 0), ("v_bias", "v.b", (G * Dv,), 0.5, 0),
            ("o_bias", "o.b", (H,), 0.5, 0), ("q_norm", "q.norm", (Hq * D,), 0.2, 1.0), ("k_norm", "k.norm", (G * D,), 0.2, 1.0),
            ("o", "o", (H, Hq * Dv), 0.3, 0)]
    rows.append(("g", "g", (Hq * Dv, H), 0.3, 0) if kind == "attention_2" else ("sink", "sink", (Hq,), 1.5, 0))
    for role, name, shape, std, mean in rows:
        wt[role], w64[name] = _w(rng, shape, std, mean)
    return wt, w64


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind,shape", [
    ("attention", dict()),
    ("attention_2", dict(heads=3, kv_heads=1, dim=24, vdim=8, scale=0.2, size=5, rot_dims=10, softcap=1.5, scaling=tiny.YARN)),
    ("attention", dict(heads=2, kv_heads=2, dim=8, vdim=40, scale=0.5, size=16, rot_dims=8)),
    ("attention_2", dict(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.125, size=33, rot_dims=32, softcap=30.0)),
    ("attention", dict(heads=1, kv_heads=1, dim=5, vdim=3, scale=1.0, size=1, rot_dims=4)),
    ("attention_2", dict(heads=4, kv_heads=4, dim=32, vdim=16, scale=0.3, size=None, rot_dims=None, softcap=None)),
    ("attention", dict(heads=8, kv_heads=2, dim=40, vdim=24, scale=0.15, size=64, rot_dims=40)),
    ("attention", dict(heads=8, kv_heads=1, dim=128, vdim=64, scale=0.09, size=40, rot_dims=64)),
    ("attention_2", dict(heads=2, kv_heads=1, dim=64, vdim=128, scale=0.12, size=None, rot_dims=2, softcap=3.0, scaling=tiny.YARN)),
])
def test_attention_alone_in_portions_and_beside_another_request(dtype, kind, shape):
    """Both kinds in several shapes (grouped and ungrouped heads, key and value sizes that differ, blocks of one
    position, no blocks, no rotation, every channel turning), 70 and 33 tokens on pages of 8 that lie scattered;
    portions end inside pages and blocks and on their borders."""
    rng = np.random.default_rng(3)
    ctx = _ctx(dtype)
    H = 40
    m = tiny.attention(**shape)
    wt, w64 = _att_weights(rng, H, m, kind)
    mixer = _make("mixer", "rotary_chunk_attention", _att_params(H, m, kind), wt, ctx)
    xs, refs = {}, {}
    for r, T in enumerate((70, 33)):
        x, x64 = _w(rng, (T, H), 1.0)
        xs[r], refs[r] = x.to(DT[dtype]).cuda(), S.attention_mixer(x64, w64, "", m, kind, 1e-5)
    from kv_cache_optimization_for_llm_b200 import ops
    on_tensor_cores = ops.choices["window_flash_attention"]
    whole = _run_in_steps(mixer, ctx, xs, [[(0, 70)], [(1, 33)]])
    # bfloat16 prompt portions of sizes that are multiples of 8 run on tensor cores, everything else does not
    took = ops.choices["window_flash_attention"] > on_tensor_cores
    assert took == (dtype == "bfloat16" and m["dim"] % 8 == 0 and m["vdim"] % 8 == 0)
    cut = _run_in_steps(mixer, ctx, xs, [[(0, 8), (1, 1)], [(0, 9), (1, 1)], [(0, 2), (1, 30)], [(0, 1), (1, 1)],
                                         [(0, 44)], [(0, 1)], [(0, 1)], [(0, 4)]])
    one = _run_in_steps(mixer, ctx, {0: xs[1]}, [[(0, 1)]] * 33)
    for r in xs:
        assert _err(whole[r], refs[r], dtype) < TOL[dtype]
        assert _err(cut[r], refs[r], dtype) < TOL[dtype]
        assert _same(whole[r], cut[r], dtype), "a token's result must not depend on the cut or on the batch"
    assert _same(one[0], whole[1], dtype), "token by token"


def _spiked(dtype, chunk, T, query, key, softcap=0.0, sink=None, gate=None, page=8, D=16, flash=False):
    """The attention kernel alone on keys and values made so that one key decides: every query and key is small but
    the pair (query, key), whose raw score is 30; the value of key j is the unit vector j.  Returns what the query at
    ``query`` reads, in a prompt (one portion) and decoded alone, and the plain answer.  ``flash``: the prompt on the
    tensor-core kernel, whose values have at most 128 channels: the value of key j is then the unit vector j mod 128."""
    from kv_cache_optimization_for_llm_b200 import ops
    from kv_cache_optimization_for_llm_b200.engine.batch import BatchBuilder, StepEntry
    ctx = _ctx(dtype)
    rng = np.random.default_rng(T + query)
    q = rng.normal(size=(T, D)) * 0.01
    k = rng.normal(size=(T, D)) * 0.01
    q[query] = 0
    q[query, 3] = 6.0
    k[key] = 0
    k[key, 3] = 5.0
    Dv = D if flash == "tcgen05" else (min(T, 128) if flash else T)
    v = np.zeros((T, Dv))
    v[np.arange(T), np.arange(T) % Dv] = 1.0
    g = np.full((T, Dv), 0.0 if gate is None else gate)
    src = torch.as_tensor(np.concatenate([q, k, v, g], axis=1), dtype=torch.float32).to(DT[dtype]).cuda()
    ref = S.masked_attention(q[:, None], k[:, None], v[:, None], 1.0, chunk or None, softcap or None,
                             None if sink is None else np.array([sink]))[:, 0]
    if gate is not None:
        ref = ref * S.sigmoid(gate)
    outs = []
    for steps in ([T], [query] + [1] * (T - query)):
        pages = torch.zeros((T // page + 2, 1, page, D + Dv), dtype=DT[dtype], device="cuda")
        tables = {0: list(range(T // page + 1))[::-1]}
        builder = BatchBuilder(1024, 4, [64], ctx.device, ctx.status)
        at, rows = 0, []
        for n in steps:
            if n == 0:
                continue
            batch = builder.build([StepEntry(0, [0] * n, at, ())], _Manager(tables, {0: 0}))
            part = src[at:at + n].contiguous()
            ops.kv_rows_append(part, D, 2 * D, pages, batch.block_tables[0], batch, 1, D, Dv)
            shape = dict(softcap=softcap, sinks=None if sink is None else _f32([sink]), chunk=chunk,
                         gate=None if gate is None else (part, 2 * D + Dv))
            if flash == "tcgen05" and n > 1:
                got = ops.flash_attention_rows_masked(part, pages, batch.block_tables[0], batch, 1, 1, D, 1.0, **shape)
            elif flash and n > 1:
                got = ops.window_flash_attention(part, pages, batch.block_tables[0], batch, 1, 1, D, Dv, 1.0, 0, 0, False, **shape)
            else:
                got = ops.window_attention(part, 0, pages, batch.block_tables[0], batch, 1, 1, D, Dv, 1.0, 0, 0, False, **shape)
            rows.append(got.float().cpu())
            at += n
        outs.append(torch.cat(rows)[query].numpy())
    assert int(ctx.status.item()) == 0
    return outs, ref[query]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_key_far_away_and_keys_at_the_edges_of_a_block(dtype):
    """One key whose score stands out among hundreds: the first position of the query's block and the last of the
    block before, on a page's border, at the sequence's first token, at the query itself; the query in a prompt and
    decoded alone; a query that is its block's first position sees only itself."""
    size, T, query = 37, 250, 245            # the query's block starts at 222
    tol = 2e-6 if dtype == "float32" else 1e-2
    for key, seen in ((222, True), (221, False), (0, False), (query, True), (224, True), (223, True), (query - 36, False),
                      (query - 37, False), (185, False)):
        (in_prompt, decoded), ref = _spiked(dtype, size, T, query, key)
        for got in (in_prompt, decoded):
            if seen:
                assert got[key] > 0.99 and abs(got[key] - ref[key]) < 1e-2, (key, got[key], ref[key])
            else:
                assert got[key] == 0 and ref[key] == 0, (key, got[key])
            assert np.abs(got - ref).max() < tol
    (in_prompt, decoded), ref = _spiked(dtype, 37, 230, 222, 221)         # the first position of a block
    assert ref[222] == 1.0 and in_prompt[222] > 0.999 and decoded[222] > 0.999 and in_prompt[221] == 0 and decoded[221] == 0
    (in_prompt, decoded), ref = _spiked(dtype, 37, 230, 221, 185)         # the last position of a block sees its first
    assert in_prompt[185] > 0.99 and decoded[185] > 0.99 and np.abs(in_prompt - ref).max() < tol
    # no blocks: a key hundreds of tokens back, and the very first one
    for key in (2, 0):
        (in_prompt, decoded), ref = _spiked(dtype, 0, 250, 249, key)
        assert in_prompt[key] > 0.99 and decoded[key] > 0.99 and np.abs(in_prompt - ref).max() < tol
    # the first tokens of a sequence: a block that is larger than the sequence so far
    (in_prompt, decoded), ref = _spiked(dtype, 64, 8, 2, 0)
    assert in_prompt[0] > 0.99 and np.abs(in_prompt - ref).max() < tol and np.abs(decoded - ref).max() < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sink_cap_and_gate_show_in_the_weights(dtype):
    """A learned score in the denominator takes weight without giving a value: with the spike's score capped at 4 and a
    sink of 4 the spiked key keeps about half; a sink far below changes nothing; the sink is not capped and counts
    once; the gate multiplies what is left."""
    T, query, key = 60, 59, 19
    tol = 1e-5 if dtype == "float32" else 2e-2
    (a, b), ref = _spiked(dtype, 0, T, query, key, softcap=4.0)
    assert 0.4 < ref[key] < 0.5 and abs(a[key] - ref[key]) < tol and abs(b[key] - ref[key]) < tol
    (a, b), ref = _spiked(dtype, 0, T, query, key, softcap=4.0, sink=4.0)
    assert 0.28 < ref[key] < 0.33 and abs(ref.sum() - 0.65) < 0.05
    assert np.abs(a - ref).max() < tol and np.abs(b - ref).max() < tol
    (a, b), ref = _spiked(dtype, 0, T, query, key, softcap=4.0, sink=40.0)      # were the sink capped, this would be the line above
    assert ref.sum() < 1e-12 and np.abs(a).max() < 1e-10 and np.abs(b).max() < 1e-10
    (a, b), ref = _spiked(dtype, 0, T, query, key, sink=-30.0)
    assert ref[key] > 0.99 and abs(a[key] - ref[key]) < tol and abs(b[key] - ref[key]) < tol
    (a, b), ref = _spiked(dtype, 16, T, query, 50, softcap=4.0, sink=1.0, gate=-1.0)
    assert np.abs(a - ref).max() < tol and np.abs(b - ref).max() < tol and ref[50] < 0.27


@pytest.mark.parametrize("wide", [False, True])
def test_prompt_portions_on_tensor_cores_see_the_same_keys_and_the_same_sink(wide, monkeypatch):
    """The kernel that bfloat16 prompt portions use (both tile heights): keys at the edges of the query's block, on tile
    borders (64 keys a tile) and far away; the sink, the cap and the gate in its softmax and on its result."""
    from kv_cache_optimization_for_llm_b200 import ops
    monkeypatch.setattr(ops, "WINDOW_FLASH_WIDE", wide)
    size, T, query = 37, 250, 245            # the query's block starts at 222
    before = ops.choices["window_flash_attention"]
    for key, seen in ((222, True), (221, False), (0, False), (query, True), (223, True), (192, False), (191, False), (185, False)):
        (in_prompt, _), ref = _spiked("bfloat16", size, T, query, key, flash=True)
        slot = key % 128
        if seen:
            assert in_prompt[slot] > 0.99 and abs(in_prompt[slot] - ref[slot]) < 1e-2, (key, in_prompt[slot], ref[slot])
        assert np.abs(in_prompt - ref).max() < 1e-2, key
    for key in (2, 0, 63, 64, 127, 128):      # no blocks: every key up to the query, across all tiles
        (in_prompt, _), ref = _spiked("bfloat16", 0, 250, 249, key, flash=True)
        assert in_prompt[key % 128] > 0.99 and np.abs(in_prompt - ref).max() < 1e-2
    (a, _), ref = _spiked("bfloat16", 0, 64, 63, 19, softcap=4.0, sink=4.0, flash=True)
    assert 0.28 < ref[19] < 0.33 and np.abs(a - ref).max() < 2e-2
    (a, _), ref = _spiked("bfloat16", 0, 64, 63, 19, softcap=4.0, sink=40.0, flash=True)
    assert np.abs(a).max() < 1e-10
    (a, _), ref = _spiked("bfloat16", 0, 64, 63, 19, softcap=4.0, sink=400.0, flash=True)     # beyond what a float holds
    assert np.abs(a).max() == 0
    (a, _), ref = _spiked("bfloat16", 16, 64, 63, 50, softcap=4.0, sink=1.0, gate=-1.0, flash=True)
    assert np.abs(a - ref).max() < 2e-2 and ref[50] < 0.27
    assert ops.choices["window_flash_attention"] >= before + 18


@pytest.mark.parametrize("D", [64, 128])
def test_long_steps_of_one_head_size_on_tcgen05_see_the_same_keys_and_the_same_sink(D):
    """The tcgen05 kernel with roles, which long bfloat16 steps with keys and values of 64 or of 128 channels use: keys
    at the edges of the query's block, on tile borders and far away; the sink, the cap and the gate."""
    from kv_cache_optimization_for_llm_b200 import ops
    size, T, query = 37, 250, 245            # the query's block starts at 222
    before = ops.choices["flash_attention_rows_masked"]
    for key, seen in ((222, True), (221, False), (0, False), (query, True), (223, True), (192, False), (191, False), (185, False)):
        (in_prompt, _), ref = _spiked("bfloat16", size, T, query, key, flash="tcgen05", D=D)
        if seen:
            assert in_prompt[key % D] > 0.99 and abs(in_prompt[key % D] - ref[key % D]) < 1e-2, (key, in_prompt[key % D])
        assert np.abs(in_prompt - ref).max() < 1e-2, key
    for key in (2, 0, 63, 64, 127, 128):      # no blocks: every key up to the query, across all tiles
        (in_prompt, _), ref = _spiked("bfloat16", 0, 250, 249, key, flash="tcgen05", D=D)
        assert in_prompt[key % D] > 0.99 and np.abs(in_prompt - ref).max() < 1e-2
    (a, _), ref = _spiked("bfloat16", 0, 64, 63, 19, softcap=4.0, flash="tcgen05", D=D)
    assert 0.4 < ref[19] < 0.5 and np.abs(a - ref).max() < 2e-2
    (a, _), ref = _spiked("bfloat16", 0, 64, 63, 19, softcap=4.0, sink=4.0, flash="tcgen05", D=D)
    assert 0.28 < ref[19] < 0.33 and np.abs(a - ref).max() < 2e-2
    (a, _), ref = _spiked("bfloat16", 0, 64, 63, 19, softcap=4.0, sink=400.0, flash="tcgen05", D=D)     # beyond what a float holds
    assert np.abs(a).max() == 0
    (a, _), ref = _spiked("bfloat16", 16, 64, 63, 50, softcap=4.0, sink=1.0, gate=-1.0, flash="tcgen05", D=D)
    assert np.abs(a - ref).max() < 2e-2 and ref[50] < 0.27
    assert ops.choices["flash_attention_rows_masked"] >= before + 18


@pytest.mark.parametrize("kind,shape", [
    ("attention", dict(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.125, size=50, rot_dims=64)),
    ("attention_2", dict(heads=4, kv_heads=1, dim=128, vdim=128, scale=0.09, size=33, rot_dims=32, softcap=30.0, scaling=tiny.YARN)),
    ("attention_2", dict(heads=2, kv_heads=2, dim=64, vdim=64, scale=0.125, size=None, rot_dims=16, softcap=5.0)),
])
def test_the_mixer_on_tcgen05_in_portions_and_beside_another_request(kind, shape, monkeypatch):
    """The whole mixer with every step that carries a run of tokens on the tcgen05 kernel (as long steps are by
    themselves), against the plain attention and against the same tokens cut otherwise."""
    from kv_cache_optimization_for_llm_b200 import ops
    monkeypatch.setattr(ops, "FLASH_ROWS_WIDE", 3)
    rng = np.random.default_rng(8)
    ctx = _ctx("bfloat16")
    H = 40
    m = tiny.attention(**shape)
    wt, w64 = _att_weights(rng, H, m, kind)
    mixer = _make("mixer", "rotary_chunk_attention", _att_params(H, m, kind), wt, ctx)
    xs, refs = {}, {}
    for r, T in enumerate((70, 33)):
        x, x64 = _w(rng, (T, H), 1.0)
        xs[r], refs[r] = x.to(torch.bfloat16).cuda(), S.attention_mixer(x64, w64, "", m, kind, 1e-5)
    before = ops.choices["flash_attention_rows_masked"]
    whole = _run_in_steps(mixer, ctx, xs, [[(0, 70)], [(1, 33)]])
    cut = _run_in_steps(mixer, ctx, xs, [[(0, 8), (1, 1)], [(0, 9), (1, 1)], [(0, 2), (1, 30)], [(0, 1), (1, 1)],
                                         [(0, 44)], [(0, 1)], [(0, 1)], [(0, 4)]])
    assert ops.choices["flash_attention_rows_masked"] >= before + 7
    for r in xs:
        assert _err(whole[r], refs[r], "bfloat16") < TOL["bfloat16"]
        assert _err(cut[r], refs[r], "bfloat16") < TOL["bfloat16"]


# --------------------------------------------------------------------------- the matrix memory

def _mlstm_weights(rng, H, m, forget_bias=2.0):
    Hh, D, Dv = m["heads"], m["dim"], m["vdim"]
    wt, w64 = {}, {}
    for role, name, shape, std, mean in (("q", "q", (Hh * D, H), 0.3, 0), ("k", "k", (Hh * D, H), 0.3, 0),
                                         ("v", "v", (Hh * Dv, H), 0.3, 0), ("g", "g", (Hh * Dv, H), 0.3, 0),
                                         ("i", "i", (Hh, H), 0.4, 0), ("f", "f", (Hh, H), 0.4, 0),
                                         ("i_bias", "i.b", (Hh,), 1.0, 0), ("f_bias", "f.b", (Hh,), 1.0, forget_bias),
                                         ("norm", "norm", (Hh * Dv,), 0.2, 1.0), ("o", "o", (H, Hh * Dv), 0.3, 0)):
        wt[role], w64[name] = _w(rng, shape, std, mean)
    return wt, w64


def _mlstm_params(H, m, eps=1e-5):
    return {"hidden_size": H, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"], "gate_cap": m["gate_cap"], "eps": eps}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [dict(), dict(heads=1, dim=5, vdim=3, gate_cap=2.0), dict(heads=2, dim=16, vdim=16, gate_cap=15.0),
                                   dict(heads=2, dim=8, vdim=72, gate_cap=6.0), dict(heads=4, dim=64, vdim=32, gate_cap=12.0),
                                   dict(heads=1, dim=130, vdim=136, gate_cap=10.0)])
def test_matrix_memory_alone_in_portions_and_beside_another_request(dtype, shape):
    """Several shapes (one head, keys that are no multiple of four wide, values wider than one block's 64 columns),
    70 and 33 tokens; the state slots start full of rubbish, which a request that starts at position 0 must not read."""
    rng = np.random.default_rng(4)
    ctx = _ctx(dtype)
    H = 40
    m = tiny.mlstm(**shape)
    wt, w64 = _mlstm_weights(rng, H, m)
    mixer = _make("mixer", "mlstm", _mlstm_params(H, m), wt, ctx)
    xs, refs = {}, {}
    for r, T in enumerate((70, 33)):
        x, x64 = _w(rng, (T, H), 1.0)
        xs[r], refs[r] = x.to(DT[dtype]).cuda(), S.mlstm_mixer(x64, w64, "", m, 1e-5)
    whole = _run_in_steps(mixer, ctx, xs, [[(0, 70)], [(1, 33)]])
    cut = _run_in_steps(mixer, ctx, xs, [[(0, 8), (1, 1)], [(0, 9), (1, 1)], [(0, 2), (1, 30)], [(0, 1), (1, 1)],
                                         [(0, 44)], [(0, 1)], [(0, 1)], [(0, 4)]])
    one = _run_in_steps(mixer, ctx, {0: xs[1]}, [[(0, 1)]] * 33)
    tol = 1e-4 if dtype == "float32" else TOL[dtype]
    for r in xs:
        assert _err(whole[r], refs[r], dtype) < tol
        assert _err(cut[r], refs[r], dtype) < tol
        assert _err(cut[r], whole[r].double().numpy(), dtype) < tol
    assert _err(one[0], whole[1].double().numpy(), dtype) < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_running_maximum_starts_at_zero_and_the_gates_are_capped(dtype):
    """The kernel alone on made-up gates.  A first token whose input gate is far below zero: with a maximum that
    starts at 0 the read-out is divided by exp(-m) = 1, not by |n . q|; raw gates far above the cap count as the cap."""
    from kv_cache_optimization_for_llm_b200 import ops
    from kv_cache_optimization_for_llm_b200.engine.batch import BatchBuilder, StepEntry
    ctx = _ctx(dtype)
    rng = np.random.default_rng(5)
    T, D, Dv, cap = 6, 8, 4, 5.0
    q, k, v = (np.round(rng.normal(size=(T, n)) * 4) / 4 for n in (D, D, Dv))
    raw_i = np.array([-3.0, -2.5, 40.0, 0.5, -60.0, 1.0])
    raw_f = np.array([1.0, 30.0, -30.0, 0.0, 2.0, 2.0])
    gi, gf = S.soft_cap(raw_i, cap), S.log_sigmoid(S.soft_cap(raw_f, cap))
    ref = S.matrix_memory(q * 0.5, k, v, gi, gf)
    src = torch.as_tensor(np.concatenate([q, k, v], axis=1), dtype=torch.float32).to(DT[dtype]).cuda()
    gates = _f32(np.stack([raw_i, raw_f], axis=1))
    state = torch.full((2, ops.mlstm_state_floats(1, D, Dv)), 9.0, dtype=torch.float32, device="cuda")
    builder = BatchBuilder(64, 4, [8], ctx.device, ctx.status)
    got, at = [], 0
    for n in (2, 1, 3):
        batch = builder.build([StepEntry(0, [0] * n, at, ())], _Manager({0: list(range(8))}, {0: 1}))
        got.append(ops.mlstm_scan(src[at:at + n].contiguous(), 0, D, 2 * D, gates[at:at + n].contiguous(), _f32([0.0]), _f32([0.0]),
                                  cap, 0.5, state, batch, 1, D, Dv).cpu())
        at += n
    got = torch.cat(got).numpy()
    assert np.abs(got - ref).max() < 1e-5 * np.abs(ref).max()
    # what a maximum that started at minus infinity would give for the first token: C^T q / |n . q|
    first_wrong = (v[0] * (k[0] @ q[0] * 0.5)) / abs(k[0] @ q[0] * 0.5)
    assert np.abs(first_wrong - ref[0]).max() > 0.1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_runs_are_walked_in_chunks_side_by_side_and_states_last_for_hundreds_of_tokens(dtype):
    """A run of 700 tokens (cut into chunks of 64 that are walked side by side) beside a short one, then 40 tokens one
    by one; forget gates near one, so that the first tokens still show at the end."""
    from kv_cache_optimization_for_llm_b200 import ops
    rng = np.random.default_rng(6)
    ctx = _ctx(dtype, max_positions=2048)
    H = 24
    m = tiny.mlstm(heads=2, dim=12, vdim=68, gate_cap=8.0)
    wt, w64 = _mlstm_weights(rng, H, m, forget_bias=30.0)      # every forget gate at its cap: log f = -0.0003
    mixer = _make("mixer", "mlstm", _mlstm_params(H, m), wt, ctx)
    xs, refs = {}, {}
    for r, T in enumerate((740, 90)):
        x, x64 = _w(rng, (T, H), 1.0)
        xs[r], refs[r] = x.to(DT[dtype]).cuda(), S.mlstm_mixer(x64, w64, "", m, 1e-5)
    before = ops.choices["mlstm_scan_chunked"]
    got = _run_in_steps(mixer, ctx, xs, [[(1, 5)], [(0, 700), (1, 1)], [(1, 84)]] + [[(0, 1)]] * 40, page=16, state_slots=4)
    assert ops.choices["mlstm_scan_chunked"] > before
    short = _run_in_steps(mixer, ctx, xs, [[(0, 200), (1, 90)], [(0, 255)], [(0, 245)]] + [[(0, 1)]] * 40, page=16,
                          state_slots=4)
    tol = 2e-4 if dtype == "float32" else TOL[dtype]
    for r in xs:
        assert _err(got[r], refs[r], dtype) < tol and _err(short[r], refs[r], dtype) < tol
    # the memory of the first tokens is still there at the end: without them the last rows are other numbers
    late = S.mlstm_mixer(xs[0][100:].double().cpu().numpy(), w64, "", m, 1e-5)
    assert np.abs(late[-1] - refs[0][-1]).max() > 1e-3 * np.abs(refs[0][-1]).max()


# --------------------------------------------------------------------------- the experts

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [dict(), dict(experts=3, top=1, ff=16, limit=2.0, shared_ff=0),
                                   dict(experts=4, top=4, ff=8, limit=0.3, shared_ff=8, shared_limit=5.0),
                                   dict(experts=9, top=3, ff=5, limit=0.9, shared_ff=3, shared_limit=0.2),
                                   dict(experts=1, top=1, ff=24, limit=1.0, shared_ff=24, shared_limit=1.0)])
def test_experts_weigh_their_input_and_limit_both_products(dtype, shape):
    """Routed experts with limits low enough that many features meet them, so that a weight on the output instead of
    the input, a limit on the wrong side, or renormalised weights would show; with and without the shared expert."""
    rng = np.random.default_rng(7)
    ctx = _ctx(dtype)
    H, T = 40, 29
    mlp = tiny.moe(**shape)
    E, F = mlp["router"]["experts"], mlp["expert"]["ff"]
    SF = mlp["shared"]["ff"] if mlp.get("shared") else 0
    wt, w64 = {}, {}
    wt["router"], w64["router"] = _w(rng, (E, H), 0.5)
    for e in range(E):
        for role, shp in (("gate", (F, H)), ("up", (F, H)), ("down", (H, F))):
            wt[f"{role}{e}"], w64[f"e{e}.{role}"] = _w(rng, shp, 0.3)
    if SF:
        for role, shp in (("gate", (SF, H)), ("up", (SF, H)), ("down", (H, SF)), ("sg", (1, H))):
            wt[f"shared_{role}"], w64[f"shared.{role}"] = _w(rng, shp, 0.3)
    params = {"hidden_size": H, "experts": E, "top": mlp["router"]["top"], "expert_ff": F, "limit": mlp["expert"]["limit"],
              "shared_ff": SF, "shared_limit": mlp["shared"]["limit"] if SF else None, "alpha": 1.702}
    ff = _make("feed_forward", "limited_experts", params, wt, ctx)
    x, x64 = _w(rng, (T, H), 1.0)
    got = ff.forward(x.to(DT[dtype]).cuda(), None)
    ref = S.moe(x64, w64, "", mlp)
    assert _err(got, ref, dtype) < TOL[dtype]
    # the wrong readings are far away: the weight on the output, and weights that sum to one
    chosen, weight = S.route(x64, w64["router"], mlp["router"]["top"])
    on_output = np.zeros_like(ref)
    for t in range(T):
        for e, c in zip(chosen[t], weight[t]):
            on_output[t] += c * S.limited_expert(x64[t][None], w64[f"e{e}.gate"], w64[f"e{e}.up"], w64[f"e{e}.down"],
                                                 mlp["expert"]["limit"])[0]
    if SF:
        on_output += S.limited_expert(x64, w64["shared.gate"], w64["shared.up"], w64["shared.down"], mlp["shared"]["limit"]) \
            * S.sigmoid(x64 @ w64["shared.sg"].T)
    assert np.sqrt(((on_output - ref) ** 2).mean()) > 0.05 * np.sqrt((ref ** 2).mean())


def test_router_scores_are_sigmoids_taken_as_they_are():
    from kv_cache_optimization_for_llm_b200 import ops
    logits = _f32([[2.0, -1.0, 0.5, 3.0, -4.0, 9.0], [0.1, 0.2, 0.3, -0.1, 0.0, 7.0], [-5.0, -6.0, -7.0, -8.0, -9.0, 1.0]])
    x = torch.zeros((3, 8), dtype=torch.float32, device="cuda")
    gate, _ = ops.route(x, None, None, 5, 0, 2, 1.0, logits, score="sigmoid", renormalize=False)     # the sixth column is not the router's
    ref = np.zeros((3, 5))
    ref[0, 3], ref[0, 0] = S.sigmoid(3.0), S.sigmoid(2.0)
    ref[1, 2], ref[1, 1] = S.sigmoid(0.3), S.sigmoid(0.2)
    ref[2, 0], ref[2, 1] = S.sigmoid(-5.0), S.sigmoid(-6.0)
    assert np.abs(gate.cpu().numpy() - ref).max() < 1e-6


# --------------------------------------------------------------------------- whole models

def _runner(folder, dtype, **kw):
    from kv_cache_optimization_for_llm_b200 import EngineConfig
    from kv_cache_optimization_for_llm_b200.engine.runner import ModelRunner
    args = dict(dtype=dtype, page_size=8, num_pages=40, max_num_seqs=3, max_num_batched_tokens=256, max_model_len=160,
                use_cuda_graphs=False)
    args.update(kw)
    return ModelRunner(folder, EngineConfig(**args))


def _logit_err(got, ref, dtype="float32"):
    """float32: the largest difference over the largest value.  bfloat16: root mean square of the differences over
    that of the values, row by row, and of the rows' figures the one that four in five stay below: where two experts'
    scores lie within a rounding of each other the choice may go either way, which changes a few rows much and says
    nothing about the kernels; all rows together must still stay below three times the limit."""
    if dtype == "float32":
        return np.abs(got - ref).max() / np.abs(ref).max()
    scale = np.sqrt((ref ** 2).mean())
    rows = np.sqrt(((got - ref) ** 2).mean(axis=-1)) / scale
    if rows.ndim == 0 or rows.size < 5:
        return float(np.max(rows))
    return max(float(np.quantile(rows, 0.8)), float(np.sqrt((rows ** 2).mean())) / 3.0)


def _close(a, b, dtype):
    """Two runs of the engine that cut the same tokens differently."""
    return _logit_err(a, b, dtype) < (5e-5 if dtype == "float32" else TOL_MODEL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_model_prefill_decoding_portions_batches_and_reuse(dtype):
    """A model with all kinds of mixer, a layer without feed-forward and layers that use another layer's tensors.
    Whole prompts; token by token; portions of 2, 3, 7, ... beside single tokens of another request; then requests
    that end and others that take over their slots and pages in a pool that holds two of them at most; 60 decoded
    tokens in a row, past every block's end."""
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    folder = tempfile.mkdtemp(prefix="kvb200_tv_")
    cfg = tiny.MIXED
    w = tiny.write_model(folder, cfg, seed=1)
    r = _runner(folder, dtype)
    assert len(r.spec.schedule) == 7 and len(r.spec.layers) == 4
    assert len(r.cache.states) == 2        # the two mLSTM applications keep a state each, with the same tensors
    rng = np.random.default_rng(5)
    seqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in (90, 37, 61, 1, 150)]
    refs = [S.forward(cfg, w, s) for s in seqs]
    tol = TOL_MODEL[dtype]
    whole = r.step([StepEntry(0, seqs[1], 0, range(37))]).cpu().numpy()
    assert _logit_err(whole, refs[1], dtype) < tol
    r.release(0)
    single = np.concatenate([r.step([StepEntry(1, [t], i, [0])]).cpu().numpy() for i, t in enumerate(seqs[1])])
    assert _logit_err(single, refs[1], dtype) < tol
    assert _close(whole, single, dtype)
    r.release(1)
    got2 = [r.step([StepEntry(12, seqs[2][:20], 0, range(20))]).cpu().numpy()]
    pos0, pos2, got0 = 0, 20, []
    for n in (2, 3, 7, 1, 8, 16, 2, 9, 5, 1, 1, 30, 2, 3):
        entries = [StepEntry(10, seqs[0][pos0:pos0 + n], pos0, range(n))]
        if pos2 < len(seqs[2]):
            entries.insert(0 if n % 2 else 1, StepEntry(12, [seqs[2][pos2]], pos2, [0]))
        if n == 7:
            entries.append(StepEntry(13, seqs[3], 0, [0]))
        out = r.step(entries).cpu().numpy()
        i = 0
        for e in entries:
            k = len(e.want)
            if e.request_id == 10:
                got0.append(out[i:i + k])
            elif e.request_id == 12:
                got2.append(out[i:i + k])
                pos2 += 1
            else:
                assert _logit_err(out[i:i + k], refs[3], dtype) < tol
                r.release(13)
            i += k
        pos0 += n
    assert pos0 == 90
    assert _logit_err(np.concatenate(got0), refs[0], dtype) < tol
    assert _logit_err(np.concatenate(got2), refs[2][:pos2], dtype) < tol
    r.check_status()
    r.release(10)
    r.release(12)
    assert r.manager.check() == ""
    long = [r.step([StepEntry(20, seqs[4][:90], 0, range(90))]).cpu().numpy()]
    for i in range(90, 150):
        long.append(r.step([StepEntry(20, [seqs[4][i]], i, [0])]).cpu().numpy())
    assert _logit_err(np.concatenate(long), refs[4], dtype) < tol
    r.check_status()
    r.release(20)
    assert all(r.manager.free_pages(g) == 40 for g in range(r.manager.num_groups()))


def test_the_stream_after_every_layer():
    """float32: the residual stream after each application of a layer, against the plain model's."""
    from kv_cache_optimization_for_llm_b200 import ops
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    folder = tempfile.mkdtemp(prefix="kvb200_tv_")
    cfg = tiny.MIXED
    w = tiny.write_model(folder, cfg, seed=3)
    r = _runner(folder, "float32")
    seq = np.random.default_rng(2).integers(0, cfg["vocab"], 30).tolist()
    _, after = S.forward(cfg, w, seq, keep_layers=True)
    seen = []
    for block in r.model.layers:
        inner = block.forward

        def spy(residual, delta, batch, cache, inner=inner):
            residual, pending = inner(residual, delta, batch, cache)
            copy = residual.clone()
            ops.add_norm(copy, pending, None, None, 0.0, torch.float32)       # what is pending joins a copy of the stream
            seen.append(copy.cpu().numpy())
            return residual, pending
        block.forward = spy
    r.step([StepEntry(0, seq, 0, [29])])
    assert len(seen) == len(after) == 7
    for i, (got, ref) in enumerate(zip(seen, after)):
        assert np.abs(got - ref).max() < 2e-5 * np.abs(ref).max(), f"after layer {i}"


@pytest.mark.parametrize("layers,width,kw", [
    # one layer of each kind alone
    ([tiny.layer("mlstm", tiny.mlstm(heads=2, dim=8, vdim=8, gate_cap=4.0), tiny.moe(experts=2, top=1, ff=8, shared_ff=8))], 32, {}),
    ([tiny.layer("attention", tiny.attention(heads=2, kv_heads=1, dim=8, vdim=8, size=6, rot_dims=8))], 32, {}),
    ([tiny.layer("attention_2", tiny.attention(heads=2, kv_heads=2, dim=8, vdim=16, size=9, rot_dims=4, softcap=2.0,
                                                scaling=tiny.YARN), tiny.moe(experts=4, top=4, ff=8, shared_ff=0))], 32, {}),
    # where the numbers that could be equal are not, constants that are 1 or absent, every channel turning, no blocks
    ([tiny.layer("attention_2", tiny.attention(heads=6, kv_heads=3, dim=24, vdim=40, scale=0.11, size=None, rot_dims=24,
                                                base=77.0, softcap=None), tiny.moe(experts=7, top=3, ff=24, limit=0.5,
                                                                                   shared_ff=40, shared_limit=3.0)),
      tiny.layer("mlstm", tiny.mlstm(heads=5, dim=20, vdim=12, gate_cap=20.0)),
      tiny.layer("attention", tiny.attention(heads=1, kv_heads=1, dim=96, vdim=16, scale=0.05, size=64, rot_dims=None),
                 tiny.moe(experts=2, top=2, ff=104, shared_ff=8)),
      tiny.layer("mlstm", tiny.mlstm(heads=5, dim=20, vdim=12, gate_cap=20.0), weights_of=1),
      tiny.layer("mlstm", tiny.mlstm(heads=1, dim=4, vdim=100, gate_cap=1.0), tiny.moe())], 104,
     dict(emb_scale=1.0, mult=1.0, logit_scale=1.0, logit_softcap=None)),
    # sizes that are no multiples of eight: nothing may rest on 16-byte rows
    ([tiny.layer("attention", tiny.attention(heads=3, kv_heads=1, dim=5, vdim=3, scale=0.4, size=7, rot_dims=2),
                 tiny.moe(experts=3, top=2, ff=9, shared_ff=5)),
      tiny.layer("mlstm", tiny.mlstm(heads=3, dim=5, vdim=7, gate_cap=3.0), tiny.moe(experts=2, top=1, ff=3, shared_ff=0)),
      tiny.layer("attention_2", tiny.attention(heads=2, kv_heads=2, dim=6, vdim=9, scale=0.4, size=3, rot_dims=6,
                                                softcap=1.0, scaling=tiny.YARN))], 36, dict(mult=2.5, logit_softcap=0.5)),
    # the same layer four times over, each application with a cache of its own
    ([tiny.layer("attention", tiny.attention(), tiny.moe())] + [tiny.layer("attention", tiny.attention(), tiny.moe(), weights_of=0)] * 3,
     48, {}),
])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_orders_of_layers_sizes_and_constants(layers, width, kw, dtype):
    """A prompt in three portions and four tokens one by one, against the plain model."""
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    folder = tempfile.mkdtemp(prefix="kvb200_tv_")
    cfg = tiny.config(layers, width=width, vocab=53, eps=1e-6, **kw)
    # a seed with which no head's read-out comes out near zero in front of its norm at any of these tokens: the norm
    # would turn float32 rounding into a difference a thousand times larger, in the plain model as much as here
    w = tiny.write_model(folder, cfg, seed=7)
    r = _runner(folder, dtype)
    seq = np.random.default_rng(1).integers(0, 53, 44).tolist()
    ref = S.forward(cfg, w, seq)
    got, pos = [], 0
    for n in (11, 2, 27, 1, 1, 1, 1):
        got.append(r.step([StepEntry(0, seq[pos:pos + n], pos, range(n))]).cpu().numpy())
        pos += n
    assert _logit_err(np.concatenate(got), ref, dtype) < TOL_MODEL[dtype]
    r.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["mixed", "attention_only"])
def test_greedy_generation_through_the_engine_and_its_scheduler(dtype, which):
    """Prompts of unequal length through ``LLM.generate``: the scheduler's portions (a token budget of 24 per step),
    decode steps replayed from CUDA graphs, the engine one step ahead, five requests in three seats.  Every sampled
    row's logits are compared with the plain model on the final sequences, and in float32 the greedy tokens themselves.
    The model without a matrix memory has no state of fixed size, so that its lone prompt portions and its steps of
    single tokens beside one portion are replayed from graphs too (with dummy tokens behind the run)."""
    from kv_cache_optimization_for_llm_b200 import LLM, SamplingParams
    from logit_hook import LogitRecorder
    folder = tempfile.mkdtemp(prefix="kvb200_tv_")
    cfg = tiny.MIXED if which == "mixed" else tiny.ATTENTION_ONLY
    w = tiny.write_model(folder, cfg, seed=4)
    llm = LLM(folder, dtype=dtype, page_size=8, num_pages=48, max_num_seqs=3, max_num_batched_tokens=24,
              max_model_len=128, use_cuda_graphs=True, run_ahead=True)
    rec = LogitRecorder(llm.engine.runner)
    rng = np.random.default_rng(9)
    prompts = [rng.integers(0, cfg["vocab"], n).tolist() for n in (3, 41, 17, 1, 30)]
    outs = llm.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True))
    assert [len(o) for o in outs] == [12] * 5
    seqs = {i: prompts[i] + outs[i] for i in range(5)}
    plain = {i: S.forward(cfg, w, seqs[i]) for i in seqs}
    if dtype == "float32":
        n, worst = rec.compare(seqs, lambda i: plain[i], TOL_MODEL[dtype], "greedy generation")
    else:       # the measure of this file's other bfloat16 comparisons: over all of a request's rows at once
        got = rec.collect(seqs)
        n = sum(len(ps) for ps, _ in got.values())
        for i, (ps, rows) in got.items():
            assert _logit_err(rows, plain[i][ps], dtype) < TOL_MODEL[dtype], f"greedy generation: request {i}"
    assert n >= 60 and llm.engine.runner._graphs
    if dtype == "float32":
        for i in seqs:
            for j, tok in enumerate(outs[i]):
                row = plain[i][len(prompts[i]) + j - 1]
                assert row[tok] >= row.max() - 1e-4 * np.abs(row).max(), (i, j)
    assert llm.engine.runner.manager.check() == ""


@pytest.mark.parametrize("dtype,flags", [("float32", ()), ("bfloat16", ()), ("float32", ("--cuda-graphs",))])
def test_replay_through_the_trace_runner(dtype, flags):
    """bin/trace_run on a Tevanex folder: each request whole, then four live requests whose portions (down to two
    tokens) run beside single tokens in a pool that holds exactly them, in four state slots; requests that end hand
    pages and slots to the ones that follow."""
    from trace_driver import TraceRun, ceil64
    folder = tempfile.mkdtemp(prefix="kvb200_tv_")
    cfg = tiny.MIXED
    w = tiny.write_model(folder, cfg, seed=9)
    rng = np.random.default_rng(2)
    seqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in (70, 33, 50, 21)]
    refs = [S.forward(cfg, w, s) for s in seqs]
    tol = TOL_MODEL[dtype]
    tr = TraceRun(folder, dtype, sum(ceil64(len(s)) for s in seqs), ("--page-size", "8") + tuple(flags))
    try:
        for r, s in enumerate(seqs):
            got = tr.step([(f"w{r}", s, range(len(s)))], end=[f"w{r}"])
            assert _logit_err(got, refs[r], dtype) < tol, f"whole request {r}"
        for round_ in range(2):         # the second round runs in slots and pages that the first gave back
            plans = {0: [5, 2, 16, 9, 2, 30] + [1] * 6, 1: [1, 1, 20, 2] + [1] * 9, 2: [33, 2, 3, 2] + [1] * 10,
                     3: [2, 2, 2, 7] + [1] * 8}
            pos = {r: 0 for r in plans}
            step = 0
            while plans:
                entries, expect, ends = [], [], []
                for r in sorted(plans):
                    if step < r:        # they start one step apart
                        continue
                    n = plans[r].pop(0)
                    entries.append((f"m{round_}_{r}", seqs[r][pos[r]:pos[r] + n], range(n)))
                    expect.append(refs[r][pos[r]:pos[r] + n])
                    pos[r] += n
                    if not plans[r]:
                        assert pos[r] == len(seqs[r])
                        ends.append(f"m{round_}_{r}")
                        del plans[r]
                got = tr.step(entries, end=ends)
                assert _logit_err(got, np.concatenate(expect), dtype) < tol, f"round {round_}, mixed step {step}"
                step += 1
    finally:
        tr.close()


def test_command_line_serves_the_design():
    """The engine's command line on a Tevanex folder: requests on standard input in the wire format, greedy tokens
    back as JSON lines; each token is the plain model's best (ties within 1e-4 allowed)."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder = tempfile.mkdtemp(prefix="kvb200_tv_")
    cfg = tiny.MIXED
    w = tiny.write_model(folder, cfg, seed=8)
    rng = np.random.default_rng(4)
    prompts = {3: rng.integers(0, cfg["vocab"], 9).tolist(), 11: rng.integers(0, cfg["vocab"], 26).tolist()}
    lines = [f"{rid} 6 1 " + " ".join(map(str, toks)) for rid, toks in prompts.items()]
    env = dict(os.environ, IGNORE_EOS="1", PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    p = subprocess.run([sys.executable, "-m", "kv_cache_optimization_for_llm_b200.cli", folder, "--dtype", "float32",
                        "--page-size", "4", "--num-pages", "64", "--max-num-seqs", "4", "--max-model-len", "64"],
                       input="\n".join(lines) + "\n", capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    out = [json.loads(line) for line in p.stdout.splitlines() if line.strip()]
    for rid, prompt in prompts.items():
        toks = [m["tok"] for m in out if m.get("id") == rid and "tok" in m]
        assert len(toks) == 6
        logits = S.forward(cfg, w, prompt + toks)
        for j, tok in enumerate(toks):
            row = logits[len(prompt) + j - 1]
            assert row[tok] >= row.max() - 1e-4 * np.abs(row).max(), (rid, j)
