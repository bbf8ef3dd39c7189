"""The Solulix design on the GPU against its plain restatement (tests/plain_solulix.py): each
mechanism alone, then whole models through the step function, the cache, the scheduler, the
generation entry point and the trace runner, in float32 and bfloat16."""

import os
import tempfile

import numpy as np
import pytest
import torch

import plain_solulix as S
import tiny_solulix as tiny

pytestmark = pytest.mark.gpu

from part_harness import DT, TOL, TOL_MODEL, _Manager, _ctx, _err, _make, _rel, _run_in_steps, _same, _w  # noqa: E402


# --------------------------------------------------------------------------- what joins the residual stream

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H", [40, 333])
def test_two_branches_rows_and_a_vector_join_the_stream_before_the_norm(dtype, H):
    from kv_cache_optimization_for_llm_b200 import ops
    rng = np.random.default_rng(H)
    T = 7
    f32 = lambda a: torch.as_tensor(a, dtype=torch.float32).cuda()
    d64 = lambda t: t.cpu().numpy().astype(np.float64)
    res0 = d64(f32(rng.normal(size=(T, H)) * 2 + 0.5))
    (a_t, a), (b_t, b) = _w(rng, (T, H), 1.5, 0.7), _w(rng, (T, H), 0.5, -0.2)
    e, vec, w = d64(f32(rng.normal(size=(T, H)))), d64(f32(rng.normal(size=H))), d64(f32(1 + 0.2 * rng.normal(size=H)))
    dev = lambda t: t.to(DT[dtype]).cuda()
    for deltas, ref_add, rows_, vec_ in (((dev(a_t), dev(b_t)), a + b, None, None), ((dev(a_t),), a, f32(e), f32(vec)),
                                         ((), 0 * a, None, f32(vec)), ((dev(a_t), dev(b_t)), a + b, f32(e), f32(vec))):
        pending = ops.PendingSum(deltas, rows_, vec_)
        want_res = res0 + ref_add + (e if rows_ is not None else 0) + (vec if vec_ is not None else 0)
        want = S.rms_norm(want_res, w, 1e-5)
        resid = f32(res0)
        pick = torch.tensor([5, 0, 5], dtype=torch.int32, device="cuda")
        picked = ops.join_norm(resid, pending, "rms", f32(w), 1e-5, DT[dtype], pick, compute_dtype=DT[dtype])
        assert np.array_equal(d64(resid), res0), "picking rows must leave the residual alone"
        assert _rel(picked, want[[5, 0, 5]]) < TOL[dtype]
        out = ops.join_norm(resid, pending, "rms", f32(w), 1e-5, DT[dtype], compute_dtype=DT[dtype])
        assert _rel(out, want) < TOL[dtype]
        assert _rel(resid, want_res) < 3e-6, "the residual is float32 in both precisions"
    # the normed embedding: float32 out whatever the compute type
    out = ops.join_norm(f32(res0), None, "rms", f32(w), 1e-5, torch.float32, compute_dtype=DT[dtype])
    assert out.dtype == torch.float32 and _rel(out, S.rms_norm(res0, w, 1e-5)) < 3e-6


# --------------------------------------------------------------------------- attention

def _attention_weights(rng, H, mx):
    Hq, G, D, Dv, taps = (mx[k] for k in ("heads", "kv_heads", "dim", "vdim", "conv"))
    wt, w64 = {}, {}
    for role, name, shape, std in (("q", "q", (Hq * D, H), 0.3), ("k", "k", (G * D, H), 0.3), ("v", "v", (G * Dv, H), 0.3),
                                   ("q_conv", "q.conv", (Hq * D, taps), 0.6), ("k_conv", "k.conv", (G * D, taps), 0.6),
                                   ("v_conv", "v.conv", (G * Dv, taps), 0.6), ("o", "o", (H, Hq * Dv), 0.3)):
        wt[role], w64[name] = _w(rng, shape, std)
    return wt, w64


def _attention_mixer(mx, wt, ctx, H):
    return _make("mixer", "conv_window_attention", {
        "hidden_size": H, "heads": mx["heads"], "kv_heads": mx["kv_heads"], "dim": mx["dim"], "vdim": mx["vdim"],
        "conv": mx["conv"], "scale": mx["scale"], "window": mx["mask"]["size"], "keep_first": mx["mask"]["keep_first"],
        "one_more": True}, wt, ctx)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [dict(), dict(heads=6, kv_heads=1, dim=24, vdim=8, conv=4, size=5, keep_first=9),
                                   dict(heads=2, kv_heads=2, dim=8, vdim=40, conv=1, size=16, keep_first=0),
                                   dict(heads=3, kv_heads=1, dim=64, vdim=64, conv=2, size=33, keep_first=1),
                                   dict(heads=1, kv_heads=1, dim=5, vdim=3, conv=7, size=1, keep_first=2),
                                   dict(heads=4, kv_heads=4, dim=32, vdim=16, conv=3, size=200, keep_first=8)])
def test_attention_alone_in_portions_and_beside_another_request(dtype, shape):
    """Several shapes (key and value sizes that differ, one tap, a window of one token, a window wider
    than the sequence, kept tokens beyond the window), 70 and 33 tokens on pages of 8 that lie
    scattered; portions end inside pages and on their borders and are shorter than the taps."""
    rng = np.random.default_rng(3)
    ctx = _ctx(dtype)
    H = 40
    mx = tiny.attention(**shape)["mixer"]
    wt, w64 = _attention_weights(rng, H, mx)
    mixer = _attention_mixer(mx, wt, ctx, H)
    xs, refs = {}, {}
    for r, T in enumerate((70, 33)):
        x, x64 = _w(rng, (T, H), 1.0)
        xs[r], refs[r] = x.to(DT[dtype]).cuda(), S.attention_mixer(x64, w64, "", mx)
    whole = _run_in_steps(mixer, ctx, xs, [[(0, 70)], [(1, 33)]])
    cut = _run_in_steps(mixer, ctx, xs, [[(0, 8), (1, 1)], [(0, 9), (1, 1)], [(0, 2), (1, 30)], [(0, 1), (1, 1)],
                                         [(0, 44)], [(0, 1)], [(0, 1)], [(0, 4)]])
    one = _run_in_steps(mixer, ctx, {0: xs[1]}, [[(0, 1)]] * 33)
    for r in xs:
        assert _err(whole[r], refs[r], dtype) < TOL[dtype]
        assert _err(cut[r], refs[r], dtype) < TOL[dtype]
        assert _same(whole[r], cut[r], dtype), "a token's result must not depend on the cut or on the batch"
    assert _same(one[0], whole[1], dtype), "token by token"


def _spiked(dtype, size, keep_first, T, query, key, page=8, D=16, wide=None):
    """The attention kernels alone on keys and values made so that one key decides: every query and key
    is small but the pair (query, key), whose score is 30; the value of key j is the unit vector j (``D`` 16) or,
    with key and value size ``D`` both (the sizes the tensor-core kernel takes), the unit vector j mod D.
    Returns what the query at ``query`` reads, in a prompt (one portion) and decoded alone, and the plain answer."""
    from kv_cache_optimization_for_llm_b200 import ops
    from kv_cache_optimization_for_llm_b200.engine.batch import BatchBuilder, StepEntry
    ctx = _ctx(dtype)
    Dv = T if D == 16 else D
    rng = np.random.default_rng(T + query)
    q = rng.normal(size=(T, D)) * 0.01
    k = rng.normal(size=(T, D)) * 0.01
    q[query] = 0
    q[query, 3] = 6.0
    k[key] = 0
    k[key, 3] = 5.0
    v = np.eye(T) if D == 16 else np.eye(D)[np.arange(T) % D]
    src = torch.as_tensor(np.concatenate([q, k, v], axis=1), dtype=torch.float32).to(DT[dtype]).cuda()
    s = (q @ k.T).astype(np.float64)
    prob = S.one_more_softmax(s, S.visible(T, size or T, keep_first))      # size 0: no window
    ref = prob @ v
    outs = []
    before = ops.choices["flash_attention_rows"]
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
            if n > 1 and ops.flash_attention_rows_supported(D, Dv, 1, page, DT[dtype]):
                got = ops.flash_attention_rows(part, pages, batch.block_tables[0], batch, 1, 1, D, 1.0, size, keep_first, True,
                                               wide=wide)
            else:
                got = ops.window_attention(part, 0, pages, batch.block_tables[0], batch, 1, 1, D, Dv, 1.0, size, keep_first, True)
            rows.append(got.float().cpu())
            at += n
        outs.append(torch.cat(rows)[query].numpy())
    assert int(ctx.status.item()) == 0
    if D != 16 and dtype == "bfloat16":
        assert ops.choices["flash_attention_rows"] > before, "the tensor-core kernel was meant to run"
    return outs, ref[query]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_key_far_away_and_keys_at_the_edges_of_the_window_and_of_the_kept_tokens(dtype):
    """One key with a score that stands out among hundreds, placed just inside and just outside the
    window, just inside and just outside the kept first tokens, on a page's border, and at the
    sequence's very first token; the query in a prompt and decoded alone."""
    size, keep = 37, 6
    T, query = 250, 245
    for key, seen in ((query - size + 1, True), (query - size, False), (keep - 1, True), (keep, False), (0, True),
                      (query, True), (216, True), (215, True), (query - 130, False)):
        (in_prompt, decoded), ref = _spiked(dtype, size, keep, T, query, key)
        for got in (in_prompt, decoded):
            if seen:
                assert got[key] > 0.99 and abs(got[key] - ref[key]) < 1e-2, (key, got[key], ref[key])
            else:
                assert got[key] == 0 and ref[key] == 0, (key, got[key])
            assert np.abs(got - ref).max() < (2e-6 if dtype == "float32" else 1e-2)
    # no window: everything up to the query counts; the one more in the denominator keeps the sum below 1
    (in_prompt, decoded), ref = _spiked(dtype, 0, 0, 250, 249, 2)
    assert in_prompt[2] > 0.99 and abs(in_prompt.sum() - ref.sum()) < 1e-2 and ref.sum() < 1.0
    # the first tokens of a sequence: the one more counts most where there are few keys
    (in_prompt, decoded), ref = _spiked(dtype, 4, 1, 8, 0, 5)
    assert abs(in_prompt[0] - ref[0]) < 1e-2 and 0.4 < ref[0] < 0.6


@pytest.mark.parametrize("wide", [0, 1, 3])
@pytest.mark.parametrize("D", [64, 128])
def test_the_same_edges_on_the_tensor_core_kernels_of_prompt_portions(D, wide):
    """bfloat16 with key and value size 64 or 128, on 64-row and 128-row tiles (mma.sync) and on the tcgen05 form with
    roles: kept first tokens that fill more than one tile of 64 keys in front of a window that starts tiles later,
    keys on both sides of every edge, and of a tile's border."""
    size, keep = 37, 70
    T, query = 400, 390
    for key, seen in ((query - size + 1, True), (query - size, False), (keep - 1, True), (keep, False), (0, True), (63, True),
                      (64, True), (query, True), (query - 6, True), (200, False), (128, False), (127, False)):
        (in_prompt, decoded), ref = _spiked("bfloat16", size, keep, T, query, key, D=D, wide=wide)
        for got in (in_prompt, decoded):
            if seen:
                assert got[key % D] > 0.97, (key, got[key % D])
            else:
                assert got[key % D] < 0.1, (key, got[key % D])
            assert np.abs(got - ref).max() < 1e-2
    # kept first tokens that the window still covers (no tile in front of the window's own), and no window at all
    for size, keep, key, seen in ((300, 20, 95, True), (300, 20, 90, False), (0, 0, 1, True)):
        (in_prompt, decoded), ref = _spiked("bfloat16", size, keep, T, query, key, D=D, wide=wide)
        assert (in_prompt[key % D] > 0.97) == seen and np.abs(in_prompt - ref).max() < 1e-2


@pytest.mark.parametrize("shape", [dict(heads=4, kv_heads=2, dim=64, vdim=64, conv=3, size=50, keep_first=70),
                                   dict(heads=3, kv_heads=1, dim=128, vdim=128, conv=2, size=100, keep_first=5),
                                   dict(heads=2, kv_heads=2, dim=64, vdim=64, conv=4, size=1000, keep_first=0)])
@pytest.mark.parametrize("wide", [None, 3])
def test_attention_on_tensor_cores_in_long_portions(shape, wide, monkeypatch):
    """The mixer in bfloat16 at sizes whose prompt portions run on tensor cores: 300 and 130 tokens, whole, and
    cut into portions beside single tokens of the other request."""
    from kv_cache_optimization_for_llm_b200 import ops
    monkeypatch.setattr(ops, "FLASH_ROWS_WIDE", wide)
    rng = np.random.default_rng(11)
    dtype = "bfloat16"
    ctx = _ctx(dtype)
    H = 40
    mx = tiny.attention(**shape)["mixer"]
    wt, w64 = _attention_weights(rng, H, mx)
    mixer = _attention_mixer(mx, wt, ctx, H)
    xs, refs = {}, {}
    for r, T in enumerate((300, 130)):
        x, x64 = _w(rng, (T, H), 1.0)
        xs[r], refs[r] = x.to(DT[dtype]).cuda(), S.attention_mixer(x64, w64, "", mx)
    before = ops.choices["flash_attention_rows"]
    whole = _run_in_steps(mixer, ctx, xs, [[(0, 300)], [(1, 130)]])
    cut = _run_in_steps(mixer, ctx, xs, [[(0, 129), (1, 1)], [(0, 2), (1, 1)], [(0, 65), (1, 100)], [(0, 1), (1, 1)],
                                         [(0, 100), (1, 27)], [(0, 1)], [(0, 1)], [(0, 1)]])
    assert ops.choices["flash_attention_rows"] >= before + 6
    if wide == 3:
        assert ops.choices["flash_attention_rows_3"] >= 6
    for r in xs:
        assert _err(whole[r], refs[r], dtype) < TOL[dtype]
        assert _err(cut[r], refs[r], dtype) < TOL[dtype]


# --------------------------------------------------------------------------- the delta rule

def _delta_weights(rng, H, mx):
    Hh, G, D, Dv, taps = (mx[k] for k in ("heads", "kv_heads", "dim", "vdim", "conv"))
    gd, hv = G * D, Hh * Dv
    wt, w64 = {}, {}
    for role, name, shape, std, mean in (
            ("q", "q", (gd, H), 0.3, 0), ("k", "k", (gd, H), 0.3, 0), ("v", "v", (hv, H), 0.3, 0),
            ("q_conv", "q.conv", (gd, taps), 0.6, 0), ("k_conv", "k.conv", (gd, taps), 0.6, 0),
            ("v_conv", "v.conv", (hv, taps), 0.6, 0), ("b", "b", (Hh, H), 0.3, 0), ("a", "a", (Hh, H), 0.3, 0),
            ("A_log", "A_log", (Hh,), 0.7, 0), ("dt_bias", "dt_bias", (Hh,), 1.0, 0), ("norm", "norm", (Dv,), 0.2, 1),
            ("g", "g", (hv, H), 0.3, 0), ("o", "o", (H, hv), 0.3, 0)):
        wt[role], w64[name] = _w(rng, shape, std, mean)
    return wt, w64


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,taps", [(4, 2, 12, 20, 4), (2, 2, 32, 32, 4), (6, 1, 8, 40, 2),
                                                          (1, 1, 64, 128, 1), (3, 3, 24, 6, 7)])
def test_gated_delta_alone_in_portions_and_beside_another_request(dtype, heads, kv_heads, dim, vdim, taps):
    """Also: portions shorter than the convolution's tail, so that the tail is shifted, not replaced,
    and forty tokens decoded one by one."""
    rng = np.random.default_rng(vdim)
    ctx = _ctx(dtype)
    H = 40
    mx = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps}
    wt, w64 = _delta_weights(rng, H, mx)
    mixer = _make("mixer", "gated_delta", {"hidden_size": H, "eps": 1e-5, **mx}, wt, ctx)
    xs, refs = {}, {}
    for r, T in enumerate((85, 19)):
        x, x64 = _w(rng, (T, H), 1.0)
        xs[r], refs[r] = x.to(DT[dtype]).cuda(), S.delta_mixer(x64, w64, "", mx, 1e-5)
    whole = _run_in_steps(mixer, ctx, xs, [[(0, 85)], [(1, 19)]])
    cut = _run_in_steps(mixer, ctx, xs, [[(0, 1), (1, 1)], [(0, 2), (1, 1)], [(0, 1), (1, 16)], [(0, 1)], [(0, 17)],
                                         [(0, 2)], [(0, 20), (1, 1)], [(0, 1)]] + [[(0, 1)]] * 40)
    for r in xs:
        assert _err(whole[r], refs[r], dtype) < TOL[dtype]
        assert _err(cut[r], refs[r], dtype) < TOL[dtype]
        assert _same(whole[r], cut[r], dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_state_is_carried_from_step_to_step_over_hundreds_of_tokens(dtype):
    """Random weights would hide a lost state behind the decay.  Here the decay is (almost) 1, so that after
    300 tokens the state decides what the next tokens read: the plain model started afresh at token 300
    answers something else altogether.  The engine's portions and single tokens must not."""
    rng = np.random.default_rng(0)
    ctx = _ctx(dtype)
    H = 40
    mx = {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 16, "conv": 2}
    wt, w64 = _delta_weights(rng, H, mx)
    wt["A_log"], w64["A_log"] = _w(rng, (2,), 0.0, -20.0)        # exp(A) ~ 2e-9: no decay to speak of
    mixer = _make("mixer", "gated_delta", {"hidden_size": H, "eps": 1e-5, **mx}, wt, ctx)
    x, x64 = _w(rng, (420, H), 1.0)
    ref = S.delta_mixer(x64, w64, "", mx, 1e-5)
    afresh = S.delta_mixer(x64[300:], w64, "", mx, 1e-5)         # what a lost state (and a lost tail) would give
    assert np.abs(ref[300:] - afresh).max() > 0.3 * np.abs(ref).max(), "the state must matter"
    got = _run_in_steps(mixer, ctx, {0: x.to(DT[dtype]).cuda()}, [[(0, 300)], [(0, 2)], [(0, 78)]] + [[(0, 1)]] * 40, page=16)
    assert _err(got[0], ref, dtype) < TOL[dtype]
    assert _err(got[0][300:], ref[300:], dtype) < TOL[dtype]


# --------------------------------------------------------------------------- the experts

def _expert_weights(rng, H, E, I, F, Sh):
    wt, w64 = {}, {}
    wt["router"], w64["router"] = _w(rng, (E + I, H), 3.0 / np.sqrt(H))
    wt["correction"], w64["correction"] = _w(rng, (E + I,), 0.1)
    for e in range(E):
        wt[f"up{e}"], w64[f"e{e}.up"] = _w(rng, (F, H), 0.3)
        wt[f"down{e}"], w64[f"e{e}.down"] = _w(rng, (H, F), 0.3)
    if Sh:
        wt["shared_up"], w64["shared.up"] = _w(rng, (Sh, H), 0.3)
        wt["shared_down"], w64["shared.down"] = _w(rng, (H, Sh), 0.3)
    return wt, w64


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,I,top,F,Sh", [(5, 1, 2, 12, 20), (3, 2, 3, 16, 0), (8, 0, 1, 8, 8), (2, 3, 5, 24, 0),
                                          (40, 2, 4, 5, 3), (1, 1, 1, 7, 0)])
def test_routed_experts_alone(dtype, E, I, top, F, Sh):
    """Several shapes: identity experts, none, all experts chosen, widths that are no multiple of 8, more
    experts than a warp has lanes.  A token's result does not depend on its neighbours."""
    from kv_cache_optimization_for_llm_b200 import ops
    rng = np.random.default_rng(E * 7 + I)
    ctx = _ctx(dtype)
    H, T = 40, 37
    wt, w64 = _expert_weights(rng, H, E, I, F, Sh)
    mlp = {"router": {"experts": E, "identity": I, "top": top, "scale": 1.7}, "expert": {"ff": F}}
    if Sh:
        mlp["shared"] = {"ff": Sh}
    ff = _make("feed_forward", "routed_experts", {"hidden_size": H, "experts": E, "identity": I, "top": top, "scale": 1.7,
                                                  "expert_ff": F, "shared_ff": Sh}, wt, ctx)
    x, x64 = _w(rng, (T, H), 1.0)
    xd = x.to(DT[dtype]).cuda()
    ref = S.moe_ff(x64, w64, "", mlp)
    got = ff.forward(xd, None)
    assert _rel(got, ref) < TOL[dtype]
    # the router itself: the chosen experts and their weights, in float32 in both precisions
    gate, idw = ops.route(xd, ff.router, ff.correction, E, I, top, 1.7)
    idx, wts = S.route(x64, w64, "", mlp["router"])
    dense = np.zeros((T, E + I))
    np.put_along_axis(dense, idx, wts, axis=1)
    assert np.abs(gate.cpu().numpy() - dense).max() < 1e-5
    if I:
        assert np.abs(idw.cpu().numpy() - dense[:, E:].sum(axis=1)).max() < 1e-5
    alone = torch.cat([ff.forward(xd[t:t + 1].contiguous(), None) for t in (0, 11, 36)])
    if dtype == "float32":
        assert torch.equal(alone, got[[0, 11, 36]])
    else:
        assert _rel(alone, ref[[0, 11, 36]]) < TOL[dtype]


# --------------------------------------------------------------------------- whole models

def _runner(folder, dtype, **kw):
    from kv_cache_optimization_for_llm_b200 import EngineConfig
    from kv_cache_optimization_for_llm_b200.engine.runner import ModelRunner
    args = dict(dtype=dtype, page_size=8, num_pages=40, max_num_seqs=3, max_num_batched_tokens=256, max_model_len=160,
                use_cuda_graphs=False)
    args.update(kw)
    return ModelRunner(folder, EngineConfig(**args))


def _logit_err(got, ref, dtype="float32"):
    if dtype == "float32":
        return np.abs(got - ref).max() / np.abs(ref).max()
    return np.sqrt(((got - ref) ** 2).mean()) / np.sqrt((ref ** 2).mean())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_model_prefill_decoding_portions_batches_and_reuse(dtype):
    """A model with every kind of layer and feed-forward, a layer without feed-forward and a repeated
    run of layers.  Whole prompts; token by token; portions of 2, 3, 7, ... beside single tokens of
    another request; then requests that end and others that take over their slots and pages in a
    pool that holds two of them at most; 60 decoded tokens in a row, past every window."""
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    folder = tempfile.mkdtemp(prefix="kvb200_sx_")
    cfg = tiny.MIXED
    w = tiny.write_model(folder, cfg, seed=1)
    r = _runner(folder, dtype)
    # eight layer runs: three attention groups, states for all layer runs but the two of the attention with one tap
    assert len(r.spec.schedule) == 8 and r.cache.group_entries == [2, 2, 1] and len(r.cache.states) == 6
    rng = np.random.default_rng(5)
    seqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in (90, 37, 61, 1, 150)]
    refs = [S.forward(cfg, w, s) for s in seqs]
    tol = TOL_MODEL[dtype]
    whole = r.step([StepEntry(0, seqs[1], 0, range(37))]).cpu().numpy()
    assert _logit_err(whole, refs[1], dtype) < tol
    r.release(0)
    single = np.concatenate([r.step([StepEntry(1, [t], i, [0])]).cpu().numpy() for i, t in enumerate(seqs[1])])
    assert _logit_err(single, refs[1], dtype) < tol
    if dtype == "float32":
        assert np.array_equal(whole, single)
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
    # the windowed groups have given back what their windows passed, but not the pages of the kept first tokens
    held = [sum(p >= 0 for p in r.manager.block_table(20, g)) for g in range(r.manager.num_groups())]
    assert held[0] < 19 and held[1] < 19, held
    r.release(20)
    assert all(r.manager.free_pages(g) == 40 for g in range(r.manager.num_groups()))


@pytest.mark.parametrize("layers,loop", [
    ([tiny.attention(heads=2, kv_heads=1, dim=8, vdim=8, conv=2, size=6, keep_first=2)], None),
    ([tiny.delta(heads=1, kv_heads=1, dim=32, vdim=16, conv=3, mlp=tiny.dense(24))], {"start": 0, "stop": 1, "times": 3}),
    ([tiny.delta(heads=2, kv_heads=1, dim=16, vdim=16, conv=3), tiny.attention(mlp=tiny.moe(experts=2, identity=0, top=2, ff=8, shared=0))],
     {"start": 1, "stop": 2, "times": 1}),
    # sizes that are no powers of two, head counts of 1, all three layers repeated twice, the loop running to the end
    ([tiny.attention(heads=5, kv_heads=5, dim=24, vdim=40, conv=3, scale=0.11, size=9, keep_first=13, mlp=tiny.dense(72)),
      tiny.delta(heads=6, kv_heads=2, dim=40, vdim=24, conv=3, mlp=tiny.moe(experts=7, identity=3, top=4, scale=2.5, ff=24, shared=40)),
      tiny.attention(heads=1, kv_heads=1, dim=96, vdim=16, conv=5, scale=0.05, size=64, keep_first=0)],
     {"start": 0, "stop": 3, "times": 2}),
])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_orders_of_layers_and_loops(layers, loop, dtype):
    """One layer alone, a lone layer three times in a row, a loop of one pass, odd sizes: a prompt in
    three portions and four tokens one by one."""
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    folder = tempfile.mkdtemp(prefix="kvb200_sx_")
    cfg = tiny.config(layers, width=40 if len(layers) < 3 else 104, vocab=53, loop=loop, eps=1e-6)
    w = tiny.write_model(folder, cfg, seed=2)
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
def test_greedy_generation_through_the_engine_and_its_scheduler(dtype):
    """Prompts of unequal length through ``LLM.generate``: the scheduler's portions (a token budget of
    24 per step), decode steps replayed from CUDA graphs, the engine one step ahead, five requests in
    three seats.  Every sampled row's logits are compared with the plain model on the final
    sequences, and in float32 the greedy tokens themselves."""
    from kv_cache_optimization_for_llm_b200 import LLM, SamplingParams
    from logit_hook import LogitRecorder
    folder = tempfile.mkdtemp(prefix="kvb200_sx_")
    cfg = tiny.MIXED
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
    n, worst = rec.compare(seqs, lambda i: plain[i], TOL_MODEL[dtype], "greedy generation")
    assert n >= 60 and llm.engine.runner._graphs
    if dtype == "float32":
        for i in seqs:
            for j, tok in enumerate(outs[i]):
                row = plain[i][len(prompts[i]) + j - 1]
                assert row[tok] >= row.max() - 1e-4 * np.abs(row).max(), (i, j)
    assert llm.engine.runner.manager.check() == ""


@pytest.mark.parametrize("dtype,flags", [("float32", ()), ("bfloat16", ()), ("float32", ("--cuda-graphs",))])
def test_replay_through_the_trace_runner(dtype, flags):
    """bin/trace_run on a Solulix folder: each request whole, then four live requests whose portions
    (down to two tokens) run beside single tokens in a pool that holds exactly them, in four state
    slots; requests that end hand pages and slots to the ones that follow."""
    from trace_driver import TraceRun, ceil64
    folder = tempfile.mkdtemp(prefix="kvb200_sx_")
    cfg = tiny.MIXED
    w = tiny.write_model(folder, cfg, seed=6)
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_are_no_multiples_of_eight(dtype):
    """A width of 36, heads of 5, 3 and 7 channels, experts 6 wide, 50 tokens in the vocabulary: nothing may rest on
    16-byte rows.  Whole, in portions and token by token."""
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    folder = tempfile.mkdtemp(prefix="kvb200_sx_")
    layers = [tiny.attention(heads=3, kv_heads=1, dim=5, vdim=3, conv=2, scale=0.4, size=7, keep_first=2,
                             mlp=tiny.moe(experts=3, identity=1, top=2, scale=1.1, ff=6, shared=10)),
              tiny.delta(heads=3, kv_heads=3, dim=7, vdim=5, conv=3, mlp=tiny.dense(18))]
    cfg = tiny.config(layers, width=36, vocab=50, loop={"start": 0, "stop": 2, "times": 2})
    w = tiny.write_model(folder, cfg, seed=3)
    r = _runner(folder, dtype)
    seq = np.random.default_rng(3).integers(0, 50, 40).tolist()
    ref = S.forward(cfg, w, seq)
    got, pos = [], 0
    for n in (13, 2, 21, 1, 1, 1, 1):
        got.append(r.step([StepEntry(0, seq[pos:pos + n], pos, range(n))]).cpu().numpy())
        pos += n
    assert _logit_err(np.concatenate(got), ref, dtype) < TOL_MODEL[dtype]
    r.check_status()


def test_command_line_serves_the_design():
    """The engine's command line on a Solulix folder: requests on standard input in the wire format, greedy tokens
    back as JSON lines; each token is the plain model's best (ties within 1e-4 allowed)."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder = tempfile.mkdtemp(prefix="kvb200_sx_")
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
