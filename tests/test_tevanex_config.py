"""Tevanex without a GPU: the configuration, the model description and its tensor names, what each layer asks of the
cache, and the plain restatement checked against second formulations of its mechanisms."""

import copy
import math

import numpy as np
import pytest

import plain_tevanex as S
import tiny_tevanex as tiny


def _parse(cfg):
    from kv_cache_optimization_for_llm_b200.registry import resolve_architecture
    arch = resolve_architecture(cfg)
    return arch, arch.parse_config(cfg)


def test_description_names_every_tensor_and_shares_layers():
    arch, cfg = _parse(tiny.MIXED)
    spec = arch.build_spec(cfg)
    # four layers have tensors of their own; the other three applications use theirs, each with its own cache
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 0, 3, 2, 1] and all(e.cache_of is None for e in spec.schedule)
    assert [layer.block for layer in spec.layers] == ["postnorm", "postnorm", "postnorm", "postnorm_mixer_only"]
    names = tiny.expected(tiny.MIXED)
    assert names["embed"].shape == (97, 40) and names["head"].shape == (97, 40) and names["final.norm"].shape == (40,)
    assert names["l0.mix.q"].shape == (36, 40) and names["l0.mix.v"].shape == (60, 40) and names["l0.mix.g"].shape == (60, 40)
    assert names["l0.mix.i"].shape == (3, 40) and names["l0.mix.f.b"].shape == (3,) and names["l0.mix.norm"].shape == (60,)
    assert names["l0.mix.o"].shape == (40, 60)
    assert names["l1.mix.q"].shape == (64, 40) and names["l1.mix.k"].shape == (32, 40) and names["l1.mix.v"].shape == (48, 40)
    assert names["l1.mix.q.norm"].shape == (64,) and names["l1.mix.k.norm"].shape == (32,) and names["l1.mix.sink"].shape == (4,)
    assert names["l1.mix.o"].shape == (40, 96) and names["l1.mix.o.b"].shape == (40,) and "l1.mix.g" not in names
    assert names["l2.mix.g"].shape == (24, 40) and "l2.mix.sink" not in names and names["l2.mix.k.b"].shape == (24,)
    assert names["l0.mlp.router"].shape == (5, 40) and names["l0.mlp.e4.gate"].shape == (12, 40)
    assert names["l0.mlp.e0.down"].shape == (40, 12) and names["l0.mlp.shared.up"].shape == (20, 40)
    assert names["l0.mlp.shared.sg"].shape == (1, 40)
    assert "l1.mlp.shared.gate" not in names and names["l1.mlp.e2.up"].shape == (16, 40)
    assert not any(n.startswith(("l3.", "l5.", "l6.", "l4.mlp", "l4.norm2")) for n in names) and "l4.norm1" in names


def test_what_each_application_asks_of_the_cache():
    import torch
    from kv_cache_optimization_for_llm_b200.cache.specs import PagedKVSpec, SlotStateSpec
    from kv_cache_optimization_for_llm_b200.models.spec import PartSpec
    from kv_cache_optimization_for_llm_b200.parts import lookup
    arch, cfg = _parse(tiny.MIXED)
    spec = arch.build_spec(cfg)
    att = spec.layers[1].parts["mixer"]
    assert att.kind == "rotary_chunk_attention" and att.params["chunk"] == 11 and att.params["sink"] and not att.params["gate"]
    assert att.params["position"].kind == "rope" and att.params["position"].params["rotary_dim"] == 8
    second = spec.layers[2].parts["mixer"]
    assert second.params["gate"] and not second.params["sink"] and second.params["softcap"] == 3.0
    assert second.params["position"].kind == "rope_interleaved" and second.params["position"].params["scaling"]["rope_type"] == "yarn"
    assert spec.layers[0].parts["mixer_post_norm"].params["scale"] == 0.4
    assert spec.lm_head.params["scale"] == 0.6 and spec.lm_head.params["softcap"] == 7.0
    assert spec.embedding.params["scale"] == 0.7


def test_what_the_config_leaves_out_is_not_there():
    cfg = tiny.config([tiny.layer("attention_2", tiny.attention(size=None, rot_dims=None, softcap=None), tiny.moe(shared_ff=0))],
                      logit_softcap=None)
    arch, parsed = _parse(cfg)
    spec = arch.build_spec(parsed)
    att = spec.layers[0].parts["mixer"].params
    assert att["chunk"] is None and att["softcap"] is None and att["position"] is None
    assert spec.layers[0].parts["feed_forward"].params["shared_ff"] == 0 and spec.lm_head.params["softcap"] is None


@pytest.mark.parametrize("breakage,needle", [
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"].pop("gate_cap"), "gate_cap"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "grouped"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "dense"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["layers"][3].update(weights_of=5), "weights_of"),
    (lambda c: c["layers"][3].update(weights_of=1), "type"),
    (lambda c: c["layers"][0].update(type="conv"), "conv"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_config_errors_name_the_key(breakage, needle):
    from kv_cache_optimization_for_llm_b200.config import ConfigError
    cfg = copy.deepcopy(tiny.MIXED)
    breakage(cfg)
    with pytest.raises(ConfigError) as e:
        _parse(cfg)
    assert needle in str(e.value)


def test_the_engines_frequencies_are_the_plain_ones():
    from kv_cache_optimization_for_llm_b200.parts.position import rope_inv_freq, yarn_inv_freq
    for dims, base, sc in ((10, 500.0, tiny.YARN), (64, 1e4, dict(factor=8.0, original=512, fast=32.0, slow=1.0)),
                           (2, 3.0, dict(factor=1.5, original=7, fast=2.0, slow=1.0))):
        f, grow = S.rotary_frequencies(dims, base, sc)
        g, grow2 = yarn_inv_freq(dims, base, sc)
        assert np.abs(g.numpy() - f).max() < 1e-15 and abs(grow - grow2) < 1e-15
        assert np.abs(rope_inv_freq(dims, base, None).numpy() - S.rotary_frequencies(dims, base)[0]).max() < 1e-15


def test_stretched_frequencies_keep_fast_waves_and_divide_slow_ones():
    sc = dict(factor=4.0, original=64, fast=8.0, slow=1.0)
    plain, _ = S.rotary_frequencies(32, 1e4)
    f, grow = S.rotary_frequencies(32, 1e4, sc)
    assert f[0] == plain[0] and abs(f[-1] - plain[-1] / 4.0) < 1e-18 and abs(grow - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    ratio = plain / f
    assert np.all(np.diff(ratio) >= -1e-12) and ratio[0] == 1.0 and abs(ratio[-1] - 4.0) < 1e-12


def test_rotation_depends_on_the_distance_only_in_both_layouts():
    rng = np.random.default_rng(0)
    f, grow = S.rotary_frequencies(6, 50.0)
    q, k = rng.normal(size=(1, 1, 8)), rng.normal(size=(1, 1, 8))
    for layout in ("half", "pairs"):
        a = S.rotate(q, [17], 6, f, grow, layout)[0, 0] @ S.rotate(k, [12], 6, f, grow, layout)[0, 0]
        b = S.rotate(q, [105], 6, f, grow, layout)[0, 0] @ S.rotate(k, [100], 6, f, grow, layout)[0, 0]
        assert abs(a - b) < 1e-12
        assert np.array_equal(S.rotate(q, [9], 6, f, grow, layout)[0, 0, 6:], q[0, 0, 6:])       # the rest passes
    # the layouts pair other channels
    assert np.abs(S.rotate(q, [3], 6, f, grow, "half") - S.rotate(q, [3], 6, f, grow, "pairs")).max() > 1e-3


def test_blocks_of_positions_are_counted_from_the_start():
    seen = [[j for j in range(12) if S.chunk_visible(i, j, 5)] for i in range(12)]
    assert seen[4] == [0, 1, 2, 3, 4] and seen[5] == [5] and seen[9] == [5, 6, 7, 8, 9] and seen[11] == [10, 11]
    assert [j for j in range(4) if S.chunk_visible(3, j, None)] == [0, 1, 2, 3]


def test_matrix_memory_is_the_unscaled_recurrence_divided_by_the_maximum():
    """With the true memory C* = sum_s exp(i_s + F_t - F_s) k_s v_s^T (and n* likewise) the read-out is
    C*^T q / (max(|n* . q|, 1) + 1e-6 exp(m)), m being max(F_t, max_s (i_s + F_t - F_s)): the maximum only guards the
    exponentials."""
    rng = np.random.default_rng(1)
    T, D, Dv = 9, 4, 3
    q, k, v = rng.normal(size=(T, D)), rng.normal(size=(T, D)), rng.normal(size=(T, Dv))
    gi, gf = rng.normal(size=T), -np.abs(rng.normal(size=T))
    got = S.matrix_memory(q, k, v, gi, gf)
    F = np.cumsum(gf)
    for t in range(T):
        w = np.array([math.exp(gi[s] + F[t] - F[s]) for s in range(t + 1)])
        C = sum(w[s] * np.outer(k[s], v[s]) for s in range(t + 1))
        n = sum(w[s] * k[s] for s in range(t + 1))
        m = max(F[t], max(gi[s] + F[t] - F[s] for s in range(t + 1)))
        ref = C.T @ q[t] / (max(abs(n @ q[t]), 1.0) + 1e-6 * math.exp(m))
        assert np.abs(got[t] - ref).max() < 1e-10


def test_an_experts_weight_is_on_its_input():
    rng = np.random.default_rng(2)
    W, F = 6, 5
    w = {"router": rng.normal(size=(3, W)), "shared.sg": rng.normal(size=(1, W))}
    for e in ("e0.", "e1.", "e2.", "shared."):
        w.update({e + "gate": rng.normal(size=(F, W)), e + "up": rng.normal(size=(F, W)), e + "down": rng.normal(size=(W, F))})
    mlp = tiny.moe(experts=3, top=2, ff=F, limit=0.7, shared_ff=F, shared_limit=0.4)
    h = rng.normal(size=(4, W))
    out = S.moe(h, w, "", mlp)
    chosen, weight = S.route(h, w["router"], 2)
    assert np.all(weight[:, 0] >= weight[:, 1]) and np.all((weight > 0) & (weight < 1))
    t = 1
    by_hand = sum(S.limited_expert(c * h[t][None], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], 0.7)[0]
                  for e, c in zip(chosen[t], weight[t]))
    by_hand = by_hand + S.limited_expert(h[t][None], w["shared.gate"], w["shared.up"], w["shared.down"], 0.4)[0] \
        * S.sigmoid(h[t] @ w["shared.sg"][0])
    assert np.abs(out[t] - by_hand).max() < 1e-12
    first = np.zeros((3, 3))
    gate, up = first.copy(), first.copy()
    gate[:, 0], up[:, 0] = [-3.0, 0.2, 5.0], [9.0, -9.0, 0.1]
    y = S.limited_expert(np.eye(3)[:1], gate, up, np.eye(3), 0.7)
    # gate limited from above only, up from both sides
    assert abs(y[0, 0] - (-3.0 * S.sigmoid(1.702 * -3.0) * 1.7)) < 1e-12 and abs(y[0, 1] - 0.2 * S.sigmoid(0.3404) * 0.3) < 1e-12
    assert abs(y[0, 2] - 0.7 * S.sigmoid(1.702 * 0.7) * 1.1) < 1e-12


def test_a_sink_takes_weight_without_a_value():
    q = np.zeros((1, 1, 2))
    k = np.zeros((1, 1, 2))
    v = np.ones((1, 1, 1))
    assert abs(S.masked_attention(q, k, v, 1.0, None, None, np.array([0.0]))[0, 0, 0] - 0.5) < 1e-15
    assert abs(S.masked_attention(q, k, v, 1.0, None, None, None)[0, 0, 0] - 1.0) < 1e-15
