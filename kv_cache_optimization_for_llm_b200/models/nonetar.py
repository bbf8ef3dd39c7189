"""The Nonetar decoder as a model description.

A token's embedding plus a sinusoidal position vector starts ``streams`` equal copies of the residual stream.
Every sublayer reads a learned weighted sum of the copies, norms it (RMS norm, weight stored around zero), and
writes its output back into all copies through a learned mixing matrix; the model's last norm reads their plain
sum.  In front of every mixer the normed row is shifted towards the previous token's, channel by channel.  Mixers
are of two kinds: a sliding-window attention (biases, per-head query and key norm, a learned factor per head, a soft
cap on the scores and a bias that grows with the distance) beside a gated diagonal linear recurrence, their results
summed with fixed weights; and a state-space-duality mixer with a matrix state per head.  The feed-forward is an
ungated dense one with the xIELU activation.  The logits are multiplied by a constant.  config.json names the layers
one by one.
"""

from __future__ import annotations

from ..config.model_config import NonetarConfig, NonetarLayerConfig
from ..registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

# what the design fixes
DECAY_SCALE = 8.0        # log a = -DECAY_SCALE * r * softplus(lam) in the diagonal recurrence
SLOPE_POWER = 8.0        # slope_h = 2^(-SLOPE_POWER * (h + 1) / heads) of the attention's distance bias
POSITION_BASE = 10000.0  # of the sinusoidal position vector


def _mixer(cfg: NonetarConfig, i: int, layer: NonetarLayerConfig) -> PartSpec:
    m, p, W = layer.mixer, f"l{i}.mix.", cfg.width
    if layer.type == "mamba2":
        return PartSpec("state_space_duality", {
            "hidden_size": W, "heads": int(m["heads"]), "vdim": int(m["vdim"]), "state": int(m["state"]),
            "groups": int(m["groups"]), "norm_groups": int(m["norm_groups"]), "conv": int(m["conv"]), "eps": cfg.norm_eps,
        }, {"in": p + "in", "conv": p + "conv", "conv_bias": p + "conv.b", "dt_bias": p + "dt_bias", "A_log": p + "A_log",
            "D": p + "D", "norm": p + "norm", "o": p + "o"})
    a, r = m["left"], m["right"]
    pl, pr = p + "left.", p + "right."
    left = PartSpec("shaped_window_attention", {
        "hidden_size": W, "heads": int(a["heads"]), "kv_heads": int(a["kv_heads"]), "dim": int(a["dim"]),
        "vdim": int(a["vdim"]), "scale": float(a["scale"]),
        "window": int(a["mask"]["size"]) if (a.get("mask") or {}).get("size") else None,
        "softcap": float(a["softcap"]) if a.get("softcap") else None, "slope_power": SLOPE_POWER, "bias": True,
        "qk_norm": True, "head_temperature": True, "eps": cfg.norm_eps, "out_scale": float(m["left_scale"]),
    }, {"q": pl + "q", "k": pl + "k", "v": pl + "v", "q_bias": pl + "q.b", "k_bias": pl + "k.b", "v_bias": pl + "v.b",
        "q_norm": pl + "q.norm", "k_norm": pl + "k.norm", "temp": pl + "temp", "o": pl + "o"}, family="mixer")
    right = PartSpec("gated_linear_recurrence", {
        "hidden_size": W, "width": int(r["width"]), "blocks": int(r["blocks"]), "conv": int(r["conv"]),
        "decay_scale": DECAY_SCALE, "out_scale": float(m["right_scale"]),
    }, {"y": pr + "y", "y_bias": pr + "y.b", "x": pr + "x", "x_bias": pr + "x.b", "conv": pr + "conv",
        "conv_bias": pr + "conv.b", "ra": pr + "ra", "ra_bias": pr + "ra.b", "ri": pr + "ri", "ri_bias": pr + "ri.b",
        "lam": pr + "lam", "o": pr + "o"}, family="mixer")
    return PartSpec("side_by_side", {"left": left, "right": right})


def build_nonetar_spec(cfg: NonetarConfig) -> ModelSpec:
    W, S, eps = cfg.width, cfg.streams, cfg.norm_eps

    def read_norm(i, q, shift):
        names = {"weight": f"l{i}.norm{q}", "in": f"l{i}.hc{q}.in"}
        if shift:
            names["shift"] = f"l{i}.shift"
        return PartSpec("hyper_rmsnorm", {"size": W, "streams": S, "eps": eps, "one_plus": True, "learned": True,
                                          "shift": shift}, names)

    def write(i, q):
        return PartSpec("hyper_write", {"streams": S, "learned": True}, {"mix": f"l{i}.hc{q}.mix", "out": f"l{i}.hc{q}.out"})

    layers = []
    for i, layer in enumerate(cfg.layers):
        parts = dict(mixer=_mixer(cfg, i, layer), mixer_norm=read_norm(i, 1, True), mixer_write=write(i, 1))
        if layer.mlp is None:
            layers.append(LayerSpec("hyper_prenorm_mixer_only", parts))
            continue
        parts.update(feed_forward=PartSpec("dense_xielu", {"hidden_size": W, "intermediate_size": int(layer.mlp["ff"])},
                                           {"up": f"l{i}.mlp.up", "down": f"l{i}.mlp.down", "act": f"l{i}.mlp.act"}),
                     ff_norm=read_norm(i, 2, False), ff_write=write(i, 2))
        layers.append(LayerSpec("hyper_prenorm", parts))
    spec = ModelSpec(
        architecture=cfg.architecture, hidden_size=W, vocab_size=cfg.vocab, max_position=cfg.max_position_embeddings,
        embedding=PartSpec("sinusoid_stream_embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "streams": S,
                                                         "base": POSITION_BASE}, {"table": "embed"}),
        layers=layers, schedule=[ScheduleEntry(i) for i in range(len(layers))],
        # the last norm reads the plain sum of the streams; the constant on the logits is multiplied into its weight
        final_norm=PartSpec("hyper_rmsnorm", {"size": W, "streams": S, "eps": eps, "one_plus": True, "learned": False,
                                              "shift": False, "scale": cfg.logit_scale}, {"weight": "final.norm"}),
        lm_head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": W}, {"weight": "head"}),
        eos_token_ids=cfg.eos_token_ids,
    )
    spec.validate()
    return spec


register_architecture("Nonetar", NonetarConfig.from_dict, build_nonetar_spec)
