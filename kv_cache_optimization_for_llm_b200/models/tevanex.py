"""The Tevanex decoder as a model description.

A token's embedding, multiplied by a constant, starts the residual stream.  The sublayers of a layer read the
stream itself, without a norm in front; their outputs pass an RMS norm and a constant factor before they join it.
Mixers are of three kinds: a matrix memory per head with exponential gates (mLSTM); and two grouped-query
attentions over blocks of positions, with biases, a norm over all of a token's queries (and keys) at once, and a
rotation of part of every head: one pairs channels half a rotation apart and counts a learned number per head into
the softmax's denominator, the other pairs neighbouring channels, stretches its frequencies (YaRN), caps its scores
and gates its output.  The feed-forward is a set of small gated experts with limited activations, chosen by sigmoid
scores that weigh the expert's input, beside a shared expert with a gate of its own.  A layer may use another layer's
tensors while keeping a cache or state of its own.  The logits are multiplied by a constant and capped.
config.json names the layers one by one.
"""

from __future__ import annotations

from ..config.model_config import TevanexConfig, TevanexLayerConfig
from ..registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

# what the design fixes
EXPERT_ALPHA = 1.702     # a(g) = g sigmoid(EXPERT_ALPHA g) in the experts


def _mixer(cfg: TevanexConfig, i: int, layer: TevanexLayerConfig) -> PartSpec:
    m, p, W = layer.mixer, f"l{i}.mix.", cfg.width
    if layer.type == "mlstm":
        return PartSpec("mlstm", {
            "hidden_size": W, "heads": int(m["heads"]), "dim": int(m["dim"]), "vdim": int(m["vdim"]),
            "gate_cap": float(m["gate_cap"]), "eps": cfg.norm_eps,
        }, {"q": p + "q", "k": p + "k", "v": p + "v", "g": p + "g", "i": p + "i", "f": p + "f", "i_bias": p + "i.b",
            "f_bias": p + "f.b", "norm": p + "norm", "o": p + "o"})
    second = layer.type == "attention_2"
    rot = m.get("rot") or None
    position = None
    if rot and int(rot["dims"]) > 0:
        if second:
            scaling = dict(rot["scaling"], rope_type="yarn") if rot.get("scaling") else None
            position = PartSpec("rope_interleaved", {"dims": int(rot["dims"]), "base": float(rot["base"]), "scaling": scaling})
        else:
            position = PartSpec("rope", {"head_dim": int(m["dim"]), "rotary_dim": int(rot["dims"]),
                                         "theta": float(rot["base"]), "scaling": None})
    names = {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o", "q_bias": p + "q.b", "k_bias": p + "k.b",
             "v_bias": p + "v.b", "o_bias": p + "o.b", "q_norm": p + "q.norm", "k_norm": p + "k.norm"}
    names.update({"g": p + "g"} if second else {"sink": p + "sink"})
    return PartSpec("rotary_chunk_attention", {
        "hidden_size": W, "heads": int(m["heads"]), "kv_heads": int(m["kv_heads"]), "dim": int(m["dim"]),
        "vdim": int(m["vdim"]), "scale": float(m["scale"]),
        "chunk": int(m["mask"]["size"]) if (m.get("mask") or {}).get("size") else None,
        "softcap": float(m["softcap"]) if second and m.get("softcap") else None,
        "sink": not second, "gate": second, "bias": True, "qk_norm": True, "eps": cfg.norm_eps, "position": position,
    }, names)


def _feed_forward(cfg: TevanexConfig, i: int, mlp) -> PartSpec:
    p, W = f"l{i}.mlp.", cfg.width
    E = int(mlp["router"]["experts"])
    shared = mlp.get("shared") or None
    names = {"router": p + "router"}
    for e in range(E):
        names.update({f"gate{e}": f"{p}e{e}.gate", f"up{e}": f"{p}e{e}.up", f"down{e}": f"{p}e{e}.down"})
    if shared:
        names.update(shared_gate=p + "shared.gate", shared_up=p + "shared.up", shared_down=p + "shared.down",
                     shared_sg=p + "shared.sg")
    return PartSpec("limited_experts", {
        "hidden_size": W, "experts": E, "top": int(mlp["router"]["top"]), "expert_ff": int(mlp["expert"]["ff"]),
        "limit": float(mlp["expert"]["limit"]), "shared_ff": int(shared["ff"]) if shared else 0,
        "shared_limit": float(shared["limit"]) if shared else None, "alpha": EXPERT_ALPHA,
    }, names)


def build_tevanex_spec(cfg: TevanexConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps

    def post_norm(name):
        # the constant on every branch rides in the weight of the norm behind it
        return PartSpec("rmsnorm", {"size": W, "eps": eps, "scale": cfg.residual_mult}, {"weight": name})

    # Only layers with tensors of their own are layers of the description; a layer that uses another's tensors is one
    # more application of that layer in the schedule, with a cache or state of its own.
    layers, index_of, schedule = [], {}, []
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is None:
            parts = dict(mixer=_mixer(cfg, i, layer), mixer_post_norm=post_norm(f"l{i}.norm1"))
            if layer.mlp is None:
                layers.append(LayerSpec("postnorm_mixer_only", parts))
            else:
                parts.update(feed_forward=_feed_forward(cfg, i, layer.mlp), ff_post_norm=post_norm(f"l{i}.norm2"))
                layers.append(LayerSpec("postnorm", parts))
            index_of[i] = len(layers) - 1
    for i, layer in enumerate(cfg.layers):
        schedule.append(ScheduleEntry(index_of[i if layer.weights_of is None else layer.weights_of]))
    spec = ModelSpec(
        architecture=cfg.architecture, hidden_size=W, vocab_size=cfg.vocab, max_position=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "scale": cfg.embedding_scale},
                           {"table": "embed"}),
        layers=layers, schedule=schedule,
        final_norm=PartSpec("rmsnorm", {"size": W, "eps": eps}, {"weight": "final.norm"}),
        lm_head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": W, "scale": cfg.logit_scale,
                                         "softcap": cfg.logit_softcap or None}, {"weight": "head"}),
        eos_token_ids=cfg.eos_token_ids,
    )
    spec.validate()
    return spec


register_architecture("Tevanex", TevanexConfig.from_dict, build_tevanex_spec)
