"""Small Tevanex configurations and weights for the tests: sizes that differ from one another wherever the design
allows it (query against key/value heads, key against value size, turning channels against the head size, blocks of
positions that are no multiple of a page, experts against chosen experts, the shared expert's width and limit against
the routed ones'), and weights drawn here."""

import json
import os

import numpy as np
import torch


def mlstm(heads=3, dim=12, vdim=20, gate_cap=9.0):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap}


def attention(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, size=11, rot_dims=8, base=3000.0, softcap=None, scaling=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size}
    if rot_dims is not None:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling is not None:
            m["rot"]["scaling"] = scaling
    if softcap is not None:
        m["softcap"] = softcap
    return m


YARN = {"factor": 3.0, "original": 40, "fast": 6.0, "slow": 0.5}


def moe(experts=5, top=2, ff=12, limit=1.1, shared_ff=20, shared_limit=0.8):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared_ff:
        m["shared"] = {"ff": shared_ff, "limit": shared_limit}
    return m


def layer(kind, mixer, mlp=None, weights_of=None):
    entry = {"type": kind, "mixer": mixer, "mlp": mlp}
    if weights_of is not None:
        entry["weights_of"] = weights_of
    return entry


def config(layers, width=40, vocab=97, emb_scale=0.7, mult=0.4, logit_scale=0.6, logit_softcap=7.0, eps=1e-5):
    cfg = {"architecture": "Tevanex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": emb_scale},
           "residual_mult": mult, "logit_scale": logit_scale, "layers": layers}
    if logit_softcap is not None:
        cfg["logit_softcap"] = logit_softcap
    return cfg


_A1 = attention()
_A2 = attention(heads=3, kv_heads=1, dim=24, vdim=8, scale=0.2, size=20, rot_dims=10, base=500.0, softcap=3.0, scaling=YARN)
_M = mlstm()
_F = moe()
# all three kinds of mixer, a layer without feed-forward, layers that use another layer's tensors (also one that comes
# before a layer of its own kind with other sizes), blocks of 11, 20 and 5 positions on pages of 8
MIXED = config([layer("mlstm", _M, _F),
                layer("attention", _A1, moe(experts=3, top=1, ff=16, limit=2.0, shared_ff=0)),
                layer("attention_2", _A2, _F),
                layer("mlstm", _M, _F, weights_of=0),
                layer("attention", attention(heads=2, kv_heads=2, dim=8, vdim=8, scale=0.5, size=5, rot_dims=8), None),
                layer("attention_2", _A2, _F, weights_of=2),
                layer("attention", _A1, moe(experts=3, top=1, ff=16, limit=2.0, shared_ff=0), weights_of=1)])


# no mixer with a state of fixed size: the engine may then replay lone prompt portions and mixed steps from graphs
ATTENTION_ONLY = config([layer("attention", _A1, _F),
                         layer("attention_2", _A2, moe(experts=4, top=2, ff=8, limit=1.5, shared_ff=8, shared_limit=1.0)),
                         layer("attention", _A1, _F, weights_of=0),
                         layer("attention_2", attention(heads=2, kv_heads=1, dim=16, vdim=16, scale=0.25, size=None, rot_dims=16,
                                                        base=100.0, softcap=6.0), None)], width=32, vocab=61)


def expected(cfg):
    from kv_cache_optimization_for_llm_b200.models.spec import expected_weights
    from kv_cache_optimization_for_llm_b200.registry import resolve_architecture
    arch = resolve_architecture(cfg)
    return expected_weights(arch.build_spec(arch.parse_config(cfg)))


def draw_weights(cfg, seed, gain=1.0):
    """Every tensor the model expects, drawn here and rounded to bfloat16 so that both precisions load the same
    numbers: matrices N(0, gain / sqrt(fan-in)), norm weights about 1, biases and sinks about 0, forget-gate biases
    about 2 so that the memories neither die at once nor stand still, routers wide enough that the choice is clear."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, ws in sorted(expected(cfg).items()):
        last = name.rsplit(".", 1)[-1]
        if name.endswith(".f.b"):
            t = 2.0 + rng.normal(size=ws.shape)
        elif name.endswith(".i.b"):
            t = rng.normal(size=ws.shape)
        elif last == "sink":
            t = rng.normal(size=ws.shape)
        elif last == "router":
            t = rng.normal(size=ws.shape) * (3.0 / np.sqrt(ws.shape[-1]))
        elif name.endswith(".mix.i") or name.endswith(".mix.f"):
            t = rng.normal(size=ws.shape) * (2.0 / np.sqrt(ws.shape[-1]))
        elif ws.kind == "vector":
            t = 1.0 + 0.2 * rng.normal(size=ws.shape)
        elif ws.kind == "bias":
            t = 0.5 * rng.normal(size=ws.shape)
        else:
            t = rng.normal(size=ws.shape) * (gain / np.sqrt(ws.shape[-1]))
        out[name] = torch.as_tensor(t, dtype=torch.float32).to(torch.bfloat16)
    return out


def write_model(folder, cfg, seed, gain=1.0, weights=None):
    from kv_cache_optimization_for_llm_b200.weights.safetensors_io import write_tensors
    os.makedirs(folder, exist_ok=True)
    tensors = weights if weights is not None else draw_weights(cfg, seed, gain)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_tensors(os.path.join(folder, "model.safetensors"), tensors, metadata={"format": "pt"})
    return {k: v.float().numpy().astype(np.float64) for k, v in tensors.items()}
