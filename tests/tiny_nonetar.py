"""Small Nonetar configurations and weights for the tests: sizes that differ from one another wherever the
design allows it (query against key/value heads, key against value size, taps, windows that are no multiple of
a page, blocks, groups), and weights drawn here."""

import json
import os

import numpy as np
import torch


def left(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, size=11, softcap=4.0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size}
    if softcap is not None:
        m["softcap"] = softcap
    return m


def right(width=36, blocks=3, conv=3):
    return {"width": width, "blocks": blocks, "conv": conv}


def parallel(left_=None, right_=None, left_scale=0.8, right_scale=1.3, mlp=None):
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": left_ or left(), "right": right_ or right(), "left_scale": left_scale, "right_scale": right_scale}}


def mamba(heads=4, vdim=12, state=10, groups=2, norm_groups=3, conv=4, mlp=None):
    return {"type": "mamba2", "mlp": mlp,
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def config(layers, width=48, vocab=101, streams=3, logit_scale=0.7, eps=1e-5):
    return {"architecture": "Nonetar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "streams": streams,
            "logit_scale": logit_scale, "layers": layers}


# both kinds of mixer, a layer without feed-forward, grouped and ungrouped heads, windows of 11, 20 and 5 tokens on
# pages of 8, an attention without cap, one without window
MIXED = config([mamba(mlp=dense(56)),
                parallel(mlp=dense(24)),
                parallel(left(heads=3, kv_heads=3, dim=8, vdim=8, scale=0.5, size=20, softcap=None), right(16, 1, 2)),
                mamba(heads=2, vdim=16, state=24, groups=1, norm_groups=1, conv=2, mlp=dense(32)),
                parallel(left(heads=6, kv_heads=1, dim=24, vdim=8, scale=0.2, size=5, softcap=1.5), right(40, 5, 4),
                         left_scale=1.1, right_scale=0.4, mlp=dense(16))])


def expected(cfg):
    from kv_cache_optimization_for_llm_b200.models.spec import expected_weights
    from kv_cache_optimization_for_llm_b200.registry import resolve_architecture
    arch = resolve_architecture(cfg)
    return expected_weights(arch.build_spec(arch.parse_config(cfg)))


def draw_weights(cfg, seed, gain=1.0):
    """Every tensor the model expects, drawn here and rounded to bfloat16 so that both precisions load the same
    numbers: matrices N(0, gain / sqrt(fan-in)), weights stored around zero and small vectors about 0, the mixing
    of the streams near the identity, step sizes and decays in a range where the states neither die at once nor
    stand still."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, ws in sorted(expected(cfg).items()):
        last = name.rsplit(".", 1)[-1]
        if name.endswith(".conv"):
            t = rng.normal(size=ws.shape) * 0.7
        elif last == "mix" and ".hc" in name:
            t = np.eye(ws.shape[0]) + 0.3 * rng.normal(size=ws.shape)
        elif ".hc" in name and last == "in":
            t = 1.0 / ws.shape[0] + 0.3 * rng.normal(size=ws.shape)
        elif ".hc" in name and last == "out":
            t = 1.0 + 0.3 * rng.normal(size=ws.shape)
        elif last == "temp":
            t = 1.0 + 0.3 * rng.normal(size=ws.shape)
        elif last == "lam":
            t = rng.normal(size=ws.shape) - 2.0          # softplus about 0.13: decays between exp(-1) and 1
        elif last == "A_log":
            t = rng.normal(size=ws.shape) * 0.5
        elif last == "shift":
            t = rng.uniform(0.0, 1.0, size=ws.shape)
        elif ws.kind == "vector":
            t = 1.0 + 0.2 * rng.normal(size=ws.shape)
        elif ws.kind == "bias":
            t = (0.2 if "norm" in last else 0.5) * rng.normal(size=ws.shape)
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
