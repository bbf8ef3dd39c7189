"""Position encodings."""

from __future__ import annotations

import math

import torch

from .base import Part
from .registry import register


def rope_inv_freq(head_dim: int, theta: float, scaling) -> torch.Tensor:
    """Rotary frequencies in float64: ``1/theta^(2i/d)``, then the llama3 rescale by
    wavelength band: long waves divided by ``factor``, short ones kept, a linear
    blend between (upstream computes the same in float32, base/src/kernels.cu:58-83)."""
    i = torch.arange(head_dim // 2, dtype=torch.float64)
    inv = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float64), 2.0 * i / head_dim)
    if not scaling:
        return inv
    kind = scaling.get("rope_type", scaling.get("type", "llama3"))
    if kind == "yarn":
        return yarn_inv_freq(head_dim, float(theta), scaling)[0]
    if kind != "llama3":
        raise ValueError(f"rope scaling of type {kind!r} is not known to this position encoding "
                         "(known: none, 'llama3', 'yarn')")
    factor = float(scaling["factor"])
    low_ff, high_ff = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    wavelen = 2.0 * math.pi / inv
    smooth = (orig / wavelen - low_ff) / (high_ff - low_ff)
    blended = (1.0 - smooth) * (inv / factor) + smooth * inv
    out = torch.where(wavelen > orig / low_ff, inv / factor,
                      torch.where(wavelen >= orig / high_ff, blended, inv))
    return out


def yarn_inv_freq(dims: int, base: float, scaling):
    """(frequencies [dims / 2] in float64, factor on cos and sin) of a rotation stretched for longer sequences than
    the ``original`` ones (YaRN): with ``pair(t) = dims ln(original / (2 pi t)) / (2 ln base)``, the pair index whose
    wave turns ``t`` times over the original length, ``lo = max(floor(pair(fast)), 0)``, ``hi = min(ceil(pair(slow)),
    dims - 1)`` and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``, pair i's frequency is
    ``f_i / factor * ramp_i + f_i (1 - ramp_i)``: fast waves stay, slow ones are divided by ``factor``.  cos and sin
    are multiplied by ``0.1 ln(factor) + 1``.  scaling: factor, original, fast, slow."""
    for key in ("factor", "original", "fast", "slow"):
        if scaling.get(key) is None:
            raise ValueError(f"rope scaling of type 'yarn' needs the key {key!r}")
    i = torch.arange(dims // 2, dtype=torch.float64)
    inv = 1.0 / torch.pow(torch.tensor(float(base), dtype=torch.float64), 2.0 * i / dims)
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return inv / factor * ramp + inv * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def _rotary_tables(ctx, kind: str, dims: int, base: float, scaling):
    """float32 cos and sin [max_positions, dims / 2] on the device, shared between equal parts; angles in float64."""
    key = (kind, dims, float(base), tuple(sorted((k, str(v)) for k, v in (scaling or {}).items())), ctx.max_positions)
    if key not in ctx.shared:
        grow = 1.0
        if not dims:
            inv = torch.zeros(0, dtype=torch.float64)
        elif scaling and scaling.get("rope_type", scaling.get("type", "llama3")) == "yarn":
            inv, grow = yarn_inv_freq(dims, base, scaling)
        else:
            inv = rope_inv_freq(dims, base, scaling)
        ang = torch.arange(ctx.max_positions, dtype=torch.float64)[:, None] * inv[None, :]
        ctx.shared[key] = ((ang.cos() * grow).to(torch.float32).to(ctx.device).contiguous(),
                           (ang.sin() * grow).to(torch.float32).to(ctx.device).contiguous())
    return ctx.shared[key]


@register("position", "rope")
class RotaryEncoding(Part):
    """Rotate-half rotary encoding with optional llama3 or YaRN frequency scaling (``scaling["rope_type"]`` "llama3" or
    "yarn"; see :func:`yarn_inv_freq`).

    Holds float32 tables ``cos, sin [max_positions, rotary_dim/2]`` whose angles
    ``pos * inv_freq`` are formed in float64 (upstream: float32 tables with each
    value stored twice, base/src/kernels.cu:85-105).  The rotation itself runs in
    the kernel that also writes keys and values to the cache.
    params: head_dim, rotary_dim, theta, scaling (dict or None)."""

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.rotary_dim = int(params["rotary_dim"])
        if self.rotary_dim % 2 or self.rotary_dim > params["head_dim"]:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim")
        self.cos, self.sin = _rotary_tables(ctx, "rope", self.rotary_dim, float(params["theta"]), params.get("scaling"))

    def tables(self):
        return self.cos, self.sin


@register("position", "rope_interleaved")
class InterleavedRotaryEncoding(Part):
    """Rotary encoding whose pairs are neighbours: dimension 2i turns with dimension 2i + 1 by
    the angle ``pos * base^(-2i/dims)`` for i < dims/2; dimensions from ``dims`` on pass unchanged.
    Holds float32 tables ``cos, sin [max_positions, dims/2]`` with angles formed in float64; the
    rotation itself runs inside the mixer's kernels.  ``scaling`` as for the rotate-half kind.
    params: dims, base, scaling (dict or None)."""

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.rotary_dim = int(params["dims"])
        if self.rotary_dim % 2 or self.rotary_dim < 0:
            raise ValueError(f"rotary dims {self.rotary_dim} must be even")
        self.cos, self.sin = _rotary_tables(ctx, "rope_interleaved", self.rotary_dim, float(params["base"]),
                                            params.get("scaling"))

    def tables(self):
        return self.cos, self.sin
