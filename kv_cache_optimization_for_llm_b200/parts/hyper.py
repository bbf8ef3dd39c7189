"""A residual stream kept as several copies (hyper-connections), and the token shift in front of a mixer.

The stream is float32 [T, S, W].  A sublayer reads ``u = sum_s in[s] x_s``, norms it, and writes back
``x_t <- sum_s mix[s, t] x_s + out[t] * y`` into every copy at once.  Nothing of this is a launch of its own
beyond one kernel per sublayer: the write stays pending (:class:`ops.PendingStreams`) until the next read, and
the kernel that carries it out also makes the next sublayer's normed input.  With one copy and
``in = mix = out = 1`` this is the ordinary pre-norm residual.
"""

from __future__ import annotations

import dataclasses

import torch

from .. import ops
from ..cache.specs import PagedWithStateSpec, SlotStateSpec, paged_part, state_part
from ..weights.loader import WeightSpec
from .base import Part
from .registry import register


@register("stream", "hyper_write")
class HyperWrite(Part):
    """How a sublayer's output ``y`` enters the ``streams`` copies of the residual stream:
    ``x_t <- sum_s mix[s, t] x_s + out[t] * y`` (``mix`` indexed [from, to]).  ``learned`` False: no tensors,
    the identity and ones (the ordinary residual add).  Nothing is launched here; the write travels on
    with ``y``.  params: streams, learned."""

    @classmethod
    def weight_specs(cls, params):
        if not params.get("learned", True):
            return {}
        s = int(params["streams"])
        return {"mix": WeightSpec((s, s), "bias"), "out": WeightSpec((s,), "bias")}

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ("streams",)

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.mix, self.out = weights.get("mix"), weights.get("out")

    def forward(self, residual, delta, embedded=None):
        """``delta``: the sublayer's output, one tensor or a tuple of up to two that are summed."""
        ys = delta if isinstance(delta, (tuple, list)) else (delta,)
        return ops.PendingStreams(ys, self.mix, self.out)


@register("norm", "hyper_rmsnorm")
class HyperRMSNorm(Part):
    """The read of a sublayer from ``streams`` copies of the residual stream and its RMS norm:
    ``u = sum_s in[s] x_s`` (``learned`` False: the plain sum), ``h = u / sqrt(mean(u^2) + eps) * w`` (``one_plus``:
    times ``1 + w``), all float32, in the kernel that first carries out the write pending from the sublayer before.
    ``scale``: a constant that multiplies the result (multiplied into the weight when the model is built).

    ``shift`` True adds the token shift: ``h_t + (h_{t-1} - h_t) * shift`` element by element, with ``h_{t-1}`` the
    previous token's row before the shift (zero in front of a sequence's first token).  The last row of a request
    is kept in ``size`` floats of its state slot, which the block asks for (``state_floats``).  For steps of single
    tokens the shift is part of the same kernel.
    params: size, streams, eps, one_plus, learned, shift, scale."""

    @classmethod
    def weight_specs(cls, params):
        n, specs = int(params["size"]), {}
        specs["weight"] = WeightSpec((n,), "bias" if params.get("one_plus") else "vector")
        if params.get("learned", True):
            specs["in"] = WeightSpec((int(params["streams"]),), "bias")
        if params.get("shift"):
            specs["shift"] = WeightSpec((n,), "bias")
        return specs

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ("streams",)

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.size, self.streams, self.eps = int(params["size"]), int(params["streams"]), float(params["eps"])
        self.one_plus = bool(params.get("one_plus"))
        self.weight = weights["weight"]
        scale = float(params.get("scale", 1.0))
        if scale != 1.0:
            self.weight = (((1.0 + self.weight) if self.one_plus else self.weight) * scale).contiguous()
            self.one_plus = False
        self.in_w = weights.get("in")
        self.shift = weights.get("shift")

    def state_floats(self) -> int:
        return self.size if self.shift is not None else 0

    def activation_widths(self):
        return [self.size] + ([2 * self.size] if self.shift is not None else [])

    def forward(self, residual, delta=None, rows=None, batch=None, state=None):
        """``state``: float32 view [slots, size] of the requests' last rows (with ``shift``)."""
        dt = self.ctx.dtype
        if self.shift is None or rows is not None:
            return ops.hyper_norm(residual, delta, self.in_w, self.weight, self.eps, self.one_plus, dt, dt, rows=rows)
        if batch.decode_only:
            return ops.hyper_norm(residual, delta, self.in_w, self.weight, self.eps, self.one_plus, dt, dt,
                                  shift=self.shift, shift_state=state, batch=batch)
        h, prev = ops.hyper_norm(residual, delta, self.in_w, self.weight, self.eps, self.one_plus, torch.float32, dt,
                                 shift_state=state, batch=batch, stage_prev=True)
        return ops.token_shift(h, prev, self.shift, state, batch, dt)


@register("block", "hyper_prenorm")
class HyperPreNormBlock(Part):
    """``x <- write1(mixer(norm1(read1(x)))); x <- write2(ff(norm2(read2(x))))`` over several copies of the residual
    stream.  The reads and norms are ``hyper_rmsnorm`` parts, the writes ``hyper_write`` parts; a write is carried out
    by the next read's kernel (of this layer, of the next one, or of the model's last norm).  When the mixer's norm
    shifts tokens, the layer asks for room for one normed row in the request's state slot beside what the mixer asks
    for, and hands each its own part of the slot."""

    part_families = {"mixer": "mixer", "mixer_norm": "norm", "mixer_write": "stream",
                     "feed_forward": "feed_forward", "ff_norm": "norm", "ff_write": "stream"}

    def __init__(self, parts):
        self.parts = dict(parts)
        self.mixer, self.mixer_norm, self.mixer_write = parts["mixer"], parts["mixer_norm"], parts["mixer_write"]
        self.feed_forward = parts.get("feed_forward")
        self.ff_norm, self.ff_write = parts.get("ff_norm"), parts.get("ff_write")
        wish = self.mixer.cache_spec()
        st = state_part(wish)
        if st is not None and st.dtype != torch.float32:
            raise ValueError("hyper_prenorm: the mixer's state must be float32 to share the slot with the shifted row")
        self.mixer_floats = 0
        if st is not None:
            self.mixer_floats = 1
            for n in st.shape:
                self.mixer_floats *= int(n)
        self.extra = int(self.mixer_norm.state_floats()) if hasattr(self.mixer_norm, "state_floats") else 0
        self._views = {}

    def cache_spec(self):
        wish = self.mixer.cache_spec()
        if not self.extra:
            return wish
        state = SlotStateSpec((self.mixer_floats + self.extra,), torch.float32)
        paged = paged_part(wish)
        return PagedWithStateSpec(paged, state) if paged is not None else state

    def _split(self, cache):
        """(the mixer's binding, the norm's rows of the slots) out of the layer's binding."""
        if not self.extra:
            return cache, None
        got = self._views.get(id(cache.state))
        if got is None or got[0] is not cache.state:
            n = self.mixer_floats
            got = (cache.state, cache.state[:, :n] if n else None, cache.state[:, n:n + self.extra])
            self._views[id(cache.state)] = got
        return dataclasses.replace(cache, state=got[1]), got[2]

    def forward(self, residual, delta, batch, cache):
        mixer_cache, rows = self._split(cache)
        h = self.mixer_norm.forward(residual, delta, batch=batch, state=rows)
        pending = self.mixer_write.forward(residual, self.mixer.forward(h, batch, mixer_cache))
        if self.feed_forward is None:
            return residual, pending
        h = self.ff_norm.forward(residual, pending)
        return residual, self.ff_write.forward(residual, self.feed_forward.forward(h, batch))


@register("block", "hyper_prenorm_mixer_only")
class HyperPreNormMixerBlock(HyperPreNormBlock):
    """The same for a layer that has no feed-forward."""

    part_families = {"mixer": "mixer", "mixer_norm": "norm", "mixer_write": "stream"}
