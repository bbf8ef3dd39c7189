"""Arrangements of a mixer and a feed-forward inside one layer."""

from __future__ import annotations

import torch

from .. import ops
from .base import Part
from .registry import register


@register("block", "prenorm")
class PreNormBlock(Part):
    """``h += mixer(norm1(h)); h += ff(norm2(h))`` (upstream: base/src/engine.cu:639-859).

    The float32 residual travels with the branch output that has not been added
    yet: each norm adds the pending ``delta`` first, so add and norm are one kernel,
    and the block hands its feed-forward output on as the next pending delta.

    A mixer or feed-forward with ``fuses_residual = True`` goes one step further (bfloat16
    only; the 32-bit path keeps every formula as it stands).  When the block is built, the
    part multiplies the weight of the norm in front of it into its own input matrices
    (``fold_input_scale``) and the norm becomes weightless.  ``forward`` then may get ``x`` as
    an ``ops.PendingNorm``, carried out by the part's first product, and gets the residual as
    ``into=``, which its last product may add to itself, returning an ``ops.Folded``."""

    # the parts this arrangement takes, by name, and the family each is looked up in
    part_families = {"mixer": "mixer", "mixer_norm": "norm", "feed_forward": "feed_forward", "ff_norm": "norm"}

    def __init__(self, parts):
        self.parts = dict(parts)
        self.mixer, self.mixer_norm = parts["mixer"], parts["mixer_norm"]
        self.feed_forward, self.ff_norm = parts["feed_forward"], parts["ff_norm"]
        for part, norm in ((self.mixer, self.mixer_norm), (self.feed_forward, self.ff_norm)):
            if (getattr(part, "fuses_residual", False) and part.ctx.dtype == torch.bfloat16
                    and hasattr(norm, "give_up_weight") and norm.weight is not None):
                part.fold_input_scale(norm.give_up_weight())

    def cache_spec(self):
        """What this layer asks of the cache: its mixer's wish."""
        return self.mixer.cache_spec()

    def forward(self, residual, delta, batch, cache):
        if getattr(self.mixer, "fuses_residual", False):
            x = self.mixer_norm.forward(residual, delta, lazy=True)
            a = self.mixer.forward(x, batch, cache, into=residual)
        else:
            a = self.mixer.forward(self.mixer_norm.forward(residual, delta), batch, cache)
        if getattr(self.feed_forward, "fuses_residual", False):
            x = self.ff_norm.forward(residual, a, lazy=True)
            f = self.feed_forward.forward(x, batch, into=residual)
        else:
            f = self.feed_forward.forward(self.ff_norm.forward(residual, a), batch)
        return residual, f


@register("block", "sandwich")
class SandwichBlock(Part):
    """``h += post1(mixer(pre1(h))); h += post2(ff(pre2(h)))``: a norm in front of each sublayer and
    one behind it, before the residual add.  A per-channel scale of a branch belongs to its post
    norm (``scaled``).  The post norm is not a launch of its own: the branch output travels on as
    an :class:`ops.PostNormed`, and the next pre norm (of this layer, of the next one, or the
    model's last norm) norms it, adds it and norms the sum in one kernel.  A feed-forward that
    ends in a bias hands it over with its output (``forward(..., bias_out=True)``)."""

    part_families = {"mixer": "mixer", "mixer_norm": "norm", "mixer_post_norm": "norm",
                     "feed_forward": "feed_forward", "ff_norm": "norm", "ff_post_norm": "norm"}

    def __init__(self, parts):
        self.parts = dict(parts)
        self.mixer, self.mixer_norm, self.mixer_post = parts["mixer"], parts["mixer_norm"], parts["mixer_post_norm"]
        self.feed_forward = parts.get("feed_forward")
        self.ff_norm, self.ff_post = parts.get("ff_norm"), parts.get("ff_post_norm")

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, residual, delta, batch, cache):
        a = self.mixer.forward(self.mixer_norm.forward(residual, delta), batch, cache)
        pending = self.mixer_post.as_pending(a)
        if self.feed_forward is None:
            return residual, pending
        x = self.ff_norm.forward(residual, pending)
        if getattr(self.feed_forward, "hands_over_bias", False):
            f, bias = self.feed_forward.forward(x, batch, bias_out=True)
        else:
            f, bias = self.feed_forward.forward(x, batch), None
        return residual, self.ff_post.as_pending(f, bias)


@register("block", "sandwich_mixer_only")
class SandwichMixerBlock(SandwichBlock):
    """The sandwich block of a layer that has no feed-forward: ``h += post1(mixer(pre1(h)))``."""

    part_families = {"mixer": "mixer", "mixer_norm": "norm", "mixer_post_norm": "norm"}


@register("block", "postnorm")
class PostNormBlock(Part):
    """``h += post1(mixer(h)); h += post2(ff(h))``: the sublayers read the residual stream itself, and only their
    outputs pass a norm (whose weight carries any constant on the branch) before they join it.  A branch output
    travels on as an :class:`ops.PostNormed`; the kernel that norms it and adds it to the float32 stream also leaves
    the copy of the new stream in the compute type that the next sublayer reads (``ops.add_norm`` with "copy"), so a
    sublayer boundary is one launch, as in the arrangements with a norm in front."""

    part_families = {"mixer": "mixer", "mixer_post_norm": "norm", "feed_forward": "feed_forward", "ff_post_norm": "norm"}

    def __init__(self, parts):
        self.parts = dict(parts)
        self.mixer, self.mixer_post = parts["mixer"], parts["mixer_post_norm"]
        self.feed_forward, self.ff_post = parts.get("feed_forward"), parts.get("ff_post_norm")

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, residual, delta, batch, cache):
        dtype = self.mixer.ctx.dtype
        x = ops.add_norm(residual, delta, "copy", None, 0.0, dtype)
        if getattr(self.mixer, "hands_over_bias", False):      # the last product's bias rides with the pending output
            pending = self.mixer_post.as_pending(*self.mixer.forward(x, batch, cache, bias_out=True))
        else:
            pending = self.mixer_post.as_pending(self.mixer.forward(x, batch, cache))
        if self.feed_forward is None:
            return residual, pending
        x = ops.add_norm(residual, pending, "copy", None, 0.0, dtype)
        return residual, self.ff_post.as_pending(self.feed_forward.forward(x, batch))


@register("block", "postnorm_mixer_only")
class PostNormMixerBlock(PostNormBlock):
    """The post-norm block of a layer that has no feed-forward: ``h += post1(mixer(h))``."""

    part_families = {"mixer": "mixer", "mixer_post_norm": "norm"}


@register("block", "parallel")
class ParallelBlock(Part):
    """``h += mixer(norm(h)) + ff(norm(h))``: one norm, whose output both sublayers read.  The two
    branch outputs travel on together as an :class:`ops.PendingSum`; the next norm (of the next
    layer, or the model's last one) adds both to the float32 residual and norms the sum in one
    kernel."""

    part_families = {"mixer": "mixer", "norm": "norm", "feed_forward": "feed_forward"}

    def __init__(self, parts):
        self.parts = dict(parts)
        self.mixer, self.norm = parts["mixer"], parts["norm"]
        self.feed_forward = parts.get("feed_forward")

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, residual, delta, batch, cache):
        x = self.norm.forward(residual, delta)
        a = self.mixer.forward(x, batch, cache)
        f = self.feed_forward.forward(x, batch) if self.feed_forward is not None else None
        return residual, ops.PendingSum((a, f))


@register("block", "parallel_mixer_only")
class ParallelMixerBlock(ParallelBlock):
    """The parallel block of a layer that has no feed-forward: ``h += mixer(norm(h))``."""

    part_families = {"mixer": "mixer", "norm": "norm"}
