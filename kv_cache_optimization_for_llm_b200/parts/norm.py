"""Norms over the model's width with the residual add fused in front of them."""

from __future__ import annotations

from .. import ops
from ..weights.loader import WeightSpec
from .base import Part
from .registry import register


@register("norm", "rmsnorm")
class RMSNorm(Part):
    """``y = v / sqrt(mean(v^2) + eps) * w`` over the whole width, plain weight
    (upstream: base/src/kernels.cu:10-36), where ``v = residual + delta`` is summed
    and kept in float32 (upstream adds in a second kernel and keeps bfloat16,
    base/src/kernels.cu:38-43).  With ``scale`` (a constant on a branch, or on the logits behind the model's last
    norm) the weight is multiplied by it once, when the model is built.

    The same part may stand behind a branch (``as_pending``): there it is not carried out at once but handed on as
    an :class:`ops.PostNormed`, and whoever brings the residual stream up to date next norms the branch output and
    adds it in one kernel.  params: size, eps, scale."""

    @classmethod
    def weight_specs(cls, params):
        return {"weight": WeightSpec((params["size"],), "vector")}

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ("elementwise",)      # the general kernels (rowwise) are loaded at first use, if a branch ever hands it a post norm or several summands

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.eps = float(params["eps"])
        self.size = int(params["size"])
        self.weight = weights["weight"]
        if params.get("scale") is not None and float(params["scale"]) != 1.0:
            self.weight = (self.weight * float(params["scale"])).contiguous()

    def activation_widths(self):
        return [self.size]

    def as_pending(self, delta, bias=None):
        """``delta`` (a branch's output, ``bias`` still to be added) with this norm pending on it."""
        return ops.PostNormed(delta, bias, "rms", self.weight, self.eps)

    def give_up_weight(self):
        """Hands the weight to a part that multiplies it into its own matrices
        (``fold_input_scale``); the norm is weightless from then on."""
        w, self.weight = self.weight, None
        return w

    def forward(self, residual, delta=None, rows=None, lazy=False):
        if isinstance(delta, ops.Folded):
            # the branch before this norm has added its output itself and left the sums of squares
            if lazy and rows is None and self.weight is None:
                return ops.PendingNorm(residual, delta.xb, delta.sumsq, self.eps, self.ctx.dtype)
            delta = None
        if isinstance(delta, ops.PostNormed):
            # a branch whose output passes a norm of its own first: the general kernel takes it in
            return ops.add_norm(residual, delta, "rms", self.weight, self.eps, self.ctx.dtype, rows)
        if isinstance(delta, ops.PendingSum):
            # several summands at once (two branches of a layer, what the start of a pass adds)
            return ops.join_norm(residual, delta, "rms", self.weight, self.eps, self.ctx.dtype, rows,
                                 compute_dtype=self.ctx.dtype)
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, self.ctx.dtype, rows)


@register("norm", "layernorm")
class LayerNorm(Part):
    """``y = (v - mean(v)) / sqrt(var(v) + eps) * w`` over the whole width, the variance being the
    mean squared deviation, a weight and no bias; ``v = residual + delta`` is summed and kept in
    float32 as for :class:`RMSNorm`.  With a ``scale`` tensor (a per-channel scale of a branch, "layer
    scale") the output is also multiplied by it; the two vectors are multiplied once, when the
    model is built.

    The same part stands behind a branch (``as_pending``): there it is not carried out at once
    but handed on as an :class:`ops.PostNormed`, and the norm in front of the next sublayer does
    post-norm, residual add and its own norm in one kernel.
    params: size, eps."""

    @classmethod
    def weight_specs(cls, params):
        specs = {"weight": WeightSpec((params["size"],), "vector")}
        if params.get("scaled"):
            specs["scale"] = WeightSpec((params["size"],), "vector")
        return specs

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ("rowwise",)

    norm_kind = "layer"

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.eps = float(params["eps"])
        self.size = int(params["size"])
        self.weight = weights["weight"]
        if params.get("scaled"):
            self.weight = (self.weight * weights["scale"]).contiguous()

    def activation_widths(self):
        return [self.size]

    def as_pending(self, delta, bias=None):
        """``delta`` (a branch's output, ``bias`` still to be added) with this norm pending on it."""
        return ops.PostNormed(delta, bias, self.norm_kind, self.weight, self.eps)

    def forward(self, residual, delta=None, rows=None, lazy=False):
        if isinstance(delta, ops.Folded):
            delta = None        # that branch has added its output to the residual itself
        if isinstance(delta, ops.PendingSum):
            return ops.join_norm(residual, delta, self.norm_kind, self.weight, self.eps, self.ctx.dtype, rows,
                                 compute_dtype=self.ctx.dtype)
        return ops.add_norm(residual, delta, self.norm_kind, self.weight, self.eps, self.ctx.dtype, rows)
