"""A feed-forward of many small experts of which every token uses a few."""

from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import WeightSpec
from .base import Part
from .registry import register


@register("feed_forward", "routed_experts")
class RoutedExperts(Part):
    """``experts`` feed-forward layers ``W_down relu(W_up h)^2`` (``expert_ff`` wide, no biases) of which a
    token uses ``top``.  The router's logits ``W_r h`` are float32; the scores are their softmax over
    all experts; the ``top`` experts with the largest ``score + correction`` are chosen and weighted with
    ``score / (sum of the chosen scores + 1e-20) * scale``.  The last ``identity`` outputs of the router
    are experts without matrices that hand their input on.  With ``shared_ff`` > 0 one more expert
    of the same form runs for every token with weight 1.

    All first matrices are stacked into one, and all second matrices side by side into another: a
    step is two products around an activation kernel that also multiplies each expert's features
    by the token's weight for it (0 where it was not chosen), so the second product's float32 sums
    add up exactly the chosen experts.  Every expert is computed for every token; what that costs
    against products over the chosen tokens only is ``experts / top`` times the experts' arithmetic
    in long steps and nothing in steps of a few tokens, which read every expert's matrices anyway.
    params: hidden_size, experts, identity, top, scale, expert_ff, shared_ff."""

    @classmethod
    def weight_specs(cls, params):
        h, E, I, F, S = (int(params[k]) for k in ("hidden_size", "experts", "identity", "expert_ff", "shared_ff"))
        specs = {"router": WeightSpec((E + I, h), "bias"), "correction": WeightSpec((E + I,), "bias")}
        for e in range(E):
            specs[f"up{e}"] = WeightSpec((F, h))
            specs[f"down{e}"] = WeightSpec((h, F))
        if S:
            specs["shared_up"] = WeightSpec((S, h))
            specs["shared_down"] = WeightSpec((h, S))
        return specs

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ("experts",) + (("gemm_f32",) if dtype == torch.float32 else ("gemm_bf16", "gemm_bf16_wide"))

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.hidden = int(params["hidden_size"])
        self.E, self.I, self.top = int(params["experts"]), int(params["identity"]), int(params["top"])
        self.F, self.S = int(params["expert_ff"]), int(params.get("shared_ff") or 0)
        self.scale = float(params["scale"])
        if not 1 <= self.top <= min(32, self.E + self.I):
            raise ValueError(f"routed_experts: {self.top} of {self.E + self.I} experts per token is refused (1 to 32)")
        ups = [weights[f"up{e}"] for e in range(self.E)] + ([weights["shared_up"]] if self.S else [])
        downs = [weights[f"down{e}"] for e in range(self.E)] + ([weights["shared_down"]] if self.S else [])
        self.width = self.E * self.F + self.S
        # the products' inner sizes are padded to multiples of 8 (16-byte rows), the padding being zeros
        self.pad = (-self.width) % 8
        if ups:
            up = torch.cat(ups, dim=0)
            down = torch.cat(downs, dim=1)
            if self.pad:
                up = torch.cat([up, up.new_zeros((self.pad, up.shape[1]))], dim=0)
                down = torch.cat([down, down.new_zeros((down.shape[0], self.pad))], dim=1)
            self.up, self.down = up.contiguous(), down.contiguous()
        else:
            self.up = self.down = None
        self.router, self.correction = weights["router"], weights["correction"]
        # The router's products are float32 sums of float32 products.  Where the compute type holds the router's
        # weights exactly (a checkpoint stored in that type), the step's matrix product kernels make them (tensor
        # cores add up bfloat16 products exactly in float32); otherwise the routing kernel does, on float32 weights.
        self.router_in_compute_type = None
        lowp = self.router.to(ctx.dtype)
        if self.hidden % 8 == 0 and torch.equal(lowp.float(), self.router):
            self.router_in_compute_type = lowp.contiguous()

    def activation_widths(self):
        w = self.width + self.pad
        return [4 * (self.E + self.I) + 2, w, w, self.hidden]

    def forward(self, x, batch):
        logits = None
        if self.router_in_compute_type is not None:
            logits = ops.linear(x, self.router_in_compute_type, out_dtype=torch.float32)
        gate, identity_weight = ops.route(x, self.router, self.correction, self.E, self.I, self.top, self.scale, logits)
        if self.up is not None:
            a = ops.expert_act(ops.linear(x, self.up), gate, self.E, self.F, self.S + self.pad)
            y = ops.linear(a, self.down)
        else:
            y = ops.new(tuple(x.shape), x.dtype, x.device)
            y.zero_()
        if identity_weight is not None:
            ops.row_axpy(y, x, identity_weight)
        return y


@register("feed_forward", "limited_experts")
class LimitedExperts(Part):
    """``experts`` gated feed-forward layers without biases, of which a token uses ``top``:

        g = min(W_gate x, limit),   u = clamp(W_up x, -limit, limit),   expert(x) = W_down (g sigmoid(alpha g) (u + 1)).

    The router's logits ``W_r h`` are float32; the scores are their sigmoids, each by itself; the ``top`` experts with
    the largest scores are chosen and weighted with their scores as they are.  The weight multiplies the expert's
    *input*: the layer's output is the sum of ``expert(w h)`` over the chosen experts.  With ``shared_ff`` > 0 one more
    expert of the same form (its own ``shared_limit``) runs for every token with weight 1, and its output is multiplied
    by ``sigmoid(w_sg . h)``, one number per token.

    All gate and up matrices are stacked into one matrix, expert after expert, and all down matrices side by side
    into another: a step is two products around an activation kernel.  Without biases ``W (w h) = w (W h)``, so the
    kernel multiplies a chosen expert's two first products by the token's weight before it limits them, and writes 0
    for an expert that was not chosen; the second product's float32 sums then add up exactly the chosen experts.  The
    shared expert's gate multiplies its activation, which for a last matrix without bias is the same as multiplying its
    output.  The router's rows and the shared gate's row are one small product with float32 results.  Every expert is
    computed for every token (see :class:`RoutedExperts` for what that costs).
    params: hidden_size, experts, top, expert_ff, limit, shared_ff, shared_limit, alpha."""

    @classmethod
    def weight_specs(cls, params):
        h, E, F, S = (int(params[k]) for k in ("hidden_size", "experts", "expert_ff", "shared_ff"))
        specs = {"router": WeightSpec((E, h))}
        for e in range(E):
            specs[f"gate{e}"] = WeightSpec((F, h))
            specs[f"up{e}"] = WeightSpec((F, h))
            specs[f"down{e}"] = WeightSpec((h, F))
        if S:
            specs.update(shared_gate=WeightSpec((S, h)), shared_up=WeightSpec((S, h)), shared_down=WeightSpec((h, S)),
                         shared_sg=WeightSpec((1, h)))
        return specs

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ("experts",) + (("gemm_f32",) if dtype == torch.float32 else ("gemm_bf16", "gemm_bf16_wide"))

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.hidden = int(params["hidden_size"])
        self.E, self.top = int(params["experts"]), int(params["top"])
        self.F, self.S = int(params["expert_ff"]), int(params.get("shared_ff") or 0)
        self.limit = float(params["limit"])
        self.shared_limit = float(params.get("shared_limit") or self.limit)
        self.alpha = float(params.get("alpha", 1.702))
        if not 1 <= self.top <= min(32, self.E):
            raise ValueError(f"limited_experts: {self.top} of {self.E} experts per token is refused (1 to 32)")
        first, second = [], []
        for e in range(self.E):
            first += [weights[f"gate{e}"], weights[f"up{e}"]]
            second.append(weights[f"down{e}"])
        if self.S:
            first += [weights["shared_gate"], weights["shared_up"]]
            second.append(weights["shared_down"])
        self.first = torch.cat(first, dim=0).contiguous()
        down = torch.cat(second, dim=1)
        # the second product's inner size is padded to a multiple of 8 (16-byte rows), the padding being zeros
        self.pad = (-down.shape[1]) % 8
        if self.pad:
            down = torch.cat([down, down.new_zeros((down.shape[0], self.pad))], dim=1)
        self.down = down.contiguous()
        # the router's rows, then the shared gate's row: float32 sums of products in the compute type
        self.small = torch.cat([weights["router"]] + ([weights["shared_sg"]] if self.S else []), dim=0).contiguous()

    def activation_widths(self):
        inner = self.E * self.F + self.S
        return [2 * inner, inner + self.pad, 6 * (self.E + 1), self.hidden]

    def forward(self, x, batch):
        logits = ops.linear(x, self.small, out_dtype=torch.float32)
        gate, _ = ops.route(x, None, None, self.E, 0, self.top, 1.0, logits, score="sigmoid", renormalize=False)
        p = ops.linear(x, self.first)
        a = ops.limited_act(p, gate, logits[:, self.E] if self.S else None, self.E, self.F, self.S, self.pad, self.limit,
                            self.shared_limit, self.alpha)
        return ops.linear(a, self.down)
