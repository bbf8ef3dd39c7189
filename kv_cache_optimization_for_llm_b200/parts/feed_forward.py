"""Feed-forward parts."""

from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import WeightSpec
from .base import Part
from .registry import register


@register("feed_forward", "swiglu")
class SwiGLU(Part):
    """``down( silu(gate(x)) * up(x) )``, no bias (upstream: base/src/engine.cu:780-855,
    base/src/kernels.cu:45-52).  gate and up are stored as one [2*I, H] matrix so
    one product feeds the activation kernel.  params: hidden_size, intermediate_size."""

    @classmethod
    def weight_specs(cls, params):
        h, i = params["hidden_size"], params["intermediate_size"]
        return {"gate": WeightSpec((i, h)), "up": WeightSpec((i, h)), "down": WeightSpec((h, i))}

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ("elementwise",) + (("gemm_f32",) if dtype == torch.float32 else ("gemm_bf16", "gemm_bf16_wide"))

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        inter = int(params["intermediate_size"])
        # gate and up rows alternate in blocks, so that a 128-row tile of the product holds
        # 64 gate features and the 64 up features of the same indices and the activation
        # can be the product's epilogue; widths that are no multiple of 64 keep [gate | up]
        self.block = 64 if inter % 64 == 0 else inter
        g, u = weights["gate"], weights["up"]
        if self.block == inter:
            self.gate_up = torch.cat([g, u], dim=0).contiguous()
        else:
            nb, h = inter // self.block, g.shape[1]
            self.gate_up = torch.stack([g.view(nb, self.block, h), u.view(nb, self.block, h)], dim=1) \
                .reshape(2 * inter, h).contiguous()
        self.down = weights["down"]

    fuses_residual = True

    def fold_input_scale(self, scale):
        """Multiplies ``scale`` [hidden] (the weight of the norm in front) into the input
        columns of the gate and up matrix, so that the norm itself can go without."""
        self.gate_up = (self.gate_up.float() * scale.float()[None, :]).to(self.gate_up.dtype).contiguous()

    def activation_widths(self):
        """Elements per token of the tensors one call produces: gate|up (when the activation is a
        kernel of its own), the activation, and the output (or its bfloat16 copy with sums)."""
        inter, hidden = self.gate_up.shape[0] // 2, self.down.shape[0]
        return [2 * inter, inter, 2 * hidden]

    def forward(self, x, batch, into=None):
        a = ops.linear_swiglu(x, self.gate_up, self.block)
        return ops.linear(a, self.down, into=into)


@register("feed_forward", "gated_dense")
class GatedDense(Part):
    """``down( act(gate(x) + b_gate) * (up(x) + b_up) ) + b_down`` with ``act`` the tanh form of GELU
    (or SiLU).  gate and up are one [2 I, H] matrix; their biases and the activation are one kernel
    behind the product.  The last bias can be handed to the caller instead of being added here
    (``bias_out``), for a norm kernel that adds it while it reads the rows anyway.
    params: hidden_size, intermediate_size, activation ("gelu_tanh" or "silu"), bias (bool)."""

    @classmethod
    def weight_specs(cls, params):
        h, i = params["hidden_size"], params["intermediate_size"]
        specs = {"gate": WeightSpec((i, h)), "up": WeightSpec((i, h)), "down": WeightSpec((h, i))}
        if params.get("bias", True):
            specs.update(gate_bias=WeightSpec((i,), "bias"), up_bias=WeightSpec((i,), "bias"),
                         down_bias=WeightSpec((h,), "bias"))
        return specs

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ("rowwise",) + (("gemm_f32",) if dtype == torch.float32 else ("gemm_bf16", "gemm_bf16_wide"))

    hands_over_bias = True

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.act = str(params.get("activation", "gelu_tanh"))
        if self.act not in ops.ACT_KINDS:
            raise ValueError(f"activation {self.act!r} is not known to this feed-forward (known: {sorted(ops.ACT_KINDS)})")
        self.gate_up = torch.cat([weights["gate"], weights["up"]], dim=0).contiguous()
        self.down = weights["down"]
        self.bias = self.down_bias = None
        if params.get("bias", True):
            self.bias = torch.cat([weights["gate_bias"], weights["up_bias"]]).contiguous()
            self.down_bias = weights["down_bias"]

    def activation_widths(self):
        inter, hidden = self.gate_up.shape[0] // 2, self.down.shape[0]
        return [2 * inter, inter, hidden]

    def forward(self, x, batch, bias_out=False):
        a = ops.bias_act_mul(ops.linear(x, self.gate_up), self.bias, self.act)
        y = ops.linear(a, self.down)
        if bias_out:
            return y, self.down_bias
        if self.down_bias is not None:
            y = y + self.down_bias.to(y.dtype)
        return y


@register("feed_forward", "dense_xielu")
class DenseXIELU(Part):
    """``down( act(up(x)) )`` without gate or bias, ``act`` the xIELU with two learned numbers (p, q):
    ``z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2``.
    params: hidden_size, intermediate_size."""

    @classmethod
    def weight_specs(cls, params):
        h, i = int(params["hidden_size"]), int(params["intermediate_size"])
        return {"up": WeightSpec((i, h)), "down": WeightSpec((h, i)), "act": WeightSpec((2,), "bias")}

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ("streams",) + (("gemm_f32",) if dtype == torch.float32 else ("gemm_bf16", "gemm_bf16_wide"))

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.up, self.down, self.act = weights["up"], weights["down"], weights["act"]

    def activation_widths(self):
        return [self.up.shape[0], self.up.shape[0], self.down.shape[0]]

    def forward(self, x, batch):
        return ops.linear(ops.xielu(ops.linear(x, self.up), self.act), self.down)
