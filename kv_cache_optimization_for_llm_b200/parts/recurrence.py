"""Mixers whose state is a linear recurrence with a decay that depends on the token: a gated diagonal
recurrence per channel, a matrix state per head with one decay per head (state-space duality), and a matrix
memory per head with exponential gates and a running maximum (mLSTM).

The first two make their projections in one product, pass part of it through a short causal convolution whose last
inputs live in the request's state slot beside the recurrence's state (float32), and walk the request's
tokens of the step in one kernel (csrc/kernels/recurrence.cu); the third has no convolution and its kernels are
csrc/kernels/mlstm.cu.  A request that starts at position 0 starts from a zero state.
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache.specs import SlotStateSpec
from ..weights.loader import WeightSpec
from .base import Part
from .delta_rule import _pad8, _stack
from .registry import register


def _gemm_modules(dtype):
    return ("gemm_f32",) if dtype == torch.float32 else ("gemm_bf16", "gemm_bf16_wide")


@register("mixer", "gated_linear_recurrence")
class GatedLinearRecurrence(Part):
    """Two branches of ``width`` channels: ``y = gelu_tanh(W_y h + b_y)`` and ``u = conv(W_x h + b_x)``, a causal
    convolution over time per channel (``conv`` taps, the last for the token itself, a bias, zeros before the
    sequence's start, no activation).  ``u`` is cut into ``blocks`` equal parts; in part b, with square matrices
    [out, in], ``r = sigmoid(Wa_b u_b + ba_b)`` and ``i = sigmoid(Wi_b u_b + bi_b)``.  Then per channel

        a = exp(-decay_scale * r * softplus(lam)),     S_t = a S_{t-1} + sqrt(1 - a^2) * i * u,

    from S = 0, and the result is ``W_o (S * y)``.  Gates, decay and state are float32.  The request's state is S
    and the convolution's last ``conv - 1`` inputs.  ``out_scale`` multiplies the result (before W_o).
    params: hidden_size, width, blocks, conv, decay_scale, out_scale."""

    @classmethod
    def weight_specs(cls, params):
        h, C, nb, taps = (int(params[k]) for k in ("hidden_size", "width", "blocks", "conv"))
        bw = C // nb
        return {"y": WeightSpec((C, h)), "y_bias": WeightSpec((C,), "bias"), "x": WeightSpec((C, h)),
                "x_bias": WeightSpec((C,), "bias"), "conv": WeightSpec((C, taps), "bias"),
                "conv_bias": WeightSpec((C,), "bias"), "ra": WeightSpec((nb, bw, bw)), "ra_bias": WeightSpec((nb, bw), "bias"),
                "ri": WeightSpec((nb, bw, bw)), "ri_bias": WeightSpec((nb, bw), "bias"), "lam": WeightSpec((C,), "bias"),
                "o": WeightSpec((h, C))}

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ("recurrence", "delta_rule") + _gemm_modules(dtype)

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.C, self.nb, self.taps = int(params["width"]), int(params["blocks"]), int(params["conv"])
        if self.C % self.nb:
            raise ValueError(f"gated_linear_recurrence: {self.C} channels do not split into {self.nb} equal blocks")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"gated_linear_recurrence: {self.taps} convolution taps are refused (1 to 16)")
        self.decay_scale = float(params.get("decay_scale", 8.0))
        self.out_scale = float(params.get("out_scale", 1.0))
        # one product makes both branches: [x | y], each starting on a multiple of 8 rows
        self.w_in, (self.at_x, self.at_y) = _stack([weights["x"], weights["y"]], ctx.dtype)
        self.x_bias, self.y_bias = weights["x_bias"], weights["y_bias"]
        self.conv_w, self.conv_bias = weights["conv"], weights["conv_bias"]
        # per block the rows that make r, then the rows that make i
        self.gates = torch.cat([weights["ra"], weights["ri"]], dim=1).contiguous()
        self.ra_bias = weights["ra_bias"].reshape(-1).contiguous()
        self.ri_bias = weights["ri_bias"].reshape(-1).contiguous()
        self.lam, self.o = weights["lam"], weights["o"]

    def cache_spec(self):
        return SlotStateSpec((self.C * self.taps,), torch.float32)      # S, then taps - 1 rows of inputs

    def activation_widths(self):
        return [self.w_in.shape[0], self.C, 4 * self.C, 4 * self.C, self.C, self.o.shape[0]]

    def readout(self, p, first, batch, cache):
        """From the product ``p`` (this mixer's columns start at ``first``) to the gated state [T, width]."""
        tails = cache.state[:, self.C:] if self.taps > 1 else None
        u = ops.conv_silu(p, first + self.at_x, self.C, self.conv_w, tails, batch, act="none", in_bias=self.x_bias,
                          out_bias=self.conv_bias)
        a, b = ops.gate_coeffs(u, self.gates, self.ra_bias, self.ri_bias, self.lam, self.decay_scale)
        return ops.diag_scan(a, b, (p, first + self.at_y), self.y_bias, self.out_scale, cache.state, batch, self.ctx.dtype)

    def forward(self, x, batch, cache):
        return ops.linear(self.readout(ops.linear(x, self.w_in), 0, batch, cache), self.o)


@register("mixer", "state_space_duality")
class StateSpaceDuality(Part):
    """A matrix state per head with one decay per head and token.  One product lays out
    [z: inner | x: inner | B: groups * state | C: groups * state | dt: heads], inner = heads * vdim.  x, B and C together
    pass a causal convolution per channel (``conv`` taps, the last for the token itself, a bias, zeros before the
    sequence's start) and SiLU.  Per head (head h reads group ``h // (heads / groups)``), with
    ``dt = softplus(dt + dt_bias)``:

        S_t = exp(-exp(A_log_h) dt) S_{t-1} + dt B_t x_t^T   (S is state x vdim),    y_t = S_t^T C_t + D_h x_t.

    The heads' y, side by side, are multiplied by ``silu(z)``, divided in ``norm_groups`` equal parts each by its own
    root mean square, multiplied by ``norm``, and projected by W_o.  Step sizes, decays and the state are float32.
    The request's state is the matrices and the convolution's last ``conv - 1`` inputs.
    params: hidden_size, heads, vdim, state, groups, norm_groups, conv, eps."""

    @classmethod
    def weight_specs(cls, params):
        h, H, Dv, N, G, taps = (int(params[k]) for k in ("hidden_size", "heads", "vdim", "state", "groups", "conv"))
        inner, ch = H * Dv, H * Dv + 2 * G * N
        return {"in": WeightSpec((2 * inner + 2 * G * N + H, h)), "conv": WeightSpec((ch, taps), "bias"),
                "conv_bias": WeightSpec((ch,), "bias"), "dt_bias": WeightSpec((H,), "bias"), "A_log": WeightSpec((H,), "bias"),
                "D": WeightSpec((H,), "bias"), "norm": WeightSpec((inner,), "vector"), "o": WeightSpec((h, inner))}

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ("recurrence", "delta_rule") + _gemm_modules(dtype)

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.H, self.Dv, self.N, self.G = (int(params[k]) for k in ("heads", "vdim", "state", "groups"))
        self.norm_groups, self.taps, self.eps = int(params["norm_groups"]), int(params["conv"]), float(params["eps"])
        if self.H % self.G:
            raise ValueError(f"state_space_duality: {self.H} heads cannot share {self.G} groups evenly")
        self.inner = self.H * self.Dv
        if self.inner % self.norm_groups:
            raise ValueError(f"state_space_duality: {self.inner} channels do not split into {self.norm_groups} equal parts")
        if not 1 <= self.N <= 256:
            raise ValueError(f"state_space_duality: a state of {self.N} rows is refused (1 to 256)")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"state_space_duality: {self.taps} convolution taps are refused (1 to 16)")
        self.channels = self.inner + 2 * self.G * self.N
        w = weights["in"]
        # [z | x B C | dt], each segment starting on a multiple of 8 rows of the product
        self.w_in, (self.at_z, self.at_xbc, self.at_dt) = _stack(
            [w[:self.inner], w[self.inner:self.inner + self.channels], w[self.inner + self.channels:]], ctx.dtype)
        self.conv_w, self.conv_bias = weights["conv"], weights["conv_bias"]
        self.dt_bias, self.A_log, self.D = weights["dt_bias"], weights["A_log"], weights["D"]
        self.norm, self.o = weights["norm"], weights["o"]
        self.matrix_floats = self.inner * self.N

    def cache_spec(self):
        return SlotStateSpec((self.matrix_floats + (self.taps - 1) * self.channels,), torch.float32)

    def activation_widths(self):
        return [self.w_in.shape[0], self.channels, 2 * self.inner, self.inner, self.o.shape[0]]

    def forward(self, x, batch, cache):
        p = ops.linear(x, self.w_in)
        tails = cache.state[:, self.matrix_floats:] if self.taps > 1 else None
        c = ops.conv_silu(p, self.at_xbc, self.channels, self.conv_w, tails, batch, out_bias=self.conv_bias)
        y = ops.ssd_scan(c, (p, self.at_dt), self.dt_bias, self.A_log, self.D, cache.state, batch, self.H, self.G,
                         self.N, self.Dv)
        g = ops.gated_group_norm(y, (p, self.at_z), self.norm, self.norm_groups, self.eps, self.ctx.dtype)
        return ops.linear(g, self.o)


@register("mixer", "mlstm")
class MatrixLSTM(Part):
    """A matrix memory per head with exponential gates (the mLSTM cell of xLSTM).  One product lays out
    [q: heads * dim | k: heads * dim | v: heads * vdim | g: heads * vdim]; a second, with float32 results, makes the raw
    gates [a: heads | b: heads].  Per head, with ``q`` multiplied by ``dim^(-1/2)``,
    ``i = cap tanh((a + b_i) / cap)`` and ``f = logsigmoid(cap tanh((b + b_f) / cap))``, and a running maximum ``m``:

        m_t = max(f + m_{t-1}, i),    C_t = exp(f + m_{t-1} - m_t) C_{t-1} + exp(i - m_t) k v^T    (C is dim x vdim),
        n_t likewise with k alone,     y_t = C_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6),

    from C = 0, n = 0, m = 0.  Every head's y is divided by its own root mean square (``eps`` inside the root); the
    heads, side by side, are multiplied by ``norm``, by ``sigmoid(g)``, and projected by W_o.  Gates, exponentials and
    the state are float32; the request's state slot holds C, n and m.
    params: hidden_size, heads, dim, vdim, gate_cap, eps."""

    @classmethod
    def weight_specs(cls, params):
        h, H, D, Dv = (int(params[k]) for k in ("hidden_size", "heads", "dim", "vdim"))
        return {"q": WeightSpec((H * D, h)), "k": WeightSpec((H * D, h)), "v": WeightSpec((H * Dv, h)),
                "g": WeightSpec((H * Dv, h)), "i": WeightSpec((H, h)), "f": WeightSpec((H, h)),
                "i_bias": WeightSpec((H,), "bias"), "f_bias": WeightSpec((H,), "bias"),
                "norm": WeightSpec((H * Dv,), "vector"), "o": WeightSpec((h, H * Dv))}

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ("mlstm",) + _gemm_modules(dtype)

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.H, self.D, self.Dv = (int(params[k]) for k in ("heads", "dim", "vdim"))
        self.cap, self.eps = float(params["gate_cap"]), float(params["eps"])
        if not 1 <= self.D <= 256:
            raise ValueError(f"mlstm: keys of {self.D} channels are refused (1 to 256)")
        if not self.cap > 0:
            raise ValueError(f"mlstm: a gate cap of {self.cap} is refused (above zero)")
        self.w_in, (self.at_q, self.at_k, self.at_v, self.at_g) = _stack(
            [weights["q"], weights["k"], weights["v"], weights["g"]], ctx.dtype)
        # the raw gates are float32 sums: their matrix stays apart from the others
        self.w_gates = torch.cat([weights["i"], weights["f"]], dim=0).contiguous()
        self.i_bias, self.f_bias = weights["i_bias"], weights["f_bias"]
        self.norm, self.o = weights["norm"], weights["o"]
        self.state_floats = ops.mlstm_state_floats(self.H, self.D, self.Dv)

    def cache_spec(self):
        return SlotStateSpec((self.state_floats,), torch.float32)

    def activation_widths(self):
        inner = self.H * self.Dv
        return [self.w_in.shape[0], 2 * (2 * self.H + 8), 2 * inner, inner, self.o.shape[0]]

    def forward(self, x, batch, cache):
        p = ops.linear(x, self.w_in)
        gates = ops.linear(x, self.w_gates, out_dtype=torch.float32)
        y = ops.mlstm_scan(p, self.at_q, self.at_k, self.at_v, gates, self.i_bias, self.f_bias, self.cap,
                           self.D ** -0.5, cache.state, batch, self.H, self.D, self.Dv)
        return ops.linear(ops.head_norm_gate(y, (p, self.at_g), self.norm, self.H, self.eps, self.ctx.dtype), self.o)
