"""Attention over a sliding window with one row [key | value] per token and key/value head in the pages: one whose
queries, keys and values pass a short convolution first and whose window keeps the sequence's first tokens; one
whose scores are shaped on their way to the softmax (a factor per head, a soft cap, a bias that grows with the
distance); one that rotates queries and keys and masks by blocks of positions; and the arrangement of two mixers
side by side."""

from __future__ import annotations

import dataclasses

import torch

from .. import ops
from ..cache.specs import PagedKVSpec, PagedWithStateSpec, SlotStateSpec, paged_part, state_part
from ..weights.loader import WeightSpec
from .base import Part
from .registry import lookup, register


@register("mixer", "conv_window_attention")
class ConvWindowAttention(Part):
    """Grouped-query attention without positions in its scores.

    q (``heads`` x ``dim``), k (``kv_heads`` x ``dim``) and v (``kv_heads`` x ``vdim``) come from one
    product with the row-stacked matrix; each channel then passes a causal convolution over time of
    ``conv`` taps (the last tap weighs the token itself, zeros before the sequence's start, no
    activation), whose last ``conv - 1`` inputs per request live in the request's state slot.  The
    convolved keys and values go to the request's pages, a row per token and key/value head holding
    [k | v].  Query i sees key j when ``j <= i and (i - j < window or j < keep_first)`` (``window`` None:
    every key up to i); scores are ``(q . k) * scale``; with ``one_more`` the softmax's denominator is
    ``1 + sum exp(s)``.  Query head h reads key/value head ``h // (heads / kv_heads)``.  Then W_o.
    Kernels: the general one (float32 arithmetic, any sizes, chunks of keys by absolute position) for
    float32, for steps of single tokens and for sizes the other refuses; for bfloat16 steps with runs
    of tokens and key and value size both 64 or 128 the tensor-core kernel of prompt portions.
    params: hidden_size, heads, kv_heads, dim, vdim, conv, scale, window, keep_first, one_more."""

    @classmethod
    def weight_specs(cls, params):
        h, H, G, D, Dv, taps = (params[k] for k in ("hidden_size", "heads", "kv_heads", "dim", "vdim", "conv"))
        return {"q": WeightSpec((H * D, h)), "k": WeightSpec((G * D, h)), "v": WeightSpec((G * Dv, h)),
                "q_conv": WeightSpec((H * D, taps), "bias"), "k_conv": WeightSpec((G * D, taps), "bias"),
                "v_conv": WeightSpec((G * Dv, taps), "bias"), "o": WeightSpec((h, H * Dv))}

    @classmethod
    def kernel_modules(cls, params, dtype):
        mods = ["window_attention", "delta_rule"]
        if dtype == torch.bfloat16 and params["dim"] == params["vdim"] and params["dim"] in (64, 128):
            mods.append("flash_attention")
        return tuple(mods) + (("gemm_f32",) if dtype == torch.float32 else ("gemm_bf16", "gemm_bf16_wide"))

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.heads, self.kv_heads = int(params["heads"]), int(params["kv_heads"])
        self.dim, self.vdim, self.taps = int(params["dim"]), int(params["vdim"]), int(params["conv"])
        if self.heads % self.kv_heads:
            raise ValueError(f"conv_window_attention: {self.heads} query heads cannot be grouped over "
                             f"{self.kv_heads} key/value heads")
        if not (1 <= self.dim <= 256 and 1 <= self.vdim <= 256):
            raise ValueError(f"conv_window_attention: head sizes {self.dim} x {self.vdim} are refused (1 to 256)")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"conv_window_attention: {self.taps} convolution taps are refused (1 to 16)")
        self.scale = float(params["scale"])
        self.window = int(params["window"]) if params.get("window") else None
        self.keep_first = int(params.get("keep_first") or 0) if self.window else 0
        self.one_more = bool(params.get("one_more"))
        self.qkv = torch.cat([weights["q"], weights["k"], weights["v"]], dim=0).contiguous()
        self.conv_w = torch.cat([weights["q_conv"], weights["k_conv"], weights["v_conv"]], dim=0).contiguous()
        self.o = weights["o"]
        self.k_off = self.heads * self.dim
        self.v_off = self.k_off + self.kv_heads * self.dim
        self.channels = self.v_off + self.kv_heads * self.vdim

    def cache_spec(self):
        paged = PagedKVSpec(self.kv_heads, self.dim + self.vdim, self.window, planes=1, keep_first=self.keep_first)
        if self.taps == 1:
            return paged
        return PagedWithStateSpec(paged, SlotStateSpec(((self.taps - 1) * self.channels,), torch.float32))

    def activation_widths(self):
        return [self.channels, self.channels, self.heads * self.vdim, self.o.shape[0]]

    def _on_tensor_cores(self, page_size):
        return ops.flash_attention_rows_supported(self.dim, self.vdim, self.heads // self.kv_heads, page_size, self.ctx.dtype)

    def query_tile_heights(self):
        """Tokens per tile of the tensor-core kernel for prompt portions (bfloat16, key and value size
        64 or 128): the step's batch lays the tiles out for them."""
        if self.ctx.dtype != torch.bfloat16 or self.dim != self.vdim or self.dim not in (64, 128):
            return []
        g = self.heads // self.kv_heads
        return [ops.flash_tokens_per_tile(g, False), ops.flash_tokens_per_tile(g, True)]

    def forward(self, x, batch, cache):
        p = ops.linear(x, self.qkv)
        table = batch.block_tables[cache.group]
        # the convolution writes the new keys and values into their pages itself where the rows allow 16-byte accesses
        fused = cache.write and ops.conv_can_append(p, 0, self.channels, self.k_off, self.v_off, self.dim, self.vdim)
        c = ops.conv_silu(p, 0, self.channels, self.conv_w, cache.state, batch, act="none",
                          append=(cache.k, table, self.k_off, self.v_off, self.kv_heads, self.dim, self.vdim) if fused else None)
        if cache.write and not fused:
            ops.kv_rows_append(c, self.k_off, self.v_off, cache.k, table, batch, self.kv_heads, self.dim, self.vdim)
        if not batch.decode_only and self._on_tensor_cores(cache.page_size) and c.stride(0) % 8 == 0:
            a = ops.flash_attention_rows(c, cache.k, table, batch, self.heads, self.kv_heads, self.dim, self.scale,
                                         self.window or 0, self.keep_first, self.one_more)
        else:
            a = ops.window_attention(c, 0, cache.k, table, batch, self.heads, self.kv_heads, self.dim, self.vdim,
                                     self.scale, self.window or 0, self.keep_first, self.one_more)
        return ops.linear(a, self.o)


@register("mixer", "shaped_window_attention")
class ShapedWindowAttention(Part):
    """Grouped-query attention whose scores are shaped on their way to the softmax, over a sliding window.

    q (``heads`` x ``dim``), k (``kv_heads`` x ``dim``) and v (``kv_heads`` x ``vdim``) come from one product with the
    row-stacked matrix; with ``bias`` each gets a bias; with ``qk_norm`` every query and key head is divided by its
    root mean square (eps inside the root) and multiplied by a weight of ``dim`` shared by the heads.  Keys and values
    go to the request's pages, a row [k | v] per token and key/value head.  No rotation.  For query i and key j

        s = (q . k) * scale * temp[h];    s <- softcap * tanh(s / softcap);    s <- s - slope_h * (i - j),

    with ``temp`` a learned number per head (``head_temperature``), ``softcap`` 0 or None for no cap, and
    ``slope_h = 2^(-slope_power * (h + 1) / heads)`` (``slope_power`` None: no distance bias).  Query i sees key j when
    ``0 <= i - j < window`` (``window`` None: every key up to i).  Ordinary softmax, float32.  ``out_scale`` multiplies
    the result.  Then W_o.
    params: hidden_size, heads, kv_heads, dim, vdim, scale, window, softcap, slope_power, bias, qk_norm,
    head_temperature, eps, out_scale."""

    @classmethod
    def weight_specs(cls, params):
        h, H, G, D, Dv = (int(params[k]) for k in ("hidden_size", "heads", "kv_heads", "dim", "vdim"))
        specs = {"q": WeightSpec((H * D, h)), "k": WeightSpec((G * D, h)), "v": WeightSpec((G * Dv, h)),
                 "o": WeightSpec((h, H * Dv))}
        if params.get("bias"):
            specs.update(q_bias=WeightSpec((H * D,), "bias"), k_bias=WeightSpec((G * D,), "bias"),
                         v_bias=WeightSpec((G * Dv,), "bias"))
        if params.get("qk_norm"):
            specs.update(q_norm=WeightSpec((D,), "vector"), k_norm=WeightSpec((D,), "vector"))
        if params.get("head_temperature"):
            specs["temp"] = WeightSpec((H,), "bias")
        return specs

    @classmethod
    def kernel_modules(cls, params, dtype):
        if dtype == torch.float32:
            return ("window_attention", "gemm_f32")
        flash = ("window_flash_attention",) if cls._flash_sizes(params, dtype) else ()
        return ("window_attention",) + flash + ("gemm_bf16", "gemm_bf16_wide")

    @staticmethod
    def _flash_sizes(params, dtype, page_size=16):
        return ops.window_flash_attention_supported(int(params["dim"]), int(params["vdim"]),
                                                    int(params["heads"]) // max(1, int(params["kv_heads"])), page_size, dtype)

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.heads, self.kv_heads = int(params["heads"]), int(params["kv_heads"])
        self.dim, self.vdim = int(params["dim"]), int(params["vdim"])
        if self.heads % self.kv_heads:
            raise ValueError(f"shaped_window_attention: {self.heads} query heads cannot be grouped over "
                             f"{self.kv_heads} key/value heads")
        if not (1 <= self.dim <= 256 and 1 <= self.vdim <= 256):
            raise ValueError(f"shaped_window_attention: head sizes {self.dim} x {self.vdim} are refused (1 to 256)")
        self.scale, self.eps = float(params["scale"]), float(params.get("eps", 1e-6))
        self.window = int(params["window"]) if params.get("window") else None
        self.softcap = float(params.get("softcap") or 0.0)
        self.out_scale = float(params.get("out_scale", 1.0))
        self.w_in, (_, self.k_off, self.v_off) = _stack_rows([weights["q"], weights["k"], weights["v"]])
        self.q_bias, self.k_bias, self.v_bias = (weights.get(n) for n in ("q_bias", "k_bias", "v_bias"))
        self.q_norm, self.k_norm = weights.get("q_norm"), weights.get("k_norm")
        self.temp = weights.get("temp")
        self.slopes = None
        if params.get("slope_power") is not None:
            power = float(params["slope_power"])
            self.slopes = torch.tensor([2.0 ** (-power * (h + 1) / self.heads) for h in range(self.heads)],
                                       dtype=torch.float32, device=ctx.device)
        self.o = weights["o"]

    def cache_spec(self):
        return PagedKVSpec(self.kv_heads, self.dim + self.vdim, self.window, planes=1)

    def activation_widths(self):
        return [self.w_in.shape[0], self.heads * self.dim, self.heads * self.vdim, self.o.shape[0]]

    def query_tile_heights(self):
        """Tokens per tile of the tensor-core kernel for prompt portions (bfloat16, sizes that are multiples of 8 up to
        128): the step's batch lays the tiles out for them."""
        if not self._flash_sizes(self.params, self.ctx.dtype):
            return []
        g = self.heads // self.kv_heads
        return [ops.rows_tokens_per_tile(g, False), ops.rows_tokens_per_tile(g, True)]

    def readout(self, p, first, batch, cache):
        """From the product ``p`` (this mixer's columns start at ``first``) to the heads' results [T, heads * vdim]."""
        table = batch.block_tables[cache.group]
        q = ops.qk_norm_append(p, first, self.k_off, self.v_off, self.q_bias, self.k_bias, self.v_bias, self.q_norm,
                               self.k_norm, self.eps, cache.k, table, batch, self.heads, self.kv_heads, self.dim,
                               self.vdim, write=cache.write)
        if not batch.decode_only and self._flash_sizes(self.params, self.ctx.dtype, cache.page_size):
            return ops.window_flash_attention(q, cache.k, table, batch, self.heads, self.kv_heads, self.dim, self.vdim,
                                              self.scale, self.window or 0, 0, False, head_scale=self.temp,
                                              slopes=self.slopes, softcap=self.softcap, out_scale=self.out_scale)
        return ops.window_attention(q, 0, cache.k, table, batch, self.heads, self.kv_heads, self.dim, self.vdim,
                                    self.scale, self.window or 0, 0, False, head_scale=self.temp, slopes=self.slopes,
                                    softcap=self.softcap, out_scale=self.out_scale)

    def forward(self, x, batch, cache):
        return ops.linear(self.readout(ops.linear(x, self.w_in), 0, batch, cache), self.o)


@register("mixer", "rotary_chunk_attention")
class RotaryChunkAttention(Part):
    """Grouped-query attention with rotated queries and keys over blocks of positions.

    q (``heads`` x ``dim``), k (``kv_heads`` x ``dim``), v (``kv_heads`` x ``vdim``) and, with ``gate``, g (``heads`` x
    ``vdim``) come from one product with the row-stacked matrix.  With ``bias`` q, k, v and the output projection have
    biases.  With ``qk_norm`` all of a token's queries together are divided by their root mean square (``eps`` inside
    the root) and multiplied by a weight of ``heads * dim``, before they are cut into heads; likewise the keys.  Then the
    first ``position.rotary_dim`` channels of every query and key head turn with the position (``position``: a part of
    the position family, "rope" pairing channel i with i + dims / 2, "rope_interleaved" 2 i with 2 i + 1; None: no
    rotation).  Keys and values go to the request's pages, a row [k | v] per token and key/value head.  For query i
    and key j

        s = (q . k) * scale;    s <- softcap * tanh(s / softcap)   (``softcap`` 0 or None: not),

    and query i sees key j <= i only when ``i // chunk == j // chunk``, the blocks counted from the sequence's start
    (``chunk`` None: every key up to i).  Softmax in float32; with ``sink`` a learned number per head joins its
    denominator as ``exp(sink_h)``, once, without a value.  With ``gate`` the heads' results are multiplied element by
    element by ``sigmoid(g)``.  Then W_o; its bias is handed to whoever adds the result to the stream.
    A block of positions never reaches further back than ``chunk`` keys, so the pages are a windowed group of that size.
    params: hidden_size, heads, kv_heads, dim, vdim, scale, chunk, softcap, sink, gate, bias, qk_norm, eps, position."""

    @classmethod
    def weight_specs(cls, params):
        h, H, G, D, Dv = (int(params[k]) for k in ("hidden_size", "heads", "kv_heads", "dim", "vdim"))
        specs = {"q": WeightSpec((H * D, h)), "k": WeightSpec((G * D, h)), "v": WeightSpec((G * Dv, h)),
                 "o": WeightSpec((h, H * Dv))}
        if params.get("bias"):
            specs.update(q_bias=WeightSpec((H * D,), "bias"), k_bias=WeightSpec((G * D,), "bias"),
                         v_bias=WeightSpec((G * Dv,), "bias"), o_bias=WeightSpec((h,), "bias"))
        if params.get("qk_norm"):
            specs.update(q_norm=WeightSpec((H * D,), "vector"), k_norm=WeightSpec((G * D,), "vector"))
        if params.get("sink"):
            specs["sink"] = WeightSpec((H,), "bias")
        if params.get("gate"):
            specs["g"] = WeightSpec((H * Dv, h))
        return specs

    @classmethod
    def kernel_modules(cls, params, dtype):
        if dtype == torch.float32:
            return ("window_attention", "gemm_f32")
        flash = ("window_flash_attention",) if cls._flash_sizes(params, dtype) else ()
        if cls._one_size(params, dtype):
            flash += ("flash_attention",)
        return ("window_attention",) + flash + ("gemm_bf16", "gemm_bf16_wide")

    @staticmethod
    def _flash_sizes(params, dtype, page_size=16):
        return ops.window_flash_attention_supported(int(params["dim"]), int(params["vdim"]),
                                                    int(params["heads"]) // max(1, int(params["kv_heads"])), page_size, dtype)

    @staticmethod
    def _one_size(params, dtype):
        """Keys and values of one size that the tcgen05 kernel of prompt portions takes (bfloat16, 64 or 128)."""
        return dtype == torch.bfloat16 and int(params["dim"]) == int(params["vdim"]) and int(params["dim"]) in (64, 128)

    hands_over_bias = True

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.heads, self.kv_heads = int(params["heads"]), int(params["kv_heads"])
        self.dim, self.vdim = int(params["dim"]), int(params["vdim"])
        if self.kv_heads < 1 or self.heads % self.kv_heads:
            raise ValueError(f"rotary_chunk_attention: {self.heads} query heads cannot be grouped over "
                             f"{self.kv_heads} key/value heads")
        if not (1 <= self.dim <= 256 and 1 <= self.vdim <= 256):
            raise ValueError(f"rotary_chunk_attention: head sizes {self.dim} x {self.vdim} are refused (1 to 256)")
        self.scale, self.eps = float(params["scale"]), float(params.get("eps", 1e-6))
        self.chunk = int(params["chunk"]) if params.get("chunk") else None
        self.softcap = float(params.get("softcap") or 0.0)
        mats = [weights["q"], weights["k"], weights["v"]] + ([weights["g"]] if params.get("gate") else [])
        self.w_in, starts = _stack_rows(mats)
        self.k_off, self.v_off = starts[1], starts[2]
        self.g_off = starts[3] if params.get("gate") else None
        self.q_bias, self.k_bias, self.v_bias = (weights.get(n) for n in ("q_bias", "k_bias", "v_bias"))
        self.o_bias = weights.get("o_bias")
        self.q_norm, self.k_norm = weights.get("q_norm"), weights.get("k_norm")
        self.sinks = weights.get("sink")
        self.o = weights["o"]
        pos = params.get("position")
        self.position, self.rot, self.layout = None, 0, "half"
        if pos is not None:
            self.position = (ctx.make("position", pos) if ctx.make is not None
                             else lookup("position", pos.kind)(pos.params, {}, ctx))
            self.rot = int(self.position.rotary_dim)
            self.layout = "pairs" if pos.kind == "rope_interleaved" else "half"
            if self.rot > self.dim:
                raise ValueError(f"rotary_chunk_attention: {self.rot} turning channels in heads of {self.dim}")

    def cache_spec(self):
        return PagedKVSpec(self.kv_heads, self.dim + self.vdim, self.chunk, planes=1)

    def activation_widths(self):
        return [self.w_in.shape[0], self.heads * self.dim, self.heads * self.vdim, self.o.shape[0]]

    def query_tile_heights(self):
        """Tokens per tile of the tensor-core kernel for prompt portions (bfloat16, sizes that are multiples of 8 up to
        128): the step's batch lays the tiles out for them."""
        if not self._flash_sizes(self.params, self.ctx.dtype):
            return []
        g = self.heads // self.kv_heads
        heights = [ops.rows_tokens_per_tile(g, False), ops.rows_tokens_per_tile(g, True)]
        if self._one_size(self.params, self.ctx.dtype):
            heights.append(ops.flash_tokens_per_tile(g, True))
        return heights

    def forward(self, x, batch, cache, bias_out=False):
        p = ops.linear(x, self.w_in)
        table = batch.block_tables[cache.group]
        cos, sin = self.position.tables() if self.rot else (None, None)
        q = ops.qk_rot_append(p, 0, self.k_off, self.v_off, self.q_bias, self.k_bias, self.v_bias, self.q_norm,
                              self.k_norm, self.eps, cos, sin, self.rot, self.layout, cache.k, table, batch, self.heads,
                              self.kv_heads, self.dim, self.vdim, write=cache.write)
        shape = dict(softcap=self.softcap, sinks=self.sinks, chunk=self.chunk or 0,
                     gate=(p, self.g_off) if self.g_off is not None else None)
        if (not batch.decode_only and self._one_size(self.params, self.ctx.dtype)
                and ops.flash_attention_rows_masked_wanted(batch, self.heads, self.kv_heads, self.dim, self.vdim,
                                                           cache.page_size, self.ctx.dtype, q)):
            # long bfloat16 steps with keys and values of one size, 64 or 128: the tcgen05 kernel with roles
            a = ops.flash_attention_rows_masked(q, cache.k, table, batch, self.heads, self.kv_heads, self.dim, self.scale,
                                                **shape)
        elif not batch.decode_only and self._flash_sizes(self.params, self.ctx.dtype, cache.page_size):
            # prompt portions in bfloat16: both products on tensor cores, the scores shaped in float32 between them
            a = ops.window_flash_attention(q, cache.k, table, batch, self.heads, self.kv_heads, self.dim, self.vdim,
                                           self.scale, 0, 0, False, **shape)
        else:
            a = ops.window_attention(q, 0, cache.k, table, batch, self.heads, self.kv_heads, self.dim, self.vdim,
                                     self.scale, 0, 0, False, **shape)
        y = ops.linear(a, self.o)
        if bias_out:
            return y, self.o_bias
        if self.o_bias is not None:
            y = y + self.o_bias.to(y.dtype)
        return y


def _stack_rows(mats):
    """Row-stacks matrices [n_i, in], each starting on a multiple of 8 rows; returns the matrix and the starts."""
    starts, rows, at = [], [], 0
    for m in mats:
        starts.append(at)
        rows.append(m)
        pad = -m.shape[0] % 8
        if pad:
            rows.append(torch.zeros((pad, m.shape[1]), dtype=m.dtype, device=m.device))
        at += m.shape[0] + pad
    return torch.cat(rows, dim=0).contiguous(), starts


@register("mixer", "side_by_side")
class SideBySide(Part):
    """Two mixers that read the same input and whose results are summed: ``left_scale * left(h) + right_scale * right(h)``.
    Each side is a mixer part with a stacked input matrix ``w_in``, a ``readout(product, first column, batch, cache)``
    and an output matrix ``o``; the weights of the sum are handed to the sides as their ``out_scale``.  One product
    with both input matrices stacked feeds both sides; the two output products are handed on together and summed by
    whoever adds them to the residual stream.  A side's pages and state slot are the layer's: at most one side
    keeps pages, and the sides' states lie one behind the other in the request's slot.
    params: left, right (mixer parts)."""

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ()

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.sides = [ctx.make("mixer", params["left"]), ctx.make("mixer", params["right"])]
        for s in self.sides:
            if not (hasattr(s, "readout") and hasattr(s, "w_in") and hasattr(s, "o")):
                raise ValueError(f"side_by_side: a mixer of kind {s.kind!r} cannot stand beside another "
                                 "(it needs w_in, readout and o)")
        self.w_in, self.starts = _stack_rows([s.w_in for s in self.sides])
        wishes = [s.cache_spec() for s in self.sides]
        paged = [paged_part(w) for w in wishes]
        if sum(p is not None for p in paged) > 1:
            raise ValueError("side_by_side: only one of the two mixers may keep pages")
        self.paged = next((p for p in paged if p is not None), None)
        self.floats = []
        for w in wishes:
            st = state_part(w)
            if st is not None and st.dtype != torch.float32:
                raise ValueError("side_by_side: the mixers' states must be float32 to share a slot")
            n = 0
            if st is not None:
                n = 1
                for d in st.shape:
                    n *= int(d)
            self.floats.append(n)
        self._views = {}

    def cache_spec(self):
        total = sum(self.floats)
        state = SlotStateSpec((total,), torch.float32) if total else None
        if self.paged is not None:
            return PagedWithStateSpec(self.paged, state) if state is not None else self.paged
        return state

    def activation_widths(self):
        own = [self.w_in.shape[0]]
        for s in self.sides:
            own += list(s.activation_widths())[1:]
        return own

    def query_tile_heights(self):
        out = []
        for s in self.sides:
            fn = getattr(s, "query_tile_heights", None)
            if fn is not None:
                out.extend(fn())
        return out

    def _bindings(self, cache):
        """Each side's view of the layer's binding: the pages as they are, its own part of the state slot."""
        state = getattr(cache, "state", None)
        if state is None or not any(self.floats):
            return [cache, cache]
        got = self._views.get(id(state))
        if got is None or got[0] is not state:
            at, views = 0, []
            for n in self.floats:
                views.append(state[:, at:at + n] if n else None)
                at += n
            got = (state, views)
            self._views[id(state)] = got
        return [dataclasses.replace(cache, state=v) for v in got[1]]

    def forward(self, x, batch, cache):
        p = ops.linear(x, self.w_in)
        outs = []
        for side, first, binding in zip(self.sides, self.starts, self._bindings(cache)):
            outs.append(ops.linear(side.readout(p, first, batch, binding), side.o))
        return tuple(outs)
