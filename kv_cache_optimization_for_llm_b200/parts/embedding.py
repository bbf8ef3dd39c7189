"""Token embedding and the LM head."""

from __future__ import annotations

from .. import ops
from ..weights.loader import WeightSpec
from .base import Part
from .registry import register


@register("embedding", "token_embedding")
class TokenEmbedding(Part):
    """``residual[t] = table[token[t]] * scale`` (upstream, without a factor: base/src/kernels.cu:279-287).
    The residual stream starts, and stays, in float32; the factor is applied there.
    params: vocab_size, hidden_size, scale (1 when absent)."""

    @classmethod
    def weight_specs(cls, params):
        return {"table": WeightSpec((params["vocab_size"], params["hidden_size"]), "matrix")}

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ("elementwise",)

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.table = weights["table"]
        self.scale = float(params.get("scale", 1.0) or 1.0)

    def forward(self, batch):
        return ops.embed_gather(self.table, batch.token_ids, batch.status, batch.sampled, self.scale)


@register("embedding", "normed_token_embedding")
class NormedTokenEmbedding(TokenEmbedding):
    """``residual[t] = rmsnorm(table[token[t]]) * weight``: the looked-up row passes an RMS norm (float32,
    eps inside the root) before it starts the residual stream.  params: vocab_size, hidden_size, eps."""

    @classmethod
    def weight_specs(cls, params):
        return {"table": WeightSpec((params["vocab_size"], params["hidden_size"]), "matrix"),
                "norm": WeightSpec((params["hidden_size"],), "vector")}

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ("elementwise", "rowwise")

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.norm_weight, self.eps = weights["norm"], float(params["eps"])

    def forward(self, batch):
        import torch
        rows = ops.embed_gather(self.table, batch.token_ids, batch.status, batch.sampled, self.scale)
        return ops.join_norm(rows, None, "rms", self.norm_weight, self.eps, torch.float32, compute_dtype=self.ctx.dtype)


@register("head", "linear_head")
class LinearHead(Part):
    """``logits = x . W^T`` in float32 output, W either its own tensor or the embedding
    table when tied (upstream: base/src/engine.cu:872-890, always tied, bfloat16
    logits).  With ``scale`` and ``softcap`` the logits become ``softcap * tanh(logits * scale / softcap)``
    (``softcap`` absent or 0: only the factor), in float32, in place.
    params: vocab_size, hidden_size, scale, softcap."""

    @classmethod
    def weight_specs(cls, params):
        return {"weight": WeightSpec((params["vocab_size"], params["hidden_size"]), "matrix")}

    @classmethod
    def kernel_modules(cls, params, dtype):
        import torch
        shaped = ("rowwise",) if (params.get("softcap") or float(params.get("scale", 1.0) or 1.0) != 1.0) else ()
        return shaped + (("gemm_f32",) if dtype == torch.float32 else ("gemm_bf16", "gemm_bf16_wide"))

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.weight = weights["weight"]
        self.scale = float(params.get("scale", 1.0) or 1.0)
        self.softcap = float(params.get("softcap") or 0.0)

    def forward(self, x):
        import torch
        logits = ops.linear(x, self.weight, out_dtype=torch.float32)
        if self.softcap or self.scale != 1.0:
            ops.scale_softcap(logits, self.scale, self.softcap)
        return logits


@register("embedding", "sinusoid_stream_embedding")
class SinusoidStreamEmbedding(TokenEmbedding):
    """``x[t] = table[token[t]] + pe(position[t])`` with the sinusoidal vector ``pe(p)[2i] = sin(p base^(-2i / W))``,
    ``pe(p)[2i + 1] = cos`` of the same angle, copied into ``streams`` residual streams: float32 [T, streams, W].
    params: vocab_size, hidden_size, streams, base."""

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ("streams",)

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.stream_copies = int(params.get("streams", 1))
        self.base = float(params.get("base", 10000.0))

    def forward(self, batch):
        return ops.embed_sinusoid_streams(self.table, batch.token_ids, batch.positions, self.stream_copies, batch.status,
                                          batch.sampled, self.base)
