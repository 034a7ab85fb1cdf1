"""The two ends of a decoder: token embedding and output head.

``TokenEmbedding`` gathers the rows of the step's tokens into the float32
residual stream (crates/prelude-core/src/models/commons/embedding.rs:29-35,
qwen3.rs:555-558, 602).  ``LinearHead`` multiplies the wanted rows, after the
final norm, with the vocabulary matrix; tied, it takes the embedding's table
itself, the same memory (qwen3.rs:637-660).  Both are parts like any other: an
architecture whose embedding is scaled, or whose logits are capped, registers
its own kind and names its spec in ``ModelSpec.embedding`` / ``ModelSpec.head``.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..config.spec import LinearHeadSpec, ScaledEmbeddingSpec, SinusoidEmbeddingSpec, TokenEmbeddingSpec
from ..ops import kernels as K
from ..ops.linear import linear
from ..weights.loader import TensorReq
from .registry import RunContext, register_part


@register_part("embedding", "token_embedding")
class TokenEmbedding:
    def __init__(self, spec: TokenEmbeddingSpec, prefix: str = ""):
        self.spec = spec
        self.table: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorReq]:
        return {self.spec.name: TensorReq((self.spec.vocab_size, self.spec.hidden_size))}

    def load(self, get, ctx: RunContext) -> None:
        self.table = get(self.spec.name).to(device=ctx.device, dtype=ctx.dtype).contiguous()

    def forward(self, batch) -> torch.Tensor:
        return K.embed_gather(batch.token_ids, self.table)


@register_part("embedding", "token_embedding_sinusoid")
class SinusoidTokenEmbedding(TokenEmbedding):
    """The token's row plus a fixed position vector of sines and cosines of the token's position
    (entry 2i: sin(p base^(-2i/hidden)), entry 2i + 1: its cosine).  The rates are made once in 64-bit; the kernel
    takes angle, sine and cosine in 64-bit and rounds the sum once to the float32 residual stream."""

    def __init__(self, spec: SinusoidEmbeddingSpec, prefix: str = ""):
        super().__init__(spec, prefix)
        self.rate: Optional[torch.Tensor] = None

    def load(self, get, ctx: RunContext) -> None:
        super().load(get, ctx)
        s = self.spec
        i = torch.arange(0, s.hidden_size, 2, dtype=torch.float64)
        self.rate = torch.pow(torch.tensor(float(s.base), dtype=torch.float64), -i / s.hidden_size).to(ctx.device).contiguous()

    def forward(self, batch) -> torch.Tensor:
        return K.embed_sinusoid(batch.token_ids, batch.positions, self.table, self.rate)


@register_part("embedding", "token_embedding_scaled")
class ScaledTokenEmbedding(TokenEmbedding):
    """The token's row times a constant, multiplied in float32 as the row enters the residual stream.  The table
    itself stays as stored, so a tied head reads it without the constant."""

    def __init__(self, spec: ScaledEmbeddingSpec, prefix: str = ""):
        super().__init__(spec, prefix)

    def forward(self, batch) -> torch.Tensor:
        return K.embed_gather_scaled(batch.token_ids, self.table, self.spec.scale)


@register_part("head", "linear_head")
class LinearHead:
    def __init__(self, spec: LinearHeadSpec, prefix: str = ""):
        self.spec = spec
        self.weight: Optional[torch.Tensor] = None

    def tensors(self) -> Tuple[Dict[str, TensorReq], Dict[str, TensorReq]]:
        """(required, optional): a tied model may still carry a copy of the head; it is not read."""
        req = {self.spec.name: TensorReq((self.spec.vocab_size, self.spec.hidden_size))}
        return ({}, req) if self.spec.tied else (req, {})

    def load(self, get, ctx: RunContext, embedding) -> None:
        if self.spec.tied:
            table = getattr(embedding, "table", None)
            if table is None or tuple(table.shape) != (self.spec.vocab_size, self.spec.hidden_size):
                raise ValueError("a tied head needs an embedding part with a [vocab, hidden] table")
            self.weight = table                          # the same memory
        else:
            self.weight = get(self.spec.name).to(device=ctx.device, dtype=ctx.dtype).contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear(x, self.weight, None, out_dtype=torch.float32)
