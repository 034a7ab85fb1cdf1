"""RMSNorm with a learned scale, alone or fused with the residual add.

y = x / sqrt(mean(x^2) + eps) * w in float32
(crates/prelude-core/src/ops/traits/norm.rs:5-12; fused add+norm protocol
crates/prelude-core/src/models/commons/linear.rs:435-501).  The scale is kept
in float32 whatever the run's type: a bfloat16 scale converts exactly, and one
stored in 32-bit keeps its bits.  A scale stored around zero (``NormSpec.offset`` 1)
is kept as ``offset + w``, added once in float32 when the tensor is loaded.

What a norm adds to the residual stream may itself be waiting for a norm
(``kernels.Normed``: the output of a sublayer that is normed before the add);
the two norms and the add between them are then one kernel.  It may also join
the stream times a constant (``kernels.Scaled``); the add multiplies then.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import NormSpec
from ..ops import kernels as K
from ..weights.loader import TensorReq
from .registry import RunContext, register_part


@register_part("norm", "rmsnorm")
class RmsNorm:
    def __init__(self, spec: NormSpec, prefix: str):
        self.spec, self.prefix = spec, prefix
        self.weight: Optional[torch.Tensor] = None
        self.dtype = None

    def tensors(self) -> Dict[str, TensorReq]:
        return {self.name: TensorReq((self.spec.dim,), "norm_zero" if self.spec.offset else "norm")}

    @property
    def name(self) -> str:
        return f"{self.prefix}{self.spec.suffix}"

    def load(self, get, ctx: RunContext) -> None:
        w = get(self.name).to(device=ctx.device, dtype=torch.float32)
        self.weight = (w + float(self.spec.offset) if self.spec.offset else w).contiguous()
        self.dtype = ctx.dtype

    def pending(self, x) -> K.Normed:
        """x as a value that this norm has yet to be applied to: whoever adds it to the residual stream applies it."""
        return K.Normed(x, self.weight, self.spec.eps)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Norm of a tensor of the run's type over its last axis."""
        return K.rmsnorm(x, self.weight, self.spec.eps)

    def add_forward(self, x: Optional[torch.Tensor], res: torch.Tensor) -> torch.Tensor:
        """res += x in place (float32), then the norm of res in the run's type."""
        if isinstance(x, K.Normed):
            return K.normed_add_rmsnorm(x, res, self.weight, self.spec.eps, self.dtype)
        if isinstance(x, K.Scaled):
            return K.scaled_add_rmsnorm(x, res, self.weight, self.spec.eps, self.dtype)
        return K.add_rmsnorm(x, res, self.weight, self.spec.eps, self.dtype)

    def gather_add_forward(self, x: Optional[torch.Tensor], res: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """norm(res[rows] + x[rows]) for the chosen rows only; res is left alone."""
        if isinstance(x, K.Normed):
            return K.normed_add_rmsnorm(x, res, self.weight, self.spec.eps, self.dtype, rows=rows)
        if isinstance(x, K.Scaled):
            return K.scaled_add_rmsnorm(x, res, self.weight, self.spec.eps, self.dtype, rows=rows)
        return K.gather_add_rmsnorm(x, res, rows, self.weight, self.spec.eps, self.dtype)
