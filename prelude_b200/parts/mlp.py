"""Gated feed-forward: down(act(gate(x)) * up(x)), no biases
(crates/prelude-core/src/models/qwen3.rs:383-448).

Gate and up rows are stored one below the other so that one product feeds the
activation kernel; the reference merges them the same way where its kernels
take the merged layout (qwen3.rs:411-419).  The activation comes from the spec;
the reference parses ``hidden_act`` and then applies SiLU regardless.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import ClampedGluSpec, GatedMlpSpec
from ..ops import kernels as K
from ..ops.linear import gated_linear_clamped, gated_linear_gelu_tanh, gated_linear_silu, linear
from ..weights.loader import TensorReq
from .registry import RunContext, register_part

_ACTIVATIONS = {"silu": K.silu_mul, "gelu_tanh": K.gelu_tanh_mul}
# the same with the activation in the epilogue of the gate/up product, where a kernel of this library takes the shape
_FUSED = {"silu": gated_linear_silu, "gelu_tanh": gated_linear_gelu_tanh}


@register_part("feed_forward", "gated_mlp")
class GatedMlp:
    def __init__(self, spec: GatedMlpSpec, prefix: str):
        if spec.activation not in _ACTIVATIONS:
            raise ValueError(f"gated feed-forward: no kernel for activation {spec.activation!r}; known: {sorted(_ACTIVATIONS)}")
        self.spec, self.prefix = spec, prefix
        self.w_gate_up = self.w_down = None

    def tensors(self) -> Dict[str, TensorReq]:
        s, p = self.spec, self.prefix
        return {
            f"{p}.{s.gate_name}": TensorReq((s.intermediate_size, s.hidden_size)),
            f"{p}.{s.up_name}": TensorReq((s.intermediate_size, s.hidden_size)),
            f"{p}.{s.down_name}": TensorReq((s.hidden_size, s.intermediate_size)),
        }

    def load(self, get, ctx: RunContext) -> None:
        s, p = self.spec, self.prefix

        def mat(name):
            return get(f"{p}.{name}").to(device=ctx.device, dtype=ctx.dtype)

        self.w_gate_up = torch.cat([mat(s.gate_name), mat(s.up_name)], dim=0).contiguous()
        self.w_down = mat(s.down_name).contiguous()

    def activation_bytes_per_token(self, elem: int) -> int:
        """The merged gate/up projection, the activation, the output (as float32 partial sums at most)."""
        return 3 * self.spec.intermediate_size * elem + 4 * self.spec.hidden_size * 4

    def forward(self, x: torch.Tensor):
        """The feed-forward of x; what comes back goes to a fused residual add, which also takes
        the partial sums of a product whose K was cut into parts."""
        act = _FUSED[self.spec.activation](x, self.w_gate_up)
        if act is None:
            act = _ACTIVATIONS[self.spec.activation](linear(x, self.w_gate_up))
        return linear(act, self.w_down, partial_sums_ok=True)


@register_part("feed_forward", "clamped_glu")
class ClampedGlu:
    """down(a * sigmoid(alpha a) * (b + 1)) with a = min(gate(x), limit) and b = clamp(up(x), -limit, limit): gate and up
    rows one below the other and one product with the unit in its epilogue where a kernel of this library takes the
    shape (a decode step: the streaming kernel; a long prompt step: the paired-block tcgen05 kernel), else the
    library product and the activation kernel; then the down projection."""

    def __init__(self, spec: ClampedGluSpec, prefix: str):
        self.spec, self.prefix = spec, prefix
        self.w_gate_up = self.w_down = None

    def tensors(self) -> Dict[str, TensorReq]:
        s, p = self.spec, self.prefix
        return {
            f"{p}.{s.gate_name}": TensorReq((s.intermediate_size, s.hidden_size)),
            f"{p}.{s.up_name}": TensorReq((s.intermediate_size, s.hidden_size)),
            f"{p}.{s.down_name}": TensorReq((s.hidden_size, s.intermediate_size)),
        }

    def load(self, get, ctx: RunContext) -> None:
        s, p = self.spec, self.prefix

        def mat(name):
            return get(f"{p}.{name}").to(device=ctx.device, dtype=ctx.dtype)

        self.w_gate_up = torch.cat([mat(s.gate_name), mat(s.up_name)], dim=0).contiguous()
        self.w_down = mat(s.down_name).contiguous()

    def activation_bytes_per_token(self, elem: int) -> int:
        return 3 * self.spec.intermediate_size * elem + 4 * self.spec.hidden_size * 4

    def forward(self, x: torch.Tensor):
        act = gated_linear_clamped(x, self.w_gate_up, self.spec.limit, self.spec.alpha)
        if act is None:
            act = K.clamped_glu(linear(x, self.w_gate_up), self.spec.limit, self.spec.alpha)
        return linear(act, self.w_down, partial_sums_ok=True)
