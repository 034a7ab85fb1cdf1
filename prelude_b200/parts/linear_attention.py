"""Linear attention with a decaying matrix state per head (``DecayedLinearAttentionSpec``).

One merged projection [v | k | q | gate]; the recurrence token by token with the state in float32, its loaders
taking SiLU of v, k and q on the way in; one norm over all heads' outputs with a learned scale, the sigmoid gate,
the output projection.  Per sequence it keeps the state [heads, head_dim, value_dim] (float32) in the sequence's
state slot.  The decays are constants of the model, one per head.  The kernels read how a step's tokens are spread
over sequences from the step's device arrays, so the mixer can be recorded.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import DecayedLinearAttentionSpec
from ..ops import kernels as K
from ..ops.linear import linear
from ..weights.loader import TensorReq
from .registry import RunContext, StateNeed, register_part


@register_part("mixer", "decayed_linear_attention")
class DecayedLinearAttention:
    def __init__(self, spec: DecayedLinearAttentionSpec, prefix: str):
        if len(spec.decays) != spec.num_heads:
            raise ValueError(f"{len(spec.decays)} decays for {spec.num_heads} heads")
        self.spec, self.prefix = spec, prefix
        self.qk_cols = spec.num_heads * spec.head_dim
        self.v_cols = spec.num_heads * spec.value_dim
        self.w_in = self.w_o = self.norm_w = self.decay = None

    def tensors(self) -> Dict[str, TensorReq]:
        s, p = self.spec, self.prefix
        return {
            f"{p}.{s.q_name}": TensorReq((self.qk_cols, s.hidden_size)),
            f"{p}.{s.k_name}": TensorReq((self.qk_cols, s.hidden_size)),
            f"{p}.{s.v_name}": TensorReq((self.v_cols, s.hidden_size)),
            f"{p}.{s.gate_name}": TensorReq((self.v_cols, s.hidden_size)),
            f"{p}.{s.norm_name}": TensorReq((self.v_cols,), "norm"),
            f"{p}.{s.o_name}": TensorReq((s.hidden_size, self.v_cols)),
        }

    def load(self, get, ctx: RunContext) -> None:
        s, p = self.spec, self.prefix

        def mat(name):
            return get(f"{p}.{name}").to(device=ctx.device, dtype=ctx.dtype)

        # the order the scan reads: values, keys, queries; then the gate
        mats = [mat(s.v_name), mat(s.k_name), mat(s.q_name), mat(s.gate_name)]
        pad = (-sum(m.shape[0] for m in mats)) % 8             # rows of the merged projection stay 16-byte aligned
        if pad:
            mats.append(torch.zeros((pad, s.hidden_size), dtype=ctx.dtype, device=ctx.device))
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.w_o = mat(s.o_name).contiguous()
        self.norm_w = get(f"{p}.{s.norm_name}").to(device=ctx.device, dtype=torch.float32).contiguous()
        self.decay = torch.tensor(list(s.decays), dtype=torch.float64).to(torch.float32).to(ctx.device)

    def activation_bytes_per_token(self, elem: int) -> int:
        return (2 * self.qk_cols + 3 * self.v_cols + 8) * elem + self.v_cols * 4 + self.spec.hidden_size * elem

    def cache_need(self) -> StateNeed:
        s = self.spec
        return StateNeed((s.num_heads, s.head_dim, s.value_dim), torch.float32)

    def forward(self, x: torch.Tensor, batch, cache, write_cache: bool = True) -> torch.Tensor:
        s = self.spec
        T = batch.n_tokens
        proj = linear(x, self.w_in)
        g0 = self.v_cols + 2 * self.qk_cols
        o = K.decay_scan(proj, self.decay, cache.state, batch, out=batch.workspace("decay_o", (T, self.v_cols), torch.float32))
        y = K.gated_group_rmsnorm(o, proj[:, g0:g0 + self.v_cols], self.norm_w, 1, s.norm_eps, gate_after=True, sigmoid_gate=True,
                                  out=batch.workspace("decay_gated", (T, self.v_cols), x.dtype))
        return linear(y, self.w_o)
