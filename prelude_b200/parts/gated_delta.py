"""The gated delta rule (``GatedDeltaSpec``): a matrix state per head that forgets by a learned decay and is corrected
towards each token's value along its key.

One merged projection [q | k | v | gate | beta | a]; a causal convolution with SiLU over q, k and v; the recurrence
token by token with the state in float32 (unit q and k, sigmoid, softplus and decay inside the scan kernel, in
float32); the norm per head with the gate after it; the output projection.  Per sequence it keeps the state
[heads, head_dim, value_dim] (float32) and the convolutions' last ``conv_taps`` - 1 inputs, both in the sequence's
state slot.  Everything that depends on how a step's tokens are spread over sequences is read by the kernels from the
step's device arrays, so the mixer can be recorded.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import GatedDeltaSpec
from ..ops import kernels as K
from ..ops.linear import linear
from ..weights.loader import TensorReq
from .registry import CombinedNeed, RunContext, StateNeed, register_part


@register_part("mixer", "gated_delta")
class GatedDelta:
    def __init__(self, spec: GatedDeltaSpec, prefix: str):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} heads do not divide over {spec.num_kv_heads} query/key heads")
        if spec.conv_taps < 1:
            raise ValueError("a convolution has at least one tap")
        if abs(spec.unit_eps - 1e-6) > 1e-12:
            raise ValueError("the scan kernel makes unit vectors with 1e-6 under the root")
        self.spec, self.prefix = spec, prefix
        self.qk_cols = spec.num_kv_heads * spec.head_dim
        self.inner = spec.num_heads * spec.value_dim
        self.channels = 2 * self.qk_cols + self.inner                       # what the convolutions cover: q, k, v
        self.proj_cols = self.channels + self.inner + 2 * spec.num_heads    # ... then gate, beta, a
        self.w_in = self.w_o = self.conv_w = self.a_log = self.dt_bias = self.norm_w = None

    def tensors(self) -> Dict[str, TensorReq]:
        s, p = self.spec, self.prefix
        req = {
            f"{p}.{s.q_name}": TensorReq((self.qk_cols, s.hidden_size)),
            f"{p}.{s.k_name}": TensorReq((self.qk_cols, s.hidden_size)),
            f"{p}.{s.v_name}": TensorReq((self.inner, s.hidden_size)),
            f"{p}.{s.q_name}{s.conv_suffix}": TensorReq((self.qk_cols, s.conv_taps), "conv"),
            f"{p}.{s.k_name}{s.conv_suffix}": TensorReq((self.qk_cols, s.conv_taps), "conv"),
            f"{p}.{s.v_name}{s.conv_suffix}": TensorReq((self.inner, s.conv_taps), "conv"),
            f"{p}.{s.beta_name}": TensorReq((s.num_heads, s.hidden_size)),
            f"{p}.{s.a_name}": TensorReq((s.num_heads, s.hidden_size)),
            f"{p}.{s.a_log_name}": TensorReq((s.num_heads,), "log_rate"),
            f"{p}.{s.dt_bias_name}": TensorReq((s.num_heads,), "bias"),
            f"{p}.{s.gate_name}": TensorReq((self.inner, s.hidden_size)),
            f"{p}.{s.norm_name}": TensorReq((s.value_dim,), "norm"),
            f"{p}.{s.o_name}": TensorReq((s.hidden_size, self.inner)),
        }
        return req

    def load(self, get, ctx: RunContext) -> None:
        s, p = self.spec, self.prefix

        def mat(name):
            return get(f"{p}.{name}").to(device=ctx.device, dtype=ctx.dtype)

        def vec(name):
            return get(f"{p}.{name}").to(device=ctx.device, dtype=torch.float32).contiguous()

        mats = [mat(s.q_name), mat(s.k_name), mat(s.v_name), mat(s.gate_name), mat(s.beta_name), mat(s.a_name)]
        pad = (-self.proj_cols) % 8                         # rows of the merged projection stay 16-byte aligned
        if pad:
            mats.append(torch.zeros((pad, s.hidden_size), dtype=ctx.dtype, device=ctx.device))
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.w_o = mat(s.o_name).contiguous()
        self.conv_w = torch.cat([vec(s.q_name + s.conv_suffix), vec(s.k_name + s.conv_suffix), vec(s.v_name + s.conv_suffix)], dim=0).contiguous()
        self.a_log, self.dt_bias = vec(s.a_log_name), vec(s.dt_bias_name)
        self.norm_w = vec(s.norm_name).repeat(s.num_heads).contiguous()     # one scale over value_dim, shared by the heads

    def activation_bytes_per_token(self, elem: int) -> int:
        return (self.proj_cols + 8 + self.channels + self.inner) * elem + self.inner * 4 + self.spec.hidden_size * elem

    def cache_need(self) -> CombinedNeed:
        s = self.spec
        return CombinedNeed((StateNeed((s.num_heads, s.head_dim, s.value_dim), torch.float32),
                             StateNeed((s.conv_taps - 1, self.channels), None)))

    def forward(self, x: torch.Tensor, batch, cache, write_cache: bool = True) -> torch.Tensor:
        s = self.spec
        T, H = batch.n_tokens, s.num_heads
        state, carried = cache.children[0].state, cache.children[1].state
        proj = linear(x, self.w_in)
        g0 = self.channels
        b0 = g0 + self.inner
        qkv, gate, beta, a = proj[:, :g0], proj[:, g0:b0], proj[:, b0:b0 + H], proj[:, b0 + H:b0 + 2 * H]
        u = K.causal_conv_silu(qkv, self.conv_w, None, carried, batch, out=batch.workspace("delta_conv", (T, self.channels), x.dtype))
        K.conv_state_update(qkv, carried, batch)
        o = K.gated_delta_scan(u, beta, a, self.a_log, self.dt_bias, state, batch, s.num_kv_heads,
                               out=batch.workspace("delta_o", (T, self.inner), torch.float32))
        y = K.gated_group_rmsnorm(o, gate, self.norm_w, H, s.norm_eps, out=batch.workspace("delta_gated", (T, self.inner), x.dtype),
                                  gate_after=True)
        return linear(y, self.w_o)
