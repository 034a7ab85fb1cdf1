"""Time mixing with a decaying matrix state per head (``WkvSpec``).

Every token is blended with the one before it, once per reader (r, k, v, gate, decay), each blend with its own
learned weights; r, k, v and the gate are projections of their blends, the decay's logarithm goes through a narrow
pair of matrices with a tanh between them.  The recurrence runs token by token with the state in float32 (the
decay's two exponentials and the bonus for the current token inside the scan kernel, in float32); each head's output
is brought to unit root mean square, scaled, gated and projected out.  Per sequence the mixer keeps the state
[heads, head_dim, head_dim] (float32) and the last token's input, both in the sequence's state slot.  The kernels
find a step's sequences through the step's device arrays, so the mixer can be recorded.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import WkvSpec
from ..ops import kernels as K
from ..ops.linear import linear
from ..weights.loader import ANY, TensorReq
from .registry import CombinedNeed, RunContext, StateNeed, register_part

_READERS = ("r", "k", "v", "g", "w")        # the order of the blends the shift kernel writes


@register_part("mixer", "wkv")
class Wkv:
    def __init__(self, spec: WkvSpec, prefix: str):
        self.spec, self.prefix = spec, prefix
        self.inner = spec.num_heads * spec.head_dim
        self.mu = self.w_r = self.w_k = self.w_v = self.w_g = self.w_1 = self.w_2 = self.w_o = None
        self.w0 = self.bonus = self.norm_w = None

    def tensors(self) -> Dict[str, TensorReq]:
        s, p = self.spec, self.prefix
        rank = ANY if s.decay_rank is None else s.decay_rank      # not a key of the configuration: the tensors' shapes give it
        req = {f"{p}.{s.mix_prefix}{n}": TensorReq((s.hidden_size,), "blend") for n in _READERS}
        for name in (s.r_name, s.k_name, s.v_name, s.gate_name):
            req[f"{p}.{name}"] = TensorReq((self.inner, s.hidden_size))
        req[f"{p}.{s.w1_name}"] = TensorReq((rank, s.hidden_size))
        req[f"{p}.{s.w2_name}"] = TensorReq((self.inner, rank))
        req[f"{p}.{s.w0_name}"] = TensorReq((self.inner,), "log_rate")
        req[f"{p}.{s.bonus_name}"] = TensorReq((s.num_heads, s.head_dim), "bias")
        req[f"{p}.{s.norm_name}"] = TensorReq((self.inner,), "norm")
        req[f"{p}.{s.o_name}"] = TensorReq((s.hidden_size, self.inner))
        return req

    def load(self, get, ctx: RunContext) -> None:
        s, p = self.spec, self.prefix

        def mat(name):
            return get(f"{p}.{name}").to(device=ctx.device, dtype=ctx.dtype).contiguous()

        def vec(name):
            return get(f"{p}.{name}").to(device=ctx.device, dtype=torch.float32).contiguous()

        self.mu = torch.stack([vec(s.mix_prefix + n) for n in _READERS]).contiguous()
        self.w_r, self.w_k, self.w_v, self.w_g = mat(s.r_name), mat(s.k_name), mat(s.v_name), mat(s.gate_name)
        self.w_1, self.w_2, self.w_o = mat(s.w1_name), mat(s.w2_name), mat(s.o_name)
        if self.w_1.shape[0] != self.w_2.shape[1]:
            raise ValueError(f"{p}: the decay's matrices meet at {self.w_1.shape[0]} and {self.w_2.shape[1]} channels")
        self.w0, self.bonus, self.norm_w = vec(s.w0_name), vec(s.bonus_name).view(-1), vec(s.norm_name)

    def activation_bytes_per_token(self, elem: int) -> int:
        s = self.spec
        return (len(_READERS) * s.hidden_size + 5 * self.inner + s.hidden_size) * elem + self.inner * 4

    def cache_need(self) -> CombinedNeed:
        s = self.spec
        return CombinedNeed((StateNeed((s.num_heads, s.head_dim, s.head_dim), torch.float32),
                             StateNeed((1, s.hidden_size), None)))

    def forward(self, x: torch.Tensor, batch, cache, write_cache: bool = True) -> torch.Tensor:
        s = self.spec
        T = batch.n_tokens
        state, carried = cache.children[0].state, cache.children[1].state
        blends = K.token_shift_mix(x, carried.view(carried.shape[0], s.hidden_size), self.mu, batch,
                                   out=batch.workspace("wkv_blends", (len(_READERS), T, s.hidden_size), x.dtype))
        K.conv_state_update(x, carried, batch)                         # the step's last input of every sequence
        r, k, v = linear(blends[0], self.w_r), linear(blends[1], self.w_k), linear(blends[2], self.w_v)
        gate = linear(blends[3], self.w_g)
        w_raw = linear(K.tanh_(linear(blends[4], self.w_1)), self.w_2)
        o = K.wkv_scan(r, k, v, w_raw, self.w0, self.bonus, state, batch, out=batch.workspace("wkv_o", (T, self.inner), torch.float32))
        y = K.gated_group_rmsnorm(o, gate, self.norm_w, s.num_heads, s.norm_eps,
                                  out=batch.workspace("wkv_gated", (T, self.inner), x.dtype), gate_after=True)
        return linear(y, self.w_o)
