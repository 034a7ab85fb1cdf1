"""Grouped-query softmax attention with the options of ``MaskedAttentionSpec``: a norm of every q and k head with one
scale shared by the heads or without a scale, before the rotation or after it; rotation by rates (or none), whose
cosine and sine may carry an amplitude; a window that keeps the first tokens visible or a mask of chunks, capped
scores, a sink per head, a gate per head on the output, and values blended with those of the first layer that shares
the blend's key.

One merged projection [q | k | v | gate]; one kernel norms, rotates, blends, stores the queries and writes keys and
values into the layer's pages; then attention over the pages (mask, cap, sink and gate inside the attention kernel)
and the output projection.  The values that later layers blend with live in a buffer of the step: they are needed for
the step's own tokens only, because what is cached is the blended value.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import MaskedAttentionSpec
from ..ops import kernels as K
from ..ops.linear import linear
from ..ops.paged_general import attention_general
from ..weights.loader import TensorReq
from .registry import KvPagesNeed, RunContext, make_part, register_part


@register_part("mixer", "masked_attention")
class MaskedAttention:
    def __init__(self, spec: MaskedAttentionSpec, prefix: str):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} query heads do not divide over {spec.num_kv_heads} key/value heads")
        if spec.window is not None and spec.chunk is not None:
            raise ValueError("a mask is a window or chunks, not both")
        if spec.keep_first and spec.window is None:
            raise ValueError("first tokens are kept behind a window only")
        self.spec, self.prefix = spec, prefix
        self.position = make_part("position", spec.position, prefix)
        self.rotary_dim = int(getattr(self.position, "rotary_dim", 0) or 0)
        if self.rotary_dim and getattr(self.position, "rates_host", None) is None:
            raise ValueError("this mixer takes a position encoding given by rates (kind 'rotary_rates'), or none")
        if self.rotary_dim > spec.head_dim:
            raise ValueError(f"a rotation of {self.rotary_dim} elements does not fit heads of {spec.head_dim}")
        self.q_cols = spec.num_heads * spec.head_dim
        self.k_cols = spec.num_kv_heads * spec.head_dim
        self.v_cols = spec.num_kv_heads * spec.value_dim
        self.o_cols = spec.num_heads * spec.value_dim
        self.g_cols = spec.num_heads if spec.head_gate else 0
        self.w_in = self.b_in = self.w_o = self.b_o = self.q_norm = self.k_norm = self.sink = None
        self.blend = 0.0

    def parts(self):
        return (self.position,)

    def tensors(self) -> Dict[str, TensorReq]:
        s, p = self.spec, self.prefix
        req = {
            f"{p}.{s.q_name}": TensorReq((self.q_cols, s.hidden_size)),
            f"{p}.{s.k_name}": TensorReq((self.k_cols, s.hidden_size)),
            f"{p}.{s.v_name}": TensorReq((self.v_cols, s.hidden_size)),
            f"{p}.{s.o_name}": TensorReq((s.hidden_size, self.o_cols)),
        }
        if s.qkv_bias:
            for name, n in ((s.q_name, self.q_cols), (s.k_name, self.k_cols), (s.v_name, self.v_cols)):
                req[f"{p}.{name}{s.bias_suffix}"] = TensorReq((n,), "bias")
        if s.o_bias:
            req[f"{p}.{s.o_name}{s.bias_suffix}"] = TensorReq((s.hidden_size,), "bias")
        if s.head_norm_eps is not None and s.head_norm_scale:
            req[f"{p}.{s.q_name}{s.norm_suffix}"] = TensorReq((s.head_dim,), "norm")
            req[f"{p}.{s.k_name}{s.norm_suffix}"] = TensorReq((s.head_dim,), "norm")
        if s.sink:
            req[f"{p}.{s.sink_name}"] = TensorReq((s.num_heads,), "bias")
        if s.head_gate:
            req[f"{p}.{s.gate_name}"] = TensorReq((s.num_heads, s.hidden_size))
        if s.value_blend is not None:
            req[f"{p}.{s.value_blend.name}"] = TensorReq((), "blend")       # the source layer carries one too and never reads it
        return req

    def load(self, get, ctx: RunContext) -> None:
        s, p = self.spec, self.prefix

        def mat(name):
            return get(f"{p}.{name}").to(device=ctx.device, dtype=ctx.dtype)

        def vec(name):
            return get(f"{p}.{name}").to(device=ctx.device, dtype=torch.float32).contiguous()

        mats = [mat(s.q_name), mat(s.k_name), mat(s.v_name)] + ([mat(s.gate_name)] if s.head_gate else [])
        rows = sum(m.shape[0] for m in mats)
        pad = (-rows) % 8                                   # rows of the merged projection stay 16-byte aligned
        if pad:
            mats.append(torch.zeros((pad, s.hidden_size), dtype=ctx.dtype, device=ctx.device))
        self.w_in = torch.cat(mats, dim=0).contiguous()
        if s.qkv_bias:
            b = [vec(s.q_name + s.bias_suffix), vec(s.k_name + s.bias_suffix), vec(s.v_name + s.bias_suffix)]
            b.append(torch.zeros(self.w_in.shape[0] - self.q_cols - self.k_cols - self.v_cols, dtype=torch.float32, device=ctx.device))
            self.b_in = torch.cat(b).contiguous()
        self.w_o = mat(s.o_name).contiguous()
        if s.o_bias:
            self.b_o = vec(s.o_name + s.bias_suffix)
        if s.head_norm_eps is not None and s.head_norm_scale:
            self.q_norm, self.k_norm = vec(s.q_name + s.norm_suffix), vec(s.k_name + s.norm_suffix)
        if s.sink:
            self.sink = vec(s.sink_name)
        if s.value_blend is not None and not s.value_blend.source:
            self.blend = float(get(f"{p}.{s.value_blend.name}").to(torch.float32))
        self.position.load(get, ctx)

    def activation_bytes_per_token(self, elem: int) -> int:
        return (2 * self.q_cols + self.k_cols + 2 * self.v_cols + self.g_cols + 2 * self.o_cols) * elem + self.spec.hidden_size * elem

    def cache_need(self) -> KvPagesNeed:
        s = self.spec
        same = s.head_dim == s.value_dim
        return KvPagesNeed(s.num_kv_heads, s.head_dim, s.window, v_heads=None if same else s.num_kv_heads,
                           v_head_dim=None if same else s.value_dim, keep_first=s.keep_first if s.window is not None else 0,
                           chunk=s.chunk)

    def forward(self, x: torch.Tensor, batch, cache, write_cache: bool = True) -> torch.Tensor:
        s = self.spec
        T = batch.n_tokens
        proj = linear(x, self.w_in, self.b_in)
        k0, v0, g0 = self.q_cols, self.q_cols + self.k_cols, self.q_cols + self.k_cols + self.v_cols
        v_other = v_copy = None
        if s.value_blend is not None and write_cache:
            shared = batch.workspace(f"value_blend.{s.value_blend.key}", (T, self.v_cols), x.dtype)
            if s.value_blend.source:
                v_copy = shared
            else:
                v_other = shared
        rates = self.position.rates if self.rotary_dim else None
        norm = None if s.head_norm_eps is None else ("after" if s.head_norm_after_rotation else "before")
        q = K.heads_prepare(
            proj[:, :k0], proj[:, k0:v0] if write_cache else None, proj[:, v0:g0] if write_cache else None,
            n_heads=s.num_heads, q_dim=s.head_dim, q_weight=self.q_norm, k_weight=self.k_norm, eps=s.head_norm_eps or 0.0,
            norm=norm, rates=rates, amplitude=float(getattr(self.position, "amplitude", 1.0)) if self.rotary_dim else 1.0,
            rot_dims=self.rotary_dim, adjacent=bool(getattr(self.position, "adjacent", False)),
            v_other=v_other, v_copy=v_copy, mix=self.blend, positions=batch.positions, table_row=batch.table_row_of_token,
            block_table=batch.block_tables[cache.group], q_out=batch.workspace("masked_q", (T, s.num_heads, s.head_dim), x.dtype),
            k_pages=cache.k_pages if write_cache else None, v_pages=cache.v_pages if write_cache else None, status=batch.status)
        gate = proj[:, g0:g0 + self.g_cols] if s.head_gate else None
        o = attention_general(q, cache.k_pages, cache.v_pages, s.value_dim, batch, cache.group, s.softmax_scale, s.window, self.sink,
                              out=batch.workspace("masked_out", (T, s.num_heads, s.value_dim), x.dtype), keep_first=s.keep_first,
                              chunk=s.chunk, softcap=s.softcap, gate=gate)
        return linear(o.view(T, self.o_cols), self.w_o, self.b_o)
