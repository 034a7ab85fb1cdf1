"""Routed experts: a mixture of SiLU-gated feed-forwards, a few per token.

The router's logits are a 32-bit product of the feed-forward's input with the
router matrix (float32 sums of exact products on the float32 units, whatever
the run's type: ``kernels.router_logits``).  Scores are their sigmoids; experts form equal groups of
neighbours, a group scores the sum of its largest scores, and only experts of
the best groups can be chosen; the chosen scores weigh the experts' outputs
(``RoutedExpertsSpec`` has the constants).  A learned correction per expert may
join the scores for the choice alone.

All experts' gate and up rows live in one tensor [experts, 2 * expert_size,
hidden] and their down rows in another [experts, hidden, expert_size].  A step
groups its (token, choice) pairs by expert on the device and runs two grouped
products over them (gate/up with the activation in the epilogue, then down)
and a weighted sum per token: five launches after the router's product, none
of whose shapes depends on what the router chose, so the part can be recorded.
"""
from __future__ import annotations

import os
from typing import Dict

import torch

from ..config.spec import RoutedExpertsSpec
from ..ops import kernels as K
from ..ops import linear as L
from ..weights.loader import TensorReq
from .registry import RunContext, register_part


# average rows per expert up to which a step's products run on the kernel that only streams the experts' weights
MOE_FEW_ROWS = int(os.environ.get("PRELUDE_MOE_FEW_ROWS", "6"))
# average rows per expert from which a step's products run on the paired-block tcgen05 kernel
MOE_PAIR_MIN_ROWS = int(os.environ.get("PRELUDE_MOE_PAIR_MIN_ROWS", "192"))


@register_part("feed_forward", "routed_experts")
class RoutedExperts:
    def __init__(self, spec: RoutedExpertsSpec, prefix: str):
        s = spec
        if s.n_experts % s.n_groups or not 0 < s.keep_groups <= s.n_groups:
            raise ValueError(f"{s.n_experts} experts do not form {s.n_groups} equal groups of which {s.keep_groups} are kept")
        if not 0 < s.top_k <= s.keep_groups * (s.n_experts // s.n_groups):
            raise ValueError(f"top_k={s.top_k} experts cannot come from {s.keep_groups} groups of {s.n_experts // s.n_groups}")
        self.spec, self.prefix = spec, prefix
        self.w_router = self.w_gate_up = self.w_down = self.correction = None

    def _expert(self, e: int, name: str) -> str:
        return f"{self.prefix}.{self.spec.expert_prefix}{e}.{name}"

    def tensors(self) -> Dict[str, TensorReq]:
        s = self.spec
        req = {f"{self.prefix}.{s.router_name}": TensorReq((s.n_experts, s.hidden_size))}
        if s.correction_name is not None:
            req[f"{self.prefix}.{s.correction_name}"] = TensorReq((s.n_experts,), "bias")
        for e in range(s.n_experts):
            req[self._expert(e, s.gate_name)] = TensorReq((s.expert_size, s.hidden_size))
            req[self._expert(e, s.up_name)] = TensorReq((s.expert_size, s.hidden_size))
            req[self._expert(e, s.down_name)] = TensorReq((s.hidden_size, s.expert_size))
        return req

    def load(self, get, ctx: RunContext) -> None:
        s = self.spec

        def mat(name):
            return get(name).to(device=ctx.device, dtype=ctx.dtype)

        self.w_router = mat(f"{self.prefix}.{s.router_name}").contiguous()
        if s.correction_name is not None:
            self.correction = get(f"{self.prefix}.{s.correction_name}").to(device=ctx.device, dtype=torch.float32).contiguous()
        self.w_gate_up = torch.stack([torch.cat([mat(self._expert(e, s.gate_name)), mat(self._expert(e, s.up_name))], dim=0)
                                      for e in range(s.n_experts)]).contiguous()
        self.w_down = torch.stack([mat(self._expert(e, s.down_name)) for e in range(s.n_experts)]).contiguous()

    def activation_bytes_per_token(self, elem: int) -> int:
        s = self.spec
        return s.top_k * (s.expert_size * elem + s.hidden_size * 4) + s.n_experts * 4 + s.hidden_size * elem

    def pair_takes(self, x: torch.Tensor) -> bool:
        """Whether a step's products run on the paired-block kernel: bfloat16, aligned sizes, and rows enough that an
        expert's 256-row tiles are mostly full (PRELUDE_MOE_PAIR_MIN_ROWS rows per expert on average, default 192)."""
        s = self.spec
        return (x.dtype == torch.bfloat16 and L.PREFILL_GEMM != "cublas" and s.hidden_size % 8 == 0 and s.expert_size % 8 == 0
                and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and x.shape[0] * s.top_k >= MOE_PAIR_MIN_ROWS * s.n_experts
                # operands no smaller than one copy box of the kernel (128 rows of 64 elements)
                and s.hidden_size >= 64 and s.expert_size >= 64 and s.n_experts * min(s.hidden_size, 2 * s.expert_size) >= 128)

    def route(self, x: torch.Tensor):
        """(experts int32 [T, top_k], weights float32 [T, top_k]) for the rows of x."""
        s = self.spec
        logits = K.router_logits(x, self.w_router)
        return K.moe_route(logits, s.top_k, s.n_groups, s.keep_groups, s.group_score_top, s.renormalize, self.correction)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        s = self.spec
        ids, weights = self.route(x)
        if self.pair_takes(x):
            # a long prompt step: rows sorted by expert, both products on the paired-block tcgen05 kernel (tiles of 256 rows)
            plan = K.moe_sort(ids, s.n_experts, 256)
            status = L.tc_status(x.device)
            h = K.moe_gemm_pair(K.moe_gather_rows(x, plan, s.top_k), self.w_gate_up, plan, True, status)
            return K.moe_combine(K.moe_gemm_pair(h, self.w_down, plan, False, status), plan, weights, x.dtype)
        # tiles of 128 rows where the experts have many rows each and the tensor-core kernel takes the shapes, else of 64
        small = x.dtype != torch.bfloat16 or s.hidden_size % 8 or s.expert_size % 8
        few = not small and x.shape[0] * s.top_k <= MOE_FEW_ROWS * s.n_experts       # a decode step: stream the weights
        plan = K.moe_sort(ids, s.n_experts, 64 if (small or few) else None)
        h = K.moe_gemm(x, self.w_gate_up, plan, gated=True, gather_div=s.top_k, few_rows=few)
        y = K.moe_gemm(h, self.w_down, plan, gated=False, out_dtype=torch.float32, few_rows=few)
        return K.moe_combine(y, plan, weights, x.dtype)
