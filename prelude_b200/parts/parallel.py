"""Several mixers side by side on the same input (``ParallelMixerSpec``): the result is the sum of their outputs,
each times its scale, added up in float32 and rounded once.  With ``member_norms`` each output is first brought to
unit root mean square over the model width and multiplied by its own learned weight; norms, scales and sum are one
kernel, and the sum is handed on in float32.  What the members keep (pages, state) forms one combined
cache need; member i runs against child i of the layer's cache."""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import ParallelMixerSpec
from ..ops import kernels as K
from ..weights.loader import TensorReq
from .registry import CombinedNeed, RunContext, make_part, register_part


@register_part("mixer", "parallel")
class ParallelMixer:
    def __init__(self, spec: ParallelMixerSpec, prefix: str):
        if not (len(spec.mixers) == len(spec.scales) == len(spec.names)) or len(spec.mixers) < 2:
            raise ValueError("a parallel mixer has two or more members, each with a scale and a name")
        self.spec, self.prefix = spec, prefix
        self.members = [make_part("mixer", m, f"{prefix}.{n}") for m, n in zip(spec.mixers, spec.names)]
        self.norms = []
        if spec.member_norms is not None:
            if len(spec.member_norms) != len(spec.mixers) or len(spec.mixers) != 2:
                raise ValueError("normed members: two mixers, each with its norm")
            if any(n.eps != spec.member_norms[0].eps for n in spec.member_norms):
                raise ValueError("the members' norms share one eps")
            self.norms = [make_part("norm", ns, f"{prefix}.{n}") for ns, n in zip(spec.member_norms, spec.names)]

    def parts(self):
        return tuple(self.members) + tuple(self.norms)

    def tensors(self) -> Dict[str, TensorReq]:
        out: Dict[str, TensorReq] = {}
        for m in self.parts():
            out.update(m.tensors())
        return out

    def load(self, get, ctx: RunContext) -> None:
        for m in self.parts():
            m.load(get, ctx)

    def activation_bytes_per_token(self, elem: int) -> int:
        return sum(getattr(m, "activation_bytes_per_token", lambda e: 0)(elem) for m in self.members)

    def cache_need(self) -> CombinedNeed:
        return CombinedNeed(tuple(m.cache_need() for m in self.members))

    def forward(self, x: torch.Tensor, batch, cache, write_cache: bool = True) -> torch.Tensor:
        outs = [m.forward(x, batch, cache.children[i], write_cache) for i, m in enumerate(self.members)]
        outs = [o.materialize(x.dtype) if isinstance(o, K.PartialSums) else o for o in outs]
        scales = self.spec.scales
        if self.norms:
            return K.normed_pair_sum(outs[0], self.norms[0].weight, scales[0], outs[1], self.norms[1].weight, scales[1],
                                     self.norms[0].spec.eps)
        y = K.scaled_sum(outs[0], scales[0], outs[1], scales[1], torch.float32 if len(outs) > 2 else x.dtype)
        for i in range(2, len(outs)):
            last = i == len(outs) - 1
            y = K.scaled_sum(y, 1.0, outs[i].float(), scales[i], x.dtype if last else torch.float32)
        return y
