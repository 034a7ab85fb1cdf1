"""Arrangement of a mixer and a feed-forward in one layer.

Pre-norm residual block with the add fused into the next norm, as the
reference's decoder layer (crates/prelude-core/src/models/qwen3.rs:486-502):

    res += delta ; x = norm1(res) ; a = mixer(x)
    res += a     ; x = norm2(res) ; return feed_forward(x)      (added by whoever comes next)

``res`` is the float32 residual stream and is updated in place.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import BlockSpec
from ..weights.loader import TensorReq
from .registry import RunContext, make_part, register_part


@register_part("block", "prenorm_residual")
class PreNormResidualBlock:
    """The block of this file's head.  With ``residual_scale`` m other than 1 every sublayer's output joins the stream
    times m (``kernels.Scaled``: the fused add multiplies while it adds, in float32); a block may then also have no
    feed-forward, and hands on its mixer's output instead."""

    def __init__(self, spec: BlockSpec, prefix: str = ""):
        self.spec = spec
        p = spec.prefix
        self.scale = float(spec.residual_scale)
        if spec.feed_forward is None and spec.ff_norm is not None:
            raise ValueError("a norm before a feed-forward that the block does not have")
        self.mixer_norm = make_part("norm", spec.mixer_norm, f"{p}.{spec.mixer_norm_name}")
        self.mixer = make_part("mixer", spec.mixer, f"{p}.{spec.mixer_name}")
        self.ff_norm = self.feed_forward = None
        if spec.feed_forward is not None:
            self.ff_norm = make_part("norm", spec.ff_norm, f"{p}.{spec.ff_norm_name}")
            self.feed_forward = make_part("feed_forward", spec.feed_forward, f"{p}.{spec.ff_name}")

    def parts(self):
        return tuple(x for x in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward) if x is not None)

    def tensors(self) -> Dict[str, TensorReq]:
        out: Dict[str, TensorReq] = {}
        for part in self.parts():
            out.update(part.tensors())
        return out

    def load(self, get, ctx: RunContext) -> None:
        for part in self.parts():
            part.load(get, ctx)

    def cache_need(self):
        return self.mixer.cache_need()

    def _out(self, y):
        if self.scale == 1.0:
            return y
        from ..ops import kernels as K
        return K.Scaled(y, self.scale)

    def forward(self, delta, res: torch.Tensor, batch, cache, write_cache: bool):
        x = self.mixer_norm.add_forward(delta, res)
        a = self._out(self.mixer.forward(x, batch, cache, write_cache))
        if self.feed_forward is None:
            return a
        x = self.ff_norm.add_forward(a, res)
        return self._out(self.feed_forward.forward(x))


@register_part("block", "sandwich_residual")
class SandwichResidualBlock:
    """A norm before and after each sublayer:

        res += delta ; a = mixer(norm1(res)) ; res += norm1b(a) ; f = ff(norm2(res)) ; return norm2b(f), pending

    The norm after a sublayer and the add and norm that follow are one kernel: what this block returns is its
    feed-forward's output with ``norm2b`` still to be applied (``kernels.Normed``), which the next block's first
    norm, or the model's final norm, applies while it adds.  A block without a feed-forward returns its mixer's
    output the same way.
    """

    def __init__(self, spec: BlockSpec, prefix: str = ""):
        if spec.mixer_post_norm is None or (spec.feed_forward is not None and (spec.ff_norm is None or spec.ff_post_norm is None)):
            raise ValueError("a sandwich block needs a norm after every sublayer it has")
        self.spec = spec
        p = spec.prefix
        self.mixer_norm = make_part("norm", spec.mixer_norm, f"{p}.{spec.mixer_norm_name}")
        self.mixer = make_part("mixer", spec.mixer, f"{p}.{spec.mixer_name}")
        self.mixer_post_norm = make_part("norm", spec.mixer_post_norm, f"{p}.{spec.mixer_post_norm_name}")
        self.ff_norm = self.feed_forward = self.ff_post_norm = None
        if spec.feed_forward is not None:
            self.ff_norm = make_part("norm", spec.ff_norm, f"{p}.{spec.ff_norm_name}")
            self.feed_forward = make_part("feed_forward", spec.feed_forward, f"{p}.{spec.ff_name}")
            self.ff_post_norm = make_part("norm", spec.ff_post_norm, f"{p}.{spec.ff_post_norm_name}")

    def parts(self):
        return tuple(x for x in (self.mixer_norm, self.mixer, self.mixer_post_norm, self.ff_norm, self.feed_forward,
                                 self.ff_post_norm) if x is not None)

    def tensors(self) -> Dict[str, TensorReq]:
        out: Dict[str, TensorReq] = {}
        for part in self.parts():
            out.update(part.tensors())
        return out

    def load(self, get, ctx: RunContext) -> None:
        for part in self.parts():
            part.load(get, ctx)

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, delta, res: torch.Tensor, batch, cache, write_cache: bool):
        x = self.mixer_norm.add_forward(delta, res)
        a = self.mixer_post_norm.pending(self.mixer.forward(x, batch, cache, write_cache))
        if self.feed_forward is None:
            return a
        x = self.ff_norm.add_forward(a, res)
        return self.ff_post_norm.pending(self.feed_forward.forward(x))


@register_part("block", "postnorm_residual")
class PostNormResidualBlock:
    """Norms on the sublayers' outputs only; the sublayers read the residual stream itself:

        res += delta ; a = mixer(res) ; res += norm1(a) ; f = ff(res) ; return norm2(f), pending

    What arrives as ``delta`` is the previous block's output with its norm still to be applied
    (``kernels.Normed``); one kernel norms it, adds it and hands the sum to the sublayer in the run's type (in
    32-bit the sublayer reads the stream in place).  A block without a feed-forward returns its mixer's output
    the same way."""

    def __init__(self, spec: BlockSpec, prefix: str = ""):
        if spec.mixer_post_norm is None or (spec.feed_forward is not None and spec.ff_post_norm is None):
            raise ValueError("a post-norm block needs a norm after every sublayer it has")
        self.spec = spec
        p = spec.prefix
        self.mixer = make_part("mixer", spec.mixer, f"{p}.{spec.mixer_name}")
        self.mixer_post_norm = make_part("norm", spec.mixer_post_norm, f"{p}.{spec.mixer_post_norm_name}")
        self.feed_forward = self.ff_post_norm = None
        if spec.feed_forward is not None:
            self.feed_forward = make_part("feed_forward", spec.feed_forward, f"{p}.{spec.ff_name}")
            self.ff_post_norm = make_part("norm", spec.ff_post_norm, f"{p}.{spec.ff_post_norm_name}")

    def parts(self):
        return tuple(x for x in (self.mixer, self.mixer_post_norm, self.feed_forward, self.ff_post_norm) if x is not None)

    def tensors(self) -> Dict[str, TensorReq]:
        out: Dict[str, TensorReq] = {}
        for part in self.parts():
            out.update(part.tensors())
        return out

    def load(self, get, ctx: RunContext) -> None:
        self.dtype = ctx.dtype
        for part in self.parts():
            part.load(get, ctx)

    def cache_need(self):
        return self.mixer.cache_need()

    def _stream(self, delta, res: torch.Tensor) -> torch.Tensor:
        """res += delta (its pending norm applied); the stream in the type the sublayers read."""
        from ..ops import kernels as K
        if delta is None:
            return res if self.dtype == torch.float32 else K.scaled_sum(res, 1.0, res, 0.0, self.dtype)
        if not isinstance(delta, K.Normed):
            raise TypeError("a post-norm block adds normed outputs to the stream")
        x = K.normed_add_rmsnorm(delta, res, None, 0.0, self.dtype, sum_out=self.dtype != torch.float32)
        return res if x is None else x

    def forward(self, delta, res: torch.Tensor, batch, cache, write_cache: bool):
        x = self._stream(delta, res)
        a = self.mixer_post_norm.pending(self.mixer.forward(x, batch, cache, write_cache))
        if self.feed_forward is None:
            return a
        x = self._stream(a, res)
        return self.ff_post_norm.pending(self.feed_forward.forward(x))
