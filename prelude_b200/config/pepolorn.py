"""Typed configuration of Pepolorn, read from its own config.json keys.

A Pepolorn folder names itself with ``"architecture": "Pepolorn"`` and gives ``vocab``, ``width``, ``norm.eps`` and a
list ``layers``; every entry has a ``type`` (which mixer), the mixer's sizes and constants under ``mixer`` and its
feed-forward under ``mlp`` (``null``: none).  An entry with ``weights_of: j`` has no tensors of its own: it runs layer
j's mixer, feed-forward and norms on a cache and state of its own.  Layers are parsed one by one: nothing is assumed
about their number, order or sizes.

Two mixers exist.  ``parallel`` runs a grouped-query attention with a mask of chunks (``left``) beside a linear
attention with a decaying matrix state (``right``) and adds their outputs, each times its scale.  ``mamba2`` is a
selective state-space mixer.  Two feed-forwards exist: ``dense``, gated by the tanh form of GELU, and ``moe``, routed
SiLU-gated experts whose router adds a learned correction to the scores for the choice alone.

What the design fixes, and what this file therefore writes down: a layer norms each sublayer's output and nothing
else, with scales stored around zero; the attention has no biases, rotates the first ``rot.dims`` elements of every
head with halves paired and ramp-scaled rates whose amplitude grows by 0.1 ln(factor), and brings every q and k head
to unit root mean square AFTER the rotation, without a learned scale; the linear attention's norm spans all heads and
its scale is stored as it is applied; a group of experts scores the sum of its two largest choice scores and the
chosen scores are not renormalized; the head is the embedding table; and the tensor names (``embed``, ``final.norm``,
``l<i>.norm1`` / ``norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Optional, Tuple

from .reader import _Reader, _is_int, _is_num
from .registry import ConfigError, extract_eos_token_ids, register_architecture
from .spec import (BlockSpec, DecayedLinearAttentionSpec, GatedMlpSpec, LayerCall, LinearHeadSpec, MaskedAttentionSpec, ModelSpec,
                   NoPositionSpec, NormSpec, ParallelMixerSpec, RotaryRampScaling, RotaryRatesSpec, RoutedExpertsSpec,
                   StateSpaceSpec)

RAMP_AMPLITUDE_SLOPE = 0.1
GROUP_SCORE_TOP = 2
MAX_POSITIONS = 1 << 20          # the design names no longest sequence; this bounds positions, not the arithmetic


def _rotary(m: _Reader, span: int, problems: list):
    if m.raw.get("rot") is None:
        return NoPositionSpec()
    rot = m.obj("rot")
    dims, base = rot.positive_int("dims"), rot.number("base", positive=True)
    if dims % 2 or dims > span:
        problems.append(f"{rot.where}: `dims`={dims} must be even and at most the head's {span} elements")
    if base == 1.0:
        problems.append(f"{rot.where}: `base` must not be 1")
    scaling = None
    if rot.raw.get("scaling") is not None:
        sc = rot.obj("scaling")
        scaling = RotaryRampScaling(factor=sc.number("factor", positive=True), original=sc.number("original", positive=True),
                                    fast=sc.number("fast", positive=True), slow=sc.number("slow", positive=True),
                                    amplitude_slope=RAMP_AMPLITUDE_SLOPE)
    return RotaryRatesSpec(dims=dims, base=base, adjacent=False, scaling=scaling)


def _chunked_attention(m: _Reader, width: int, eps: float, problems: list) -> MaskedAttentionSpec:
    heads, kv_heads, dim = m.positive_int("heads"), m.positive_int("kv_heads"), m.positive_int("dim")
    if heads % kv_heads:
        problems.append(f"{m.where}: heads={heads} is not a multiple of kv_heads={kv_heads}")
    chunk = m.obj("mask").positive_int("size") if m.raw.get("mask") is not None else None
    return MaskedAttentionSpec(hidden_size=width, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, value_dim=m.positive_int("vdim"),
                               softmax_scale=m.number("scale", positive=True), position=_rotary(m, dim, problems),
                               head_norm_eps=eps, head_norm_scale=False, head_norm_after_rotation=True, chunk=chunk)


def _decayed_linear_attention(m: _Reader, width: int, eps: float, problems: list) -> DecayedLinearAttentionSpec:
    heads = m.positive_int("heads")
    decays = m.raw.get("decay")
    if not isinstance(decays, list) or len(decays) != heads or not all(_is_num(d) and d >= 0.0 for d in decays):
        problems.append(f"{m.where}: `decay` must list one non-negative number for each of the {heads} heads")
        decays = [1.0] * heads
    return DecayedLinearAttentionSpec(hidden_size=width, num_heads=heads, head_dim=m.positive_int("dim"), value_dim=m.positive_int("vdim"),
                                      decays=tuple(float(d) for d in decays), norm_eps=eps)


def _state_space(m: _Reader, width: int, eps: float, problems: list) -> StateSpaceSpec:
    heads, groups, parts = m.positive_int("heads"), m.positive_int("groups"), m.positive_int("norm_groups")
    vdim = m.positive_int("vdim")
    if heads % groups:
        problems.append(f"{m.where}: heads={heads} is not a multiple of groups={groups}")
    if (heads * vdim) % parts:
        problems.append(f"{m.where}: {heads * vdim} inner channels do not form {parts} equal parts")
    return StateSpaceSpec(hidden_size=width, num_heads=heads, head_dim=vdim, state=m.positive_int("state"), groups=groups,
                          conv_taps=m.positive_int("conv"), norm_groups=parts, norm_eps=eps)


def _feed_forward(f: _Reader, width: int, problems: list):
    kind = f.raw.get("kind")
    if kind == "dense":
        return GatedMlpSpec(hidden_size=width, intermediate_size=f.positive_int("ff"), activation="gelu_tanh", gate_name="gate",
                            up_name="up", down_name="down")
    if kind == "moe":
        r = f.obj("router")
        experts, top = r.positive_int("experts"), r.positive_int("top")
        count = keep = 1
        if r.raw.get("groups") is not None:
            g = r.obj("groups")
            count, keep = g.positive_int("count"), g.positive_int("keep")
        if experts % count or keep > count:
            problems.append(f"{r.where}: {experts} experts do not form {count} equal groups of which {keep} are kept")
        elif top > keep * (experts // count):
            problems.append(f"{r.where}: top={top} experts cannot come from {keep} groups of {experts // count}")
        return RoutedExpertsSpec(hidden_size=width, expert_size=f.obj("expert").positive_int("ff"), n_experts=experts, top_k=top,
                                 n_groups=count, keep_groups=keep, group_score_top=GROUP_SCORE_TOP, renormalize=False,
                                 correction_name="correction")
    problems.append(f"{f.where}: unknown kind {kind!r}; known: ['dense', 'moe']")
    return None


@register_architecture("Pepolorn", aliases=("Pepolorn", "PepolornModel"), model_types=("pepolorn",))
@dataclass(frozen=True)
class PepolornConfig:
    vocab: int
    width: int
    norm_eps: float
    blocks: Tuple[BlockSpec, ...]          # one per layer that has tensors of its own
    order: Tuple[int, ...]                 # for every layer, in running order, the block whose weights it runs
    eos_token_ids: Tuple[int, ...] = ()
    raw: Optional[dict] = None

    @classmethod
    def from_dict(cls, raw: dict) -> "PepolornConfig":
        problems: list = []
        top = _Reader(raw, "config", problems)
        vocab, width = top.positive_int("vocab"), top.positive_int("width")
        eps = top.obj("norm").number("eps", positive=True)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            problems.append("config: `layers` must be a non-empty list")
            layers = []
        norm = NormSpec(dim=width, eps=eps, offset=1.0, suffix="")

        def source_of(i: int) -> Optional[int]:
            """The layer whose tensors layer i runs (itself, unless it says ``weights_of``), or None with a problem noted."""
            seen, j = set(), i
            while isinstance(layers[j], dict) and layers[j].get("weights_of") is not None:
                seen.add(j)
                j = layers[j]["weights_of"]
                if not _is_int(j) or not 0 <= j < len(layers) or j in seen:
                    problems.append(f"layers[{i}]: `weights_of` must lead to another layer with tensors of its own, got {j!r}")
                    return None
            return j

        def block(i: int, prefix: str) -> Optional[BlockSpec]:
            rd = _Reader(layers[i], f"layers[{i}]", problems)
            kind = rd.raw.get("type")
            m = rd.obj("mixer")
            if kind == "parallel":
                mixer = ParallelMixerSpec(
                    mixers=(_chunked_attention(m.obj("left"), width, eps, problems),
                            _decayed_linear_attention(m.obj("right"), width, eps, problems)),
                    scales=(m.number("left_scale"), m.number("right_scale")), names=("left", "right"))
            elif kind == "mamba2":
                mixer = _state_space(m, width, eps, problems)
            else:
                problems.append(f"layers[{i}]: unknown layer type {kind!r}; known: ['mamba2', 'parallel']")
                return None
            ff = None
            if rd.raw.get("mlp") is not None:
                ff = _feed_forward(_Reader(rd.raw["mlp"], f"layers[{i}].mlp", problems), width, problems)
            return BlockSpec(mixer=mixer, feed_forward=ff, mixer_norm=None, ff_norm=None, prefix=prefix, mixer_name="mix",
                             ff_name="mlp", kind="postnorm_residual", mixer_post_norm=norm,
                             ff_post_norm=norm if ff is not None else None, mixer_post_norm_name="norm1",
                             ff_post_norm_name="norm2")

        # a layer that runs another's weights is a second call of that layer's block; were its constants to differ from
        # that layer's, it would be a block of its own over the same tensors
        blocks: list = []
        order: list = []
        for i in range(len(layers)):
            j = source_of(i)
            spec = None if j is None else block(i, f"l{j}")
            if spec is None:
                continue
            if spec not in blocks:
                blocks.append(spec)
            order.append(blocks.index(spec))
        try:
            eos = extract_eos_token_ids(raw)
        except ConfigError as e:
            problems.append(str(e))
            eos = ()
        if problems:
            raise ConfigError("failed to parse Pepolorn config: " + "; ".join(problems))
        return cls(vocab=vocab, width=width, norm_eps=eps, blocks=tuple(blocks), order=tuple(order), eos_token_ids=eos,
                   raw=copy.deepcopy(raw))

    def to_dict(self) -> dict:
        return copy.deepcopy(self.raw)

    def to_model_spec(self) -> ModelSpec:
        norm = NormSpec(dim=self.width, eps=self.norm_eps, offset=1.0, suffix="")
        return ModelSpec(architecture="Pepolorn", vocab_size=self.vocab, hidden_size=self.width, max_positions=MAX_POSITIONS,
                         blocks=self.blocks, order=tuple(LayerCall(block=b) for b in self.order), final_norm=norm,
                         tie_embeddings=True, embed_name="embed", final_norm_name="final.norm", head_name="head",
                         eos_token_ids=self.eos_token_ids,
                         head=LinearHeadSpec(self.vocab, self.width, tied=True, name="head"))
