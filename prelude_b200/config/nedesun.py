"""Typed configuration of Nedesun, read from its own config.json keys.

A Nedesun folder names itself with ``"architecture": "Nedesun"`` and gives ``vocab``, ``width``, ``norm.eps``,
``residual_mult``, ``embedding.scale`` and a list ``layers``; every entry has a ``type`` (which mixer), the mixer's
sizes and constants under ``mixer`` and its feed-forward under ``mlp`` (``null``: none).  Layers are parsed one by one:
nothing is assumed about their number, order or sizes.

Three mixers exist.  ``attention``: grouped-query attention with biases, a rotation of the first ``rot.dims`` elements
of every head (halves paired), capped scores, a mask of chunks, values blended with those of the first such layer
(``v_mix``) and a gate per head.  ``wkv``: time mixing with a decaying matrix state per head.  ``parallel``: a
windowed attention that keeps the first tokens visible, with a norm per head and a sink (``left``), beside the gated
delta rule (``right``); each side's output is normed over the width and the result is half their sum.

What the design fixes, and what this file therefore writes down: pre-norm layers whose sublayers join the stream
times ``residual_mult``; which mixer has which options; the unit vectors' 1e-6; a SiLU-gated feed-forward; a head
tied to the unscaled embedding table; and the tensor names (``embed``, ``final.norm``, ``l<i>.norm1`` / ``norm2``,
``l<i>.mix.*``, ``l<i>.mlp.*``).  The decay's inner width of ``wkv`` is no key of the configuration: the tensors give it.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Optional, Tuple

from .reader import _Reader
from .registry import ConfigError, extract_eos_token_ids, register_architecture
from .spec import (BlockSpec, GatedDeltaSpec, GatedMlpSpec, LayerCall, LinearHeadSpec, MaskedAttentionSpec, ModelSpec,
                   NoPositionSpec, NormSpec, ParallelMixerSpec, RotaryRatesSpec, ScaledEmbeddingSpec, ValueBlendSpec, WkvSpec)

UNIT_EPS = 1e-6
MAX_POSITIONS = 1 << 20          # the design names no longest sequence; this bounds positions, not the arithmetic
VALUE_BLEND_KEY = "v_mix"


def _heads(m: _Reader, problems: list) -> Tuple[int, int, int, int]:
    heads, kv_heads = m.positive_int("heads"), m.positive_int("kv_heads")
    if heads % kv_heads:
        problems.append(f"{m.where}: heads={heads} is not a multiple of kv_heads={kv_heads}")
    return heads, kv_heads, m.positive_int("dim"), m.positive_int("vdim")


def _chunked_attention(m: _Reader, width: int, first_blend: bool, problems: list) -> MaskedAttentionSpec:
    heads, kv_heads, dim, vdim = _heads(m, problems)
    position = NoPositionSpec()
    if m.raw.get("rot") is not None:
        rot = m.obj("rot")
        dims, base = rot.positive_int("dims"), rot.number("base", positive=True)
        if dims % 2 or dims > dim:
            problems.append(f"{rot.where}: `dims`={dims} must be even and at most the head's {dim} elements")
        position = RotaryRatesSpec(dims=dims, base=base, adjacent=False, scaling=None)
    chunk = m.obj("mask").positive_int("size") if m.raw.get("mask") is not None else None
    softcap = m.number("softcap", positive=True) if m.raw.get("softcap") is not None else None
    blend = ValueBlendSpec(key=VALUE_BLEND_KEY, source=first_blend) if m.raw.get("v_mix") else None
    return MaskedAttentionSpec(hidden_size=width, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, value_dim=vdim,
                               softmax_scale=m.number("scale", positive=True), position=position, qkv_bias=True, o_bias=True,
                               chunk=chunk, softcap=softcap, head_gate=True, value_blend=blend)


def _window_attention(m: _Reader, width: int, eps: float, problems: list) -> MaskedAttentionSpec:
    heads, kv_heads, dim, vdim = _heads(m, problems)
    window, keep = None, 0
    if m.raw.get("mask") is not None:
        mask = m.obj("mask")
        window = mask.positive_int("size")
        if mask.raw.get("keep_first") is not None:
            keep = mask.raw["keep_first"]
            if isinstance(keep, bool) or not isinstance(keep, int) or keep < 0:
                problems.append(f"{mask.where}: `keep_first` must be a non-negative integer")
                keep = 0
    return MaskedAttentionSpec(hidden_size=width, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, value_dim=vdim,
                               softmax_scale=m.number("scale", positive=True), position=NoPositionSpec(), head_norm_eps=eps,
                               window=window, keep_first=keep, sink=True)


def _gated_delta(m: _Reader, width: int, eps: float, problems: list) -> GatedDeltaSpec:
    heads, kv_heads, dim, vdim = _heads(m, problems)
    return GatedDeltaSpec(hidden_size=width, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, value_dim=vdim,
                          conv_taps=m.positive_int("conv"), norm_eps=eps, unit_eps=UNIT_EPS)


@register_architecture("Nedesun", aliases=("Nedesun", "NedesunModel"), model_types=("nedesun",))
@dataclass(frozen=True)
class NedesunConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    embedding_scale: float
    blocks: Tuple[BlockSpec, ...]
    eos_token_ids: Tuple[int, ...] = ()
    raw: Optional[dict] = None

    @classmethod
    def from_dict(cls, raw: dict) -> "NedesunConfig":
        problems: list = []
        top = _Reader(raw, "config", problems)
        vocab, width = top.positive_int("vocab"), top.positive_int("width")
        eps = top.obj("norm").number("eps", positive=True)
        mult = top.number("residual_mult")
        scale = top.obj("embedding").number("scale")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            problems.append("config: `layers` must be a non-empty list")
            layers = []
        norm = NormSpec(dim=width, eps=eps, suffix="")
        blocks = []
        blend_cols = None
        for i, layer in enumerate(layers):
            rd = _Reader(layer, f"layers[{i}]", problems)
            kind = rd.raw.get("type")
            m = rd.obj("mixer")
            if kind == "attention":
                mixer = _chunked_attention(m, width, blend_cols is None, problems)
                if mixer.value_blend is not None:
                    cols = mixer.num_kv_heads * mixer.value_dim
                    if blend_cols is not None and cols != blend_cols:
                        problems.append(f"layers[{i}].mixer: blended values of {cols} elements against the first such layer's {blend_cols}")
                    blend_cols = cols if blend_cols is None else blend_cols
            elif kind == "wkv":
                mixer = WkvSpec(hidden_size=width, num_heads=m.positive_int("heads"), head_dim=m.positive_int("dim"), decay_rank=None,
                                norm_eps=eps)
            elif kind == "parallel":
                mixer = ParallelMixerSpec(
                    mixers=(_window_attention(m.obj("left"), width, eps, problems), _gated_delta(m.obj("right"), width, eps, problems)),
                    scales=(0.5, 0.5), names=("left", "right"),
                    member_norms=(NormSpec(dim=width, eps=eps, suffix=".out"), NormSpec(dim=width, eps=eps, suffix=".out")))
            else:
                problems.append(f"layers[{i}]: unknown layer type {kind!r}; known: ['attention', 'parallel', 'wkv']")
                continue
            ff = None
            mlp = rd.raw.get("mlp")
            if mlp is not None:
                f = _Reader(mlp, f"layers[{i}].mlp", problems)
                if f.raw.get("kind") != "dense":
                    problems.append(f"layers[{i}].mlp: unknown kind {f.raw.get('kind')!r}; known: ['dense']")
                else:
                    ff = GatedMlpSpec(hidden_size=width, intermediate_size=f.positive_int("ff"), activation="silu",
                                      gate_name="gate", up_name="up", down_name="down")
            blocks.append(BlockSpec(mixer=mixer, feed_forward=ff, mixer_norm=norm, ff_norm=norm if ff is not None else None,
                                    prefix=f"l{i}", mixer_name="mix", ff_name="mlp", mixer_norm_name="norm1", ff_norm_name="norm2",
                                    kind="prenorm_residual", residual_scale=mult))
        try:
            eos = extract_eos_token_ids(raw)
        except ConfigError as e:
            problems.append(str(e))
            eos = ()
        if problems:
            raise ConfigError("failed to parse Nedesun config: " + "; ".join(problems))
        return cls(vocab=vocab, width=width, norm_eps=eps, residual_mult=mult, embedding_scale=scale, blocks=tuple(blocks),
                   eos_token_ids=eos, raw=copy.deepcopy(raw))

    def to_dict(self) -> dict:
        return copy.deepcopy(self.raw)

    def to_model_spec(self) -> ModelSpec:
        norm = NormSpec(dim=self.width, eps=self.norm_eps, suffix="")
        return ModelSpec(architecture="Nedesun", vocab_size=self.vocab, hidden_size=self.width, max_positions=MAX_POSITIONS,
                         blocks=self.blocks, order=tuple(LayerCall(block=i) for i in range(len(self.blocks))), final_norm=norm,
                         tie_embeddings=True, embed_name="embed", final_norm_name="final.norm", head_name="head",
                         eos_token_ids=self.eos_token_ids,
                         embedding=ScaledEmbeddingSpec(self.vocab, self.width, self.embedding_scale, name="embed"),
                         head=LinearHeadSpec(self.vocab, self.width, tied=True, name="head"))
