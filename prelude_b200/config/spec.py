"""Architecture-neutral description of a decoder: what the model builder reads.

An architecture's typed configuration (for instance ``Qwen3Config``) turns its
config.json keys into one ``ModelSpec``.  Everything below the configuration —
parts, cache manager, step function, scheduler — sees only these records, so a
part never knows which model it is in, and another architecture is another
function from config.json to a ``ModelSpec``.

Every spec class carries a ``kind`` string; ``prelude_b200.parts.registry`` maps
(part family, kind) to the class that implements it.  A new kind of mixer,
feed-forward, norm or position encoding is a new spec dataclass plus a part
class registered under its kind.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """Root-mean-square norm over ``dim`` with a learned scale: x / sqrt(mean(x^2) + eps) * (offset + w).
    ``offset`` is 0 where the scale is stored as it is applied and 1 where it is stored around zero;
    ``suffix`` is what follows the part's prefix in the tensor's name."""
    dim: int
    eps: float
    kind: str = "rmsnorm"
    offset: float = 0.0
    suffix: str = ".weight"


@dataclass(frozen=True)
class RopeSpec:
    """Rotary position encoding, half-split pairing (j, j + rotary_dim/2)."""
    head_dim: int
    rotary_dim: int
    theta: float
    max_positions: int
    kind: str = "rope_half"


@dataclass(frozen=True)
class NoPositionSpec:
    """No position encoding inside the mixer."""
    kind: str = "none"


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query softmax attention over a paged key/value cache."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    softmax_scale: float
    position: object                      # RopeSpec | NoPositionSpec | ...
    qk_norm_eps: Optional[float] = None   # per-head RMSNorm of q and k when set
    bias: bool = False
    window: Optional[int] = None          # keys visible: pos_q - window < pos_k <= pos_q
    kind: str = "attention"


@dataclass(frozen=True)
class QueryTemperatureSpec:
    """Queries at position p are scaled by 1 + coef * ln(floor((p + 1) / every) + 1): attention sharpens
    as a sequence grows, in steps of ``every`` positions."""
    coef: float
    every: int


@dataclass(frozen=True)
class DiffAttentionSpec:
    """Differential attention over a paged cache: every query head holds two score maps (two queries and two
    keys of ``head_dim``) over the same values of ``value_dim``; the head's output is map 1 minus lambda
    times map 2, divided by its root mean square and scaled by ``1 - lambda_init``, with
    lambda = exp(<lq1, lk1>) - exp(<lq2, lk2>) + lambda_init.  ``gated``: the concatenated heads are
    multiplied with sigmoid of a projection of the mixer's input before the output projection.
    The ``*_name`` fields are the tensors' names below the mixer's prefix."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    softmax_scale: float
    lambda_init: float
    norm_eps: float
    query_temperature: Optional[QueryTemperatureSpec] = None
    gated: bool = True
    window: Optional[int] = None
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    gate_name: str = "g"
    o_name: str = "o"
    lambda_names: Tuple[str, str, str, str] = ("lq1", "lk1", "lq2", "lk2")
    kind: str = "diff_attention"


@dataclass(frozen=True)
class RotaryBandScaling:
    """Rates rescaled by wavelength l = 2 pi / f: kept where l < original / high, divided by ``factor`` where
    l > original / low, and blended linearly in original / l between the two."""
    factor: float
    low: float
    high: float
    original: float
    kind: str = "bands"


@dataclass(frozen=True)
class RotaryRampScaling:
    """Rates blended between f and f / factor along a ramp over the pair index i: with
    turn(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(turn(fast)), 0),
    hi = min(ceil(turn(slow)), dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) the rate is
    f_i / factor * ramp_i + f_i (1 - ramp_i); cosine and sine are both multiplied by
    ``amplitude_slope`` ln(factor) + 1."""
    factor: float
    original: float
    fast: float
    slow: float
    amplitude_slope: float = 0.1
    kind: str = "ramp"


@dataclass(frozen=True)
class RotaryRatesSpec:
    """Rotary position encoding given by its rates instead of tables: angle = position * rate_i in 32-bit inside
    the kernel, rate_i = base^(-2i/dims) rescaled by ``scaling`` (None: as they are).  ``adjacent``: rate i turns
    elements 2i and 2i + 1 of the rotated span; otherwise i and i + dims / 2.  No longest sequence is built in."""
    dims: int
    base: float
    adjacent: bool = False
    scaling: Optional[object] = None      # RotaryBandScaling | RotaryRampScaling | None
    kind: str = "rotary_rates"


@dataclass(frozen=True)
class GqaSpec:
    """Grouped-query softmax attention over a paged cache with the options that designs combine: keys and values
    of different sizes, biases on q, k and v, an RMS norm over the whole of the q projection and of the k
    projection (all heads at once, ``whole_qk_norm_eps``), a rotation of the first ``position.dims`` elements of
    every head, a window (position i sees j with 0 <= i - j < window), and a learned sink per head whose
    exponential joins the softmax's denominator.  The ``*_name`` fields are the tensors below the mixer's prefix;
    a bias is ``<name><bias_suffix>``, a norm scale ``<name><norm_suffix>``."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    softmax_scale: float
    position: object
    qkv_bias: bool = False
    whole_qk_norm_eps: Optional[float] = None
    window: Optional[int] = None
    sink: bool = False
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    o_name: str = "o"
    sink_name: str = "sink"
    bias_suffix: str = ".b"
    norm_suffix: str = ".norm"
    kind: str = "gqa"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Attention whose keys and values come from one cached latent per token.  Queries: c_q = norm(W_dq x),
    q = W_uq c_q, per head [``head_dim`` plain | ``rot_dim`` rotated].  W_dkv x gives ``kv_rank`` + ``rot_dim``
    rows: the first, normed, are the latent c; the rest, rotated, are a key part that all heads share.  Head h's
    plain key is W_uk,h c and its value W_uv,h c; the score is (q_plain . k_plain + q_rot . k_rot) * scale.
    Only c and the rotated key part are cached.  ``sink``: a learned number per head joins the denominator."""
    hidden_size: int
    num_heads: int
    head_dim: int
    rot_dim: int
    value_dim: int
    kv_rank: int
    q_rank: int
    softmax_scale: float
    norm_eps: float
    position: object
    sink: bool = False
    window: Optional[int] = None
    dq_name: str = "dq"
    uq_name: str = "uq"
    dkv_name: str = "dkv"
    uk_name: str = "uk"
    uv_name: str = "uv"
    o_name: str = "o"
    sink_name: str = "sink"
    norm_suffix: str = ".norm"
    kind: str = "latent_attention"


@dataclass(frozen=True)
class StateSpaceSpec:
    """A selective state-space mixer with scalar decay per head.  W_in x is laid out [z | x | B | C | dt] with
    inner = heads * head_dim, B and C of ``groups`` * ``state`` each, dt of ``heads``.  x, B and C pass a causal
    convolution per channel over ``conv_taps`` tokens (last tap: the current token) with bias, then SiLU.
    dt = softplus(dt + dt_bias).  Per head (its group: h // (heads / groups)) the state S [state, head_dim] moves as
    S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T and y_t = S_t^T C_t + D x_t.  y * silu(z) is brought to unit
    root mean square in ``norm_groups`` equal parts, scaled, and projected out.  The state and the last
    ``conv_taps`` - 1 inputs of the convolution are carried per sequence."""
    hidden_size: int
    num_heads: int
    head_dim: int
    state: int
    groups: int
    conv_taps: int
    norm_groups: int
    norm_eps: float
    in_name: str = "in"
    conv_name: str = "conv"
    conv_bias_name: str = "conv.b"
    dt_bias_name: str = "dt_bias"
    a_log_name: str = "A_log"
    d_name: str = "D"
    norm_name: str = "norm"
    o_name: str = "o"
    kind: str = "state_space"


@dataclass(frozen=True)
class ValueBlendSpec:
    """Values blended across layers: the first layer of a model that names ``key`` keeps its values of the step's
    tokens (``source``); every later layer with the same key replaces its own values by
    (1 - lambda) v + lambda v_source, lambda a learned number (``name``), before they are cached."""
    key: str
    source: bool
    name: str = "vmix"


@dataclass(frozen=True)
class MaskedAttentionSpec:
    """Grouped-query softmax attention over a paged cache whose options are per head: an RMS norm of every q head and
    every k head over its own elements with one scale shared by all heads (``head_norm_eps``; ``head_norm_scale``
    False: no learned scale; ``head_norm_after_rotation``: the rotated head is normed instead of the head being
    normed and then rotated, which differs where the rotation's amplitude is not 1), a rotation of the
    first ``position.dims`` elements of every head (or none), and one of two masks.  ``window``: position i sees j
    with 0 <= i - j < window, and also every j < ``keep_first``.  ``chunk``: i sees j <= i only inside its own run
    of ``chunk`` positions, counted from position 0.  ``softcap``: score <- softcap * tanh(score / softcap) after
    the scale.  ``sink``: a learned number per head joins the softmax's denominator.  ``head_gate``: head h's output
    is multiplied by sigmoid((W_gate x)_h).  ``value_blend``: see ``ValueBlendSpec``.  Biases on q, k, v
    (``qkv_bias``) and on the output projection (``o_bias``) are ``<name><bias_suffix>``."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    softmax_scale: float
    position: object                       # RotaryRatesSpec | NoPositionSpec
    qkv_bias: bool = False
    o_bias: bool = False
    head_norm_eps: Optional[float] = None
    head_norm_scale: bool = True
    head_norm_after_rotation: bool = False
    window: Optional[int] = None
    keep_first: int = 0
    chunk: Optional[int] = None
    softcap: Optional[float] = None
    sink: bool = False
    head_gate: bool = False
    value_blend: Optional[ValueBlendSpec] = None
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    o_name: str = "o"
    gate_name: str = "g"
    sink_name: str = "sink"
    bias_suffix: str = ".b"
    norm_suffix: str = ".norm"
    kind: str = "masked_attention"


@dataclass(frozen=True)
class GatedDeltaSpec:
    """The gated delta rule.  q and k are ``num_kv_heads`` x ``head_dim``, v is ``num_heads`` x ``value_dim``; each
    passes a causal convolution per channel over ``conv_taps`` tokens (last tap: the current token, no bias) and
    SiLU; q and k become unit vectors per head (x / sqrt(sum x^2 + ``unit_eps``)), q times head_dim^(-1/2).
    beta = sigmoid(W_b x), g = exp(-exp(A_log) softplus(W_a x + dt_bias)), one of each per head.  Per head (its q/k
    head: h // (heads / kv heads)) the state S [head_dim, value_dim] moves as S <- g S; u = beta (v - S^T k);
    S <- S + k u^T; o = S^T q.  o is brought to unit root mean square per head (``norm_eps``), scaled by a weight
    over value_dim that the heads share, multiplied by silu(W_g x), and projected out.  The state (float32) and
    the convolutions' last ``conv_taps`` - 1 inputs are carried per sequence."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    conv_taps: int
    norm_eps: float
    unit_eps: float = 1e-6
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    conv_suffix: str = ".conv"
    beta_name: str = "b"
    a_name: str = "a"
    a_log_name: str = "A_log"
    dt_bias_name: str = "dt_bias"
    gate_name: str = "g"
    norm_name: str = "norm"
    o_name: str = "o"
    kind: str = "gated_delta"


@dataclass(frozen=True)
class WkvSpec:
    """Time mixing with a decaying matrix state per head.  With x' the previous token's input (zeros before the
    first), each of r, k, v, g, w reads its own blend x + (x' - x) mu_s.  r, k, v are projections of their blends
    (``num_heads`` x ``head_dim``), the gate is silu(W_g blend_g), the decay w = exp(-exp(W_w2 tanh(W_w1 blend_w) + w0))
    per head and key channel (``decay_rank``: rows of W_w1).  Per head o_t = (S + diag(u) k_t v_t^T)^T r_t, then
    S <- diag(w_t) S + k_t v_t^T.  o is brought to unit root mean square per head (``norm_eps``), times a weight
    over all heads' channels, times the gate, and projected out.  The state (float32) and the previous token's
    input are carried per sequence."""
    hidden_size: int
    num_heads: int
    head_dim: int
    decay_rank: Optional[int]          # None: the decay's matrices give it by their shapes
    norm_eps: float
    mix_prefix: str = "mu."
    r_name: str = "r"
    k_name: str = "k"
    v_name: str = "v"
    gate_name: str = "g"
    w1_name: str = "w1"
    w2_name: str = "w2"
    w0_name: str = "w0"
    bonus_name: str = "u"
    norm_name: str = "norm"
    o_name: str = "o"
    kind: str = "wkv"


@dataclass(frozen=True)
class DecayedLinearAttentionSpec:
    """Linear attention with a decaying matrix state per head and a decay that is a constant of the model.
    q = silu(W_q x) and k = silu(W_k x) are ``num_heads`` x ``head_dim``, v = silu(W_v x) is ``num_heads`` x
    ``value_dim``.  Per head S_t = decays[h] S_(t-1) + k_t v_t^T and o_t = S_t^T q_t, with no other scale.  The
    concatenated heads are brought to unit root mean square together (``norm_eps``), times a learned scale over all
    of them, times sigmoid(W_g x), and projected out.  The state [head_dim, value_dim] (float32) is carried per
    sequence."""
    hidden_size: int
    num_heads: int
    head_dim: int
    value_dim: int
    decays: Tuple[float, ...]
    norm_eps: float
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    gate_name: str = "g"
    norm_name: str = "norm"
    o_name: str = "o"
    kind: str = "decayed_linear_attention"


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Several mixers side by side on the same input; the result is the sum of their outputs, each times its
    scale.  ``names[i]`` is mixer i's prefix below this mixer's.  With ``member_norms`` every member's output is
    first brought to unit root mean square over the model width and multiplied by a learned weight
    (``<prefix>.<names[i]><member_norms[i].suffix>``)."""
    mixers: Tuple[object, ...]
    scales: Tuple[float, ...]
    names: Tuple[str, ...]
    member_norms: Optional[Tuple[NormSpec, ...]] = None
    kind: str = "parallel"


@dataclass(frozen=True)
class ClampedGluSpec:
    """down(a * sigmoid(alpha * a) * (b + 1)) with a = min(gate(x), limit), b = clamp(up(x), -limit, limit); no biases."""
    hidden_size: int
    intermediate_size: int
    limit: float
    alpha: float = 1.702
    gate_name: str = "gate"
    up_name: str = "up"
    down_name: str = "down"
    kind: str = "clamped_glu"


@dataclass(frozen=True)
class RoutedExpertsSpec:
    """A mixture of ``n_experts`` SiLU-gated feed-forwards of ``expert_size``, ``top_k`` per token.  The router's
    scores are sigmoid(W_router x) in 32-bit.  Experts form ``n_groups`` equal runs of neighbours; a group's
    score is the sum of its ``group_score_top`` largest scores, and only experts of the ``keep_groups`` best
    groups can be chosen.  The chosen experts' outputs are added up weighted by their scores
    (``renormalize``: divided by the scores' sum first).  With ``correction_name`` a learned number per expert
    (``<prefix>.<correction_name>``) is added to the scores wherever they decide the choice (group scores and the
    experts chosen; the sums may be negative, and an expert outside the kept groups counts as minus infinity); the
    weights stay the scores without it.  Expert e's tensors are ``<prefix>.<expert_prefix><e>.<name>``."""
    hidden_size: int
    expert_size: int
    n_experts: int
    top_k: int
    n_groups: int = 1
    keep_groups: int = 1
    group_score_top: int = 2
    renormalize: bool = False
    correction_name: Optional[str] = None
    router_name: str = "router"
    expert_prefix: str = "e"
    gate_name: str = "gate"
    up_name: str = "up"
    down_name: str = "down"
    kind: str = "routed_experts"


@dataclass(frozen=True)
class GatedMlpSpec:
    """down(act(gate(x)) * up(x)), no biases; ``activation``: "silu", or "gelu_tanh" (the tanh form of GELU)."""
    hidden_size: int
    intermediate_size: int
    activation: str = "silu"
    gate_name: str = "gate_proj.weight"
    up_name: str = "up_proj.weight"
    down_name: str = "down_proj.weight"
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class BlockSpec:
    """One layer: which mixer, which feed-forward, which norms, how arranged.

    ``prefix`` is the layer's tensor-name prefix; the four ``*_name`` fields are
    the sub-prefixes of its parts below it.
    """
    mixer: object
    feed_forward: object
    mixer_norm: NormSpec
    ff_norm: NormSpec
    prefix: str
    mixer_name: str = "self_attn"
    ff_name: str = "mlp"
    mixer_norm_name: str = "input_layernorm"
    ff_norm_name: str = "post_attention_layernorm"
    kind: str = "prenorm_residual"
    # kind "sandwich_residual": a norm after each sublayer as well, applied to its output before the residual add;
    # there ``feed_forward`` (with its norms) may be None: a layer that is a mixer only.
    # kind "postnorm_residual": only the norms after the sublayers (``mixer_norm`` and ``ff_norm`` are None): the
    # sublayers read the residual stream itself
    mixer_post_norm: Optional[NormSpec] = None
    ff_post_norm: Optional[NormSpec] = None
    mixer_post_norm_name: str = "post_mixer_norm"
    ff_post_norm_name: str = "post_ff_norm"
    # kind "prenorm_residual" only: every sublayer's output is multiplied by this before it joins the stream; there
    # too ``feed_forward`` (with ``ff_norm``) may be None
    residual_scale: float = 1.0


@dataclass(frozen=True)
class TokenEmbeddingSpec:
    """A table of ``vocab_size`` rows of ``hidden_size``: the residual stream starts as the rows of the step's tokens."""
    vocab_size: int
    hidden_size: int
    name: str = "model.embed_tokens.weight"
    kind: str = "token_embedding"


@dataclass(frozen=True)
class ScaledEmbeddingSpec:
    """The token's row of the table times ``scale``; a tied head takes the table itself, without the scale."""
    vocab_size: int
    hidden_size: int
    scale: float
    name: str = "model.embed_tokens.weight"
    kind: str = "token_embedding_scaled"


@dataclass(frozen=True)
class SinusoidEmbeddingSpec:
    """The token's row of the table plus a fixed position vector: entry 2i is sin(p * base^(-2i/hidden_size)),
    entry 2i + 1 the cosine of the same angle, p the token's position in its sequence."""
    vocab_size: int
    hidden_size: int
    name: str = "model.embed_tokens.weight"
    base: float = 10000.0
    kind: str = "token_embedding_sinusoid"


@dataclass(frozen=True)
class LinearHeadSpec:
    """logits = x W^T over the vocabulary; ``tied`` takes the embedding's table for W."""
    vocab_size: int
    hidden_size: int
    tied: bool
    name: str = "lm_head.weight"
    kind: str = "linear_head"


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``block`` indexes ``ModelSpec.blocks`` (a block may be named more than once:
    its weights are shared).  ``cache`` names the cache this call uses; by
    default every call has a cache of its own, numbered by its place in the
    order.  A call with ``writes_cache=False`` reads the cache of the earlier
    call that owns it and stores nothing.
    """
    block: int
    cache: Optional[int] = None
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    blocks: Tuple[BlockSpec, ...]
    order: Tuple[LayerCall, ...]
    final_norm: NormSpec
    tie_embeddings: bool
    embed_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm"
    head_name: str = "lm_head.weight"
    eos_token_ids: Tuple[int, ...] = field(default_factory=tuple)
    # The two ends of the model are parts as well.  Left at None they are the plain ones that the fields above
    # describe (a table gather; a linear head, tied or not); an architecture with a scaled embedding, learned
    # positions added to it, or a capped or scaled head names its own spec here.
    embedding: Optional[object] = None
    head: Optional[object] = None
    # name patterns (shell style) of tensors that checkpoints of the architecture carry and the model does not read
    ignored_tensors: Tuple[str, ...] = field(default_factory=tuple)

    def embedding_spec(self) -> object:
        return self.embedding or TokenEmbeddingSpec(self.vocab_size, self.hidden_size, self.embed_name)

    def head_spec(self) -> object:
        return self.head or LinearHeadSpec(self.vocab_size, self.hidden_size, self.tie_embeddings, self.head_name)

    def resolved_order(self) -> Tuple[LayerCall, ...]:
        """The run order with every ``cache`` filled in and checked."""
        out = []
        for n, call in enumerate(self.order):
            if not 0 <= call.block < len(self.blocks):
                raise ValueError(f"order[{n}] names block {call.block}, model has {len(self.blocks)}")
            cache = n if call.cache is None else call.cache
            if call.writes_cache:
                if cache != n:
                    raise ValueError(f"order[{n}] writes a cache, so it must own it (cache={cache})")
            else:
                if not (0 <= cache < n and out[cache].writes_cache):
                    raise ValueError(f"order[{n}] reads cache {cache}, which no earlier call owns")
            out.append(LayerCall(call.block, cache, call.writes_cache))
        return tuple(out)
