"""Plain, slow, whole-sequence implementation of the Pepolorn decoder.

The oracle of the Pepolorn tests.  It shares no code with the ``prelude_b200``
package: it takes the parsed config.json and a ``dict`` of tensors keyed by
their safetensors names, runs a whole sequence at once with no cache, and
returns the logits of every position (and, on request, the residual stream
after every layer).  One function per mechanism; the recurrences are explicit
loops over tokens.

The design, in this file's notation (D = width, t = position from 0):

  norm        n(x; g) = x / sqrt(mean(x^2) + eps) * (1 + g)          (scales stored around zero)
  layer       r <- r + n(mixer(r); g1) ;  r <- r + n(ff(r); g2)      (the sublayers read r itself)
  mixers      'parallel': a_l * chunked_attention(r) + a_r * decayed_linear_attention(r);  'mamba2'
  ff          dense: W_d [ gelu_tanh(W_g x) * W_u x ];  routed: sum over the chosen experts e of s_e W_d,e [ silu(W_g,e x) * W_u,e x ]
  output      logits = E n(r; g_final), E the embedding table
  a layer with 'weights_of': j runs layer j's tensors on a state of its own

All arithmetic is done in ``dtype`` (float64 by default); bfloat16 weights
convert exactly.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def zero_centred_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * (1.0 + g)


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


# -- rotation ---------------------------------------------------------------------------------------
def ramped_rates(dims: int, base: float, sc: Optional[dict]) -> Tuple[List[float], float]:
    """(rates, amplitude).  Pair i turns at base^(-2i/dims); with a scaling the rate is blended towards rate / factor
    along a ramp over i, and cosine and sine both grow by 0.1 ln(factor) + 1."""
    plain = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if sc is None:
        return plain, 1.0

    def where(turns: float) -> float:
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(where(sc["fast"])), 0)
    hi = min(math.ceil(where(sc["slow"])), dims - 1)
    rates = []
    for i, f in enumerate(plain):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        rates.append(f / sc["factor"] * ramp + f * (1.0 - ramp))
    return rates, 0.1 * math.log(sc["factor"]) + 1.0


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, rates: List[float], amplitude: float) -> torch.Tensor:
    """x [T, heads, d]: entry i of the first 2 * len(rates) goes with entry i + len(rates); the rest pass."""
    n = len(rates)
    ang = positions.to(x.dtype).reshape(-1, 1, 1) * torch.tensor(rates, dtype=x.dtype).reshape(1, 1, -1)
    c, s = ang.cos() * amplitude, ang.sin() * amplitude
    out = x.clone()
    u, v = x[..., :n], x[..., n:2 * n]
    out[..., :n] = u * c - v * s
    out[..., n:2 * n] = v * c + u * s
    return out


# -- softmax attention over chunks --------------------------------------------------------------------
def chunk_mask(T: int, size: Optional[int], start: int = 0) -> torch.Tensor:
    """[T, T] of who sees whom: j <= i, and (with ``size``) both in the same run of ``size`` positions from 0."""
    i = torch.arange(start, start + T).reshape(-1, 1)
    j = torch.arange(start, start + T).reshape(1, -1)
    seen = j <= i
    if size is not None:
        seen = seen & (torch.div(i, size, rounding_mode="floor") == torch.div(j, size, rounding_mode="floor"))
    return seen


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, seen: torch.Tensor) -> torch.Tensor:
    """q [T, H, d], k [T, H, d], v [T, H, e], seen [T, T] -> [T, H, e]."""
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~seen, -math.inf)
    return torch.einsum("hij,jhe->ihe", torch.softmax(s, dim=-1), v)


def chunked_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """Grouped-query attention without biases: partial rotation of paired halves with ramped rates, then every q and k
    head brought to unit root mean square (no scale), scores times ``scale``, a mask of chunks."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).reshape(T, H, d)
    k = (h @ w["k"].T).reshape(T, G, d)
    v = (h @ w["v"].T).reshape(T, G, e)
    if m.get("rot") is not None:
        rot = m["rot"]
        rates, amp = ramped_rates(rot["dims"], rot["base"], rot.get("scaling"))
        pos = torch.arange(T)
        q, k = rotate_halves(q, pos, rates, amp), rotate_halves(k, pos, rates, amp)
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    rep = H // G
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    size = m["mask"]["size"] if m.get("mask") else None
    o = softmax_attention(q, k, v, m["scale"], chunk_mask(T, size))
    return o.reshape(T, H * e) @ w["o"].T


# -- linear attention with a fixed decay per head -------------------------------------------------------
def decayed_state(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor) -> torch.Tensor:
    """q, k [T, H, d], v [T, H, e], decay [H]:  S_t = decay S_(t-1) + k_t v_t^T ;  o_t = S_t^T q_t."""
    T, H, d = q.shape
    e = v.shape[-1]
    S = torch.zeros(H, d, e, dtype=q.dtype)
    o = torch.empty(T, H, e, dtype=q.dtype)
    for t in range(T):
        S = decay.reshape(H, 1, 1) * S + k[t].reshape(H, d, 1) * v[t].reshape(H, 1, e)
        o[t] = torch.einsum("hde,hd->he", S, q[t])
    return o


def decayed_linear_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w["q"].T).reshape(T, H, d)
    k = silu(h @ w["k"].T).reshape(T, H, d)
    v = silu(h @ w["v"].T).reshape(T, H, e)
    o = decayed_state(q, k, v, torch.tensor(m["decay"], dtype=h.dtype)).reshape(T, H * e)
    o = unit_rms(o, eps) * w["norm"]                       # one norm over all heads, plain scale
    o = o * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


# -- state-space mixer ----------------------------------------------------------------------------------
def causal_conv(u: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """u [T, C], taps [C, K] (last column: the current token), zeros before the start."""
    T, C = u.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=u.dtype), u], dim=0)
    out = bias.reshape(1, C).expand(T, C).clone()
    for j in range(K):
        out = out + padded[j:j + T] * taps[:, j].reshape(1, C)
    return out


def selective_state(x: torch.Tensor, B: torch.Tensor, C: torch.Tensor, dt: torch.Tensor, a_log: torch.Tensor,
                    D: torch.Tensor) -> torch.Tensor:
    """x [T, H, P], B and C [T, H, N] (already spread over the heads), dt [T, H]:
    S_t = exp(-exp(a_log) dt_t) S_(t-1) + dt_t B_t x_t^T ;  y_t = S_t^T C_t + D x_t."""
    T, H, P = x.shape
    N = B.shape[-1]
    S = torch.zeros(H, N, P, dtype=x.dtype)
    y = torch.empty_like(x)
    for t in range(T):
        keep = torch.exp(-torch.exp(a_log) * dt[t])
        S = keep.reshape(H, 1, 1) * S + dt[t].reshape(H, 1, 1) * B[t].reshape(H, N, 1) * x[t].reshape(H, 1, P)
        y[t] = torch.einsum("hnp,hn->hp", S, C[t]) + D.reshape(H, 1) * x[t]
    return y


def mamba2(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = h @ w["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w["conv"], w["conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N).repeat_interleave(H // G, dim=1)
    C = xbc[:, inner + G * N:].reshape(T, G, N).repeat_interleave(H // G, dim=1)
    dt = softplus(dt + w["dt_bias"])
    y = selective_state(x, B, C, dt, w["A_log"], w["D"]).reshape(T, inner)
    y = y * silu(z)                                        # the gate comes before the norm
    parts = m["norm_groups"]
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w["norm"]
    return y @ w["o"].T


# -- feed-forwards ----------------------------------------------------------------------------------------
def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor]) -> torch.Tensor:
    return (gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def route(h: torch.Tensor, w_router: torch.Tensor, correction: torch.Tensor, r: dict) -> Tuple[torch.Tensor, torch.Tensor]:
    """(experts [T, top], weights [T, top]).  s = sigmoid(W h); the choice goes by s + correction, restricted to the
    ``keep`` groups of neighbours whose two largest choice scores sum highest; the weights are s itself."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ w_router.T)
    choice = s + correction
    groups = r.get("groups")
    if groups is not None and groups["keep"] < groups["count"]:
        n = groups["count"]
        per = E // n
        by_group = choice.reshape(-1, n, per)
        score = by_group.topk(min(2, per), dim=-1).values.sum(dim=-1)
        best = score.topk(groups["keep"], dim=-1).indices
        allowed = torch.zeros_like(score, dtype=torch.bool).scatter_(1, best, True)
        choice = choice.masked_fill(~allowed.repeat_interleave(per, dim=1), -math.inf)
    ids = choice.topk(top, dim=-1).indices
    return ids, torch.gather(s, 1, ids)


def route_margin(h: torch.Tensor, w_router: torch.Tensor, correction: torch.Tensor, r: dict) -> torch.Tensor:
    """[T]: by how much each token's choice is decided: the smaller of the gap between the last kept group and the
    first one dropped, and the gap between the last chosen expert and the best allowed one not chosen.  A test in
    reduced precision leaves out tokens whose gap is within the rounding."""
    E, top = r["experts"], r["top"]
    choice = torch.sigmoid(h @ w_router.T) + correction
    margin = torch.full((h.shape[0],), math.inf, dtype=h.dtype)
    groups = r.get("groups")
    if groups is not None and groups["keep"] < groups["count"]:
        per = E // groups["count"]
        score = choice.reshape(-1, groups["count"], per).topk(min(2, per), dim=-1).values.sum(dim=-1)
        ranked = score.sort(dim=-1, descending=True).values
        margin = ranked[:, groups["keep"] - 1] - ranked[:, groups["keep"]]
        allowed = torch.zeros_like(score, dtype=torch.bool).scatter_(1, score.topk(groups["keep"], dim=-1).indices, True)
        choice = choice.masked_fill(~allowed.repeat_interleave(per, dim=1), -math.inf)
    ranked = choice.sort(dim=-1, descending=True).values
    if top < E:
        margin = torch.minimum(margin, ranked[:, top - 1] - ranked[:, top])
    return margin


def routed_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], mlp: dict) -> torch.Tensor:
    ids, weights = route(h, w["router"], w["correction"], mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(ids[t].tolist(), weights[t]):
            x = h[t]
            out[t] += s * ((silu(w[f"e{e}.gate"] @ x) * (w[f"e{e}.up"] @ x)) @ w[f"e{e}.down"].T)
    return out


# -- the model ------------------------------------------------------------------------------------------------
def sub(tensors: Dict[str, torch.Tensor], prefix: str, dtype) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(dtype) for k, v in tensors.items() if k.startswith(prefix)}


def mixer(kind: str, h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    if kind == "parallel":
        left = chunked_attention(h, sub(w, "left.", h.dtype), m["left"], eps)
        right = decayed_linear_attention(h, sub(w, "right.", h.dtype), m["right"], eps)
        return m["left_scale"] * left + m["right_scale"] * right
    if kind == "mamba2":
        return mamba2(h, w, m, eps)
    raise ValueError(f"unknown layer type {kind!r}")


def feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], mlp: dict) -> torch.Tensor:
    if mlp["kind"] == "dense":
        return dense_ff(h, w)
    if mlp["kind"] == "moe":
        return routed_ff(h, w, mlp)
    raise ValueError(f"unknown feed-forward {mlp['kind']!r}")


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens, dtype=torch.float64, layers_out: Optional[list] = None,
            margins_out: Optional[list] = None):
    """Logits [T, vocab] of a whole sequence; ``layers_out`` collects the residual stream after every layer,
    ``margins_out`` every router's ``route_margin``."""
    eps = cfg["norm"]["eps"]
    table = tensors["embed"].to(dtype)
    r = table[torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        src = i
        while cfg["layers"][src].get("weights_of") is not None:
            src = cfg["layers"][src]["weights_of"]
        a = mixer(layer["type"], r, sub(tensors, f"l{src}.mix.", dtype), layer["mixer"], eps)
        r = r + zero_centred_norm(a, tensors[f"l{src}.norm1"].to(dtype), eps)
        if layer.get("mlp") is not None:
            fw = sub(tensors, f"l{src}.mlp.", dtype)
            if margins_out is not None and layer["mlp"]["kind"] == "moe":
                margins_out.append(route_margin(r, fw["router"], fw["correction"], layer["mlp"]["router"]))
            f = feed_forward(r, fw, layer["mlp"])
            r = r + zero_centred_norm(f, tensors[f"l{src}.norm2"].to(dtype), eps)
        if layers_out is not None:
            layers_out.append(r.clone())
    return zero_centred_norm(r, tensors["final.norm"].to(dtype), eps) @ table.T
