"""Plain, slow, whole-sequence implementation of the Nedesun decoder.

The oracle of the Nedesun tests.  It shares no code with the ``prelude_b200``
package: it takes the parsed config.json and a ``dict`` of tensors keyed by
their safetensors names, runs a whole sequence at once with no cache, and
returns the logits of every position (and, on request, the residual stream
after every layer).  One function per mechanism; recurrences are explicit loops
over the tokens.

The design, in this file's notation (D = width, t = position from 0, a = residual multiplier):

  norm        n(x; g) = x / sqrt(mean(x^2) + eps) * g
  embedding   r_t = E[token_t] * c
  layer       r <- r + a * mixer(n(r; g1)) ;  r <- r + a * ff(n(r; g2))    (the second only where there is a ff)
  mixers      'attention' (chunked, capped, gated), 'wkv' (decaying matrix state with a bonus for the current
              token), 'parallel' (window attention with kept first tokens and a sink, beside a gated delta rule)
  ff          W_d [ silu(W_g x) * W_u x ]
  output      logits = E n(r; g_final)

All arithmetic is done in ``dtype`` (float64 by default); bfloat16 weights convert exactly.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_norm(x: torch.Tensor, g: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if g is None else y * g


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


# -- which keys a query sees ----------------------------------------------------------------------
def visible(n: int, window: Optional[int] = None, keep_first: int = 0, chunk: Optional[int] = None) -> torch.Tensor:
    """[n, n] booleans: entry (i, j) says whether position i sees position j.  Always j <= i.  With a window, j must
    lie within the last ``window`` positions (i - j < window) or among the first ``keep_first``; with a chunk, i
    and j must lie in the same run of ``chunk`` positions counted from 0."""
    see = torch.zeros(n, n, dtype=torch.bool)
    for i in range(n):
        for j in range(i + 1):
            ok = True
            if window is not None:
                ok = i - j < window or j < keep_first
            if chunk is not None:
                ok = ok and (i // chunk == j // chunk)
            see[i, j] = ok
    return see


# -- rotation -------------------------------------------------------------------------------------
def rotate_half_pairs(x: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, size]: element i of the first ``dims`` is paired with element i + dims / 2; the pair at position
    t turns by t * base^(-2i/dims).  What lies beyond ``dims`` passes unchanged."""
    T = x.shape[0]
    half = dims // 2
    out = x.clone()
    for i in range(half):
        f = base ** (-2.0 * i / dims)
        ang = torch.arange(T, dtype=x.dtype) * f
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        a, b = x[:, :, i], x[:, :, i + half]
        out[:, :, i] = a * c - b * s
        out[:, :, i + half] = b * c + a * s
    return out


# -- softmax attention with the options ----------------------------------------------------------
def softmax_attention(q, k, v, scale: float, see: torch.Tensor, softcap: Optional[float] = None,
                      sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, e] -> [T, H, e].  Head h reads key/value head h // (H / G).  A sink adds
    exp(sink_h) to head h's denominator and nothing to its numerator."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap is not None:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~see, -math.inf)
        if sink is not None:
            s = torch.cat([s, sink[h].expand(T, 1)], dim=1)
        p = torch.softmax(s, dim=-1)
        out[:, h] = p[:, :T] @ v[:, g]
    return out


def chunked_attention(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, shared_v: dict) -> torch.Tensor:
    """Mixer 'attention'.  ``shared_v`` carries the first value-mixing layer's values along the layers."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[f"{p}.q"].T + w[f"{p}.q.b"]).view(T, H, d)
    k = (h @ w[f"{p}.k"].T + w[f"{p}.k.b"]).view(T, G, d)
    v = (h @ w[f"{p}.v"].T + w[f"{p}.v.b"]).view(T, G, e)
    rot = m.get("rot")
    if rot is not None:
        q, k = rotate_half_pairs(q, rot["dims"], rot["base"]), rotate_half_pairs(k, rot["dims"], rot["base"])
    if m.get("v_mix"):
        if "first" not in shared_v:
            shared_v["first"] = v
        else:
            lam = w[f"{p}.vmix"]
            v = (1.0 - lam) * v + lam * shared_v["first"]
    mask = m.get("mask")
    see = visible(T, chunk=mask["size"] if mask else None)
    o = softmax_attention(q, k, v, m["scale"], see, softcap=m.get("softcap"))
    gate = torch.sigmoid(h @ w[f"{p}.g"].T)                      # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * e) @ w[f"{p}.o"].T + w[f"{p}.o.b"]


def window_sink_attention(h, w, p: str, m: dict, eps: float) -> torch.Tensor:
    """Left member of 'parallel': no biases, no rotation, per-head norm of q and k, window with kept first tokens, sink."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm((h @ w[f"{p}.q"].T).view(T, H, d), w[f"{p}.q.norm"], eps)
    k = rms_norm((h @ w[f"{p}.k"].T).view(T, G, d), w[f"{p}.k.norm"], eps)
    v = (h @ w[f"{p}.v"].T).view(T, G, e)
    mask = m.get("mask")
    see = visible(T, window=mask["size"], keep_first=mask.get("keep_first", 0)) if mask else visible(T)
    o = softmax_attention(q, k, v, m["scale"], see, sink=w[f"{p}.sink"])
    return o.reshape(T, H * e) @ w[f"{p}.o"].T


# -- recurrences ----------------------------------------------------------------------------------
def causal_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, n]: y_t = sum_j taps[:, j] * x_(t - (n - 1 - j)), zeros before the start."""
    T, C = x.shape
    n = taps.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(n):
            s = t - (n - 1 - j)
            if s >= 0:
                y[t] += taps[:, j] * x[s]
    return y


def gated_delta_rule(h, w, p: str, m: dict, eps: float) -> torch.Tensor:
    """Right member of 'parallel'."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[f"{p}.q"].T, w[f"{p}.q.conv"])).view(T, G, d)
    k = silu(causal_conv(h @ w[f"{p}.k"].T, w[f"{p}.k.conv"])).view(T, G, d)
    v = silu(causal_conv(h @ w[f"{p}.v"].T, w[f"{p}.v.conv"])).view(T, H, e)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[f"{p}.b"].T)                                        # [T, H]
    decay = torch.exp(-torch.exp(w[f"{p}.A_log"]) * softplus(h @ w[f"{p}.a"].T + w[f"{p}.dt_bias"]))
    gate = silu(h @ w[f"{p}.g"].T).view(T, H, e)
    o = torch.zeros(T, H, e, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(d, e, dtype=h.dtype)
        for t in range(T):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            o[t, hd] = S.T @ q[t, g]
    o = rms_norm(o, w[f"{p}.norm"], eps) * gate
    return o.reshape(T, H * e) @ w[f"{p}.o"].T


def wkv(h, w, p: str, m: dict, eps: float) -> torch.Tensor:
    """Mixer 'wkv'."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)

    def mix(s):
        return h + (prev - h) * w[f"{p}.mu.{s}"]

    r = (mix("r") @ w[f"{p}.r"].T).view(T, H, d)
    k = (mix("k") @ w[f"{p}.k"].T).view(T, H, d)
    v = (mix("v") @ w[f"{p}.v"].T).view(T, H, d)
    gate = silu(mix("g") @ w[f"{p}.g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mix("w") @ w[f"{p}.w1"].T) @ w[f"{p}.w2"].T + w[f"{p}.w0"])).view(T, H, d)
    bonus = w[f"{p}.u"]
    o = torch.zeros(T, H, d, dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros(d, d, dtype=h.dtype)
        for t in range(T):
            kv = torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = (S + bonus[hd][:, None] * kv).T @ r[t, hd]
            S = decay[t, hd][:, None] * S + kv
    o = rms_norm(o, None, eps).reshape(T, H * d) * w[f"{p}.norm"] * gate
    return o @ w[f"{p}.o"].T


def parallel(h, w, p: str, m: dict, eps: float) -> torch.Tensor:
    left = rms_norm(window_sink_attention(h, w, f"{p}.left", m["left"], eps), w[f"{p}.left.out"], eps)
    right = rms_norm(gated_delta_rule(h, w, f"{p}.right", m["right"], eps), w[f"{p}.right.out"], eps)
    return 0.5 * (left + right)


def feed_forward(x, w, p: str) -> torch.Tensor:
    return (silu(x @ w[f"{p}.gate"].T) * (x @ w[f"{p}.up"].T)) @ w[f"{p}.down"].T


# -- the model ------------------------------------------------------------------------------------
def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; ``layers_out`` collects the residual stream after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    a = cfg["residual_mult"]
    r = w["embed"][torch.tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    shared_v: dict = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        h = rms_norm(r, w[f"{p}.norm1"], eps)
        kind = layer["type"]
        if kind == "attention":
            y = chunked_attention(h, w, f"{p}.mix", layer["mixer"], eps, shared_v)
        elif kind == "wkv":
            y = wkv(h, w, f"{p}.mix", layer["mixer"], eps)
        elif kind == "parallel":
            y = parallel(h, w, f"{p}.mix", layer["mixer"], eps)
        else:
            raise ValueError(f"unknown layer type {kind!r}")
        r = r + a * y
        if layer.get("mlp") is not None:
            r = r + a * feed_forward(rms_norm(r, w[f"{p}.norm2"], eps), w, f"{p}.mlp")
        if layers_out is not None:
            layers_out.append(r.clone())
    return rms_norm(r, w["final.norm"], eps) @ w["embed"].T
