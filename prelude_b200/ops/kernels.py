"""Thin tensor wrappers over the C launchers of the kernel library.

Each function checks what the C side cannot see (devices, types, contiguity),
allocates the output with torch, and launches on torch's current stream, so the
calls can be captured in a CUDA graph.  Nothing here computes: if the library
is missing the call raises.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import library as _l
from .library import KernelLibraryError, check

F32, BF16 = 0, 1


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelLibraryError(f"kernels take float32 or bfloat16, not {dtype}")


def _stream() -> int:
    return _l.current_stream_ptr()


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def kv_swizzled(dtype: torch.dtype, head_dim: int) -> bool:
    """Whether key/value pages of this type and head size store the 16-byte chunks
    of a token row permuted (chunk c of token r at position c ^ (r & 7)).  The rule
    is a function of the page tensor alone, so the kernel that writes a page and
    the kernels that read it always agree."""
    return dtype == torch.bfloat16 and head_dim % 64 == 0


def _need(t: torch.Tensor, name: str, dtype=None, contiguous=True) -> None:
    if not t.is_cuda:
        raise KernelLibraryError(f"{name} must live on a CUDA device")
    if dtype is not None and t.dtype != dtype:
        raise KernelLibraryError(f"{name} must be {dtype}, is {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelLibraryError(f"{name} must be contiguous")


def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """res[t, :] = table[ids[t], :] as float32 (the residual stream)."""
    _need(ids, "ids", torch.int32)
    _need(table, "table")
    T, (V, H) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    check(_l.library().pb_embed_gather(ids.data_ptr(), table.data_ptr(), dtype_code(table.dtype), out.data_ptr(),
                                       T, H, V, _stream()), "embed_gather")
    return out


def embed_sinusoid(ids: torch.Tensor, positions: torch.Tensor, table: torch.Tensor, rate: torch.Tensor,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """res[t, 2i] = table[ids[t], 2i] + sin(p_t rate[i]), res[t, 2i+1] = table[ids[t], 2i+1] + cos(p_t rate[i]), float32;
    ``rate`` is float64 [ceil(width / 2)]."""
    _need(ids, "ids", torch.int32)
    _need(positions, "positions", torch.int32)
    _need(table, "table")
    _need(rate, "rate", torch.float64)
    T, (V, H) = ids.numel(), table.shape
    if positions.numel() != T or rate.numel() != (H + 1) // 2:
        raise KernelLibraryError("embed_sinusoid: one position per token and one rate per pair of columns")
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    check(_l.library().pb_embed_sinusoid(ids.data_ptr(), positions.data_ptr(), table.data_ptr(), dtype_code(table.dtype),
                                         rate.data_ptr(), out.data_ptr(), T, H, V, _stream()), "embed_sinusoid")
    return out


class Normed:
    """A sublayer's output that is normed before it joins the residual stream: the value is
    ``x / sqrt(mean(x^2) + eps) * weight`` (weight float32, as applied), not computed yet.  The fused residual
    add takes it as it is and norms, adds and norms again in one pass, in float32."""

    def __init__(self, x: torch.Tensor, weight: torch.Tensor, eps: float):
        self.x, self.weight, self.eps = x, weight, float(eps)

    @property
    def shape(self):
        return self.x.shape


def normed_add_rmsnorm(x: "Normed", res: torch.Tensor, weight: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype,
                       rows: Optional[torch.Tensor] = None, sum_out: bool = False) -> Optional[torch.Tensor]:
    """res += norm(x) (in place, unless ``rows`` picks rows: then res is left alone); returns rmsnorm(res) * weight
    in ``out_dtype`` for every row, or for the chosen ones; with ``weight`` None only the sum is made, and with
    ``sum_out`` it is also returned in ``out_dtype`` (for a sublayer that reads the stream itself)."""
    xt = x.x.materialize(out_dtype) if isinstance(x.x, PartialSums) else x.x
    _need(xt, "x", out_dtype)
    _need(x.weight, "x.weight", torch.float32)
    _need(res, "res", torch.float32)
    total, width = res.shape
    if tuple(xt.shape) != tuple(res.shape) or x.weight.numel() != width:
        raise KernelLibraryError(f"normed_add_rmsnorm: x {tuple(xt.shape)} against residual {tuple(res.shape)}")
    out = None
    n_out = total
    if rows is not None:
        _need(rows, "rows", torch.int32)
        n_out = rows.numel()
        if weight is None:
            raise KernelLibraryError("normed_add_rmsnorm: chosen rows need the norm that follows")
    if weight is not None:
        _need(weight, "weight", torch.float32)
    if weight is not None or sum_out:
        out = torch.empty((n_out, width), dtype=out_dtype, device=res.device)
    check(_l.library().pb_normed_add_rmsnorm(xt.data_ptr(), x.weight.data_ptr(), x.eps, res.data_ptr(), _ptr(rows), n_out, total,
                                             _ptr(weight), _ptr(out), dtype_code(out_dtype), width, float(eps), _stream()),
          "normed_add_rmsnorm")
    return out


class PartialSums:
    """The output of a product whose K was cut into parts: ``parts`` is float32
    [n, rows, width] and the value is their sum.  The residual add takes it as
    it is and adds the parts up in float32; anyone else calls ``materialize``."""

    def __init__(self, parts: torch.Tensor):
        if parts.dim() != 3 or parts.dtype != torch.float32 or not parts.is_contiguous():
            raise KernelLibraryError("PartialSums: a dense float32 [parts, rows, width] tensor is needed")
        self.parts = parts

    @property
    def shape(self):
        return self.parts.shape[1:]

    def materialize(self, dtype: torch.dtype) -> torch.Tensor:
        return self.parts.sum(dim=0).to(dtype)


def clamped_glu(gate_up: torch.Tensor, limit: float, alpha: float) -> torch.Tensor:
    """[T, 2I] (gate columns first) -> a sigmoid(alpha a) (b + 1), a = min(gate, limit), b = clamp(up, -limit, limit); [T, I]."""
    _need(gate_up, "gate_up")
    T, two_i = gate_up.shape
    if two_i % 2:
        raise KernelLibraryError("clamped_glu: merged projection must have an even number of columns")
    out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    check(_l.library().pb_clamped_glu(gate_up.data_ptr(), out.data_ptr(), dtype_code(gate_up.dtype), T, two_i // 2,
                                      float(limit), float(alpha), _stream()), "clamped_glu")
    return out


def _x_args(x, out_dtype: torch.dtype, what: str):
    """(pointer, parts, stride) of the addend of a fused add: a tensor of the run's type, partial sums, or nothing."""
    if x is None:
        return None, 0, 0
    if isinstance(x, PartialSums):
        _need(x.parts, what)
        return x.parts.data_ptr(), x.parts.shape[0], x.parts.stride(0)
    _need(x, what, out_dtype)
    return x.data_ptr(), 0, 0


def add_rmsnorm(x, res: torch.Tensor, weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """res += x (when x is given: a tensor of ``out_dtype`` or ``PartialSums``); returns
    rmsnorm(res) * weight in ``out_dtype``."""
    _need(res, "res", torch.float32)
    _need(weight, "weight", torch.float32)
    rows, width = res.shape
    if x is not None and tuple(x.shape) != tuple(res.shape):
        raise KernelLibraryError(f"add_rmsnorm: x {tuple(x.shape)} against residual {tuple(res.shape)}")
    if weight.numel() != width:
        raise KernelLibraryError(f"add_rmsnorm: weight has {weight.numel()} elements, rows have {width}")
    ptr, parts, stride = _x_args(x, out_dtype, "x")
    if out is None:
        out = torch.empty((rows, width), dtype=out_dtype, device=res.device)
    check(_l.library().pb_add_rmsnorm(ptr, parts, stride, res.data_ptr(), weight.data_ptr(), out.data_ptr(),
                                      dtype_code(out_dtype), rows, width, float(eps), _stream()), "add_rmsnorm")
    return out


def gather_add_rmsnorm(x, res: torch.Tensor, rows: torch.Tensor, weight: torch.Tensor,
                       eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """rmsnorm(res[rows] + x[rows]) * weight for the chosen rows; res is not changed."""
    _need(res, "res", torch.float32)
    _need(rows, "rows", torch.int32)
    _need(weight, "weight", torch.float32)
    if x is not None and tuple(x.shape) != tuple(res.shape):
        raise KernelLibraryError(f"gather_add_rmsnorm: x {tuple(x.shape)} against residual {tuple(res.shape)}")
    ptr, parts, stride = _x_args(x, out_dtype, "x")
    total, width = res.shape
    out = torch.empty((rows.numel(), width), dtype=out_dtype, device=res.device)
    check(_l.library().pb_gather_add_rmsnorm(ptr, parts, stride, res.data_ptr(), rows.data_ptr(), weight.data_ptr(),
                                             out.data_ptr(), dtype_code(out_dtype), rows.numel(), total, width,
                                             float(eps), _stream()), "gather_add_rmsnorm")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    _need(x, "x")
    _need(weight, "weight", torch.float32)
    width = x.shape[-1]
    rows = x.numel() // width
    if weight.numel() != width:
        raise KernelLibraryError(f"rmsnorm: weight has {weight.numel()} elements, rows have {width}")
    out = torch.empty_like(x)
    check(_l.library().pb_rmsnorm(x.data_ptr(), weight.data_ptr(), out.data_ptr(), dtype_code(x.dtype), rows, width,
                                  float(eps), _stream()), "rmsnorm")
    return out


def qknorm_rope_kvwrite(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                        q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                        cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int,
                        positions: torch.Tensor, token_seq: Optional[torch.Tensor],
                        block_table: Optional[torch.Tensor], k_pages: Optional[torch.Tensor],
                        v_pages: Optional[torch.Tensor], write_kv: bool,
                        status: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                        interleaved: bool = False) -> torch.Tensor:
    """q/k norm + rotation, q to a dense [T, nH, D] tensor (``out`` if given), k and v into their pages.
    Angle j turns the pair (j, j + rotary_dim / 2), or with ``interleaved`` the pair (2 j, 2 j + 1).

    ``qkv`` is the merged projection [T, (nH + 2 nKV) D] (or [T, nH D] when
    nothing is written).  Pages are [num_pages, nKV, page_size, D].
    """
    _need(qkv, "qkv", contiguous=False)
    if qkv.dim() != 2 or qkv.stride(1) != 1:
        raise KernelLibraryError("qknorm_rope_kvwrite: the projection must be [tokens, columns] with dense rows")
    T = qkv.shape[0]
    q_cols, kv_cols = n_heads * head_dim, n_kv_heads * head_dim
    want = q_cols + (2 * kv_cols if write_kv else 0)
    if qkv.shape[1] < want:
        raise KernelLibraryError(f"qknorm_rope_kvwrite: projection has {qkv.shape[1]} columns, needs {want}")
    esz = qkv.element_size()
    base = qkv.data_ptr()
    if out is None:
        q_out = torch.empty((T, n_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    else:
        _need(out, "out", qkv.dtype)
        if tuple(out.shape) != (T, n_heads, head_dim):
            raise KernelLibraryError(f"qknorm_rope_kvwrite: out is {tuple(out.shape)}, q is {(T, n_heads, head_dim)}")
        q_out = out
    max_pos, page_size, num_pages, stride = 0, 0, 0, 0
    if cos is not None:
        _need(cos, "cos", torch.float32)
        _need(sin, "sin", torch.float32)
        max_pos = cos.shape[0]
        if cos.shape[1] * 2 != rotary_dim:
            raise KernelLibraryError("qknorm_rope_kvwrite: table width does not match rotary_dim")
    if write_kv:
        _need(k_pages, "k_pages", qkv.dtype)
        _need(v_pages, "v_pages", qkv.dtype)
        _need(block_table, "block_table", torch.int32)
        _need(token_seq, "token_seq", torch.int32)
        num_pages, page_size = k_pages.shape[0], k_pages.shape[2]
        if (k_pages.shape[1], k_pages.shape[3]) != (n_kv_heads, head_dim) or k_pages.shape != v_pages.shape:
            raise KernelLibraryError(f"qknorm_rope_kvwrite: pages {tuple(k_pages.shape)} do not fit "
                                     f"{n_kv_heads} heads of {head_dim}")
        stride = block_table.shape[1]
    for w, n in ((q_weight, "q_weight"), (k_weight, "k_weight")):
        if w is not None:
            _need(w, n, torch.float32)
            if w.numel() != head_dim:
                raise KernelLibraryError(f"qknorm_rope_kvwrite: {n} has {w.numel()} elements, heads have {head_dim}")
    _need(positions, "positions", torch.int32)
    check(_l.library().pb_qknorm_rope_kvwrite(
        base, base + q_cols * esz, base + (q_cols + kv_cols) * esz, qkv.stride(0), q_out.data_ptr(),
        _ptr(k_pages) if write_kv else None, _ptr(v_pages) if write_kv else None, dtype_code(qkv.dtype),
        _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(cos), _ptr(sin), rotary_dim if cos is not None else 0,
        1 if interleaved else 0, max_pos, positions.data_ptr(), _ptr(token_seq), _ptr(block_table), stride, page_size, num_pages, T, n_heads,
        n_kv_heads, head_dim, 1 if write_kv else 0, 1 if (write_kv and kv_swizzled(qkv.dtype, head_dim)) else 0,
        _ptr(status), _stream()), "qknorm_rope_kvwrite")
    return q_out


def paged_attention_ref(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, positions: torch.Tensor,
                        token_seq: torch.Tensor, block_table: torch.Tensor, scale: float,
                        window: Optional[int] = None, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Plain paged attention, q [T, nH, D] -> [T, nH, D]."""
    _need(q, "q")
    _need(k_pages, "k_pages", q.dtype)
    _need(v_pages, "v_pages", q.dtype)
    _need(positions, "positions", torch.int32)
    _need(token_seq, "token_seq", torch.int32)
    _need(block_table, "block_table", torch.int32)
    T, nH, D = q.shape
    num_pages, nKV, page_size, Dk = k_pages.shape
    if Dk != D or v_pages.shape != k_pages.shape:
        raise KernelLibraryError("paged_attention_ref: q and pages disagree on the head size")
    out = torch.empty_like(q)
    check(_l.library().pb_paged_attention_ref(
        q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(), dtype_code(q.dtype),
        positions.data_ptr(), token_seq.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size,
        num_pages, T, nH, nKV, D, float(scale), int(window) if window else 0, 1 if kv_swizzled(q.dtype, D) else 0,
        _ptr(status), _stream()), "paged_attention_ref")
    return out


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """[T, 2I] (gate columns first) -> silu(gate) * up, [T, I]."""
    _need(gate_up, "gate_up")
    T, two_i = gate_up.shape
    if two_i % 2:
        raise KernelLibraryError("silu_mul: merged projection must have an even number of columns")
    out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    check(_l.library().pb_silu_mul(gate_up.data_ptr(), out.data_ptr(), dtype_code(gate_up.dtype), T, two_i // 2,
                                   _stream()), "silu_mul")
    return out


def gelu_tanh_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """gelu(gate) * up, the tanh form of GELU, on a merged projection [T, 2 I] -> [T, I]."""
    _need(gate_up, "gate_up")
    T, two_i = gate_up.shape
    if two_i % 2:
        raise KernelLibraryError("gelu_tanh_mul: the merged projection has an even number of columns")
    out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    check(_l.library().pb_gelu_tanh_mul(gate_up.data_ptr(), out.data_ptr(), dtype_code(gate_up.dtype), T, two_i // 2, _stream()),
          "gelu_tanh_mul")
    return out


def gemm_ref(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
             out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a [M, K] times w [N, K] transposed (+ bias) on the float32 units."""
    _need(a, "a", contiguous=False)
    _need(w, "w", a.dtype, contiguous=False)
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1]:
        raise KernelLibraryError(f"gemm: a {tuple(a.shape)} against w {tuple(w.shape)}")
    if a.stride(1) != 1 or w.stride(1) != 1:
        raise KernelLibraryError("gemm: rows must be dense")
    M, K = a.shape
    N = w.shape[0]
    out_dtype = out_dtype or a.dtype
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != N:
            raise KernelLibraryError(f"gemm: bias has {bias.numel()} elements, output has {N} columns")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    check(_l.library().pb_gemm_ref(a.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), dtype_code(a.dtype),
                                   dtype_code(out_dtype), M, N, K, a.stride(0), w.stride(0), out.stride(0), _stream()),
          "gemm_ref")
    return out


def argmax(logits: torch.Tensor) -> torch.Tensor:
    """Row-wise argmax of float32 logits, ties to the smaller index; int32 [rows]."""
    _need(logits, "logits", torch.float32, contiguous=False)
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelLibraryError("argmax: logits must be [rows, vocab] with dense rows")
    rows, vocab = logits.shape
    out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    lib = _l.library()
    scratch = torch.empty(max(1, lib.pb_sample_scratch_floats(rows, vocab)), dtype=torch.float32, device=logits.device)
    check(lib.pb_argmax(logits.data_ptr(), logits.stride(0), rows, vocab, out.data_ptr(), scratch.data_ptr(), _stream()),
          "argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, seeds: torch.Tensor, counters: torch.Tensor,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row: greedy where temperature < 1e-7, else a Philox draw from softmax(logits / T).
    The tokens go to ``out`` (int32 [rows]) when given."""
    _need(logits, "logits", torch.float32, contiguous=False)
    _need(temperature, "temperature", torch.float32)
    _need(seeds, "seeds", torch.int64)
    _need(counters, "counters", torch.int64)
    rows, vocab = logits.shape
    if not (temperature.numel() == seeds.numel() == counters.numel() == rows):
        raise KernelLibraryError("sample: one temperature, seed and counter per row")
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    else:
        _need(out, "out", torch.int32)
        if out.numel() != rows:
            raise KernelLibraryError("sample: out holds one token per row")
    lib = _l.library()
    scratch = torch.empty(max(1, lib.pb_sample_scratch_floats(rows, vocab)), dtype=torch.float32, device=logits.device)
    check(lib.pb_sample(logits.data_ptr(), logits.stride(0), rows, vocab, temperature.data_ptr(), seeds.data_ptr(),
                        counters.data_ptr(), out.data_ptr(), scratch.data_ptr(), _stream()), "sample")
    return out


def softmax_temperature(logits: torch.Tensor, temperature: torch.Tensor) -> torch.Tensor:
    _need(logits, "logits", torch.float32, contiguous=False)
    _need(temperature, "temperature", torch.float32)
    rows, vocab = logits.shape
    out = torch.empty((rows, vocab), dtype=torch.float32, device=logits.device)
    check(_l.library().pb_softmax_temperature(logits.data_ptr(), logits.stride(0), rows, vocab,
                                              temperature.data_ptr(), out.data_ptr(), _stream()), "softmax_temperature")
    return out


def philox_uniform(seed: int, counter: int) -> float:
    """The uniform number in [0, 1) the sampler draws for (seed, counter); host-side, for tests."""
    return float(_l.library().pb_philox_uniform(seed & (2**64 - 1), counter & (2**64 - 1)))


def scatter_i32(dst: torch.Tensor, idx: torch.Tensor, val: torch.Tensor, status: Optional[torch.Tensor] = None) -> None:
    """dst.view(-1)[idx[i]] = val[i] on the device (block-table updates before a captured step)."""
    _need(dst, "dst", torch.int32)
    _need(idx, "idx", torch.int32)
    _need(val, "val", torch.int32)
    if idx.numel() != val.numel():
        raise KernelLibraryError("scatter_i32: one value per index")
    check(_l.library().pb_scatter_i32(dst.data_ptr(), dst.numel(), idx.data_ptr(), val.data_ptr(), idx.numel(),
                                      _ptr(status), _stream()), "scatter_i32")


def decode_advance(tokens: torch.Tensor, positions: torch.Tensor, kv_len: Optional[torch.Tensor],
                   counters: Optional[torch.Tensor], sampled: torch.Tensor, max_positions: int) -> None:
    """tokens = sampled; positions += 1; kv_len = positions + 1; counters += 1: a decode step that feeds itself."""
    _need(tokens, "tokens", torch.int32)
    _need(positions, "positions", torch.int32)
    _need(sampled, "sampled", torch.int32)
    if kv_len is not None:
        _need(kv_len, "kv_len", torch.int32)
    if counters is not None:
        _need(counters, "counters", torch.int64)
    check(_l.library().pb_decode_advance(tokens.data_ptr(), positions.data_ptr(), _ptr(kv_len), _ptr(counters),
                                         sampled.data_ptr(), tokens.numel(), int(max_positions), _stream()), "decode_advance")


def _cols(t: torch.Tensor, name: str) -> None:
    _need(t, name, contiguous=False)
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelLibraryError(f"{name} must be [tokens, columns] with dense rows")


def kv_write_pages(k: torch.Tensor, v: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, positions: torch.Tensor,
                   token_row: torch.Tensor, block_table: torch.Tensor, status: Optional[torch.Tensor] = None) -> None:
    """A step's keys [T, key heads * dk] and values [T, value heads * dv] (columns of a projection) into their
    pages [pages, heads, page_size, d]: key and value heads may differ in number and size."""
    _cols(k, "k")
    _cols(v, "v")
    _need(k_pages, "k_pages", k.dtype)
    _need(v_pages, "v_pages", k.dtype)
    _need(positions, "positions", torch.int32)
    _need(token_row, "token_row", torch.int32)
    _need(block_table, "block_table", torch.int32)
    T = k.shape[0]
    num_pages, nk, page_size, dk = k_pages.shape
    _, nv, _, dv = v_pages.shape
    if k.shape[1] != nk * dk or v.shape != (T, nv * dv) or v_pages.shape[0] != num_pages or v_pages.shape[2] != page_size:
        raise KernelLibraryError(f"kv_write_pages: keys {tuple(k.shape)}, values {tuple(v.shape)} do not fit pages "
                                 f"{tuple(k_pages.shape)}, {tuple(v_pages.shape)}")
    check(_l.library().pb_kv_write_pages(
        k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), k_pages.data_ptr(), v_pages.data_ptr(), dtype_code(k.dtype),
        positions.data_ptr(), token_row.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size, num_pages, T,
        nk, dk, nv, dv, 1 if kv_swizzled(k.dtype, dk) else 0, 1 if kv_swizzled(k.dtype, dv) else 0, _ptr(status), _stream()),
        "kv_write_pages")


def diff_attention_ref(q: torch.Tensor, gate: Optional[torch.Tensor], k_pages: torch.Tensor, v_pages: torch.Tensor,
                       positions: torch.Tensor, token_row: torch.Tensor, block_table: torch.Tensor, n_heads: int,
                       scale: float, temp_coef: float, temp_every: int, lam: float, norm_eps: float, out_scale: float,
                       window: Optional[int] = None, status: Optional[torch.Tensor] = None,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Plain differential attention: q [T, heads * 2 * dim] and gate [T, heads * vdim] (columns of a projection, gate
    may be None) against keys [pages, 2 * kv heads, page_size, dim] and values [pages, kv heads, page_size, vdim];
    returns [T, heads, vdim]: (map 0 - lam * map 1) at unit root mean square, times out_scale, times sigmoid(gate)."""
    _cols(q, "q")
    _need(k_pages, "k_pages", q.dtype)
    _need(v_pages, "v_pages", q.dtype)
    _need(positions, "positions", torch.int32)
    _need(token_row, "token_row", torch.int32)
    _need(block_table, "block_table", torch.int32)
    T = q.shape[0]
    num_pages, nk, page_size, dim = k_pages.shape
    _, n_kv, _, vdim = v_pages.shape
    if nk != 2 * n_kv or q.shape[1] != n_heads * 2 * dim or n_heads % n_kv:
        raise KernelLibraryError(f"diff_attention: q {tuple(q.shape)} with {n_heads} heads does not fit keys {tuple(k_pages.shape)} "
                                 f"and values {tuple(v_pages.shape)}")
    if gate is not None:
        _cols(gate, "gate")
        if gate.dtype != q.dtype or tuple(gate.shape) != (T, n_heads * vdim):
            raise KernelLibraryError(f"diff_attention: gate {tuple(gate.shape)} is not [tokens, heads * vdim]")
    if out is None:
        out = torch.empty((T, n_heads, vdim), dtype=q.dtype, device=q.device)
    check(_l.library().pb_diff_attention_ref(
        q.data_ptr(), q.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0, k_pages.data_ptr(), v_pages.data_ptr(),
        out.data_ptr(), dtype_code(q.dtype), positions.data_ptr(), token_row.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], page_size, num_pages, T, n_heads, n_kv, dim, vdim, float(scale), float(temp_coef), int(temp_every),
        float(lam), float(norm_eps), float(out_scale), int(window) if window else 0, 1 if kv_swizzled(q.dtype, dim) else 0,
        1 if kv_swizzled(q.dtype, vdim) else 0, _ptr(status), _stream()), "diff_attention_ref")
    return out


def router_logits(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [T, K] times w [E, K] transposed as float32 [T, E]: exact products, float32 sums in an order that depends on K alone."""
    _cols(x, "x")
    _need(w, "w", x.dtype)
    T, Kdim = x.shape
    if w.dim() != 2 or w.shape[1] != Kdim:
        raise KernelLibraryError(f"router_logits: x {tuple(x.shape)} against w {tuple(w.shape)}")
    out = torch.empty((T, w.shape[0]), dtype=torch.float32, device=x.device)
    check(_l.library().pb_router_logits(x.data_ptr(), x.stride(0), w.data_ptr(), out.data_ptr(), dtype_code(x.dtype), T, w.shape[0],
                                        Kdim, _stream()), "router_logits")
    return out


def moe_route(logits: torch.Tensor, top: int, groups: int, keep: int, group_top: int, renormalize: bool,
              correction: Optional[torch.Tensor] = None):
    """float32 router logits [T, E] -> (experts int32 [T, top], weights float32 [T, top]).  ``correction`` float32 [E]
    joins the scores for the choice (groups and experts) only; the weights are the scores without it."""
    _need(logits, "logits", torch.float32)
    T, E = logits.shape
    if correction is not None:
        _need(correction, "correction", torch.float32)
        if correction.numel() != E:
            raise KernelLibraryError(f"moe_route: a correction of {correction.numel()} numbers for {E} experts")
    ids = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    check(_l.library().pb_moe_route(logits.data_ptr(), _ptr(correction), T, E, top, groups, keep, group_top, 1 if renormalize else 0,
                                    ids.data_ptr(), weights.data_ptr(), _stream()), "moe_route")
    return ids, weights


class MoePlan:
    """Where a step's (token, choice) slots sit once grouped by expert; all on the device."""

    def __init__(self, offsets, order, place_of, tile_expert, tile_row0, max_tiles, tile_rows):
        self.offsets, self.order, self.place_of = offsets, order, place_of
        self.tile_expert, self.tile_row0, self.max_tiles, self.tile_rows = tile_expert, tile_row0, max_tiles, tile_rows


def moe_sort(ids: torch.Tensor, n_experts: int, tile_rows: Optional[int] = None) -> MoePlan:
    """Group the slots by expert.  ``tile_rows`` (64 or 128; default: the library's choice by rows per expert) is the
    height of the row tiles the products then run on."""
    _need(ids, "ids", torch.int32)
    n_slots = ids.numel()
    lib = _l.library()
    tile_rows = tile_rows or lib.pb_moe_tile_rows(n_slots, n_experts)
    max_tiles = -(-n_slots // tile_rows) + n_experts
    ints = torch.empty(n_experts + 1 + 2 * n_slots + 2 * max_tiles, dtype=torch.int32, device=ids.device)
    o = [0, n_experts + 1, n_experts + 1 + n_slots, n_experts + 1 + 2 * n_slots, n_experts + 1 + 2 * n_slots + max_tiles]
    plan = MoePlan(ints[o[0]:o[1]], ints[o[1]:o[2]], ints[o[2]:o[3]], ints[o[3]:o[4]], ints[o[4]:], max_tiles, tile_rows)
    check(lib.pb_moe_sort(ids.data_ptr(), n_slots, n_experts, plan.offsets.data_ptr(), plan.order.data_ptr(),
                          plan.place_of.data_ptr(), plan.tile_expert.data_ptr(), plan.tile_row0.data_ptr(), max_tiles, tile_rows, _stream()),
          "moe_sort")
    return plan


def moe_gemm(a: torch.Tensor, w: torch.Tensor, plan: MoePlan, gated: bool, gather_div: int = 0,
             out_dtype: Optional[torch.dtype] = None, few_rows: bool = False) -> torch.Tensor:
    """The experts' products over the plan's places.  a [rows, K]; w [E, N (2 N when gated: gate rows, then up rows), K];
    row of place p is ``order[p] // gather_div`` (the token of a slot) or, with gather_div 0, p itself.  Returns
    [places, N]: a W_e^T, or silu(a Wg_e^T) * (a Wu_e^T).  ``few_rows``: the experts have a row or a few each (a decode
    step): the kernel that only streams the weights, where it takes the operands (bfloat16, K in multiples of 8)."""
    _cols(a, "a")
    _need(w, "w", a.dtype)
    E, rows_w, Kdim = w.shape
    if a.shape[1] != Kdim or (gated and rows_w % 2):
        raise KernelLibraryError(f"moe_gemm: a {tuple(a.shape)} against w {tuple(w.shape)}")
    N = rows_w // 2 if gated else rows_w
    out_dtype = out_dtype or a.dtype
    if plan.tile_rows != 64 and (a.dtype != torch.bfloat16 or Kdim % 8 or a.stride(0) % 8 or a.data_ptr() % 16):
        raise KernelLibraryError("moe_gemm: a plan of 128-row tiles is for bfloat16 operands with K in multiples of 8")
    places = plan.order.numel()
    out = torch.empty((places, N), dtype=out_dtype, device=a.device)
    if (few_rows and plan.tile_rows == 64 and a.dtype == torch.bfloat16 and Kdim % 8 == 0 and a.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
        check(_l.library().pb_moe_gemv(a.data_ptr(), a.stride(0), plan.order.data_ptr() if gather_div else None, max(1, gather_div),
                                       w.data_ptr(), w.stride(0), N, Kdim, 1 if gated else 0, plan.tile_expert.data_ptr(),
                                       plan.tile_row0.data_ptr(), plan.offsets.data_ptr(), plan.max_tiles, out.data_ptr(), out.stride(0),
                                       dtype_code(out_dtype), _stream()), "moe_gemv")
        return out
    check(_l.library().pb_moe_gemm(a.data_ptr(), a.stride(0), plan.order.data_ptr() if gather_div else None, max(1, gather_div),
                                   w.data_ptr(), w.stride(0), N, Kdim, 1 if gated else 0, plan.tile_expert.data_ptr(),
                                   plan.tile_row0.data_ptr(), plan.offsets.data_ptr(), plan.max_tiles, plan.tile_rows, out.data_ptr(), out.stride(0),
                                   dtype_code(a.dtype), dtype_code(out_dtype), _stream()), "moe_gemm")
    return out


def moe_gather_rows(x: torch.Tensor, plan: MoePlan, div: int) -> torch.Tensor:
    """The rows of x in the order of the plan's places: out[place] = x[order[place] // div]."""
    _cols(x, "x")
    places = plan.order.numel()
    out = torch.empty((places, x.shape[1]), dtype=x.dtype, device=x.device)
    check(_l.library().pb_moe_gather_rows(x.data_ptr(), x.stride(0), plan.order.data_ptr(), int(div), out.data_ptr(),
                                          dtype_code(x.dtype), places, x.shape[1], _stream()), "moe_gather_rows")
    return out


def moe_gemm_pair(a_sorted: torch.Tensor, w: torch.Tensor, plan: MoePlan, gated: bool, status: torch.Tensor,
                  max_pairs: int = 0) -> torch.Tensor:
    """The experts' products on the paired-block tcgen05 kernel: a_sorted [places, K] bfloat16 holds the rows in the
    order of their places (``moe_gather_rows``), the plan has row tiles of 256; w as for ``moe_gemm``.  bfloat16 out."""
    _need(a_sorted, "a_sorted", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    E, rows_w, Kdim = w.shape
    if plan.tile_rows != 256 or a_sorted.shape != (plan.order.numel(), Kdim) or (gated and rows_w % 2):
        raise KernelLibraryError("moe_gemm_pair: a plan of 256-row tiles and rows sorted by place are needed")
    N = rows_w // 2 if gated else rows_w
    out = torch.empty((a_sorted.shape[0], N), dtype=torch.bfloat16, device=a_sorted.device)
    check(_l.library().pb_gemm_pair_grouped_bf16(
        a_sorted.data_ptr(), w.data_ptr(), out.data_ptr(), a_sorted.shape[0], rows_w, E, Kdim, a_sorted.stride(0), Kdim,
        out.stride(0), 1 if gated else 0, plan.tile_expert.data_ptr(), plan.tile_row0.data_ptr(), plan.offsets.data_ptr(),
        plan.max_tiles, max_pairs, status.data_ptr(), _stream()), "gemm_pair (grouped)")
    return out


def moe_combine(y: torch.Tensor, plan: MoePlan, weights: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """out[t] = sum_c weights[t, c] * y[place of slot (t, c)], float32 sums; y [places, width] float32 or of out_dtype."""
    _need(y, "y")
    if y.dtype not in (torch.float32, out_dtype):
        raise KernelLibraryError("moe_combine: y is float32 or of the output's type")
    _need(weights, "weights", torch.float32)
    T, top = weights.shape
    out = torch.empty((T, y.shape[1]), dtype=out_dtype, device=y.device)
    check(_l.library().pb_moe_combine(y.data_ptr(), dtype_code(y.dtype), plan.place_of.data_ptr(), weights.data_ptr(), out.data_ptr(),
                                      dtype_code(out_dtype), T, top, y.shape[1], _stream()), "moe_combine")
    return out


# -- mixers whose norm spans more than a head, rotation by rates, general paged attention ---------------------------
def gemm_ref_batched(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[b] = a[b] w[b]^T on the float32 units for a [B, M, K], w [B, N, K], out [B, M, N], each given as a view with
    dense rows (the products' operands may interleave: a [tokens, heads, size] tensor seen heads first)."""
    for t, name in ((a, "a"), (w, "w"), (out, "out")):
        _need(t, name, contiguous=False)
        if t.dim() != 3 or t.stride(2) != 1:
            raise KernelLibraryError(f"gemm_ref_batched: {name} must be [batch, rows, cols] with dense rows")
    B, M, Kd = a.shape
    N = w.shape[1]
    if w.shape != (B, N, Kd) or out.shape != (B, M, N) or w.dtype != a.dtype:
        raise KernelLibraryError(f"gemm_ref_batched: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    check(_l.library().pb_gemm_ref_batched(a.data_ptr(), w.data_ptr(), out.data_ptr(), dtype_code(a.dtype), dtype_code(out.dtype),
                                           M, N, Kd, a.stride(1), w.stride(1), out.stride(1), B, a.stride(0), w.stride(0),
                                           out.stride(0), _stream()), "gemm_ref_batched")
    return out


def qkv_prepare(q_in: torch.Tensor, k_in: Optional[torch.Tensor], v_in: Optional[torch.Tensor], *, n_heads: int, q_dim: int,
                q_weight: Optional[torch.Tensor] = None, k_weight: Optional[torch.Tensor] = None, k_norm_cols: int = 0,
                eps: float = 0.0, rates: Optional[torch.Tensor] = None, rot_dims: int = 0, adjacent: bool = False,
                amplitude: float = 1.0, q_rot_off: int = 0, k_rot_off: int = 0, positions: torch.Tensor,
                table_row: torch.Tensor, block_table: Optional[torch.Tensor] = None, q_out: torch.Tensor,
                q_split: Optional[int] = None, q_out2: Optional[torch.Tensor] = None, q2_off: int = 0,
                k_pages: Optional[torch.Tensor] = None, v_pages: Optional[torch.Tensor] = None, swizzle_k: bool = False,
                swizzle_v: bool = False, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Norm over whole projections, rotation by rates, queries to ``q_out`` (and their second part to ``q_out2``),
    keys and values into pages; see csrc/qkv_prepare.cu.  ``q_in``, ``k_in``, ``v_in`` are [T, cols] views with dense
    rows (columns of one merged projection); ``k_pages`` None: nothing is cached."""
    T = q_in.shape[0]
    dt = q_in.dtype
    for t, name in ((q_in, "q_in"), (k_in, "k_in"), (v_in, "v_in")):
        if t is not None:
            _need(t, name, dt, contiguous=False)
            if t.dim() != 2 or t.stride(1) != 1 or t.shape[0] != T:
                raise KernelLibraryError(f"qkv_prepare: {name} must be [tokens, cols] with dense rows")
    for t, name in ((q_weight, "q_weight"), (k_weight, "k_weight"), (rates, "rates")):
        if t is not None:
            _need(t, name, torch.float32)
    _need(positions, "positions", torch.int32)
    _need(table_row, "table_row", torch.int32)
    q_split = q_dim if q_split is None else q_split
    _need(q_out, "q_out", dt)
    if q_in.shape[1] != n_heads * q_dim or q_out.numel() != T * n_heads * q_split:
        raise KernelLibraryError(f"qkv_prepare: q_in {tuple(q_in.shape)}, q_out {tuple(q_out.shape)} for {n_heads} heads of {q_dim}")
    if q_weight is not None and q_weight.numel() != n_heads * q_dim:
        raise KernelLibraryError("qkv_prepare: the query norm's scale covers the whole projection")
    if rates is not None and rates.numel() * 2 != rot_dims:
        raise KernelLibraryError("qkv_prepare: one rate per rotated pair")
    q2_stride = 0
    if q_split < q_dim:
        _need(q_out2, "q_out2", dt)
        if q_out2.dim() != 3 or q_out2.shape[:2] != (T, n_heads) or q2_off + (q_dim - q_split) > q_out2.shape[2]:
            raise KernelLibraryError(f"qkv_prepare: q_out2 {tuple(q_out2.shape)} has no room for {q_dim - q_split} elements from {q2_off}")
        q2_stride = q_out2.shape[2]
    G = kd = Gv = vd = page_size = num_pages = stride = 0
    if k_pages is not None:
        _need(k_pages, "k_pages", dt)
        _need(block_table, "block_table", torch.int32)
        num_pages, G, page_size, kd = k_pages.shape
        stride = block_table.shape[1]
        if k_in is None or k_in.shape[1] != G * kd:
            raise KernelLibraryError(f"qkv_prepare: keys {None if k_in is None else tuple(k_in.shape)} against pages {tuple(k_pages.shape)}")
        if k_weight is not None and k_weight.numel() < k_norm_cols:
            raise KernelLibraryError("qkv_prepare: the key norm's scale is shorter than the columns it covers")
        if v_pages is not None and v_pages.numel() > 0:
            _need(v_pages, "v_pages", dt)
            _, Gv, _, vd = v_pages.shape
            if v_in is None or v_in.shape[1] != Gv * vd or v_pages.shape[0] != num_pages or v_pages.shape[2] != page_size:
                raise KernelLibraryError(f"qkv_prepare: values against pages {tuple(v_pages.shape)}")
        else:
            v_pages = None
    check(_l.library().pb_qkv_prepare(
        q_in.data_ptr(), q_in.stride(0), _ptr(k_in), 0 if k_in is None else k_in.stride(0), _ptr(v_in),
        0 if v_in is None else v_in.stride(0), dtype_code(dt), _ptr(q_weight), _ptr(k_weight), int(k_norm_cols), float(eps),
        _ptr(rates), int(rot_dims), 1 if adjacent else 0, float(amplitude), int(q_rot_off), int(k_rot_off), positions.data_ptr(),
        table_row.data_ptr(), _ptr(block_table), stride, page_size, num_pages, q_out.data_ptr(), q_split, _ptr(q_out2), q2_stride,
        int(q2_off), _ptr(k_pages), _ptr(v_pages), T, n_heads, q_dim, G, kd, Gv, vd, 1 if swizzle_k else 0, 1 if swizzle_v else 0,
        _ptr(status), _stream()), "qkv_prepare")
    return q_out


def attention_paged(q: torch.Tensor, k_pages: torch.Tensor, v_pages: Optional[torch.Tensor], value_dim: int, positions: torch.Tensor,
                    table_row: torch.Tensor, block_table: torch.Tensor, scale: float, window: Optional[int] = None,
                    sink: Optional[torch.Tensor] = None, swizzle_k: bool = False, swizzle_v: bool = False,
                    status: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, keep_first: int = 0,
                    chunk: Optional[int] = None, softcap: Optional[float] = None, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, H, kd] against pages [P, G, page, kd]; values from ``v_pages`` [P, Gv, page, value_dim], or, with
    ``v_pages`` None, the first ``value_dim`` elements of the key rows.  ``keep_first``: positions below it stay visible
    behind the window; ``chunk``: keys of the query's own run of positions only; ``softcap``: scores capped by tanh;
    ``gate`` [T, H] (a view with dense rows): its sigmoid multiplies the head's output.  float32 arithmetic; see
    csrc/attention_paged.cu."""
    _need(q, "q")
    _need(k_pages, "k_pages", q.dtype)
    _need(positions, "positions", torch.int32)
    _need(table_row, "table_row", torch.int32)
    _need(block_table, "block_table", torch.int32)
    T, H, kd = q.shape
    num_pages, G, page_size, kd2 = k_pages.shape
    if kd2 != kd:
        raise KernelLibraryError(f"attention_paged: queries of {kd}, keys of {kd2}")
    if v_pages is None:
        vp, Gv, v_row = k_pages, G, kd
        if value_dim > kd:
            raise KernelLibraryError("attention_paged: values that are part of the keys cannot be longer than they")
        swizzle_v = swizzle_k
    else:
        _need(v_pages, "v_pages", q.dtype)
        vp, Gv, v_row = v_pages, v_pages.shape[1], v_pages.shape[3]
        if v_row != value_dim or v_pages.shape[0] != num_pages or v_pages.shape[2] != page_size:
            raise KernelLibraryError(f"attention_paged: value pages {tuple(v_pages.shape)} against key pages {tuple(k_pages.shape)}")
    if sink is not None:
        _need(sink, "sink", torch.float32)
        if sink.numel() != H:
            raise KernelLibraryError("attention_paged: one sink per query head")
    if gate is not None:
        _need(gate, "gate", q.dtype, contiguous=False)
        if tuple(gate.shape) != (T, H) or gate.stride(1) != 1:
            raise KernelLibraryError("attention_paged: one gate per token and query head, rows dense")
    if out is None:
        out = torch.empty((T, H, value_dim), dtype=q.dtype, device=q.device)
    else:
        _need(out, "out", q.dtype)
        if tuple(out.shape) != (T, H, value_dim):
            raise KernelLibraryError(f"attention_paged: out is {tuple(out.shape)}, the result {(T, H, value_dim)}")
    check(_l.library().pb_attention_paged(
        q.data_ptr(), k_pages.data_ptr(), vp.data_ptr(), out.data_ptr(), dtype_code(q.dtype), _ptr(sink), positions.data_ptr(),
        table_row.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size, num_pages, T, H, G, kd, value_dim, v_row, Gv,
        float(scale), int(window or 0), int(keep_first or 0), int(chunk or 0), float(softcap or 0.0), _ptr(gate),
        0 if gate is None else gate.stride(0), 1 if swizzle_k else 0, 1 if swizzle_v else 0, _ptr(status), _stream()), "attention_paged")
    return out


# -- the state-space mixer ------------------------------------------------------------------------------------------
def causal_conv_silu(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], carried: torch.Tensor, batch,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(conv(x) + bias) per channel; x [T, C] a view with dense rows, weight float32 [C, taps], bias float32 [C] or
    None, carried [slots, taps - 1, C] of x's type (the sequences' last inputs of earlier steps)."""
    _need(x, "x", contiguous=False)
    _need(weight, "weight", torch.float32)
    if bias is not None:
        _need(bias, "bias", torch.float32)
    _need(carried, "carried", x.dtype)
    T, C = x.shape
    taps = weight.shape[1]
    if x.stride(1) != 1 or weight.shape[0] != C or (bias is not None and bias.numel() != C) or tuple(carried.shape[1:]) != (taps - 1, C):
        raise KernelLibraryError(f"causal_conv_silu: x {tuple(x.shape)}, weight {tuple(weight.shape)}, carried {tuple(carried.shape)}")
    if out is None:
        out = torch.empty((T, C), dtype=x.dtype, device=x.device)
    check(_l.library().pb_causal_conv_silu(x.data_ptr(), x.stride(0), weight.data_ptr(), _ptr(bias), carried.data_ptr(),
                                           out.data_ptr(), dtype_code(x.dtype), batch.token_seq.data_ptr(), batch.positions.data_ptr(),
                                           batch.q_start.data_ptr(), batch.state_slots.data_ptr(), T, C, taps, _stream()),
          "causal_conv_silu")
    return out


def conv_state_update(x: torch.Tensor, carried: torch.Tensor, batch) -> None:
    """The last taps - 1 rows of x of every sequence of the step, into its slot of ``carried``."""
    _need(x, "x", contiguous=False)
    _need(carried, "carried", x.dtype)
    check(_l.library().pb_conv_state_update(x.data_ptr(), x.stride(0), carried.data_ptr(), dtype_code(x.dtype), batch.cu_q.data_ptr(),
                                            batch.state_slots.data_ptr(), batch.cu_q.numel() - 1, x.shape[1], carried.shape[1] + 1,
                                            _stream()), "conv_state_update")


def ssm_scan(u: torch.Tensor, dt: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor,
             state: torch.Tensor, batch, groups: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The recurrence over the step's tokens, sequence by sequence; u [T, heads * P + 2 * groups * N] dense, dt [T, heads] a
    view with dense rows, state float32 [slots, heads, N, P]; returns y float32 [T, heads * P]."""
    _need(u, "u")
    _need(dt, "dt", u.dtype, contiguous=False)
    for t, name in ((dt_bias, "dt_bias"), (a_log, "a_log"), (d_skip, "d_skip"), (state, "state")):
        _need(t, name, torch.float32)
    T = u.shape[0]
    _, heads, N, P = state.shape
    if u.shape[1] != heads * P + 2 * groups * N or tuple(dt.shape) != (T, heads) or dt.stride(1) != 1:
        raise KernelLibraryError(f"ssm_scan: u {tuple(u.shape)}, dt {tuple(dt.shape)}, state {tuple(state.shape)}, {groups} groups")
    if out is None:
        out = torch.empty((T, heads * P), dtype=torch.float32, device=u.device)
    check(_l.library().pb_ssm_scan(u.data_ptr(), dt.data_ptr(), dt.stride(0), dtype_code(u.dtype), dt_bias.data_ptr(), a_log.data_ptr(),
                                   d_skip.data_ptr(), state.data_ptr(), out.data_ptr(), batch.cu_q.data_ptr(),
                                   batch.state_slots.data_ptr(), batch.cu_q.numel() - 1, heads, P, N, groups, _stream()), "ssm_scan")
    return out


# tokens of a step from which the linear attention's inputs are activated once, in place, ahead of the scan: every block
# of a head's columns would otherwise activate the head's keys and queries anew
DECAY_SCAN_ACTIVATE_AHEAD = 64


def decay_scan(proj: torch.Tensor, decay: torch.Tensor, state: torch.Tensor, batch, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Linear attention with a decaying state over the step's tokens, sequence by sequence: per head
    S <- decay_h S + k v^T, o = S^T q with q, k, v the SiLU of the projection's columns.  proj [T, >= H (P + 2 N)] a view
    with dense rows laid out [v: H P | k: H N | q: H N | ...], decay float32 [H], state float32 [slots, H, N, P];
    returns o float32 [T, H P].  A step of many tokens has the SiLU taken in place first (``proj`` then holds the
    activated values); a step of few leaves it to the scan's loaders.  See csrc/ssm.cu."""
    T = proj.shape[0]
    _rows_view(proj, "proj", T, None)
    _need(decay, "decay", torch.float32)
    _need(state, "state", torch.float32)
    _, H, N, P = state.shape
    if proj.shape[1] < H * (P + 2 * N) or decay.numel() != H:
        raise KernelLibraryError(f"decay_scan: proj {tuple(proj.shape)}, state {tuple(state.shape)}, {decay.numel()} decays")
    if out is None:
        out = torch.empty((T, H * P), dtype=torch.float32, device=proj.device)
    ahead = T >= DECAY_SCAN_ACTIVATE_AHEAD
    if ahead:
        check(_l.library().pb_silu_cols(proj.data_ptr(), proj.stride(0), dtype_code(proj.dtype), T, H * (P + 2 * N), _stream()), "silu_cols")
    check(_l.library().pb_decay_scan(proj.data_ptr(), proj.stride(0), dtype_code(proj.dtype), decay.data_ptr(), state.data_ptr(),
                                     out.data_ptr(), batch.cu_q.data_ptr(), batch.state_slots.data_ptr(), batch.cu_q.numel() - 1, H, P, N,
                                     1 if ahead else 0, _stream()), "decay_scan")
    return out


def gated_group_rmsnorm(y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, parts: int, eps: float,
                        out: Optional[torch.Tensor] = None, gate_after: bool = False, sigmoid_gate: bool = False) -> torch.Tensor:
    """y * silu(z) brought to unit root mean square in ``parts`` equal parts, times weight; with ``gate_after`` y
    brought to unit root mean square in parts, times weight, times silu(z); with ``sigmoid_gate`` the gate is
    sigmoid(z) instead of silu(z).  y float32 [T, inner], z a view [T, inner] with dense rows of the run's type,
    which the result has too."""
    _need(y, "y", torch.float32)
    _need(z, "z", contiguous=False)
    _need(weight, "weight", torch.float32)
    T, inner = y.shape
    if tuple(z.shape) != (T, inner) or z.stride(1) != 1 or weight.numel() != inner:
        raise KernelLibraryError(f"gated_group_rmsnorm: y {tuple(y.shape)}, z {tuple(z.shape)}")
    if out is None:
        out = torch.empty((T, inner), dtype=z.dtype, device=y.device)
    check(_l.library().pb_gated_group_rmsnorm(y.data_ptr(), z.data_ptr(), z.stride(0), weight.data_ptr(), out.data_ptr(),
                                              dtype_code(z.dtype), T, inner, parts, float(eps), 1 if gate_after else 0,
                                              1 if sigmoid_gate else 0, _stream()),
          "gated_group_rmsnorm")
    return out


def scaled_sum(a: torch.Tensor, sa: float, b: torch.Tensor, sb: float, out_dtype: torch.dtype) -> torch.Tensor:
    """sa * a + sb * b in float32, rounded once to ``out_dtype``."""
    _need(a, "a")
    _need(b, "b", a.dtype)
    if a.shape != b.shape:
        raise KernelLibraryError(f"scaled_sum: {tuple(a.shape)} against {tuple(b.shape)}")
    out = torch.empty(a.shape, dtype=out_dtype, device=a.device)
    check(_l.library().pb_scaled_sum(a.data_ptr(), float(sa), b.data_ptr(), float(sb), out.data_ptr(), dtype_code(a.dtype),
                                     dtype_code(out_dtype), a.numel(), _stream()), "scaled_sum")
    return out


# -- a residual stream that takes its sublayers' outputs times a constant ------------------------------------------------
class Scaled:
    """A sublayer's output that joins the residual stream times a constant: the value is ``scale * x`` (x a tensor of
    the run's type or ``PartialSums``), not computed yet.  The fused residual add multiplies while it adds, in float32."""

    def __init__(self, x, scale: float):
        self.x, self.scale = x, float(scale)

    @property
    def shape(self):
        return self.x.shape


def scaled_add_rmsnorm(x: "Scaled", res: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
                       rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """res += scale * x (in place, unless ``rows`` picks rows: then res is left alone); returns rmsnorm(res) * weight in
    ``out_dtype`` for every row, or for the chosen ones."""
    _need(res, "res", torch.float32)
    _need(weight, "weight", torch.float32)
    total, width = res.shape
    if tuple(x.shape) != tuple(res.shape) or weight.numel() != width:
        raise KernelLibraryError(f"scaled_add_rmsnorm: x {tuple(x.shape)} against residual {tuple(res.shape)}")
    ptr, parts, stride = _x_args(x.x, out_dtype, "x")
    n_out = total
    if rows is not None:
        _need(rows, "rows", torch.int32)
        n_out = rows.numel()
    out = torch.empty((n_out, width), dtype=out_dtype, device=res.device)
    check(_l.library().pb_scaled_add_rmsnorm(ptr, parts, stride, x.scale, res.data_ptr(), _ptr(rows), n_out, total, weight.data_ptr(),
                                             out.data_ptr(), dtype_code(out_dtype), width, float(eps), _stream()), "scaled_add_rmsnorm")
    return out


def normed_pair_sum(a: torch.Tensor, wa: torch.Tensor, sa: float, b: torch.Tensor, wb: torch.Tensor, sb: float, eps: float) -> PartialSums:
    """sa * a / rms(a) * wa + sb * b / rms(b) * wb over the rows of a and b [T, width], in float32: returned as a sum of
    one part, which the residual add takes without a rounding in between."""
    _need(a, "a")
    _need(b, "b", a.dtype)
    _need(wa, "wa", torch.float32)
    _need(wb, "wb", torch.float32)
    T, width = a.shape
    if a.shape != b.shape or wa.numel() != width or wb.numel() != width:
        raise KernelLibraryError(f"normed_pair_sum: {tuple(a.shape)} against {tuple(b.shape)}")
    out = torch.empty((1, T, width), dtype=torch.float32, device=a.device)
    check(_l.library().pb_normed_pair_sum(a.data_ptr(), wa.data_ptr(), float(sa), b.data_ptr(), wb.data_ptr(), float(sb), float(eps),
                                          out.data_ptr(), dtype_code(a.dtype), T, width, _stream()), "normed_pair_sum")
    return PartialSums(out)


def embed_gather_scaled(ids: torch.Tensor, table: torch.Tensor, scale: float) -> torch.Tensor:
    """res[t, :] = table[ids[t], :] * scale as float32 (the residual stream)."""
    _need(ids, "ids", torch.int32)
    _need(table, "table")
    T, (V, H) = ids.numel(), table.shape
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    check(_l.library().pb_embed_gather_scaled(ids.data_ptr(), table.data_ptr(), dtype_code(table.dtype), float(scale), out.data_ptr(),
                                              T, H, V, _stream()), "embed_gather_scaled")
    return out


def tanh_(x: torch.Tensor) -> torch.Tensor:
    """tanh of a dense tensor, in place (float32 arithmetic)."""
    _need(x, "x")
    check(_l.library().pb_tanh(x.data_ptr(), x.data_ptr(), dtype_code(x.dtype), x.numel(), _stream()), "tanh")
    return x


def _rows_view(t: torch.Tensor, name: str, rows: int, dtype) -> None:
    _need(t, name, dtype, contiguous=False)
    if t.dim() != 2 or t.stride(1) != 1 or t.shape[0] != rows:
        raise KernelLibraryError(f"{name} must be [tokens, cols] with dense rows, is {tuple(t.shape)}")


def heads_prepare(q_in: torch.Tensor, k_in: Optional[torch.Tensor], v_in: Optional[torch.Tensor], *, n_heads: int, q_dim: int,
                  q_weight: Optional[torch.Tensor] = None, k_weight: Optional[torch.Tensor] = None, eps: float = 0.0,
                  norm: Optional[str] = None, rates: Optional[torch.Tensor] = None, amplitude: float = 1.0, rot_dims: int = 0,
                  adjacent: bool = False,
                  v_other: Optional[torch.Tensor] = None, v_copy: Optional[torch.Tensor] = None, mix: float = 0.0,
                  positions: torch.Tensor, table_row: torch.Tensor, block_table: Optional[torch.Tensor] = None,
                  q_out: torch.Tensor, k_pages: Optional[torch.Tensor] = None, v_pages: Optional[torch.Tensor] = None,
                  status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-head norm (one scale for all heads, or none: ``norm`` is None for no norm, "before" or "after" the rotation;
    left out it is "before" where scales are given), rotation by rates with cosine and sine times ``amplitude``, values
    blended with another layer's; queries to
    ``q_out``, keys and values into pages; see csrc/heads_prepare.cu.  ``q_in``, ``k_in``, ``v_in`` are [T, cols] views
    with dense rows; ``v_other`` / ``v_copy`` dense [T, value cols]; ``k_pages`` None: nothing is cached."""
    T, dt = q_in.shape[0], q_in.dtype
    _rows_view(q_in, "q_in", T, dt)
    if norm is None and (q_weight is not None or k_weight is not None):
        norm = "before"
    if norm not in (None, "before", "after"):
        raise KernelLibraryError(f"heads_prepare: norm is None, 'before' or 'after', not {norm!r}")
    norm_code = {None: 0, "before": 1, "after": 2}[norm]
    for t, name in ((q_weight, "q_weight"), (k_weight, "k_weight"), (rates, "rates")):
        if t is not None:
            _need(t, name, torch.float32)
    _need(positions, "positions", torch.int32)
    _need(table_row, "table_row", torch.int32)
    _need(q_out, "q_out", dt)
    if q_in.shape[1] != n_heads * q_dim or q_out.numel() != T * n_heads * q_dim:
        raise KernelLibraryError(f"heads_prepare: q_in {tuple(q_in.shape)}, q_out {tuple(q_out.shape)} for {n_heads} heads of {q_dim}")
    if q_weight is not None and q_weight.numel() != q_dim:
        raise KernelLibraryError("heads_prepare: the query norm's scale covers one head")
    if rates is not None and rates.numel() * 2 != rot_dims:
        raise KernelLibraryError("heads_prepare: one rate per rotated pair")
    G = kd = Gv = vd = page_size = num_pages = stride = ld_other = 0
    if k_pages is not None:
        _need(k_pages, "k_pages", dt)
        _need(block_table, "block_table", torch.int32)
        num_pages, G, page_size, kd = k_pages.shape
        stride = block_table.shape[1]
        if k_in is None:
            raise KernelLibraryError("heads_prepare: key pages without keys")
        _rows_view(k_in, "k_in", T, dt)
        if k_in.shape[1] != G * kd or (k_weight is not None and k_weight.numel() != kd):
            raise KernelLibraryError(f"heads_prepare: keys {tuple(k_in.shape)} against pages {tuple(k_pages.shape)}")
        if v_pages is not None:
            _need(v_pages, "v_pages", dt)
            _, Gv, _, vd = v_pages.shape
            if v_in is None:
                raise KernelLibraryError("heads_prepare: value pages without values")
            _rows_view(v_in, "v_in", T, dt)
            if v_in.shape[1] != Gv * vd or v_pages.shape[0] != num_pages or v_pages.shape[2] != page_size:
                raise KernelLibraryError(f"heads_prepare: values {tuple(v_in.shape)} against pages {tuple(v_pages.shape)}")
            for t, name in ((v_other, "v_other"), (v_copy, "v_copy")):
                if t is not None:
                    _need(t, name, dt)
                    if tuple(t.shape) != (T, Gv * vd):
                        raise KernelLibraryError(f"heads_prepare: {name} {tuple(t.shape)} against values {tuple(v_in.shape)}")
                    ld_other = Gv * vd
    elif v_other is not None or v_copy is not None:
        raise KernelLibraryError("heads_prepare: blended values need pages")
    check(_l.library().pb_heads_prepare(
        q_in.data_ptr(), q_in.stride(0), _ptr(k_in), 0 if k_in is None else k_in.stride(0), _ptr(v_in),
        0 if v_in is None else v_in.stride(0), dtype_code(dt), _ptr(q_weight), _ptr(k_weight), norm_code, float(eps), _ptr(rates),
        float(amplitude), int(rot_dims),
        1 if adjacent else 0, _ptr(v_other), _ptr(v_copy), ld_other, float(mix), positions.data_ptr(), table_row.data_ptr(),
        _ptr(block_table), stride, page_size, num_pages, q_out.data_ptr(), _ptr(k_pages), _ptr(v_pages), T, n_heads, q_dim, G, kd, Gv,
        vd, _ptr(status), _stream()), "heads_prepare")
    return q_out


def gated_delta_scan(u: torch.Tensor, beta: torch.Tensor, a: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
                     state: torch.Tensor, batch, kv_heads: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The gated delta rule over the step's tokens, sequence by sequence; u [T, 2 G D + H E] laid out [q | k | v] (the
    convolutions' outputs), beta and a [T, H] views with dense rows, state float32 [slots, H, D, E]; returns o float32
    [T, H E].  See csrc/delta_rule.cu."""
    T = u.shape[0]
    _rows_view(u, "u", T, None)
    _rows_view(beta, "beta", T, u.dtype)
    _rows_view(a, "a", T, u.dtype)
    for t, name in ((a_log, "a_log"), (dt_bias, "dt_bias"), (state, "state")):
        _need(t, name, torch.float32)
    _, H, D, E = state.shape
    if u.shape[1] != 2 * kv_heads * D + H * E or beta.shape[1] != H or a.shape[1] != H or a_log.numel() != H or dt_bias.numel() != H:
        raise KernelLibraryError(f"gated_delta_scan: u {tuple(u.shape)}, state {tuple(state.shape)}, {kv_heads} query/key heads")
    if out is None:
        out = torch.empty((T, H * E), dtype=torch.float32, device=u.device)
    check(_l.library().pb_gated_delta_scan(u.data_ptr(), u.stride(0), beta.data_ptr(), beta.stride(0), a.data_ptr(), a.stride(0),
                                           dtype_code(u.dtype), a_log.data_ptr(), dt_bias.data_ptr(), state.data_ptr(), out.data_ptr(),
                                           batch.cu_q.data_ptr(), batch.state_slots.data_ptr(), batch.cu_q.numel() - 1, H, kv_heads, D, E,
                                           _stream()), "gated_delta_scan")
    return out


def token_shift_mix(x: torch.Tensor, carried: torch.Tensor, mu: torch.Tensor, batch, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[s, t] = x_t + (x_(t-1) - x_t) * mu[s]; x [T, width] dense, carried [slots, width] (the sequences' last input of
    earlier steps), mu float32 [n, width]; returns [n, T, width] of x's type."""
    _need(x, "x")
    _need(carried, "carried", x.dtype)
    _need(mu, "mu", torch.float32)
    T, width = x.shape
    n = mu.shape[0]
    if mu.shape[1] != width or carried.shape[1] != width:
        raise KernelLibraryError(f"token_shift_mix: x {tuple(x.shape)}, mu {tuple(mu.shape)}, carried {tuple(carried.shape)}")
    if out is None:
        out = torch.empty((n, T, width), dtype=x.dtype, device=x.device)
    check(_l.library().pb_token_shift_mix(x.data_ptr(), carried.data_ptr(), mu.data_ptr(), out.data_ptr(), dtype_code(x.dtype),
                                          batch.token_seq.data_ptr(), batch.positions.data_ptr(), batch.q_start.data_ptr(),
                                          batch.state_slots.data_ptr(), T, width, n, _stream()), "token_shift_mix")
    return out


def wkv_scan(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w: torch.Tensor, w0: torch.Tensor, bonus: torch.Tensor,
             state: torch.Tensor, batch, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The decaying-state recurrence with a bonus for the current token over the step's tokens, sequence by sequence; r, k,
    v, w [T, H D] views with dense rows (w before its exponentials), w0 and bonus float32 [H D], state float32
    [slots, H, D, D]; returns o float32 [T, H D].  See csrc/wkv.cu."""
    T = r.shape[0]
    for t, name in ((r, "r"), (k, "k"), (v, "v"), (w, "w")):
        _rows_view(t, name, T, r.dtype)
    for t, name in ((w0, "w0"), (bonus, "bonus"), (state, "state")):
        _need(t, name, torch.float32)
    _, H, D, D2 = state.shape
    if D != D2 or any(t.shape[1] != H * D for t in (r, k, v, w)) or w0.numel() != H * D or bonus.numel() != H * D:
        raise KernelLibraryError(f"wkv_scan: r {tuple(r.shape)}, state {tuple(state.shape)}")
    if out is None:
        out = torch.empty((T, H * D), dtype=torch.float32, device=r.device)
    check(_l.library().pb_wkv_scan(r.data_ptr(), r.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), w.data_ptr(),
                                   w.stride(0), dtype_code(r.dtype), w0.data_ptr(), bonus.data_ptr(), state.data_ptr(), out.data_ptr(),
                                   batch.cu_q.data_ptr(), batch.state_slots.data_ptr(), batch.cu_q.numel() - 1, H, D, _stream()), "wkv_scan")
    return out
