"""General paged attention over a step's batch: keys and values of different sizes, values that are part of the
cached key rows, a window, a sink.  Picks the kernel for the type and shape; which one ran changes the rounding,
never what is computed.

float32 always runs the plain warp-per-row kernel.  bfloat16 runs the tensor-core kernel where it takes the shape
(key size in multiples of 16, value size in multiples of 32 up to 512), prompt portions and single tokens alike; a
step of few rows has its keys dealt to several blocks per row (PRELUDE_GENERAL_ATTN=plain turns it off).
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import kernels as K
from . import library as _l
from .attention import _prefill_plan, _sm_count
from .library import check

KERNEL = os.environ.get("PRELUDE_GENERAL_ATTN", "auto")
MAX_SPLITS = 32


def tc_takes(q: torch.Tensor, k_pages: torch.Tensor, v_pages: Optional[torch.Tensor], value_dim: int) -> bool:
    if KERNEL == "plain" or q.dtype != torch.bfloat16:
        return False
    H, kd, G = q.shape[1], q.shape[2], k_pages.shape[1]
    if v_pages is not None and v_pages.shape[1] != G:
        return False
    return bool(_l.library().pb_attention_paged_tc_supported(H, G, kd, value_dim, 1 if v_pages is None else 0))


def attention_general(q: torch.Tensor, k_pages: torch.Tensor, v_pages: Optional[torch.Tensor], value_dim: int, batch, group: int,
                      scale: float, window: Optional[int], sink: Optional[torch.Tensor], out: Optional[torch.Tensor] = None,
                      keep_first: int = 0, chunk: Optional[int] = None, softcap: Optional[float] = None,
                      gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, H, kd] of the batch's tokens against the pages of cache group ``group``; ``v_pages`` None: the values are
    the first ``value_dim`` elements of the key rows.  ``keep_first``, ``chunk``, ``softcap``, ``gate``: as for
    ``kernels.attention_paged``.  While a step is being captured piece by piece, the tensor-core
    kernel is launched between the pieces: its grid follows how the step's tokens are spread over requests."""
    T, H, kd = q.shape
    if out is None:
        out = torch.empty((T, H, value_dim), dtype=q.dtype, device=q.device)
    if not tc_takes(q, k_pages, v_pages, value_dim):
        # one warp per row whatever the step holds: the launch has the shape of the token count alone
        return K.attention_paged(q, k_pages, v_pages, value_dim, batch.positions, batch.table_row_of_token, batch.block_tables[group],
                                 scale, window, sink, status=batch.status, out=out, keep_first=keep_first, chunk=chunk,
                                 softcap=softcap, gate=gate)
    recorder = batch.extras.get("recorder")
    if recorder is not None and recorder.capturing and not batch.decode_only:
        recorder.run_between_pieces(lambda: attention_general(q, k_pages, v_pages, value_dim, batch, group, scale, window, sink, out,
                                                              keep_first, chunk, softcap, gate))
        return out
    lib = _l.library()
    table = batch.block_tables[group]
    num_pages, G, page_size, _ = k_pages.shape
    if batch.decode_only:
        tile_seq = tile_tok0 = None
        n_tiles = T
    else:
        tile_seq, tile_tok0, n_tiles = _prefill_plan(batch, lib.pb_attention_paged_tc_tile_tokens(H, G))
        if n_tiles == 0:
            return out
    # few rows: deal each row's keys to several blocks, until the device is about twice full
    max_ctx = batch.max_kv_len if batch.max_kv_len else table.shape[1] * page_size
    if window:
        max_ctx = min(max_ctx, window + (keep_first or 0) + batch.max_q_len + 64)
    elif chunk:
        max_ctx = min(max_ctx, chunk + 32)
    blocks = n_tiles * G * (-(-(H // G) // 32))
    splits = 1
    if blocks < _sm_count(q.device):
        key_tiles = -(-max_ctx // 32)
        splits = max(1, min(MAX_SPLITS, -(-2 * _sm_count(q.device) // blocks), key_tiles))
        splits = -(-key_tiles // -(-key_tiles // splits))               # as many blocks as have tiles to work on
    scratch = None
    if splits > 1:
        scratch = batch.workspace("general_attention_parts", (lib.pb_attention_paged_tc_scratch_floats(T, H, value_dim, splits),), torch.float32)
    vp = k_pages if v_pages is None else v_pages
    check(lib.pb_attention_paged_tc_bf16(
        q.data_ptr(), k_pages.data_ptr(), vp.data_ptr(), out.data_ptr(), K._ptr(sink), batch.positions.data_ptr(),
        batch.table_row_of_token.data_ptr(), table.data_ptr(), table.shape[1], batch.cu_q.data_ptr(), K._ptr(tile_seq), K._ptr(tile_tok0),
        n_tiles, page_size, num_pages, T, H, G, kd, value_dim, vp.shape[3], 1 if v_pages is None else 0, float(scale), int(window or 0),
        int(keep_first or 0), int(chunk or 0), float(softcap or 0.0), K._ptr(gate), 0 if gate is None else gate.stride(0),
        splits, K._ptr(scratch), batch.status.data_ptr(), _l.current_stream_ptr(q.device)), "attention_paged_tc")
    return out
