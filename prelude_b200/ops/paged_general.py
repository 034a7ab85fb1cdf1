"""General paged attention over a step's batch: keys and values of different sizes, values that are part of the
cached key rows, a window, a sink.  Picks the kernel for the type and shape; which one ran changes the rounding,
never what is computed.

float32 always runs the plain warp-per-row kernel.  bfloat16 runs the tensor-core kernel where it takes the shape
(key size in multiples of 16, value size in multiples of 32 up to 512), prompt portions and single tokens alike; a
step of few rows has its keys dealt to several blocks per row (PRELUDE_GENERAL_ATTN=plain turns it off).  Prompt
portions that fill the tcgen05 prompt kernel's blocks go to that kernel where it takes the shape (keys and values of
one size, 64 or 128, in pages of their own; PRELUDE_GENERAL_PROMPT_ATTN=mma turns it off): it knows the same masks,
cap, sink and gate and reads the same pages, permuting them on their way into shared memory.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import kernels as K
from . import library as _l
from .attention import TC_MIN_FILL, _prefill_plan, _sm_count
from .library import check

KERNEL = os.environ.get("PRELUDE_GENERAL_ATTN", "auto")
PROMPT_KERNEL = os.environ.get("PRELUDE_GENERAL_PROMPT_ATTN", "auto")
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
        # The tcgen05 prompt kernel works on 256 query rows at a time and pays for all of them: it takes the portions
        # that fill at least TC_MIN_FILL of a block's tokens, this kernel the shorter ones and the single tokens.  Both
        # write disjoint rows of `out`.
        long_min, long_tiles = None, 0
        if (PROMPT_KERNEL != "mma" and v_pages is not None and kd == value_dim and v_pages.shape[3] == kd
                and lib.pb_attention_prefill_tc_plain_pages_supported(H, G, kd, page_size)):
            tc_tokens = lib.pb_attention_prefill_tc_tile_tokens(H, G)
            long_min = 1 if PROMPT_KERNEL == "tc" else max(2, int(tc_tokens * TC_MIN_FILL))
            tile_seq, tile_tok0, long_tiles = _prefill_plan(batch, tc_tokens, long_min, None)
            if long_tiles:
                check(lib.pb_attention_prefill_tc_masked_bf16(
                    q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(), table.data_ptr(), table.shape[1],
                    batch.positions.data_ptr(), batch.table_row_of_token.data_ptr(), batch.cu_q.data_ptr(), batch.q_start.data_ptr(),
                    tile_seq.data_ptr(), tile_tok0.data_ptr(), long_tiles, page_size, num_pages, T, H, G, kd, float(scale), int(window or 0), 0,
                    int(keep_first or 0), int(chunk or 0), float(softcap or 0.0), K._ptr(sink), K._ptr(gate),
                    0 if gate is None else gate.stride(0), batch.status.data_ptr(), _l.current_stream_ptr(q.device)),
                    "attention_prefill_tc_masked")
        tile_seq, tile_tok0, n_tiles = _prefill_plan(batch, lib.pb_attention_paged_tc_tile_tokens(H, G), 0, long_min)
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
    # (putting the parts together writes every row of the step: not beside rows that the prompt kernel wrote)
    if blocks < _sm_count(q.device) and (batch.decode_only or not long_tiles):
        key_tiles = -(-max_ctx // 32)
        splits = max(1, min(MAX_SPLITS, 2 * _sm_count(q.device) // blocks, key_tiles))    # two blocks a multiprocessor: one wave
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
