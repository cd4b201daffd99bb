"""Host side of the tensor-core attention kernels (csrc/attention_fast.cu): choice between the
decode kernel (every sequence brings one token) and the prefill kernel, scratch for the splits."""
from __future__ import annotations

from typing import Callable, Optional

import torch

from . import kernels as K
from .build import kernel, module


def decode_splits(n_tokens: int, nkv: int, max_ctx: int) -> int:
    return int(module("attention_fast").lib.gg_attn_decode_splits(int(n_tokens), int(nkv), int(max_ctx)))


def attn_decode(q, k_pool, v_pool, out, positions, seq_of_token, table, page_size, n_tokens, nq, nkv, d,
                scale, window, splits, part_o=None, part_ml=None) -> None:
    from .tcgen05_gemm import status_word
    kernel("attention_fast", "gg_attn_decode")(
        q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(),
        part_o.data_ptr() if part_o is not None else 0, part_ml.data_ptr() if part_ml is not None else 0,
        positions.data_ptr(), seq_of_token.data_ptr(), table.data_ptr(), table.shape[-1], page_size,
        k_pool.shape[0], n_tokens, nq, nkv, d, float(scale), int(window), int(splits),
        status_word(q.device).data_ptr(), torch.cuda.current_stream().cuda_stream)


def decode_tma_splits(n_tokens: int, nkv: int, max_ctx: int, cluster: bool = False) -> int:
    return int(module("attention_fast").lib.gg_attn_decode_tma_splits(int(n_tokens), int(nkv), int(max_ctx),
                                                                      int(bool(cluster))))


def attn_decode_tma(q, k_pool, v_pool, out, positions, seq_of_token, table, page_size, n_tokens, nq, nkv, d,
                    scale, window, splits, part_o=None, part_ml=None, cluster: bool = False) -> None:
    """Decode attention with the cache streamed through a TMA ring (pools: [page][nkv][64][d]).
    cluster=True merges the splits inside thread-block clusters (no scratch, no second kernel)."""
    from .tcgen05_gemm import status_word
    kernel("attention_fast", "gg_attn_decode_tma")(
        q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(),
        part_o.data_ptr() if part_o is not None else 0, part_ml.data_ptr() if part_ml is not None else 0,
        positions.data_ptr(), seq_of_token.data_ptr(), table.data_ptr(), table.shape[-1], page_size,
        k_pool.shape[0], n_tokens, nq, nkv, d, float(scale), int(window), int(splits), int(bool(cluster)),
        status_word(q.device).data_ptr(), torch.cuda.current_stream().cuda_stream)


def attn_prefill(q, k_pool, v_pool, out, cu_seqlens, ctx_lens, seq_of_token, table, page_size, n_seqs,
                 max_tiles, nq, nkv, d, scale, window) -> None:
    from .tcgen05_gemm import status_word
    kernel("attention_fast", "gg_attn_prefill")(
        q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(), cu_seqlens.data_ptr(),
        ctx_lens.data_ptr(), seq_of_token.data_ptr(), table.data_ptr(), table.shape[-1], page_size,
        k_pool.shape[0], n_seqs, max_tiles, nq, nkv, d, float(scale), int(window),
        status_word(q.device).data_ptr(), torch.cuda.current_stream().cuda_stream)


def attn_prefill_tc(q, k_pool, v_pool, out, cu_seqlens, ctx_lens, seq_of_token, table, page_size, n_tokens,
                    n_seqs, max_tiles, nq, nkv, d, scale, window) -> None:
    """Prefill attention on tcgen05: 128-query tiles, S and O in tensor memory."""
    from .tcgen05_gemm import status_word
    kernel("attention_fast", "gg_attn_prefill_tc")(
        q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(), cu_seqlens.data_ptr(),
        ctx_lens.data_ptr(), seq_of_token.data_ptr(), table.data_ptr(), table.shape[-1], page_size,
        k_pool.shape[0], n_tokens, n_seqs, max_tiles, nq, nkv, d, float(scale), int(window),
        status_word(q.device).data_ptr(), torch.cuda.current_stream().cuda_stream)


def try_make(nq: int, nkv: int, d: int, scale: float, window: int) -> Optional[Callable]:
    """f(q, k_pool, v_pool, out, ctx, table, page_size) for bfloat16, or None when the sizes are
    outside what the tensor-core kernels take (head size 64 or 128, at most 16 query heads per kv
    head); then the plain kernel serves."""
    if d not in (64, 128) or nq % nkv or nq // nkv > 16:
        return None

    def run(q, k_pool, v_pool, out, ctx, table, page_size):
        T = ctx.n_tokens
        if page_size != 64 or q.dtype != torch.bfloat16:
            K.attention_plain(q, k_pool, v_pool, out, ctx.positions, ctx.seq_of_token, table, page_size,
                              T, nq, nkv, d, scale, window)
            return
        if ctx.decode:
            splits = decode_tma_splits(T, nkv, ctx.max_ctx, cluster=True)
            attn_decode_tma(q, k_pool, v_pool, out, ctx.positions, ctx.seq_of_token, table, page_size, T, nq, nkv, d,
                            scale, window, splits, cluster=True)
        elif ctx.max_new >= 32:
            # 128-query tiles on tcgen05 (S and O in tensor memory)
            max_tiles = T // 128 + ctx.n_seqs
            attn_prefill_tc(q, k_pool, v_pool, out, ctx.cu_seqlens, ctx.ctx_lens, ctx.seq_of_token, table, page_size,
                            T, ctx.n_seqs, max_tiles, nq, nkv, d, scale, window)
        else:
            # a few tokens per sequence: 64-query tiles on mma.sync waste less
            max_tiles = T // 64 + ctx.n_seqs
            attn_prefill(q, k_pool, v_pool, out, ctx.cu_seqlens, ctx.ctx_lens, ctx.seq_of_token, table, page_size,
                         ctx.n_seqs, max_tiles, nq, nkv, d, scale, window)

    return run
