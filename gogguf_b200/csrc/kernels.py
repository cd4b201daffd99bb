"""Python face of the CUDA kernels: one thin function per launcher.

Arguments are torch tensors on the GPU; every function launches on torch's current stream and
allocates nothing (outputs and scratch are passed in).  There is no CPU or library fallback: a
tensor that is not on a CUDA device, or a missing compiler, raises.
"""
from __future__ import annotations

from typing import Optional

import torch

from .build import KernelError, kernel

F32, BF16 = 0, 1


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {dt}")


def _p(t: Optional[torch.Tensor]) -> int:
    if t is None:
        return 0
    if not t.is_cuda:
        raise KernelError("kernel argument is not on a CUDA device (there is no CPU path)")
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need(t: torch.Tensor, dt: torch.dtype, what: str) -> None:
    if t.dtype != dt:
        raise KernelError(f"{what} must be {dt}, got {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")


# ------------------------------------------------------------------------------- elementwise
def embed_gather(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, :] (float32) = table[tokens[t], :]; negative ids give zero rows."""
    _need(tokens, torch.int32, "tokens")
    _need(out, torch.float32, "out")
    V, H = table.shape
    kernel("elementwise", "gg_embed_gather")(_p(table), dtype_code(table.dtype), _p(tokens), _p(out),
                                              tokens.numel(), H, V, _stream())


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = rmsnorm(x[rows[r]] or x[r]) * weight; x float32, weight float32, out float32/bfloat16."""
    _need(x, torch.float32, "x")
    _need(weight, torch.float32, "norm weight")
    H = x.shape[-1]
    R = rows.numel() if rows is not None else x.numel() // H
    if rows is not None:
        _need(rows, torch.int32, "rows")
    if weight.numel() != H or out.shape[-1] != H or out.numel() < R * H:
        raise KernelError("rmsnorm: shapes disagree")
    kernel("elementwise", "gg_rmsnorm")(_p(x), _p(rows), _p(weight), _p(out), dtype_code(out.dtype),
                                         R, H, float(eps), _stream())


def row_stats(x: torch.Tensor, xhat: torch.Tensor, ssq: torch.Tensor) -> None:
    """xhat = bfloat16(x) and ssq[t, p] = sum of x[t, 128 p : 128 p + 128]^2 for float32 rows x [T, H]."""
    _need(x, torch.float32, "x")
    _need(xhat, torch.bfloat16, "xhat")
    _need(ssq, torch.float32, "ssq")
    H = x.shape[-1]
    T = x.numel() // H
    if xhat.numel() != T * H or ssq.numel() != T * ((H + 127) // 128):
        raise KernelError("row_stats: shapes disagree")
    kernel("elementwise", "gg_row_stats")(_p(x), _p(xhat), _p(ssq), T, H, _stream())


def rope_tables(positions: torch.Tensor, inv_freq: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> None:
    _need(positions, torch.int32, "positions")
    _need(inv_freq, torch.float64, "inv_freq")
    _need(cos, torch.float32, "cos")
    _need(sin, torch.float32, "sin")
    T, half = positions.numel(), inv_freq.numel()
    kernel("elementwise", "gg_rope_tables")(_p(positions), _p(inv_freq), _p(cos), _p(sin), T, half, _stream())


def qk_norm_rope_cache(qkv: torch.Tensor, q_out: torch.Tensor, q_weight: Optional[torch.Tensor],
                       k_weight: Optional[torch.Tensor], eps: float, cos: torch.Tensor, sin: torch.Tensor,
                       positions: torch.Tensor, seq_of_token: torch.Tensor, page_table: torch.Tensor,
                       page_size: int, k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                       n_tokens: int, nq: int, nkv: int, d: int, rot: int) -> None:
    if q_out.dtype != qkv.dtype or (k_pool is not None and k_pool.dtype != qkv.dtype):
        raise KernelError("qk_norm_rope_cache: qkv, q_out and the cache must share one dtype")
    from .tcgen05_gemm import status_word
    kernel("elementwise", "gg_qk_norm_rope_cache")(
        _p(qkv), dtype_code(qkv.dtype), _p(q_out), _p(q_weight), _p(k_weight), float(eps), _p(cos), _p(sin),
        _p(positions), _p(seq_of_token), _p(page_table), page_table.shape[-1], page_size,
        k_pool.shape[0] if k_pool is not None else 0, _p(k_pool), _p(v_pool),
        n_tokens, nq, nkv, d, rot, _p(status_word(qkv.device)), _stream())


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, n_tokens: int, inter: int) -> None:
    if gate_up.dtype != out.dtype:
        raise KernelError("swiglu: input and output must share one dtype")
    kernel("elementwise", "gg_swiglu")(_p(gate_up), dtype_code(gate_up.dtype), _p(out), n_tokens, inter, _stream())


def residual_add(x: torch.Tensor, delta: torch.Tensor) -> None:
    _need(x, torch.float32, "x")
    if delta.numel() != x.numel() or not delta.is_contiguous():
        raise KernelError("residual_add: shapes disagree")
    kernel("elementwise", "gg_residual_add")(_p(x), _p(delta), dtype_code(delta.dtype), x.numel(), _stream())


def feed_tokens(tokens: torch.Tensor, src: torch.Tensor, sampled: torch.Tensor, n: int) -> None:
    """tokens[i] = sampled[src[i]] where src[i] >= 0 (all int32, on the device)."""
    _need(tokens, torch.int32, "tokens")
    _need(src, torch.int32, "src")
    _need(sampled, torch.int32, "sampled")
    kernel("elementwise", "gg_feed_tokens")(_p(tokens), _p(src), _p(sampled), n, _stream())


# ------------------------------------------------------------------------------- matrix product
def gemm_plain(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
               m: Optional[int] = None) -> None:
    """out[M, N] (+)= x[M, K] @ w[N, K]^T on the CUDA cores with float32 accumulation."""
    N, K = w.shape
    M = x.shape[0] if m is None else m
    if x.shape[-1] != K or out.shape[-1] != N:
        raise KernelError(f"gemm: x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)} disagree")
    if x.stride(-1) != 1 or out.stride(-1) != 1 or not w.is_contiguous():
        raise KernelError("gemm: operands must be row-major")
    kernel("gemm_plain", "gg_gemm_plain")(_p(x), dtype_code(x.dtype), _p(w), dtype_code(w.dtype), _p(out),
                                           dtype_code(out.dtype), int(accumulate), M, N, K,
                                           x.stride(0), out.stride(0), _stream())


# ------------------------------------------------------------------------------- attention
def attention_plain(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                    positions: torch.Tensor, seq_of_token: torch.Tensor, page_table: torch.Tensor,
                    page_size: int, n_tokens: int, nq: int, nkv: int, d: int, scale: float, window: int) -> None:
    if not (q.dtype == k_pool.dtype == v_pool.dtype == out.dtype):
        raise KernelError("attention: q, cache and out must share one dtype")
    from .tcgen05_gemm import status_word
    kernel("attention_plain", "gg_attention_plain")(
        _p(q), _p(k_pool), _p(v_pool), _p(out), dtype_code(q.dtype), _p(positions), _p(seq_of_token),
        _p(page_table), page_table.shape[-1], page_size, k_pool.shape[0], n_tokens, nq, nkv, d, float(scale),
        int(window), _p(status_word(q.device)), _stream())


def wait_probe(limit_cycles: int, code: int, status: torch.Tensor) -> torch.Tensor:
    """Run the package's bounded wait on a barrier nothing arrives at (csrc/diagnostics.cu) and return the
    kernel's report (5 int32 on the device): both roles' return values, their elapsed cycles / 1024, the
    abort flag.  `status` is the int32 status word the code is to land in."""
    report = torch.full((5,), -1, dtype=torch.int32, device=status.device)
    kernel("diagnostics", "gg_wait_probe")(int(limit_cycles), int(code), _p(status), _p(report), _stream())
    return report


# ------------------------------------------------------------------------------- sampling
_argmax_scratch = {}


def argmax(logits: torch.Tensor, out: torch.Tensor, rows: Optional[int] = None) -> None:
    _need(logits, torch.float32, "logits")
    _need(out, torch.int32, "out")
    R = logits.shape[0] if rows is None else rows
    scratch = _argmax_scratch.get(logits.device)
    if scratch is None or scratch.numel() < R * 128:
        scratch = _argmax_scratch[logits.device] = torch.empty(max(R, 64) * 128, dtype=torch.int32,
                                                                device=logits.device)
    kernel("sampling", "gg_argmax")(_p(logits), logits.stride(0), _p(out), R, logits.shape[1],
                                     _p(scratch), scratch.numel(), _stream())


def repeat_penalty(logits: torch.Tensor, hist: torch.Tensor, hist_len: torch.Tensor, ring_rows: torch.Tensor,
                   penalty: float, rows: int) -> None:
    """In place on logits[:rows]: every distinct id in the sequences' rings is penalised once."""
    _need(logits, torch.float32, "logits")
    for t, n in ((hist, "hist"), (hist_len, "hist_len"), (ring_rows, "ring_rows")):
        _need(t, torch.int32, n)
    kernel("sampling", "gg_repeat_penalty")(_p(logits), logits.stride(0), rows, logits.shape[1], _p(hist), _p(hist_len),
                                             _p(ring_rows), hist.shape[1], float(penalty), _stream())


def history_append(tokens: torch.Tensor, ring_rows: torch.Tensor, hist: torch.Tensor, hist_len: torch.Tensor,
                   hist_pos: torch.Tensor, rows: int) -> None:
    """Append tokens[r] to the ring of sequence ring_rows[r]."""
    for t, n in ((tokens, "tokens"), (hist, "hist"), (hist_len, "hist_len"), (hist_pos, "hist_pos"), (ring_rows, "ring_rows")):
        _need(t, torch.int32, n)
    kernel("sampling", "gg_history_append")(_p(tokens), _p(ring_rows), _p(hist), _p(hist_len), _p(hist_pos),
                                             hist.shape[1], rows, _stream())


TOPK_MAX = 1024      # largest top-k the on-device chain takes (csrc/sampling.cu)


_topk_scratch = {}
_sample_scratch = {}


def sample_topk(logits: torch.Tensor, temp: float, top_k: int, top_p: float, min_p: float, uniforms: torch.Tensor,
                out: torch.Tensor, rows: Optional[int] = None) -> None:
    """The sampling chain with a top-k on the device: temperature, top-k, min-p, softmax, top-p, draw."""
    _need(logits, torch.float32, "logits")
    _need(uniforms, torch.float64, "uniforms")
    _need(out, torch.int32, "out")
    R = logits.shape[0] if rows is None else rows
    V = logits.shape[1]
    words = -(-V // 8192) * min(int(top_k), V) * R          # what gg_sample_topk_scratch_words says
    buf = _topk_scratch.get(logits.device)
    if buf is None or buf.numel() < words:
        buf = _topk_scratch[logits.device] = torch.empty(max(words, 1 << 16), dtype=torch.int64, device=logits.device)
    kernel("sampling", "gg_sample_topk")(_p(logits), logits.stride(0), float(temp), int(top_k), float(top_p),
                                          float(min_p), _p(uniforms), _p(out), R, V, _p(buf), buf.numel(), _stream())


_nucleus_scratch = {}


def sample_nucleus(logits: torch.Tensor, temp: float, top_p: float, min_p: float, uniforms: torch.Tensor,
                   out: torch.Tensor, flags: torch.Tensor, rows: Optional[int] = None) -> None:
    """Top-p and / or min-p without a top-k: candidates are each row's 1,024 largest logits, the softmax runs over
    the whole row; flags[r] = 1 where the answer may lie beyond the candidates (out[r] is then not to be used)."""
    _need(logits, torch.float32, "logits")
    _need(uniforms, torch.float64, "uniforms")
    _need(out, torch.int32, "out")
    _need(flags, torch.int32, "flags")
    R = logits.shape[0] if rows is None else rows
    V = logits.shape[1]
    slices = -(-V // 8192)
    nbytes = R * 128 * 4 + R * slices * 8 + R * slices * min(V, 1024) * 8
    buf = _nucleus_scratch.get(logits.device)
    if buf is None or buf.numel() * 8 < nbytes:
        buf = _nucleus_scratch[logits.device] = torch.empty(max(-(-nbytes // 8), 1 << 16), dtype=torch.int64,
                                                            device=logits.device)
    kernel("sampling", "gg_sample_nucleus")(_p(logits), logits.stride(0), float(temp), float(top_p), float(min_p),
                                             _p(uniforms), _p(out), _p(flags), R, V, _p(buf), buf.numel() * 8, _stream())


def sample(logits: torch.Tensor, temps: torch.Tensor, uniforms: torch.Tensor, out: torch.Tensor,
           rows: Optional[int] = None) -> None:
    _need(logits, torch.float32, "logits")
    _need(temps, torch.float32, "temps")
    _need(uniforms, torch.float64, "uniforms")
    _need(out, torch.int32, "out")
    R = logits.shape[0] if rows is None else rows
    V = logits.shape[1]
    words = R * 128 + 2 * R * (-(-V // 8192))
    scratch = _sample_scratch.get(logits.device)
    if scratch is None or scratch.numel() < words:
        scratch = _sample_scratch[logits.device] = torch.empty(max(words, 1 << 14), dtype=torch.int32, device=logits.device)
    kernel("sampling", "gg_sample")(_p(logits), logits.stride(0), _p(temps), _p(uniforms), _p(out), R, V,
                                     _p(scratch), scratch.numel(), _stream())
