"""Host side of the tcgen05 tensor-core product (csrc/gemm_tcgen05.cu)."""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch

from .build import KernelError, kernel, module

OUT_BF16, OUT_F32, OUT_F32_ACC, OUT_SWIGLU = 0, 1, 2, 3

_status: Dict[torch.device, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """One int32 on the device that kernels write to when a bounded wait runs out or, in the debug build,
    when a page table holds an index or page id out of range."""
    device = torch.device(device)
    t = _status.get(device)
    if t is None:
        t = _status[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return t


def check_status(device: torch.device) -> None:
    """Raise if a kernel left a code in the status word since the last check (reads one int: a sync)."""
    t = _status.get(torch.device(device))
    if t is None:
        return
    v = int(t.item())
    if v != 0:
        t.zero_()
        if 41 <= v <= 48:
            who = {41: "attention_plain", 42: "attn_decode", 43: "attn_prefill", 44: "attn_decode_tma",
                   45: "attn_prefill_tc", 46: "qk_norm_rope_cache", 47: "qk_norm_rope_cache (16-byte form)",
                   48: "the q/k/v product's cache write"}[v]
            raise KernelError(f"debug build: kernel {who} met a page-table index or page id out of range (code {v}); "
                              "it read page 0 (a reader) or wrote nothing (a writer), results of that step are invalid")
        raise KernelError(f"a bounded wait inside a kernel ran out (code {v}: 1 TMA producer, 2 MMA issuer, "
                          "3 epilogue of a product, 11-12 decode attention, 21-28 prefill attention); "
                          "results of that step are invalid")


def splits_for(M: int, N: int, K: int, cluster: bool = False) -> int:
    raw = module("gemm_tcgen05").lib.gg_gemm_tc_splits
    return int(raw(int(M), int(N), int(K), int(bool(cluster))))


def pair_scratch_elems(M: int, N: int, K: int) -> int:
    """Floats of scratch with which a product of more than 128 tokens splits K over the CTA pairs (0: no split)."""
    import ctypes
    n = ctypes.c_longlong(0)
    raw = module("gemm_tcgen05").lib.gg_gemm_tc_pair_scratch_elems
    raw(int(M), int(N), int(K), ctypes.byref(n))
    return int(n.value)


def qkv_rope_takes(m: int) -> bool:
    """Does `gemm_tc_qkv_rope` take m tokens?  Up to 128 always (decode form); more in the CTA-pair form, which
    GOGGUF_B200_GEMM_PAIR=0 switches off."""
    import os
    return m <= 128 or os.environ.get("GOGGUF_B200_GEMM_PAIR", "1") != "0"


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Rows in blocks of 64 gate rows then their 64 up rows: the layout the fused SwiGLU epilogue reads."""
    I, K = gate.shape
    if I % 64:
        raise KernelError("interleave_gate_up: the intermediate size must be a multiple of 64")
    return torch.stack([gate.view(I // 64, 64, K), up.view(I // 64, 64, K)], dim=1).reshape(2 * I, K).contiguous()


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
            m: Optional[int] = None, scratch: Optional[torch.Tensor] = None, cluster: bool = False,
            swiglu: bool = False) -> None:
    """out[M, N] (+)= x[M, K] @ w[N, K]^T, bfloat16 operands, float32 accumulation on the tensor cores.

    Small M splits K.  cluster=True: the partial sums are added inside thread-block clusters (no scratch).
    cluster=False: they go through `scratch` (splits_for(M, N, K) * M * N floats) and a second kernel."""
    N, K = w.shape
    M = x.shape[0] if m is None else m
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc takes bfloat16 operands")
    if swiglu:
        if out.dtype != torch.bfloat16 or accumulate or out.shape[-1] != N // 2:
            raise KernelError("gemm_tc: the fused SwiGLU writes bfloat16 [M, N / 2]")
        mode = OUT_SWIGLU
    elif out.dtype == torch.bfloat16:
        if accumulate:
            raise KernelError("gemm_tc: sums are kept in float32")
        mode = OUT_BF16
    elif out.dtype == torch.float32:
        mode = OUT_F32_ACC if accumulate else OUT_F32
    else:
        raise KernelError(f"gemm_tc: output dtype {out.dtype}")
    if x.stride(-1) != 1 or out.stride(-1) != 1 or not w.is_contiguous():
        raise KernelError("gemm_tc: operands must be row-major")
    st = status_word(x.device)
    kernel("gemm_tcgen05", "gg_gemm_tc")(
        x.data_ptr(), w.data_ptr(), out.data_ptr(), mode, M, N, K, x.stride(0), out.stride(0),
        scratch.data_ptr() if scratch is not None else 0, scratch.numel() if scratch is not None else 0,
        int(bool(cluster)), st.data_ptr(), torch.cuda.current_stream().cuda_stream)


def gemm_tc_norm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
                 m: Optional[int] = None, swiglu: bool = False, in_ssq: Optional[torch.Tensor] = None,
                 eps: float = 0.0, out_ssq: Optional[torch.Tensor] = None,
                 out_xhat: Optional[torch.Tensor] = None, scratch: Optional[torch.Tensor] = None) -> None:
    """`gemm_tc` with an RMSNorm folded in on either side (K splits inside clusters).

    in_ssq [M, ceil(K / 128)]: x is the bfloat16 copy of raw residual rows and w carries the norm's weight;
    every output row is multiplied by 1 / sqrt(sum(in_ssq[row]) / K + eps).  out_ssq [M, ceil(N / 128)] and
    out_xhat [M, N] (accumulate only): the kernel also writes the bfloat16 copy of the updated rows and
    their partial sums of squares, the inputs of the next folded product.  scratch: room for the partial tiles
    of a K split at more than 128 tokens (`pair_scratch_elems`); without it the product runs unsplit."""
    N, K = w.shape
    M = x.shape[0] if m is None else m
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc_norm takes bfloat16 operands")
    if swiglu:
        if out.dtype != torch.bfloat16 or accumulate or out.shape[-1] != N // 2:
            raise KernelError("gemm_tc_norm: the fused SwiGLU writes bfloat16 [M, N / 2]")
        mode = OUT_SWIGLU
    elif out.dtype == torch.bfloat16:
        if accumulate:
            raise KernelError("gemm_tc_norm: sums are kept in float32")
        mode = OUT_BF16
    elif out.dtype == torch.float32:
        mode = OUT_F32_ACC if accumulate else OUT_F32
    else:
        raise KernelError(f"gemm_tc_norm: output dtype {out.dtype}")
    if x.stride(-1) != 1 or out.stride(-1) != 1 or not w.is_contiguous():
        raise KernelError("gemm_tc_norm: operands must be row-major")
    in_parts = 0
    if in_ssq is not None:
        in_parts = (K + 127) // 128
        if in_ssq.dtype != torch.float32 or not in_ssq.is_contiguous() or in_ssq.shape[-1] != in_parts \
                or in_ssq.numel() < M * in_parts:
            raise KernelError("gemm_tc_norm: in_ssq must be float32 [M, ceil(K / 128)]")
    if out_ssq is not None:
        if not accumulate or out_xhat is None:
            raise KernelError("gemm_tc_norm: row statistics are written by the accumulating form only")
        if out_ssq.dtype != torch.float32 or out_ssq.shape[-1] != (N + 127) // 128 or not out_ssq.is_contiguous() \
                or out_xhat.dtype != torch.bfloat16 or not out_xhat.is_contiguous() or out_xhat.shape[-1] != N \
                or out_ssq.numel() < M * ((N + 127) // 128) or out_xhat.numel() < M * N:
            raise KernelError("gemm_tc_norm: out_ssq is float32 [M, ceil(N / 128)], out_xhat bfloat16 [M, N]")
    st = status_word(x.device)
    kernel("gemm_tcgen05", "gg_gemm_tc_norm")(
        x.data_ptr(), w.data_ptr(), out.data_ptr(), mode, M, N, K, x.stride(0), out.stride(0),
        in_ssq.data_ptr() if in_ssq is not None else 0, in_parts, float(eps),
        out_ssq.data_ptr() if out_ssq is not None else 0, out_xhat.data_ptr() if out_xhat is not None else 0,
        scratch.data_ptr() if scratch is not None else 0, scratch.numel() if scratch is not None else 0,
        st.data_ptr(), torch.cuda.current_stream().cuda_stream)


def gemm_tc_qkv_rope(x: torch.Tensor, w: torch.Tensor, m: int, q_out: torch.Tensor, qw: Optional[torch.Tensor],
                     kw: Optional[torch.Tensor], eps: float, cos: torch.Tensor, sin: torch.Tensor,
                     positions: torch.Tensor, seq_of_token: torch.Tensor, page_table: torch.Tensor, page_size: int,
                     k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor], nq: int, nkv: int,
                     in_ssq: Optional[torch.Tensor] = None, in_eps: float = 0.0,
                     scratch: Optional[torch.Tensor] = None) -> None:
    """The q/k/v projection of a step (head size 128; any m, see `qkv_rope_takes`) with the per-head q/k RMSNorm,
    the rotation and the cache write in the product's epilogue (csrc/gemm_tcgen05.cu, gg_gemm_tc_qkv_rope).
    scratch: room for the partial tiles of a K split at more than 128 tokens (`pair_scratch_elems`); the kernel that
    adds them then does the per-head work."""
    N, K = w.shape
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or q_out.dtype != torch.bfloat16:
        raise KernelError("gemm_tc_qkv_rope takes bfloat16 operands")
    if N != (nq + 2 * nkv) * 128 or not qkv_rope_takes(m) or q_out.numel() < m * nq * 128 or not q_out.is_contiguous():
        raise KernelError("gemm_tc_qkv_rope: head size 128, q_out [m, nq * 128]; more than 128 tokens only in the "
                          "CTA-pair form")
    if cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.shape[-1] != 64 or sin.shape[-1] != 64 \
            or not cos.is_contiguous() or not sin.is_contiguous():
        raise KernelError("gemm_tc_qkv_rope: cos and sin are float32 [m, 64]")
    for t in (positions, seq_of_token, page_table):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError("gemm_tc_qkv_rope: integer inputs are contiguous int32")
    for t in (qw, kw):
        if t is not None and (t.dtype != torch.float32 or t.numel() != 128):
            raise KernelError("gemm_tc_qkv_rope: norm weights are float32 [128]")
    if k_pool is not None and (k_pool.dtype != torch.bfloat16 or v_pool is None or v_pool.dtype != torch.bfloat16):
        raise KernelError("gemm_tc_qkv_rope: the cache pools are bfloat16")
    in_parts = (K + 127) // 128 if in_ssq is not None else 0
    st = status_word(x.device)
    kernel("gemm_tcgen05", "gg_gemm_tc_qkv_rope")(
        x.data_ptr(), w.data_ptr(), m, K, x.stride(0), in_ssq.data_ptr() if in_ssq is not None else 0, in_parts,
        float(in_eps), q_out.data_ptr(), qw.data_ptr() if qw is not None else 0, kw.data_ptr() if kw is not None else 0,
        float(eps), cos.data_ptr(), sin.data_ptr(), positions.data_ptr(), seq_of_token.data_ptr(),
        page_table.data_ptr(), page_table.shape[-1], int(page_size), k_pool.shape[0] if k_pool is not None else 0,
        k_pool.data_ptr() if k_pool is not None else 0, v_pool.data_ptr() if v_pool is not None else 0,
        nq, nkv, scratch.data_ptr() if scratch is not None else 0, scratch.numel() if scratch is not None else 0,
        st.data_ptr(), torch.cuda.current_stream().cuda_stream)


def make_linear(weight: torch.Tensor, swiglu: bool = False) -> Optional[Callable]:
    """A callable f(x, out, accumulate, m, ws, in_ssq=None, eps=0.0, out_ssq=None, out_xhat=None) for this
    weight, or None if its sizes are not taken (K must be a multiple of 8 so that rows start on 16-byte
    boundaries for TMA).  swiglu=True: the weight is interleaved gate/up (see `interleave_gate_up`) and
    out is [M, N / 2].  The keyword arguments are those of `gemm_tc_norm`; a call that has to fall back
    to the plain kernel refuses them."""
    N, K = weight.shape
    if K % 8 != 0 or weight.data_ptr() % 16 != 0:
        return None
    if swiglu and (N % 128 != 0 or N < 256):
        return None

    split_room: Dict[int, int] = {}      # tokens -> floats of scratch with which the prefill form splits K

    def run(x, out, accumulate, m, ws, in_ssq=None, eps=0.0, out_ssq=None, out_xhat=None):
        folded = in_ssq is not None or out_ssq is not None
        if x.stride(0) % 8 != 0 or x.data_ptr() % 16 != 0:
            if swiglu or folded:
                raise KernelError("fused product: activations must be 16-byte aligned rows")
            from . import kernels as Kn
            Kn.gemm_plain(x, weight, out, accumulate, m)
            return
        M = x.shape[0] if m is None else m
        scratch = None
        if M > 128 and ws is not None:
            need = split_room.get(M)
            if need is None:
                need = split_room[M] = pair_scratch_elems(M, N, K)
            if need:
                scratch = ws.get("gemm_partial_tiles", (need,), torch.float32)
        if folded:
            gemm_tc_norm(x, weight, out, accumulate, m, swiglu, in_ssq, eps, out_ssq, out_xhat, scratch)
        else:
            gemm_tc(x, weight, out, accumulate, m, scratch, cluster=True, swiglu=swiglu)

    return run
