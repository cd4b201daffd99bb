"""What the parts share: the runtime description, the per-step context, workspaces, and the
linear projection that every part with a matrix uses.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

import torch

from ..csrc import kernels as K


@dataclass
class Runtime:
    """How a model is run: compute dtype, device, and whether the tensor-core kernels are used.

    dtype float32: everything is true 32-bit on the CUDA cores (no reduced-precision matrix mode).
    dtype bfloat16: activations and the cache are bfloat16; the residual stream, norms, softmax,
    rotary angles and logits stay float32.  `fast=False` keeps bfloat16 storage but runs the plain
    kernels (the twins the fast kernels are checked against).
    """
    dtype: torch.dtype
    device: torch.device
    fast: bool = True
    # fast bfloat16 path only: a block's pre-norm is folded into the product that follows it (see RowStats)
    fold_norms: bool = True

    def matrix(self, t: torch.Tensor) -> torch.Tensor:
        """A projection matrix as the compute path keeps it: float32 in the 32-bit path; in the
        bfloat16 path a bfloat16 tensor stays bfloat16 and a tensor stored in 32-bit stays 32-bit."""
        t = t.to(self.device)
        if self.dtype == torch.float32:
            return t.float().contiguous()
        return t.contiguous()

    def vector(self, t: torch.Tensor) -> torch.Tensor:
        """Norm weights are applied in float32 whatever they were stored in."""
        return t.to(self.device).float().contiguous()


class Workspace:
    """Named scratch buffers that are reused from step to step and grow on demand."""

    def __init__(self, device):
        self.device = device
        self._bufs: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}

    def get(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[key] = buf
        return buf[:n].view(*shape)


@dataclass
class StepContext:
    """Everything a part may need to know about the step it runs in.

    All tensors are int32 on the device.  `n_tokens` rows are processed; rows whose
    `seq_of_token` is negative are padding and must not change any result.
    """
    runtime: Runtime
    ws: Workspace
    n_tokens: int                 # rows in this step (padding included)
    n_seqs: int                   # sequences in this step (padding included)
    tokens: torch.Tensor          # [n_tokens] token ids (-1 on padding)
    positions: torch.Tensor       # [n_tokens] absolute position of each token
    seq_of_token: torch.Tensor    # [n_tokens] row of the batch the token belongs to (-1 on padding)
    cu_seqlens: torch.Tensor      # [n_seqs + 1] prefix sums of the new-token counts
    slots: torch.Tensor           # [n_seqs] cache slot of each sequence
    ctx_lens: torch.Tensor        # [n_seqs] length of each sequence after this step (0 on padding)
    page_tables: Dict[int, torch.Tensor]  # KV group -> [n_seqs, width]
    max_new: int                  # most new tokens of one sequence (host)
    max_ctx: int                  # longest sequence after this step (host; an upper bound under a graph)
    decode: bool                  # every sequence brings exactly one token
    shared: Dict[Any, Any] = field(default_factory=dict)   # per-step values parts share (rotary tables)


class RowStats:
    """The residual stream as a product with a folded RMSNorm reads it.

    RMSNorm(x) W^T = (x / rms(x)) (W diag(w))^T: the norm's weight w goes into the matrix once, when the
    model is built; the product reads `xhat`, the bfloat16 copy of the raw float32 rows, and multiplies
    each accumulator row by 1 / sqrt(sum(ssq[row]) / H + eps) in float32.  `ssq` holds, per row, the sums
    of squares over blocks of 128 columns.  A product that adds into the residual stream can write both
    for the rows it has just updated (`Linear(..., emit=stats)`), so in a chain of such products no norm
    kernel runs at all.  `fresh` says whether xhat and ssq describe the residual rows as they are now:
    a block clears it before a part writes to the residual, a product that emitted sets it, and
    `ensure` runs the stand-alone kernel when it is not set (after the embedding, after a part that
    does not emit).
    """

    def __init__(self, xhat: torch.Tensor, ssq: torch.Tensor):
        self.xhat, self.ssq = xhat, ssq
        self.fresh = False

    def ensure(self, x: torch.Tensor) -> "RowStats":
        if not self.fresh:
            K.row_stats(x, self.xhat, self.ssq)
            self.fresh = True
        return self


class Linear:
    """y = x W^T for a weight W[N, K]; float32 accumulation, optional add into a float32 output.

    The bfloat16 path uses the tcgen05 tensor-core kernel when the sizes allow it and the plain CUDA
    core kernel otherwise (and always in the 32-bit path and for a matrix stored in 32-bit).

    `fold_input_norm` turns the projection into one that reads `RowStats` instead of normalised rows;
    `emit=stats` asks an accumulating product to write the statistics of the rows it updates.
    """

    def __init__(self, weight: torch.Tensor, rt: Runtime, swiglu: bool = False):
        self.rt = rt
        self.weight = rt.matrix(weight)
        self.out_features, self.in_features = self.weight.shape
        self.swiglu = swiglu
        self.folded_eps: Optional[float] = None
        self._fast = None
        if rt.fast and rt.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16:
            from ..csrc import tcgen05_gemm
            self._fast = tcgen05_gemm.make_linear(self.weight, swiglu=swiglu)
        if swiglu and self._fast is None:
            raise ValueError("Linear: the fused SwiGLU form needs the tensor-core kernel")

    @property
    def can_fold(self) -> bool:
        return self._fast is not None and self.rt.fold_norms

    def fold_input_norm(self, norm_weight: torch.Tensor, eps: float) -> None:
        """Multiply the norm's weight into the columns of this matrix (float32 product, rounded once)."""
        if not self.can_fold:
            raise ValueError("Linear: this projection has no tensor-core form to fold a norm into")
        from ..csrc import tcgen05_gemm
        w = (self.weight.float() * norm_weight.to(self.weight.device).float()[None, :]).to(torch.bfloat16).contiguous()
        self.weight = w
        self._fast = tcgen05_gemm.make_linear(w, swiglu=self.swiglu)
        self.folded_eps = float(eps)

    @property
    def tensor_core(self) -> bool:
        return self._fast is not None

    def qkv_rope(self, x, m: int, ws: Optional[Workspace] = None, **outputs) -> None:
        """This projection as the q/k/v projection of a step, with q/k norm, rotation and cache write
        in its epilogue (`csrc.tcgen05_gemm.gemm_tc_qkv_rope`, whose keyword arguments `outputs` are).  With a
        workspace, a product of a few hundred tokens may split K over the CTA pairs."""
        from ..csrc import tcgen05_gemm
        if ws is not None and m > 128:
            need = tcgen05_gemm.pair_scratch_elems(m, self.weight.shape[0], self.weight.shape[1])
            if need:
                outputs["scratch"] = ws.get("gemm_partial_tiles", (need,), torch.float32)
        if self.folded_eps is not None:
            if not isinstance(x, RowStats):
                raise TypeError("Linear: a projection with a folded norm reads RowStats, not normalised rows")
            outputs.update(in_ssq=x.ssq, in_eps=self.folded_eps)
            x = x.xhat
        tcgen05_gemm.gemm_tc_qkv_rope(x, self.weight, m, **outputs)

    def __call__(self, x, out: torch.Tensor, accumulate: bool = False, m: Optional[int] = None,
                 ws: Optional[Workspace] = None, emit: Optional[RowStats] = None) -> None:
        kw = {}
        if self.folded_eps is not None:
            if not isinstance(x, RowStats):
                raise TypeError("Linear: a projection with a folded norm reads RowStats, not normalised rows")
            kw.update(in_ssq=x.ssq, eps=self.folded_eps)
            x = x.xhat
        elif isinstance(x, RowStats):
            raise TypeError("Linear: RowStats given to a projection without a folded norm")
        if (emit is not None and accumulate and self._fast is not None and x.dtype == torch.bfloat16
                and x.data_ptr() != emit.xhat.data_ptr() and out.shape[-1] == emit.xhat.shape[-1]
                and out.is_contiguous()):
            kw.update(out_ssq=emit.ssq, out_xhat=emit.xhat)
            emit.fresh = True
        if self._fast is not None and x.dtype == torch.bfloat16:
            self._fast(x, out, accumulate, m, ws, **kw)
        else:
            K.gemm_plain(x, self.weight, out, accumulate, m)
