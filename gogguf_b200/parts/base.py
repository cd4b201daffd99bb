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


class Linear:
    """y = x W^T for a weight W[N, K]; float32 accumulation, optional add into a float32 output.

    The bfloat16 path uses the tcgen05 tensor-core kernel when the sizes allow it and the plain CUDA
    core kernel otherwise (and always in the 32-bit path and for a matrix stored in 32-bit).
    """

    def __init__(self, weight: torch.Tensor, rt: Runtime):
        self.rt = rt
        self.weight = rt.matrix(weight)
        self.out_features, self.in_features = self.weight.shape
        self._fast = None
        if rt.fast and rt.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16:
            from ..csrc import tcgen05_gemm
            self._fast = tcgen05_gemm.make_linear(self.weight)

    def __call__(self, x: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
                 m: Optional[int] = None, ws: Optional[Workspace] = None) -> None:
        if self._fast is not None and x.dtype == torch.bfloat16:
            self._fast(x, out, accumulate, m, ws)
        else:
            K.gemm_plain(x, self.weight, out, accumulate, m)
