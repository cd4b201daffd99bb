"""Binding of `Linear` to the tcgen05 tensor-core product (bfloat16 operands).

`try_make(weight)` returns a callable ``f(x, out, accumulate, m, ws)`` or None when the sizes
are outside what the kernel takes (then the plain kernel is used).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch


def try_make(weight: torch.Tensor) -> Optional[Callable]:
    from ..csrc import tcgen05_gemm
    return tcgen05_gemm.make_linear(weight)
