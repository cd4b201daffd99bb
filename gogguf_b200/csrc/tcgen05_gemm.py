"""Host side of the tcgen05 tensor-core product: tensor maps, tile choice, launch."""
from __future__ import annotations

from typing import Callable, Optional

import torch


def make_linear(weight: torch.Tensor) -> Optional[Callable]:
    """A callable f(x, out, accumulate, m, ws) for this weight, or None if its sizes are not taken."""
    return None
