"""gogguf_b200: a small, whole Qwen3 inference library for NVIDIA B200 (sm_100a)."""
from . import config  # noqa: F401  (registers architectures)

__version__ = "0.1.0"
