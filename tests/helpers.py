"""Shared test material: tiny configurations that differ in every size and option, model folders
made in temporary directories, and comparison helpers."""
from __future__ import annotations

import json
import os
from typing import Dict, List, Sequence

import numpy as np
import torch

# Two tiny Qwen3 configurations that differ in every size and option, plus one with windows.
TINY_A = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
    intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
    tie_word_embeddings=True, max_position_embeddings=512,
)
TINY_B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=1, head_dim=32,
    intermediate_size=160, vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5,
    tie_word_embeddings=False, max_position_embeddings=640,
)
# windows on two of four layers, sizes that are no power of two, head_dim 48, vocabulary 331
TINY_W = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=4, hidden_size=72, num_attention_heads=3, num_key_value_heads=3, head_dim=48,
    intermediate_size=104, vocab_size=331, rope_theta=50000.0, rms_norm_eps=3e-6,
    tie_word_embeddings=False, max_position_embeddings=512,
    sliding_window=37, layer_types=["sliding_attention", "full_attention", "full_attention", "sliding_attention"],
)
# head size 64 and 4 query heads per kv head: the sizes the tensor-core attention kernels take
TINY_M = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=136, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
    intermediate_size=200, vocab_size=523, rope_theta=200000.0, rms_norm_eps=2e-6,
    tie_word_embeddings=True, max_position_embeddings=1024,
    sliding_window=90, layer_types=["full_attention", "sliding_attention"],
)
# head size 128, one kv head for four query heads, widths that take the tensor-core products' fused paths
TINY_L = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=1, head_dim=128,
    intermediate_size=448, vocab_size=1000, rope_theta=1000000.0, rms_norm_eps=1e-6,
    tie_word_embeddings=False, max_position_embeddings=2048,
)
TINY = {"L": (TINY_L, 11, 0.03, 0.05), "M": (TINY_M, 9, 0.04, 0.05), "A": (TINY_A, 0, 0.02, 0.02), "B": (TINY_B, 1, 0.03, 0.05), "W": (TINY_W, 5, 0.05, 0.1)}


def make_folder(tmp, name: str, store_dtype: str = "float32", scale: float = 1.0) -> str:
    """Write tiny model `name` with the product's random-weights mode; returns the folder."""
    from gogguf_b200.config import config_from_dict
    from gogguf_b200.engine.model import write_random_model
    cfg, seed, std, nstd = TINY[name]
    folder = os.path.join(str(tmp), f"tiny_{name}_{store_dtype}")
    if not os.path.isdir(folder):
        write_random_model(config_from_dict(cfg), seed, folder, dtype=store_dtype, std=std * scale, norm_std=nstd)
    return folder


def read_folder(folder: str):
    """config dict and tensors, read with the third-party safetensors package (not the product's reader)."""
    from safetensors import safe_open
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    w: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            w[k] = f.get_tensor(k)
    return cfg, w


def random_tokens(vocab: int, n: int, seed: int) -> List[int]:
    rng = np.random.default_rng(seed)
    return [int(x) for x in rng.integers(0, vocab, size=n)]


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """max |a-b| relative to the scale of b (its max abs), a robust figure for logits."""
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


# tolerances: float32 engine against the float32/float64 plain implementation, and bfloat16 engine.
# The bfloat16 bound is for models whose weights were scaled up (make_folder(scale=4)) and for drawn
# configurations: rounding activations to bfloat16 alone costs up to 2.5e-2 there (the plain kernels show the
# same).  Tests of fixed configurations use tighter bounds beside it (tests/test_gpu_whole.py,
# tests/test_gpu_bench_shapes.py), and each kernel alone is held to 8e-3.
TOL_F32 = 2e-5
TOL_BF16 = 4e-2
