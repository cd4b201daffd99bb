"""Grouped-query attention mixer with optional per-head q/k RMSNorm and a position encoding.

Order of operations as in the reference (pkg/model/qwen3/model.go:215-260): q, k, v projections
without bias; each q and k head normed over its `head_dim` slice with one shared weight (before the
rotation); rotation of q and k; k (normed, rotated) and v (raw) appended to the cache; attention of
every new token over the cached positions it may see; output projection added to the residual.
Score scale is 1/sqrt(head_dim) unless the spec gives `scale` (pkg/ops/attention.go:24).
"""
from __future__ import annotations

import math
import os
from typing import Dict, Optional

import torch

from ..cache.sequence_cache import KVRequest, KVView
from ..config.spec import PartSpec
from ..csrc import kernels as K
from ..csrc import tcgen05_gemm
from ..weights.loader import TensorDecl
from .base import Linear, Runtime, StepContext
from .registry import POSITIONS, lookup, register_mixer

MAX_HEAD_DIM = 256


@register_mixer("attention")
class AttentionMixer:
    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        h, nq, nkv, d = spec["hidden_size"], spec["num_heads"], spec["num_kv_heads"], spec["head_dim"]
        t = {
            "q_proj.weight": TensorDecl(shape=(nq * d, h)),
            "k_proj.weight": TensorDecl(shape=(nkv * d, h)),
            "v_proj.weight": TensorDecl(shape=(nkv * d, h)),
            "o_proj.weight": TensorDecl(shape=(h, nq * d)),
        }
        if spec.get("qk_norm"):
            t["q_norm.weight"] = TensorDecl(shape=(d,), init="ones_normal")
            t["k_norm.weight"] = TensorDecl(shape=(d,), init="ones_normal")
        return t

    @classmethod
    def cache_request(cls, spec: PartSpec) -> KVRequest:
        return KVRequest(num_kv_heads=int(spec["num_kv_heads"]), head_dim=int(spec["head_dim"]),
                         window=spec.get("window"))

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.rt = rt
        self.hidden = int(spec["hidden_size"])
        self.nq = int(spec["num_heads"])
        self.nkv = int(spec["num_kv_heads"])
        self.d = int(spec["head_dim"])
        if self.nq % self.nkv:
            raise ValueError(f"attention: {self.nq} query heads are not a multiple of {self.nkv} kv heads")
        if self.d > MAX_HEAD_DIM or self.d % 2:
            raise ValueError(f"attention: head_dim={self.d} is not supported (even, at most {MAX_HEAD_DIM})")
        self.window = int(spec.get("window") or 0)
        self.scale = float(spec.get("scale") or 1.0 / math.sqrt(self.d))
        self.eps = float(spec.get("qk_norm_eps", 0.0))
        pos = dict(spec["position"])
        self.position = lookup(POSITIONS, pos["kind"], "position encoding")(pos, rt)
        self.rot = int(pos.get("rotary_dim", self.d))
        if self.rot > self.d:
            raise ValueError("attention: rotary_dim exceeds head_dim")
        q, k, v = (rt.matrix(weights[n]) for n in ("q_proj.weight", "k_proj.weight", "v_proj.weight"))
        if not (q.dtype == k.dtype == v.dtype):
            q, k, v = q.float(), k.float(), v.float()
        # rows: all q heads, then all k heads, then all v heads
        self.qkv = Linear(torch.cat([q, k, v], dim=0), rt)
        self.o = Linear(weights["o_proj.weight"], rt)
        if spec.get("qk_norm"):
            self.q_norm = rt.vector(weights["q_norm.weight"])
            self.k_norm = rt.vector(weights["k_norm.weight"])
        else:
            self.q_norm = self.k_norm = None
        self._fast = None
        if rt.fast and rt.dtype == torch.bfloat16:
            from ..csrc import fast_attention
            self._fast = fast_attention.try_make(self.nq, self.nkv, self.d, self.scale, self.window)
        # head size 128 with a full rotation by cos/sin tables: the decode form of the q/k/v product can do
        # the per-head work itself (one head per 128-row weight tile)
        self._fused_rope = (self.qkv.tensor_core and self.d == 128 and self.rot == self.d
                            and os.environ.get("GOGGUF_B200_FUSE_QKV_ROPE", "1") != "0")

    def absorb_norm(self, norm) -> bool:
        """Take the block's pre-norm into the q/k/v projection; `forward` then gets RowStats as `h`."""
        if not self.qkv.can_fold or norm.size != self.hidden:
            return False
        self.qkv.fold_input_norm(norm.weight, norm.eps)
        return True

    def prepare(self, ctx: StepContext) -> None:
        self.position.tables(ctx)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext, cache: KVView,
                writes_cache: bool = True) -> None:
        T, nq, nkv, d = ctx.n_tokens, self.nq, self.nkv, self.d
        dt = self.rt.dtype
        q = ctx.ws.get("attn_q", (T, nq * d), dt)
        o = ctx.ws.get("attn_out", (T, nq * d), dt)
        cos, sin = self.position.tables(ctx)
        table = ctx.page_tables[cache.group]
        if self._fused_rope and tcgen05_gemm.qkv_rope_takes(T):
            # norm, rotation and cache write happen in the projection's epilogue
            self.qkv.qkv_rope(h, T, ws=ctx.ws, q_out=q, qw=self.q_norm, kw=self.k_norm, eps=self.eps, cos=cos, sin=sin,
                              positions=ctx.positions, seq_of_token=ctx.seq_of_token, page_table=table,
                              page_size=cache.page_size, k_pool=cache.k if writes_cache else None,
                              v_pool=cache.v if writes_cache else None, nq=nq, nkv=nkv)
        else:
            qkv = ctx.ws.get("attn_qkv", (T, (nq + 2 * nkv) * d), dt)
            self.qkv(h, qkv, ws=ctx.ws)
            K.qk_norm_rope_cache(qkv, q, self.q_norm, self.k_norm, self.eps, cos, sin, ctx.positions,
                                 ctx.seq_of_token, table, cache.page_size,
                                 cache.k if writes_cache else None, cache.v if writes_cache else None,
                                 T, nq, nkv, d, self.rot)
        if self._fast is not None:
            self._fast(q, cache.k, cache.v, o, ctx, table, cache.page_size)
        else:
            K.attention_plain(q, cache.k, cache.v, o, ctx.positions, ctx.seq_of_token, table,
                              cache.page_size, T, nq, nkv, d, self.scale, self.window)
        self.o(o, residual, accumulate=True, ws=ctx.ws, emit=ctx.shared.get("row_stats"))
