"""Typed configuration of the Qwen3 dense decoder, read from its config.json keys.

The reference reads the same ten hyper-parameters from GGUF metadata
(pkg/model/qwen3/config.go:24-101): context length, embedding width, feed
forward width, block count, head counts, a head size decoupled from
``hidden/heads`` (config.go:70-73), the norm epsilon (default 1e-6,
config.go:60-63) and the rotary base (default 1e6, config.go:65-68).  The lm
head is the embedding when no separate output matrix exists
(pkg/model/qwen3/tensors.go:36-48); here ``tie_word_embeddings`` says so.

Everything the block structure needs is turned into a `ModelSpec` by
`to_spec`; no size lives anywhere else.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from .registry import ConfigError, register_architecture
from .spec import BlockSpec, ModelSpec, PartSpec, ScheduleEntry, default_schedule

_FULL = "full_attention"
_SLIDING = "sliding_attention"


def _req_int(d: Dict[str, Any], key: str) -> int:
    if key not in d or d[key] is None:
        raise ConfigError(f"qwen3 config: required key {key!r} is missing")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"qwen3 config: {key!r} must be an integer, got {v!r}")
    if v <= 0:
        raise ConfigError(f"qwen3 config: {key!r} must be positive, got {v}")
    return v


@register_architecture("Qwen3ForCausalLM", "qwen3")
@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    # one entry per layer: "full_attention" or "sliding_attention"
    layer_types: Tuple[str, ...]
    sliding_window: Optional[int]
    eos_token_ids: Tuple[int, ...] = ()
    initializer_range: float = 0.02

    # ------------------------------------------------------------------ parse
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen3Config":
        hidden = _req_int(d, "hidden_size")
        heads = _req_int(d, "num_attention_heads")
        layers = _req_int(d, "num_hidden_layers")
        kv_heads = d.get("num_key_value_heads")
        kv_heads = heads if kv_heads is None else _req_int(d, "num_key_value_heads")
        # head size: its own key, else hidden/heads (config.go:70-73)
        if d.get("head_dim") is not None:
            head_dim = _req_int(d, "head_dim")
        else:
            if hidden % heads:
                raise ConfigError(
                    f"qwen3 config: no 'head_dim' and hidden_size={hidden} is not divisible by "
                    f"num_attention_heads={heads}")
            head_dim = hidden // heads
        if heads % kv_heads:
            raise ConfigError(
                f"qwen3 config: num_attention_heads={heads} is not a multiple of "
                f"num_key_value_heads={kv_heads}")
        if head_dim % 2:
            raise ConfigError(f"qwen3 config: head_dim={head_dim} must be even for rotary pairs")
        if d.get("attention_bias"):
            raise ConfigError("qwen3 config: attention_bias=true is not supported (the projections have no bias)")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"qwen3 config: hidden_act={act!r} is not supported (only 'silu')")
        if d.get("rope_scaling") not in (None, {}):
            raise ConfigError("qwen3 config: rope_scaling is not supported (plain rotary positions only)")

        eps = float(d.get("rms_norm_eps", 1e-6))          # config.go:60-63
        theta = float(d.get("rope_theta", 1000000.0))      # config.go:65-68
        if not eps > 0:
            raise ConfigError(f"qwen3 config: rms_norm_eps must be > 0, got {eps}")
        if not theta > 0:
            raise ConfigError(f"qwen3 config: rope_theta must be > 0, got {theta}")

        window = d.get("sliding_window")
        if window is not None:
            if isinstance(window, bool) or not isinstance(window, int) or window <= 0:
                raise ConfigError(f"qwen3 config: sliding_window must be a positive integer or null, got {window!r}")
        lt = d.get("layer_types")
        if lt is not None:
            if not isinstance(lt, (list, tuple)) or len(lt) != layers:
                raise ConfigError(f"qwen3 config: layer_types must list {layers} entries")
            for t in lt:
                if t not in (_FULL, _SLIDING):
                    raise ConfigError(f"qwen3 config: unknown layer type {t!r}")
            layer_types = tuple(lt)
        elif d.get("use_sliding_window") and window is not None:
            first_sliding = int(d.get("max_window_layers", layers))
            layer_types = tuple(_SLIDING if i >= first_sliding else _FULL for i in range(layers))
        else:
            layer_types = tuple(_FULL for _ in range(layers))
        if _SLIDING in layer_types and window is None:
            raise ConfigError("qwen3 config: sliding_attention layers need 'sliding_window'")

        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(x) for x in eos)
        else:
            eos_ids = (int(eos),)

        return cls(
            vocab_size=_req_int(d, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_req_int(d, "intermediate_size"),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            max_position_embeddings=_req_int(d, "max_position_embeddings"),
            rms_norm_eps=eps,
            rope_theta=theta,
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            layer_types=layer_types,
            sliding_window=window,
            eos_token_ids=eos_ids,
            initializer_range=float(d.get("initializer_range", 0.02)),
        )

    # ------------------------------------------------------------------ write
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": ["Qwen3ForCausalLM"],
            "model_type": "qwen3",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "initializer_range": self.initializer_range,
        }
        if _SLIDING in self.layer_types:
            d["layer_types"] = list(self.layer_types)
            d["sliding_window"] = self.sliding_window
            d["use_sliding_window"] = True
        else:
            d["sliding_window"] = None
            d["use_sliding_window"] = False
        if self.eos_token_ids:
            d["eos_token_id"] = (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                                 else list(self.eos_token_ids))
        return d

    # ------------------------------------------------------------- derived
    @property
    def q_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def parameter_count(self) -> int:
        h, i = self.hidden_size, self.intermediate_size
        per_layer = (self.q_width + 2 * self.kv_width) * h + h * self.q_width \
            + 3 * h * i + 2 * h + 2 * self.head_dim
        n = self.num_hidden_layers * per_layer + self.vocab_size * h + h
        if not self.tie_word_embeddings:
            n += self.vocab_size * h
        return n

    def kv_bytes_per_token(self, itemsize: int = 2) -> int:
        return 2 * self.num_hidden_layers * self.kv_width * itemsize

    # -------------------------------------------------------------- aliases
    def tensor_aliases(self) -> Dict[str, str]:
        """The reference's GGUF tensor names (pkg/model/qwen3/tensors.go:19-34, norms.go:16-45) mapped to
        the checkpoint names; a folder may use either."""
        m = {"token_embd.weight": "model.embed_tokens.weight", "output_norm.weight": "model.norm.weight",
             "output.weight": "lm_head.weight"}
        per_layer = {
            "attn_norm.weight": "input_layernorm.weight", "ffn_norm.weight": "post_attention_layernorm.weight",
            "attn_q.weight": "self_attn.q_proj.weight", "attn_k.weight": "self_attn.k_proj.weight",
            "attn_v.weight": "self_attn.v_proj.weight", "attn_output.weight": "self_attn.o_proj.weight",
            "attn_q_norm.weight": "self_attn.q_norm.weight", "attn_k_norm.weight": "self_attn.k_norm.weight",
            "ffn_gate.weight": "mlp.gate_proj.weight", "ffn_up.weight": "mlp.up_proj.weight",
            "ffn_down.weight": "mlp.down_proj.weight",
        }
        for i in range(self.num_hidden_layers):
            for a, b in per_layer.items():
                m[f"blk.{i}.{a}"] = f"model.layers.{i}.{b}"
        return m

    # ---------------------------------------------------------------- spec
    def to_spec(self) -> ModelSpec:
        """Block structure of the reference's forwardBlock (pkg/model/qwen3/model.go:198-288)."""
        blocks: List[BlockSpec] = []
        rope = {"kind": "rope_neox", "theta": self.rope_theta, "rotary_dim": self.head_dim}
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            window = self.sliding_window if self.layer_types[i] == _SLIDING else None
            mixer = PartSpec(
                kind="attention",
                prefix=p + "self_attn.",
                params=dict(
                    hidden_size=self.hidden_size,
                    num_heads=self.num_attention_heads,
                    num_kv_heads=self.num_key_value_heads,
                    head_dim=self.head_dim,
                    qk_norm=True,                      # model.go:227-233
                    qk_norm_eps=self.rms_norm_eps,     # same eps as the other norms
                    window=window,
                    position=rope,
                ),
            )
            ffn = PartSpec(
                kind="swiglu",
                prefix=p + "mlp.",
                params=dict(hidden_size=self.hidden_size, intermediate_size=self.intermediate_size),
            )
            n1 = PartSpec(kind="rmsnorm", prefix=p + "input_layernorm.",
                          params=dict(size=self.hidden_size, eps=self.rms_norm_eps))
            n2 = PartSpec(kind="rmsnorm", prefix=p + "post_attention_layernorm.",
                          params=dict(size=self.hidden_size, eps=self.rms_norm_eps))
            blocks.append(BlockSpec(arrangement="pre_norm", mixer=mixer, feed_forward=ffn,
                                    mixer_norm=n1, feed_forward_norm=n2))
        spec = ModelSpec(
            architecture="Qwen3ForCausalLM",
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            max_positions=self.max_position_embeddings,
            blocks=tuple(blocks),
            schedule=default_schedule(self.num_hidden_layers),
            embedding=PartSpec(kind="embedding", prefix="model.embed_tokens.",
                               params=dict(vocab_size=self.vocab_size, hidden_size=self.hidden_size)),
            final_norm=PartSpec(kind="rmsnorm", prefix="model.norm.",
                                params=dict(size=self.hidden_size, eps=self.rms_norm_eps)),
            head=PartSpec(kind="linear_head", prefix="lm_head.",
                          params=dict(vocab_size=self.vocab_size, hidden_size=self.hidden_size,
                                      tied_to="model.embed_tokens.weight" if self.tie_word_embeddings else None)),
            stop_token_ids=self.eos_token_ids,
        )
        spec.validate()
        return spec
