"""A plain, slow implementation of the Qwen3 dense decoder: whole sequences, no cache.

Written from the formulas of the reference's CPU path (magomedcoder/gogguf); each
function cites the file and lines it restates.  The reference's own model code
is Go and cannot be compiled or imported here (no Go toolchain, no network), so
this file rests on the formulas, not on a run of the reference.

It shares no code with the `gogguf_b200` package: it takes a parsed config.json
(a dict) and a dict of tensors by checkpoint name, and works on the CPU in
float32 with float64 in the places where the reference widens (the norm's
inverse square root, rotary angles and rotation, the softmax's exp and sum, the
SiLU's exp).  With ``wide=True`` all arithmetic is float64, which gives a
tighter oracle for the 32-bit engine path.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


# --------------------------------------------------------------------------- config
def plain_config(cfg: dict) -> dict:
    """The numbers the forward pass needs, with the reference's defaults.

    pkg/model/qwen3/config.go:24-101: eps default 1e-6 (:60-63), rotary base
    default 1e6 (:65-68), head size from its own key else hidden/heads (:70-73).
    """
    heads = cfg["num_attention_heads"]
    layers = cfg["num_hidden_layers"]
    c = dict(
        layers=layers,
        hidden=cfg["hidden_size"],
        heads=heads,
        kv_heads=cfg.get("num_key_value_heads") or heads,
        head_dim=cfg.get("head_dim") or cfg["hidden_size"] // heads,
        inter=cfg["intermediate_size"],
        vocab=cfg["vocab_size"],
        eps=float(cfg.get("rms_norm_eps", 1e-6)),
        theta=float(cfg.get("rope_theta", 1e6)),
        tied=bool(cfg.get("tie_word_embeddings", False)),
    )
    window = cfg.get("sliding_window")
    lt = cfg.get("layer_types")
    if lt is None:
        if cfg.get("use_sliding_window") and window is not None:
            first = cfg.get("max_window_layers", layers)
            lt = ["sliding_attention" if i >= first else "full_attention" for i in range(layers)]
        else:
            lt = ["full_attention"] * layers
    c["windows"] = [window if t == "sliding_attention" else None for t in lt]
    return c


# --------------------------------------------------------------------------- parts
def embed(table: torch.Tensor, tokens: Sequence[int]) -> torch.Tensor:
    """x = E[tok]: a row gather, no scaling (pkg/model/qwen3/model.go:169-196, row offset :192-193)."""
    return table[torch.as_tensor(list(tokens), dtype=torch.long)].clone()


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, wide: bool = False) -> torch.Tensor:
    """out = x * (1/sqrt(mean(x^2) + eps)) * w over the last axis.

    pkg/ops/rmsnorm.go:16-25: sum of squares in float32, eps added to the mean
    inside the root, the inverse root taken in float64 and cast to float32,
    then (x*scale)*w (:10-14).
    """
    if wide:
        x64 = x.double()
        scale = 1.0 / torch.sqrt((x64 * x64).mean(dim=-1, keepdim=True) + eps)
        return x64 * scale * w.double()
    xf = x.float()
    mean = (xf * xf).sum(dim=-1, keepdim=True) / xf.shape[-1]
    scale = (1.0 / torch.sqrt((mean + torch.tensor(eps, dtype=torch.float32)).double())).float()
    return xf * scale * w.float()


def rope_tables(positions: Sequence[int], head_dim: int, theta: float):
    """cos/sin tables: angle(pos, i) = pos * theta^(-2i/d), i < d/2, in float64, stored float32.

    pkg/ops/rope_tables.go:6-20.  Returned as float64 tensors holding the
    float32-rounded values.
    """
    half = head_dim // 2
    pos = torch.as_tensor(list(positions), dtype=torch.float64)[:, None]
    i = torch.arange(half, dtype=torch.float64)[None, :]
    ang = pos * torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * i / head_dim)
    return torch.cos(ang).float().double(), torch.sin(ang).float().double()


def rope_neox(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, wide: bool = False) -> torch.Tensor:
    """NeoX rotation of x[T, heads, d]: pairs (i, i+d/2), computed in float64, stored float32.

    pkg/ops/rope_heads.go:30-38: x0' = x0*c - x1*s ; x1' = x0*s + x1*c.
    """
    half = x.shape[-1] // 2
    x64 = x.double()
    x0, x1 = x64[..., :half], x64[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    out = torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)
    return out if wide else out.float()


def softmax_rows(s: torch.Tensor, wide: bool = False) -> torch.Tensor:
    """softmax over the last axis: max in float32, exp and sum in float64, e stored float32,
    scaled by float32(1/sum) (pkg/ops/softmax.go:6-21).  -inf entries give 0."""
    if wide:
        m = s.max(dim=-1, keepdim=True).values
        e = torch.exp(s - m)
        return e / e.sum(dim=-1, keepdim=True)
    m = s.max(dim=-1, keepdim=True).values
    e = torch.exp((s - m).double())
    total = e.sum(dim=-1, keepdim=True)
    return e.float() * (1.0 / total).float()


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: Optional[int] = None,
              wide: bool = False, q_pos: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Causal grouped-query attention over one whole sequence.

    q[T, heads, d], k and v [T, kv_heads, d] (k already normed and rotated, v raw).
    pkg/ops/attention.go:10-47: query head h reads kv head h div (heads/kv_heads) (:27);
    score = dot(q, k) * float32(1/sqrt(d)) (:24,:33); softmax over the visible keys;
    out = sum_t p_t * v_t (:38-43).  A token sees keys 0..pos, itself included
    (pkg/model/qwen3/model.go:244-246); with a window w only the last w of them.

    `q_pos`: q holds only the queries at these positions (for long sequences of which a few rows are
    wanted); default: one query per key.  Queries are taken in blocks so that a long sequence fits.
    """
    Tk = k.shape[0]
    Tq, H, d = q.shape
    G = H // k.shape[1]
    dt = torch.float64 if wide else torch.float32
    scale = torch.tensor(1.0 / math.sqrt(d), dtype=dt)
    pos = torch.arange(Tk) if q_pos is None else torch.as_tensor(list(q_pos), dtype=torch.long)
    j = torch.arange(Tk)[None, :]
    out = torch.empty(Tq, H, d, dtype=dt)
    kt, vt = k.to(dt), v.to(dt)
    block = max(1, min(Tq, (1 << 24) // max(Tk, 1)))
    for a in range(0, Tq, block):
        i = pos[a:a + block, None]
        visible = j <= i
        if window is not None:
            visible &= j > i - window
        for h in range(H):
            g = h // G
            s = (q[a:a + block, h, :].to(dt) @ kt[:, g, :].T) * scale
            s = s.masked_fill(~visible, float("-inf"))
            p = softmax_rows(s, wide)
            out[a:a + block, h, :] = p.to(dt) @ vt[:, g, :]
    return out


def silu(x: torch.Tensor, wide: bool = False) -> torch.Tensor:
    """x / (1 + exp(-x)) with the exp in float64 (pkg/ops/ops.go:316-318)."""
    if wide:
        return x / (1.0 + torch.exp(-x))
    return x / (1.0 + torch.exp(-x.double()).float())


def swiglu_ffn(h: torch.Tensor, w_gate, w_up, w_down, wide: bool = False) -> torch.Tensor:
    """down( silu(gate h) * (up h) ) (pkg/model/qwen3/model.go:273-286; pkg/ops/inplace.go:14-19)."""
    dt = torch.float64 if wide else torch.float32
    g = h.to(dt) @ w_gate.to(dt).T
    u = h.to(dt) @ w_up.to(dt).T
    return (silu(g, wide) * u) @ w_down.to(dt).T


def attention_mixer(h, w, prefix, c, positions, window, wide=False, rows=None):
    """q,k,v projections, per-head q/k RMSNorm, rotary, attention, output projection.
    `rows`: compute the output only for these rows of h (keys and values still come from all rows).

    pkg/model/qwen3/model.go:215-260: no bias (:215-225); each head's slice is normed with one
    [d] weight shared by the heads and the model's eps (:227-233, :663-676) BEFORE the rotation
    (:235-236); v is left as it is.
    """
    dt = torch.float64 if wide else torch.float32
    T = h.shape[0]
    d = c["head_dim"]
    hq = h if rows is None else h[list(rows)]
    q = (hq.to(dt) @ w[prefix + "q_proj.weight"].to(dt).T).reshape(hq.shape[0], c["heads"], d)
    k = (h.to(dt) @ w[prefix + "k_proj.weight"].to(dt).T).reshape(T, c["kv_heads"], d)
    v = (h.to(dt) @ w[prefix + "v_proj.weight"].to(dt).T).reshape(T, c["kv_heads"], d)
    q = rms_norm(q, w[prefix + "q_norm.weight"], c["eps"], wide)
    k = rms_norm(k, w[prefix + "k_norm.weight"], c["eps"], wide)
    cos, sin = rope_tables(positions, d, c["theta"])
    k = rope_neox(k, cos, sin, wide)
    if rows is None:
        q = rope_neox(q, cos, sin, wide)
        o = attention(q, k, v, window, wide)
    else:
        idx = list(rows)
        q = rope_neox(q, cos[idx], sin[idx], wide)
        o = attention(q, k, v, window, wide, q_pos=[positions[r] for r in idx])
    return o.reshape(-1, c["heads"] * d) @ w[prefix + "o_proj.weight"].to(dt).T


def block(x, w, layer, c, positions, wide=False, rows=None):
    """One pre-norm block with two residual adds (pkg/model/qwen3/model.go:198-288).
    `rows`: return only these rows (the attention still reads every row's keys and values)."""
    p = f"model.layers.{layer}."
    h = rms_norm(x, w[p + "input_layernorm.weight"], c["eps"], wide)
    a = attention_mixer(h, w, p + "self_attn.", c, positions, c["windows"][layer], wide, rows)
    x = (x if rows is None else x[list(rows)]) + a
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], c["eps"], wide)
    x = x + swiglu_ffn(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                       w[p + "mlp.down_proj.weight"], wide)
    return x


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], wide: bool = False,
            taps: Optional[list] = None, rows: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence starting at position 0 (`rows`: only of these positions;
    the last block and the head then run on those rows alone, which keeps long sequences affordable).

    pkg/model/qwen3/model.go:112-167 (embed, blocks in order) and :578-610 (final norm, then
    the head, which is the embedding matrix when no separate head exists, tensors.go:36-48).
    `taps`, if given, receives the hidden state after the embedding and after each block.
    """
    c = plain_config(cfg)
    dt = torch.float64 if wide else torch.float32
    x = embed(w["model.embed_tokens.weight"], tokens).to(dt)
    if taps is not None:
        taps.append(x.clone())
    positions = list(range(len(tokens)))
    for layer in range(c["layers"]):
        x = block(x, w, layer, c, positions, wide, rows if layer == c["layers"] - 1 else None)
        if taps is not None:
            taps.append(x.clone())
    h = rms_norm(x, w["model.norm.weight"], c["eps"], wide)
    head = w["model.embed_tokens.weight"] if c["tied"] or "lm_head.weight" not in w else w["lm_head.weight"]
    return h @ head.to(dt).T


# --------------------------------------------------------------------------- sampling
def greedy(logits: Sequence[float]) -> int:
    """First index of the maximum, strict '>' (pkg/sampler/greedy.go:4-17)."""
    best = 0
    for i in range(1, len(logits)):
        if logits[i] > logits[best]:
            best = i
    return best


def repeat_penalty(logits: List[float], history: Sequence[int], penalty: float, last_n: int) -> None:
    """Each distinct id of the last n of the history once: logit>0 ? /penalty : *penalty
    (pkg/sampler/penalties.go:5-32); n = 0 means 64 (pkg/runtime/session.go:87-91)."""
    if penalty == 1 or not history:
        return
    h = list(history[-last_n:]) if last_n > 0 and len(history) > last_n else list(history)
    seen = set()
    for t in h:
        if t < 0 or t >= len(logits) or t in seen:
            continue
        seen.add(t)
        logits[t] = logits[t] / penalty if logits[t] > 0 else logits[t] * penalty


def uniform01(seed: int, stream: int, step: int) -> float:
    """The engine's counter-based uniform draw, restated: splitmix64 finaliser over
    (seed, stream, step), top 53 bits / 2^53.  (The reference draws from one PCG stream per
    sampler object, pkg/sampler/chain.go:23; a batch needs draws that do not depend on the
    neighbours, so the stream is keyed by the request instead.)"""
    M = (1 << 64) - 1

    def mix(z):
        z = (z + 0x9E3779B97F4A7C15) & M
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
        return z ^ (z >> 31)

    z = mix(seed & M)
    z = mix(z ^ (stream & M))
    z = mix(z ^ (step & M))
    return (z >> 11) / float(1 << 53)


def sample(logits: Sequence[float], temp: float, top_k: int, top_p: float, min_p: float, u: float) -> int:
    """The reference's sampling chain (pkg/sampler/chain.go:18-70) with the uniform draw given.

    greedy when temp<=0 and no top-k and no top-p (:19-21); temperature in float64 (probs.go:40-49);
    top-k keeps the k largest (:77-103); min-p masks prob < min_p*max (penalties.go:35-54); masked
    logits become -1e10 (:57-61); softmax in float64 (probs.go:20-38); top-p keeps the sorted
    prefix until the sum reaches p-1e-6 (:105-133); the draw walks the ids in order subtracting
    their probability from r = u*sum and returns the first id at which r <= 0 (:135-166).
    """
    import numpy as np
    n = len(logits)
    if temp <= 0 and top_k <= 0 and (top_p <= 0 or top_p >= 1):
        return greedy(logits)
    x = np.asarray(logits, dtype=np.float32).copy()
    if temp > 0 and temp != 1:
        x = (x.astype(np.float64) * (1.0 / float(temp))).astype(np.float32)
    mask = np.ones(n, dtype=bool)
    if 0 < top_k < n:
        order = np.argsort(-x.astype(np.float64), kind="stable")
        keep = np.zeros(n, dtype=bool)
        keep[order[:top_k]] = True
        mask &= keep
    if min_p > 0:
        e = np.exp((x - x.max()).astype(np.float64))
        p = e / e.sum()
        x[p < float(min_p) * p.max()] = np.float32(-1e10)
        mask &= ~(x <= -1e9)
    x[~mask] = np.float32(-1e10)
    e = np.exp((x - x.max()).astype(np.float64))
    probs = e / e.sum()
    if 0 < top_p < 1:
        idx = [i for i in range(n) if mask[i]]
        idx.sort(key=lambda i: -probs[i])
        keep = np.zeros(n, dtype=bool)
        cum = 0.0
        for i in idx:
            keep[i] = True
            cum += probs[i]
            if cum >= float(np.float32(top_p)) - 1e-6:
                break
        mask &= keep
    total = float(probs[mask].sum())
    if total <= 0:
        return greedy(probs.astype(np.float32))
    r = u * total
    last = 0
    for i in range(n):
        if not mask[i]:
            continue
        last = i
        r -= probs[i]
        if r <= 0:
            return i
    return last


def generate_greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], n: int,
                    stop: Sequence[int] = (), wide: bool = False) -> List[int]:
    """Greedy continuation by re-running the whole sequence each step.

    pkg/runtime/session.go:50-81 and :133-159: a stop token ends the sequence and is neither
    appended nor fed.
    """
    seq = list(prompt)
    out: List[int] = []
    for _ in range(n):
        logits = forward(cfg, w, seq, wide)[-1]
        t = greedy(logits.tolist())
        if t in stop:
            break
        out.append(t)
        seq.append(t)
    return out
