"""The step function: run the tokens a step brings, for a batch of sequences, from the cache.

A step is a list of entries, one per sequence: its cache slot, its next tokens (one or many; the
lengths may differ) and the places among these tokens whose logits are wanted.  The tokens of all
entries are packed without padding into one [T, hidden] activation; each token carries its
sequence and its absolute position, which is the sequence's cached length plus its index in the
entry - the cache index and the position are one number (the reference passes `startPos`
separately from its cache counter, pkg/model/qwen3/model.go:112-134, and the two can disagree,
pkg/runtime/conversation.go:120-125).  Only the wanted rows go through the final norm and the head
(the reference computes logits for the last token of a call only, model.go:127).

Everything is checked on the host before the first launch; a refused step leaves the cache as it was.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.sequence_cache import SequenceCache
from ..parts.base import StepContext, Workspace
from .model import Model


class StepError(ValueError):
    """A step that cannot run: unknown slot, token id out of range, context overflow, bad index."""


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


def _pad4(n: int) -> int:
    return (n + 3) & ~3


class StepLayout:
    """Packs the integer inputs of a step into one host buffer and one device buffer."""

    def __init__(self, n_tokens: int, n_seqs: int, n_want: int, group_widths: Sequence[int]):
        self.n_tokens, self.n_seqs, self.n_want = n_tokens, n_seqs, n_want
        self.group_widths = list(group_widths)
        off = 0
        self.off: Dict[str, Tuple[int, int]] = {}
        for name, n in (("tokens", n_tokens), ("positions", n_tokens), ("seq_of_token", n_tokens),
                        ("cu_seqlens", n_seqs + 1), ("slots", n_seqs), ("ctx_lens", n_seqs),
                        ("token_src", n_seqs), ("logit_rows", max(n_want, 1))):
            self.off[name] = (off, n)
            off += _pad4(n)
        for g, w in enumerate(self.group_widths):
            self.off[f"pages{g}"] = (off, n_seqs * w)
            off += _pad4(n_seqs * w)
        self.total = off

    def view(self, buf, name: str):
        o, n = self.off[name]
        return buf[o:o + n]


class Stepper:
    """Owns the workspace of one (model, cache) pair and runs steps on it."""

    def __init__(self, model: Model, cache: SequenceCache):
        self.model = model
        self.cache = cache
        self.ws = Workspace(model.rt.device)
        self._host: Optional[torch.Tensor] = None
        self._dev: Optional[torch.Tensor] = None
        self._copied: Optional[torch.cuda.Event] = None

    # ------------------------------------------------------------------ host side
    def _check(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        V = self.model.spec.vocab_size
        limit = self.model.spec.max_positions
        seen = set()
        for e in entries:
            if e.slot in seen:
                raise StepError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if not self.cache.slots.is_held(e.slot):
                raise StepError(f"slot {e.slot} is not open")
            if len(e.tokens) == 0:
                raise StepError(f"slot {e.slot}: no tokens")
            for t in e.tokens:
                if not (0 <= int(t) < V):
                    raise StepError(f"slot {e.slot}: token id {t} is outside the vocabulary (0..{V - 1})")
            for w in e.want:
                if not (0 <= int(w) < len(e.tokens)):
                    raise StepError(f"slot {e.slot}: wanted place {w} is outside its {len(e.tokens)} tokens")
            if self.cache.lengths[e.slot] + len(e.tokens) > limit:
                raise StepError(f"slot {e.slot}: {self.cache.lengths[e.slot]} cached + {len(e.tokens)} new tokens "
                                f"exceed the model's context of {limit}")

    def _buffers(self, n: int) -> Tuple[torch.Tensor, torch.Tensor]:
        if self._host is None or self._host.numel() < n:
            cap = max(1024, 1 << (n - 1).bit_length())
            self._host = torch.empty(cap, dtype=torch.int32, pin_memory=self.model.rt.device.type == "cuda")
            self._dev = torch.empty(cap, dtype=torch.int32, device=self.model.rt.device)
        return self._host, self._dev

    def build_context(self, entries: Sequence[StepEntry], host: Optional[torch.Tensor] = None,
                      dev: Optional[torch.Tensor] = None, pad_seqs: int = 0, table_width: Optional[int] = None,
                      ws: Optional[Workspace] = None, token_src: Optional[Sequence[int]] = None,
                      wait_host: bool = True) -> Tuple[StepContext, StepLayout, torch.Tensor]:
        """Fill the integer inputs for `entries` (pages must be reserved already) and copy them to the device.

        `pad_seqs` > len(entries) pads the batch with empty rows (one padding token each), which the
        kernels skip; used when a captured graph of a larger batch is replayed.
        """
        cache = self.cache
        slots = [e.slot for e in entries]
        counts = [len(e.tokens) for e in entries]
        B = max(len(entries), pad_seqs)
        n_pad = B - len(entries)
        T = sum(counts) + n_pad
        n_want = sum(len(e.want) for e in entries)
        width = table_width if table_width is not None else cache.table_width(slots)
        lay = StepLayout(T, B, max(n_want, pad_seqs), [width] * len(cache.groups))
        if host is None:
            host, dev = self._buffers(lay.total)
        if self._copied is not None and wait_host:
            self._copied.synchronize()      # the previous step's copy has left the host buffer
        h = host.numpy()
        tok, pos, sot = lay.view(h, "tokens"), lay.view(h, "positions"), lay.view(h, "seq_of_token")
        cu, sl, cl, rows = (lay.view(h, "cu_seqlens"), lay.view(h, "slots"), lay.view(h, "ctx_lens"),
                            lay.view(h, "logit_rows"))
        src = lay.view(h, "token_src")
        src[:] = -1
        if token_src is not None:
            src[:len(entries)] = np.asarray(token_src, dtype=np.int32)
        r = 0
        cu[0] = 0
        wi = 0
        rows[:] = -1
        for b, e in enumerate(entries):
            n = counts[b]
            start = cache.lengths[e.slot]
            tok[r:r + n] = np.asarray(e.tokens, dtype=np.int32)
            pos[r:r + n] = np.arange(start, start + n, dtype=np.int32)
            sot[r:r + n] = b
            for w in e.want:
                rows[wi] = r + int(w)
                wi += 1
            r += n
            cu[b + 1] = r
            sl[b] = e.slot
            cl[b] = start + n
        for b in range(len(entries), B):
            tok[r] = -1
            pos[r] = 0
            sot[r] = -1
            r += 1
            cu[b + 1] = r
            sl[b] = 0
            cl[b] = 0
        for g in range(len(cache.groups)):
            pt = lay.view(h, f"pages{g}").reshape(B, width)
            pt[:] = 0
            if entries:
                pt[:len(entries)] = np.asarray(cache.page_table(g, slots, width), dtype=np.int32)
        dev[:lay.total].copy_(host[:lay.total], non_blocking=True)
        if dev.is_cuda:
            if self._copied is None:
                self._copied = torch.cuda.Event()
            self._copied.record()
        ctx = StepContext(
            runtime=self.model.rt, ws=ws or self.ws, n_tokens=T, n_seqs=B,
            tokens=lay.view(dev, "tokens"), positions=lay.view(dev, "positions"),
            seq_of_token=lay.view(dev, "seq_of_token"), cu_seqlens=lay.view(dev, "cu_seqlens"),
            slots=lay.view(dev, "slots"), ctx_lens=lay.view(dev, "ctx_lens"),
            page_tables={g: lay.view(dev, f"pages{g}").view(B, width) for g in range(len(cache.groups))},
            max_new=max(counts) if counts else 1,
            max_ctx=max((cache.lengths[s] + n for s, n in zip(slots, counts)), default=1),
            decode=all(n == 1 for n in counts),
        )
        return ctx, lay, lay.view(dev, "logit_rows")

    # ------------------------------------------------------------------ device side
    def run_layers(self, ctx: StepContext) -> torch.Tensor:
        """Embedding and all scheduled blocks; returns the float32 residual stream [T, hidden]."""
        m = self.model
        x = ctx.ws.get("residual", (ctx.n_tokens, m.spec.hidden_size), torch.float32)
        m.embedding.forward(ctx.tokens, x)
        for b in m.blocks:
            prep = getattr(b.mixer, "prepare", None)
            if prep is not None:
                prep(ctx)
        for i, e in enumerate(m.spec.schedule):
            block = m.blocks[e.block]
            block.forward(x, ctx, self.cache.view(i), e.cache_of is None)
            stats = ctx.shared.get("row_stats")
            if stats is not None and not getattr(block, "keeps_row_stats", False):
                stats.fresh = False     # an arrangement that does not know of the statistics changed the rows
        return x

    def run_head(self, ctx: StepContext, x: torch.Tensor, rows: torch.Tensor, n_rows: int) -> torch.Tensor:
        """Final norm and head on the gathered rows; float32 logits [n_rows, vocab]."""
        m = self.model
        hn = ctx.ws.get("head_normed", (n_rows, m.spec.hidden_size), m.rt.dtype)
        logits = ctx.ws.get("logits", (n_rows, m.spec.vocab_size), torch.float32)
        m.final_norm.forward(x, hn, rows[:n_rows])
        m.head.forward(hn, logits, ctx, m=n_rows)
        return logits

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run one step.  Returns float32 logits [wanted, vocab] on the device (None if nothing is
        wanted), in the order of the entries and of their `want`.  The tensor is workspace memory:
        it is valid until the next step."""
        self._check(entries)
        slots = [e.slot for e in entries]
        counts = [len(e.tokens) for e in entries]
        self.cache.plan(slots, counts)          # raises before anything ran if the cache is full
        ctx, lay, rows = self.build_context(entries)
        x = self.run_layers(ctx)
        logits = self.run_head(ctx, x, rows, lay.n_want) if lay.n_want else None
        self.cache.commit(slots, counts)
        return logits
