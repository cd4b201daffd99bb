"""The step function: run the tokens a step brings, for a batch of sequences, from the cache.

A step is a list of entries, one per sequence: its cache slot, its next tokens (one or many; the
lengths may differ) and the places among these tokens whose logits are wanted.  The tokens of all
entries are packed without padding into one [T, hidden] activation; each token carries its
sequence and its absolute position, which is the sequence's cached length plus its index in the
entry - the cache index and the position are one number (the reference passes `startPos`
separately from its cache counter, pkg/model/qwen3/model.go:112-134, and the two can disagree,
pkg/runtime/conversation.go:120-125).  Only the wanted rows go through the final norm and the head
(the reference computes logits for the last token of a call only, model.go:127).

Everything is checked on the host before the first launch; a refused step leaves the cache as it was,
and so does a step that fails between reserving its pages and committing its lengths.  `step` refuses
the whole step at the first bad entry; `try_step` gives every entry a status of its own and runs the
others (the reference returns the error of its one sequence, pkg/runtime/session.go:69-72).

`taps` (a `LayerTaps`) hands out the residual rows of the wanted places after the embedding and after
every scheduled block, as the reference's debug hooks do for its last token
(pkg/model/qwen3/debug.go:4-9, fired at pkg/model/qwen3/model.go:141-162).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.sequence_cache import SequenceCache
from ..parts.base import StepContext, Workspace
from .model import Model


from ..csrc.build import DEBUG as _DEBUG


class StepError(ValueError):
    """A step, or one entry of it, that cannot run.  `code` is one of "empty_step", "duplicate_slot",
    "unknown_slot", "no_tokens", "bad_token", "bad_want", "context_overflow", "cache_full"."""

    def __init__(self, message: str, code: str = "bad_entry"):
        super().__init__(message)
        self.code = code


@dataclass
class LayerTaps:
    """Per-layer hooks of an eager step, in the manner of the reference's DebugHooks
    (pkg/model/qwen3/debug.go:4-9).  Every function gets float32 rows on the device, one per wanted
    place of the step, in the order of the logits: `on_embed(rows[wanted, hidden])` after the embedding,
    `on_layer(i, rows)` after schedule entry i, `on_layer_logits(i, logits[wanted, vocab])` the final
    norm and head applied to those rows (computed only if the hook is set), `on_logits(logits)` the
    step's own result.  The tensors are copies: a hook may keep them."""
    on_embed: Optional[Callable[[torch.Tensor], None]] = None
    on_layer: Optional[Callable[[int, torch.Tensor], None]] = None
    on_layer_logits: Optional[Callable[[int, torch.Tensor], None]] = None
    on_logits: Optional[Callable[[torch.Tensor], None]] = None


@dataclass
class StepOutcome:
    """What `try_step` gives back: `status[i]` is None for an entry that ran and the `StepError` that
    refused it otherwise; `logits` holds the wanted rows of the entries that ran, in their order."""
    logits: Optional[torch.Tensor]
    status: List[Optional[StepError]]

    @property
    def ran(self) -> List[int]:
        return [i for i, s in enumerate(self.status) if s is None]


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
    def _check_entry(self, e: StepEntry, seen: set) -> Optional[StepError]:
        """Why entry `e` cannot run, or None.  `seen` holds the slots of the entries before it."""
        V = self.model.spec.vocab_size
        limit = self.model.spec.max_positions
        if e.slot in seen:
            return StepError(f"slot {e.slot} appears twice in one step", "duplicate_slot")
        if not self.cache.slots.is_held(e.slot):
            return StepError(f"slot {e.slot} is not open", "unknown_slot")
        n = len(e.tokens)
        if n == 0:
            return StepError(f"slot {e.slot}: no tokens", "no_tokens")
        try:
            toks = np.asarray(e.tokens, dtype=np.int64)
        except (TypeError, ValueError, OverflowError):
            return StepError(f"slot {e.slot}: token ids must be integers", "bad_token")
        if toks.ndim != 1:
            return StepError(f"slot {e.slot}: token ids must be a flat list", "bad_token")
        bad = np.nonzero((toks < 0) | (toks >= V))[0]
        if bad.size:
            return StepError(f"slot {e.slot}: token id {int(toks[bad[0]])} is outside the vocabulary "
                             f"(0..{V - 1})", "bad_token")
        for w in e.want:
            if not (0 <= int(w) < n):
                return StepError(f"slot {e.slot}: wanted place {w} is outside its {n} tokens", "bad_want")
        if self.cache.lengths[e.slot] + n > limit:
            return StepError(f"slot {e.slot}: {self.cache.lengths[e.slot]} cached + {n} new tokens "
                             f"exceed the model's context of {limit}", "context_overflow")
        return None

    def _check(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one entry", "empty_step")
        seen: set = set()
        for e in entries:
            err = self._check_entry(e, seen)
            if err is not None:
                raise err
            seen.add(e.slot)

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
    def run_layers(self, ctx: StepContext, taps: Optional[LayerTaps] = None,
                   tap_rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Embedding and all scheduled blocks; returns the float32 residual stream [T, hidden].
        With `taps`, the rows `tap_rows` of the stream are handed out after the embedding and after
        every scheduled block (a debugging aid: it copies, and the head runs once more per block if
        `on_layer_logits` is set)."""
        m = self.model
        x = ctx.ws.get("residual", (ctx.n_tokens, m.spec.hidden_size), torch.float32)
        m.embedding.forward(ctx.tokens, x)
        tapping = taps is not None and tap_rows is not None and tap_rows.numel() > 0
        if tapping and taps.on_embed is not None:
            taps.on_embed(x.index_select(0, tap_rows.long()))
        for b in m.blocks:
            for part in getattr(b, "parts", {}).values():
                prep = getattr(part, "prepare", None)
                if prep is not None:
                    prep(ctx)
        for i, e in enumerate(m.spec.schedule):
            block = m.blocks[e.block]
            block.forward(x, ctx, self.cache.view(i), e.cache_of is None)
            stats = ctx.shared.get("row_stats")
            if stats is not None and not getattr(block, "keeps_row_stats", False):
                stats.fresh = False     # an arrangement that does not know of the statistics changed the rows
            if tapping:
                if taps.on_layer is not None:
                    taps.on_layer(i, x.index_select(0, tap_rows.long()))
                if taps.on_layer_logits is not None:
                    n = int(tap_rows.numel())
                    hn = ctx.ws.get("tap_normed", (n, m.spec.hidden_size), m.rt.dtype)
                    lg = ctx.ws.get("tap_logits", (n, m.spec.vocab_size), torch.float32)
                    m.final_norm.forward(x, hn, tap_rows)
                    m.head.forward(hn, lg, ctx, m=n)
                    taps.on_layer_logits(i, lg.clone())
        return x

    def run_head(self, ctx: StepContext, x: torch.Tensor, rows: torch.Tensor, n_rows: int) -> torch.Tensor:
        """Final norm and head on the gathered rows; float32 logits [n_rows, vocab]."""
        m = self.model
        hn = ctx.ws.get("head_normed", (n_rows, m.spec.hidden_size), m.rt.dtype)
        logits = ctx.ws.get("logits", (n_rows, m.spec.vocab_size), torch.float32)
        m.final_norm.forward(x, hn, rows[:n_rows])
        m.head.forward(hn, logits, ctx, m=n_rows)
        return logits

    def step(self, entries: Sequence[StepEntry], taps: Optional[LayerTaps] = None) -> Optional[torch.Tensor]:
        """Run one step.  Returns float32 logits [wanted, vocab] on the device (None if nothing is
        wanted), in the order of the entries and of their `want`.  The tensor is workspace memory:
        it is valid until the next step.  A bad entry refuses the whole step (`StepError`)."""
        self._check(entries)
        return self._run(entries, taps)

    def try_step(self, entries: Sequence[StepEntry], taps: Optional[LayerTaps] = None) -> StepOutcome:
        """Run the entries that can run and say, entry by entry, why the others cannot.  An entry that is
        refused changes nothing: its slot keeps its length and pages.  If the cache cannot hold the
        step, entries are left out from the end until it can ("cache_full")."""
        status: List[Optional[StepError]] = []
        seen: set = set()
        for e in entries:
            err = self._check_entry(e, seen)
            status.append(err)
            if err is None:
                seen.add(e.slot)
        good = [i for i, st in enumerate(status) if st is None]
        while good:
            need = self.cache.pages_short([entries[i].slot for i in good], [len(entries[i].tokens) for i in good])
            if need <= 0:
                break
            i = good.pop()
            status[i] = StepError(f"slot {entries[i].slot}: the cache has no room for its "
                                  f"{len(entries[i].tokens)} tokens in this step", "cache_full")
        logits = self._run([entries[i] for i in good], taps) if good else None
        return StepOutcome(logits=logits, status=status)

    def _run(self, entries: Sequence[StepEntry], taps: Optional[LayerTaps] = None) -> Optional[torch.Tensor]:
        """The checked entries, eagerly: reserve, pack, launch, commit."""
        slots = [e.slot for e in entries]
        counts = [len(e.tokens) for e in entries]
        self.cache.plan(slots, counts)          # raises before anything ran if the cache is full
        try:
            ctx, lay, rows = self.build_context(entries)
            x = self.run_layers(ctx, taps, rows[:lay.n_want] if lay.n_want else None)
            logits = self.run_head(ctx, x, rows, lay.n_want) if lay.n_want else None
        except BaseException:
            self.cache.unplan(slots)            # the pages reserved for this step go back
            raise
        self.cache.commit(slots, counts)
        if _DEBUG and self.model.rt.device.type == "cuda":
            from ..csrc.tcgen05_gemm import check_status
            check_status(self.model.rt.device)      # debug build: a page table out of range raises here
        if taps is not None and taps.on_logits is not None and logits is not None:
            taps.on_logits(logits.clone())
        return logits
