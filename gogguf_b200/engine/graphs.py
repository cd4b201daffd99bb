"""Decode steps as CUDA graphs.

A decode step (every sequence brings one token and wants its logits) launches a few hundred small
kernels; their launch cost would bound the step.  `GraphStepper` captures the device side of such
a step once per (batch bucket, page-table width bucket) and replays it: the integer inputs (tokens,
positions, slots, lengths, page tables) live in a fixed device buffer that is refilled by one copy
before each replay, so lengths and pages may change from step to step without a new capture.  A
batch smaller than its bucket is padded with rows that the kernels skip.  Every other step (prompts,
several tokens per sequence, wanted places other than the one token) runs eagerly through
`Stepper.step`.

The reference captures one graph per cached matrix product (host-to-device copy + kernel +
device-to-host copy, pkg/gpu/cuda/driver.c:1396-1557); here the whole step is one graph.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import Workspace
from .step import StepEntry, StepLayout, Stepper

BATCH_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)


def _bucket(n: int, buckets: Sequence[int]) -> Optional[int]:
    for b in buckets:
        if n <= b:
            return b
    return None


@dataclass
class _Captured:
    graph: torch.cuda.CUDAGraph
    host: torch.Tensor
    dev: torch.Tensor
    ws: Workspace
    logits: torch.Tensor
    layout: StepLayout
    kernels: int
    host2: Optional[torch.Tensor] = None       # second pinned buffer: steps may be enqueued one ahead
    copied: Optional[list] = None              # events: the copy out of each pinned buffer has been done
    turn: int = 0


class GraphStepper(Stepper):
    def __init__(self, model, cache, min_width: int = 16):
        super().__init__(model, cache)
        self.min_width = min_width
        self._graphs: Dict[Tuple[int, int], _Captured] = {}
        self.replays = 0
        # a part that reads back to the host or allocates while it runs declares `capturable = False`;
        # such a model is stepped eagerly, and `decode_from_device` is not offered for it
        self.capturable = all(getattr(p, "capturable", True) for p in model.parts())

    def _width_bucket(self, slots: Sequence[int]) -> int:
        w = max(self.cache.table_width(slots), self.min_width)
        return 1 << (w - 1).bit_length()

    def _capture(self, entries: Sequence[StepEntry], bucket: int, width: int) -> _Captured:
        dev_t = self.model.rt.device
        lay = StepLayout(bucket, bucket, bucket, [width] * len(self.cache.groups))
        host = torch.empty(lay.total, dtype=torch.int32, pin_memory=True)
        dev = torch.empty(lay.total, dtype=torch.int32, device=dev_t)
        ws = Workspace(dev_t)
        cap = _Captured(graph=torch.cuda.CUDAGraph(), host=host, dev=dev, ws=ws, logits=None, layout=lay, kernels=0)

        def run():
            ctx, lay2, rows = self.build_context(entries, host=host, dev=dev, pad_seqs=bucket,
                                                 table_width=width, ws=ws)
            ctx.max_ctx = width * self.cache.page_size      # an upper bound: lengths change between replays
            x = self.run_layers(ctx)
            return self.run_head(ctx, x, rows, bucket)

        # warm-up on a side stream: allocates the workspace, sets kernel attributes, compiles what is missing
        side = torch.cuda.Stream(device=dev_t)
        side.wait_stream(torch.cuda.current_stream(dev_t))
        with torch.cuda.stream(side):
            run()
        torch.cuda.current_stream(dev_t).wait_stream(side)
        torch.cuda.synchronize(dev_t)
        from ..csrc import build
        n0 = build.launch_count()
        with torch.cuda.graph(cap.graph):
            # the copy of the integer inputs stays outside the graph: it is re-issued before every replay
            ctx, lay2, rows = self._context_for_capture(entries, cap, bucket, width)
            x = self.run_layers(ctx)
            cap.logits = self.run_head(ctx, x, rows, bucket)
        cap.kernels = build.launch_count() - n0
        cap.host2 = torch.empty(lay.total, dtype=torch.int32, pin_memory=True)
        cap.copied = [None, None]
        return cap

    def _context_for_capture(self, entries, cap: _Captured, bucket: int, width: int):
        # same views as build_context makes, without touching host memory or copying
        from ..parts.base import StepContext
        lay, dev = cap.layout, cap.dev
        B = bucket
        ctx = StepContext(
            runtime=self.model.rt, ws=cap.ws, n_tokens=B, n_seqs=B,
            tokens=lay.view(dev, "tokens"), positions=lay.view(dev, "positions"),
            seq_of_token=lay.view(dev, "seq_of_token"), cu_seqlens=lay.view(dev, "cu_seqlens"),
            slots=lay.view(dev, "slots"), ctx_lens=lay.view(dev, "ctx_lens"),
            page_tables={g: lay.view(dev, f"pages{g}").view(B, width) for g in range(len(self.cache.groups))},
            max_new=1, max_ctx=width * self.cache.page_size, decode=True)
        return ctx, lay, lay.view(dev, "logit_rows")

    def _run(self, entries: Sequence[StepEntry], taps=None) -> Optional[torch.Tensor]:
        """Checked entries: a plain decode step replays its graph, everything else runs eagerly
        (prompts, several tokens per sequence, other wanted places, a step with layer taps, a model
        one of whose parts says it cannot be captured)."""
        decode = all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries) and len(entries) > 0
        if (not decode or taps is not None or not self.capturable
                or _bucket(len(entries), BATCH_BUCKETS) is None):
            return super()._run(entries, taps)
        return self._enqueue_decode(entries, None, None)

    def decode_from_device(self, slots: Sequence[int], sampled: torch.Tensor, rows: Sequence[int]
                           ) -> Optional[torch.Tensor]:
        """Enqueue one decode step whose input tokens are still on the device: sequence i of `slots`
        takes `sampled[rows[i]]` (an int32 tensor that a sampling kernel wrote earlier on this stream).
        Nothing is read back and the host does not wait, so the caller may enqueue this step while it
        is still reading the previous step's ids.  Returns the logits view [len(slots), vocab]."""
        entries = [StepEntry(s, [0], want=[0]) for s in slots]
        if not self.capturable:
            raise ValueError("a part of this model cannot be captured in a CUDA graph; step it eagerly")
        if _bucket(len(entries), BATCH_BUCKETS) is None:
            raise ValueError(f"no captured batch size holds {len(entries)} sequences")
        self._check(entries)
        return self._enqueue_decode(entries, sampled, list(rows))

    def _enqueue_decode(self, entries, sampled, rows):
        slots = [e.slot for e in entries]
        counts = [1] * len(entries)
        bucket = _bucket(len(entries), BATCH_BUCKETS)
        self.cache.plan(slots, counts)
        try:
            return self._replay(entries, slots, counts, bucket, sampled, rows)
        except BaseException:
            self.cache.unplan(slots)
            raise

    def _replay(self, entries, slots, counts, bucket, sampled, rows):
        width = self._width_bucket(slots)
        key = (bucket, width)
        cap = self._graphs.get(key)
        if cap is None:
            cap = self._graphs[key] = self._capture(entries, bucket, width)
        # two pinned buffers in turn: the one filled now was last copied from two steps ago
        t = cap.turn
        cap.turn ^= 1
        host = cap.host if t == 0 else cap.host2
        if cap.copied[t] is not None:
            cap.copied[t].synchronize()
        self.build_context(entries, host=host, dev=cap.dev, pad_seqs=bucket, table_width=width, ws=cap.ws,
                           token_src=rows, wait_host=False)
        if cap.copied[t] is None:
            cap.copied[t] = torch.cuda.Event()
        cap.copied[t].record()
        if sampled is not None:
            from ..csrc import kernels as K
            lay = cap.layout
            K.feed_tokens(lay.view(cap.dev, "tokens"), lay.view(cap.dev, "token_src"), sampled, len(entries))
        cap.graph.replay()
        self.replays += 1
        self.last_graph_kernels = cap.kernels
        self.last_h2d_bytes = cap.layout.total * 4
        self.cache.commit(slots, counts)
        return cap.logits[:len(entries)]
