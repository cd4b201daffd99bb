"""Per-phase device timing of a generation, behind a flag.

With `LoadOptions(timing=True)` the generation loop brackets its phases with CUDA events on the launching
stream: every prefill step, every decode step, every sampling call.  Nothing is synchronised while the loop
runs (events are only recorded); `PhaseTimer.report()` synchronises once and adds the intervals up.  The
figures are the reference's bench figures (cmd/tools/bench.go:302-364: prefill ms and tokens a second, time to
the first token, decode ms and tokens a second, total), measured on the device instead of by the host's
clock, plus the split of the decode time into model steps and sampling that the reference's one-token loop
cannot show.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch


@dataclass
class PhaseReport:
    prompt_tokens: int = 0
    decode_tokens: int = 0
    prefill_ms: float = 0.0
    prefill_steps: int = 0
    ttft_ms: float = 0.0            # start of the first prefill step -> end of the first sampling call
    decode_ms: float = 0.0          # decode steps and their sampling calls, on the device
    decode_steps: int = 0
    step_ms: float = 0.0            # of decode_ms: the model's steps
    sampling_ms: float = 0.0        # of decode_ms: the sampling kernels (and a repeat penalty's)
    total_ms: float = 0.0           # first event -> last event on the device
    host_ms: float = 0.0            # the host's clock around the same call

    @property
    def prefill_tps(self) -> float:
        return self.prompt_tokens / (self.prefill_ms / 1e3) if self.prefill_ms > 0 else 0.0

    @property
    def decode_tps(self) -> float:
        return self.decode_tokens / (self.decode_ms / 1e3) if self.decode_ms > 0 else 0.0

    @property
    def total_tps(self) -> float:
        n = self.prompt_tokens + self.decode_tokens
        return n / (self.total_ms / 1e3) if self.total_ms > 0 else 0.0

    def lines(self) -> List[str]:
        """The reference's report lines (cmd/tools/bench.go:296-299), with the decode split added."""
        return [
            f"Prefill ({self.prompt_tokens} tok, {self.prefill_steps} step{'s' if self.prefill_steps != 1 else ''}): "
            f"{self.prefill_ms:.1f} ms ({self.prefill_tps:.1f} tok/s)",
            f"TTFT: {self.ttft_ms:.1f} ms",
            f"Decode ({self.decode_tokens} tok, {self.decode_steps} steps): {self.decode_ms:.1f} ms "
            f"({self.decode_tps:.1f} tok/s; model {self.step_ms:.1f} ms, sampling {self.sampling_ms:.1f} ms)",
            f"Total: {self.total_ms:.1f} ms on the device, {self.host_ms:.1f} ms by the host's clock "
            f"({self.total_tps:.1f} tok/s)",
        ]

    def to_dict(self) -> Dict[str, float]:
        d = {k: getattr(self, k) for k in self.__dataclass_fields__}
        d.update(prefill_tps=self.prefill_tps, decode_tps=self.decode_tps, total_tps=self.total_tps)
        return d


class PhaseTimer:
    """Collects (phase, start event, end event, tokens) while a generation runs."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.enabled = self.device.type == "cuda"
        self.reset()

    def reset(self) -> None:
        self._spans: List[Tuple[str, object, object, int]] = []
        self._open: Optional[Tuple[str, object, int]] = None
        self._t0 = time.perf_counter()
        self._t1 = self._t0

    def begin(self, phase: str, tokens: int = 0) -> None:
        """phase: "prefill", "decode" or "sample"."""
        if not self.enabled:
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._open = (phase, ev, tokens)

    def end(self) -> None:
        if not self.enabled or self._open is None:
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        phase, start, tokens = self._open
        self._spans.append((phase, start, ev, tokens))
        self._open = None
        self._t1 = time.perf_counter()

    def report(self) -> PhaseReport:
        r = PhaseReport(host_ms=(self._t1 - self._t0) * 1e3)
        if not self.enabled or not self._spans:
            return r
        torch.cuda.synchronize(self.device)
        first = self._spans[0][1]
        first_sample_end = None
        for phase, a, b, tokens in self._spans:
            ms = a.elapsed_time(b)
            if phase == "prefill":
                r.prefill_ms += ms
                r.prefill_steps += 1
                r.prompt_tokens += tokens
            elif phase == "decode":
                r.step_ms += ms
                r.decode_steps += 1
                r.decode_tokens += tokens
            elif phase == "sample":
                if first_sample_end is None:
                    first_sample_end = b
                    r.decode_tokens += tokens          # the tokens drawn from the prompts' logits
                else:
                    r.sampling_ms += ms
        r.decode_ms = r.step_ms + r.sampling_ms
        r.ttft_ms = first.elapsed_time(first_sample_end) if first_sample_end is not None else r.prefill_ms
        r.total_ms = first.elapsed_time(self._spans[-1][2])
        return r
