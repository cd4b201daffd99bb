"""Choosing the next token: greedy, temperature, top-k, top-p, min-p, repeat penalty.

Options and their meaning follow the reference's sampler (pkg/sampler/chain.go:9-70):
`temp` 0 = greedy; `top_k` 0 = off; `top_p` 1 = off; `min_p` 0 = off; `seed` seeds the draws.
Greedy sampling, plain temperature sampling, and the whole chain whenever a top-k of at most 1,024 is
set run on the GPU (csrc/sampling.cu) over the whole batch, with the repeat penalty too once the
sequences' last ids have been put on the device (`Sampler.begin`).  Top-p or min-p without a top-k
also has a kernel, which answers from each row's 1,024 largest logits and flags the rows for which
that may not be the whole answer; the host reads the flags every step (so this configuration does not
run a step ahead) and takes flagged rows, like everything with a penalty but no kernel path, through
this module's host chain.  The order is
the reference's: penalty, temperature, top-k, min-p, mask to -1e10, softmax, top-p, draw.

Random draws are counter based: u = uniform01(seed, stream, step) with `stream` the request's index
and `step` the number of tokens it has generated, so a sequence's draws do not depend on what else
is in its batch.  (The reference draws from one PCG stream per sampler object, chain.go:23; its bit
stream is not reproduced.)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

_M64 = (1 << 64) - 1


def _mix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def uniform01(seed: int, stream: int, step: int) -> float:
    """A uniform number in [0, 1) that depends only on (seed, stream, step)."""
    z = _mix64(seed & _M64)
    z = _mix64(z ^ (stream & _M64))
    z = _mix64(z ^ (step & _M64))
    return (z >> 11) / float(1 << 53)


@dataclass(frozen=True)
class SamplerConfig:
    """pkg/sampler/chain.go:9-15."""
    temp: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    seed: int = 0

    @property
    def greedy(self) -> bool:
        """chain.go:19-21: no temperature, no top-k, no top-p."""
        return self.temp <= 0 and self.top_k <= 0 and (self.top_p <= 0 or self.top_p >= 1)

    @property
    def device_chain(self) -> bool:
        """The chain with a top-k has a kernel (any top-p and min-p with it)."""
        return 0 < self.top_k <= 1024

    @property
    def on_device(self) -> bool:
        """Greedy, plain temperature and top-k chains have kernels; top-p or min-p without a top-k run on the host."""
        return self.greedy or self.device_chain or \
            (self.top_k <= 0 and (self.top_p <= 0 or self.top_p >= 1) and self.min_p <= 0)


def greedy(logits: Sequence[float]) -> int:
    """First index of the maximum (pkg/sampler/greedy.go:4-17); -1 for no logits."""
    a = np.asarray(logits)
    if a.size == 0:
        return -1
    return int(np.argmax(a))


def apply_repeat_penalty(logits: np.ndarray, history: Sequence[int], penalty: float, last_n: int) -> None:
    """In place; each distinct id among the last `last_n` of the history once
    (pkg/sampler/penalties.go:5-32)."""
    if penalty == 1 or logits.size == 0 or len(history) == 0:
        return
    h = history[-last_n:] if last_n > 0 and len(history) > last_n else history
    for t in set(int(x) for x in h):
        if 0 <= t < logits.size:
            logits[t] = logits[t] / penalty if logits[t] > 0 else logits[t] * penalty


def _softmax64(x: np.ndarray) -> np.ndarray:
    e = np.exp((x - x.max()).astype(np.float64))
    return e / e.sum()


def sample_host(logits: np.ndarray, cfg: SamplerConfig, u: float) -> int:
    """The whole chain on one row of float32 logits with the uniform draw `u` given."""
    n = logits.size
    if n == 0:
        return -1
    if cfg.greedy:
        return greedy(logits)
    x = logits.astype(np.float32, copy=True)
    if cfg.temp > 0 and cfg.temp != 1:
        x = (x.astype(np.float64) * (1.0 / float(cfg.temp))).astype(np.float32)
    mask = np.ones(n, dtype=bool)
    if 0 < cfg.top_k < n:
        order = np.argsort(-x.astype(np.float64), kind="stable")
        keep = np.zeros(n, dtype=bool)
        keep[order[:cfg.top_k]] = True
        mask &= keep
    if cfg.min_p > 0:
        p = _softmax64(x)
        x[p < float(cfg.min_p) * p.max()] = np.float32(-1e10)
        mask &= ~(x <= -1e9)
    x[~mask] = np.float32(-1e10)
    probs = _softmax64(x)
    if 0 < cfg.top_p < 1:
        idx = np.flatnonzero(mask)
        idx = idx[np.argsort(-probs[idx], kind="stable")]
        cum = np.cumsum(probs[idx])
        cut = int(np.searchsorted(cum, float(np.float32(cfg.top_p)) - 1e-6, side="left"))
        keep = np.zeros(n, dtype=bool)
        keep[idx[:cut + 1]] = True
        mask &= keep
    allowed = np.flatnonzero(mask)
    total = float(probs[allowed].sum())
    if total <= 0:
        return greedy(probs.astype(np.float32))
    r = u * total
    run = np.cumsum(probs[allowed])
    hit = np.flatnonzero(r - run <= 0)
    return int(allowed[hit[0]]) if hit.size else int(allowed[-1])


class PendingSample:
    """Ids that a sampling kernel has written on the device and that are on their way to the host."""

    def __init__(self, device_tokens: torch.Tensor, pinned: torch.Tensor, event, rows: int):
        self.device_tokens, self._pinned, self._event, self.rows = device_tokens, pinned, event, rows

    def tokens(self) -> List[int]:
        self._event.synchronize()
        return self._pinned[:self.rows].tolist()


class Sampler:
    """Samples one token per row of a [rows, vocab] float32 logits tensor."""

    # what the top-k kernel's shared memory holds: k candidates of each 8,192-logit slice of a row, 8 bytes each
    TOPK_SLICE, TOPK_SMEM = 8192, 160 * 1024

    def __init__(self, cfg: SamplerConfig, repeat_penalty: float = 1.0, repeat_last_n: int = 64,
                 vocab_size: Optional[int] = None):
        self.cfg = cfg
        # The chain with a top-k has a kernel as long as the slices' candidates fit its shared memory (top-k
        # 1,024 up to a vocabulary of 163,840); beyond that the host chain takes the rows, as it does for
        # every configuration without a kernel.
        self.device_chain = cfg.device_chain
        if self.device_chain and vocab_size:
            slices = -(-int(vocab_size) // self.TOPK_SLICE)
            self.device_chain = slices * min(cfg.top_k, int(vocab_size)) * 8 <= self.TOPK_SMEM
        self.on_device = cfg.on_device and (self.device_chain or not cfg.device_chain)
        self.repeat_penalty = float(repeat_penalty)
        self.repeat_last_n = int(repeat_last_n) if repeat_last_n else 64   # 0 means 64 (session.go:87-91)
        self._out: Optional[torch.Tensor] = None
        self._outs = None
        self._turn = 0
        self._rings = None        # device rings of the sequences' last ids (repeat penalty on the device)
        self._ring_of = {}

    @property
    def device_only(self) -> bool:
        """True when every row can be sampled by kernels alone (with a repeat penalty: after `begin`)."""
        return self.on_device and (not self.penalised or self._rings is not None)

    def begin(self, streams: Sequence[int], prompts: Sequence[Sequence[int]], device) -> None:
        """Put the last `repeat_last_n` ids of each request's prompt on the device, one ring per request, so
        that the penalty can be applied, and every sampled id appended, without the host.  Only needed (and
        only done) with a repeat penalty and a configuration whose sampling runs on the device."""
        if not (self.penalised and self.on_device):
            return
        n, rows = self.repeat_last_n, len(streams)
        hist = torch.full((rows, n), -1, dtype=torch.int32)
        lens = torch.zeros(rows, dtype=torch.int32)
        for r, p in enumerate(prompts):
            tail = list(p)[-n:]
            hist[r, :len(tail)] = torch.tensor(tail, dtype=torch.int32)
            lens[r] = len(tail)
        pos = lens % n
        self._rings = (hist.to(device), lens.to(device), pos.to(torch.int32).to(device))
        self._ring_of = {int(s): r for r, s in enumerate(streams)}
        self._ring_rows = [(torch.empty(max(rows, 1), dtype=torch.int32, pin_memory=True),
                            torch.empty(max(rows, 1), dtype=torch.int32, device=device)) for _ in range(2)]

    def sample_async(self, logits: torch.Tensor, streams: Sequence[int], steps: Sequence[int]) -> PendingSample:
        """Greedy or temperature sampling on the device without waiting for the result: the ids stay in
        a device buffer (the next decode step can take them from there) and are copied to pinned host
        memory behind the kernel.  Two sets of buffers are used in turn, so one sample may be outstanding
        while the next is enqueued."""
        if not (logits.is_cuda and self.device_only):
            raise ValueError("sample_async needs CUDA logits and a sampler configuration that runs on the device")
        from ..csrc import kernels as K
        rows = len(streams)
        cap = max(rows, 64)
        if self._outs is None or self._outs[0][0].numel() < cap:
            self._outs = [(torch.empty(cap, dtype=torch.int32, device=logits.device),
                           torch.empty(cap, dtype=torch.int32, pin_memory=True),
                           torch.empty(cap, dtype=torch.float64, pin_memory=True),
                           torch.empty(cap, dtype=torch.float64, device=logits.device),
                           torch.empty(cap, dtype=torch.float32, device=logits.device)) for _ in range(2)]
        out, pinned, u_host, u_dev, temps = self._outs[self._turn]
        ring_rows = None
        if self.penalised:
            # the rows' rings: the penalty edits the logits in place before the sampling kernel reads them
            rr_host, rr_dev = self._ring_rows[self._turn]
            rr_host[:rows] = torch.tensor([self._ring_of[int(s)] for s in streams], dtype=torch.int32)
            rr_dev[:rows].copy_(rr_host[:rows], non_blocking=True)
            ring_rows = rr_dev
            K.repeat_penalty(logits, self._rings[0], self._rings[1], ring_rows, self.repeat_penalty, rows)
        self._turn ^= 1
        if self.cfg.greedy:
            K.argmax(logits, out, rows)
        else:
            u_host[:rows] = torch.tensor([uniform01(self.cfg.seed, s, k) for s, k in zip(streams, steps)],
                                         dtype=torch.float64)
            u_dev[:rows].copy_(u_host[:rows], non_blocking=True)
            if self.device_chain:
                K.sample_topk(logits, self.cfg.temp, self.cfg.top_k, self.cfg.top_p, self.cfg.min_p, u_dev, out, rows)
            else:
                temps[:rows].fill_(float(self.cfg.temp))
                K.sample(logits, temps, u_dev, out, rows)
        if ring_rows is not None:
            K.history_append(out, ring_rows, self._rings[0], self._rings[1], self._rings[2], rows)
        pinned[:rows].copy_(out[:rows], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        return PendingSample(out, pinned, ev, rows)

    @property
    def penalised(self) -> bool:
        return self.repeat_penalty > 0 and self.repeat_penalty != 1

    def sample(self, logits: torch.Tensor, streams: Sequence[int], steps: Sequence[int],
               histories: Optional[Sequence[Sequence[int]]] = None) -> List[int]:
        """`streams[r]`: request index of row r; `steps[r]`: tokens it has generated so far;
        `histories[r]`: prompt + generated ids (only read when a repeat penalty is set)."""
        rows = len(streams)
        us = [uniform01(self.cfg.seed, s, k) for s, k in zip(streams, steps)]
        if logits.is_cuda and self.on_device and not self.penalised:
            from ..csrc import kernels as K
            if self._out is None or self._out.numel() < rows:
                self._out = torch.empty(max(rows, 64), dtype=torch.int32, device=logits.device)
            out = self._out[:rows]
            if self.cfg.greedy:
                K.argmax(logits, out, rows)
            else:
                uni = torch.tensor(us, dtype=torch.float64).to(logits.device, non_blocking=True)
                if self.device_chain:
                    K.sample_topk(logits, self.cfg.temp, self.cfg.top_k, self.cfg.top_p, self.cfg.min_p, uni, out, rows)
                else:
                    temps = torch.full((rows,), float(self.cfg.temp), dtype=torch.float32).to(logits.device, non_blocking=True)
                    K.sample(logits, temps, uni, out, rows)
            return out.cpu().tolist()
        if (logits.is_cuda and not self.penalised and self.cfg.temp > 0 and self.cfg.top_k <= 0
                and logits.dtype == torch.float32 and logits.shape[1] >= 2048):
            # top-p and / or min-p without a top-k: a kernel answers from each row's 1,024 largest logits and
            # says for which rows that is not certain to be the whole answer; only those go through the host chain
            from ..csrc import kernels as K
            if self._out is None or self._out.numel() < 2 * rows:
                self._out = torch.empty(2 * max(rows, 64), dtype=torch.int32, device=logits.device)
            out, flags = self._out[:rows], self._out[rows:2 * rows]
            uni = torch.tensor(us, dtype=torch.float64).to(logits.device, non_blocking=True)
            K.sample_nucleus(logits, self.cfg.temp, self.cfg.top_p, self.cfg.min_p, uni, out, flags, rows)
            both = self._out[:2 * rows].cpu().tolist()
            res, unsure = both[:rows], both[rows:]
            for r in range(rows):
                if unsure[r]:
                    res[r] = sample_host(logits[r].detach().to("cpu", torch.float32).numpy().copy(), self.cfg, us[r])
            return res
        host = logits[:rows].detach().to("cpu", torch.float32).numpy()
        res = []
        for r in range(rows):
            row = host[r].copy()
            if self.penalised and histories is not None:
                apply_repeat_penalty(row, histories[r], self.repeat_penalty, self.repeat_last_n)
            res.append(sample_host(row, self.cfg, us[r]))
        return res


class FunctionSampler:
    """A caller's own sampling function in the place of the chain: `fn(logits) -> id`, with the row's float32
    logits as a numpy array (sampler.Func, pkg/sampler/temperature.go:9; GenerateParams.Sampler,
    pkg/runtime/context.go:15).  The repeat penalty is applied before the call, as for the chain
    (session.go:83-96).  The rows come to the host every step, so the loop does not run ahead of it."""

    device_only = False

    def __init__(self, fn, repeat_penalty: float = 1.0, repeat_last_n: int = 64):
        self.fn = fn
        self.repeat_penalty = float(repeat_penalty)
        self.repeat_last_n = int(repeat_last_n) if repeat_last_n else 64

    @property
    def penalised(self) -> bool:
        return self.repeat_penalty > 0 and self.repeat_penalty != 1

    def begin(self, streams, prompts, device) -> None:
        pass

    def sample(self, logits: torch.Tensor, streams: Sequence[int], steps: Sequence[int],
               histories: Optional[Sequence[Sequence[int]]] = None) -> List[int]:
        rows = len(streams)
        host = logits[:rows].detach().to("cpu", torch.float32).numpy()
        res = []
        for r in range(rows):
            row = host[r].copy()
            if self.penalised and histories is not None:
                apply_repeat_penalty(row, histories[r], self.repeat_penalty, self.repeat_last_n)
            res.append(int(self.fn(row)))
        return res


def make_sampler(sampler, repeat_penalty: float = 1.0, repeat_last_n: int = 64, vocab_size: Optional[int] = None):
    """The sampler of a request: a `SamplerConfig` gives the chain, a function is called as it is.
    `vocab_size`, where known, lets the sampler decide at once which of its kernels take rows of that length."""
    if isinstance(sampler, SamplerConfig):
        return Sampler(sampler, repeat_penalty, repeat_last_n, vocab_size)
    if callable(sampler):
        return FunctionSampler(sampler, repeat_penalty, repeat_last_n)
    raise TypeError(f"a sampler is a SamplerConfig or a function of a row of logits, not {type(sampler).__name__}")
