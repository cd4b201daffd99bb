"""The generation loop above the step function.

One *batch* is a set of requests that start together: their prompts, of unequal lengths, run in one
prefill step; then every live sequence goes on by one token per step.  A sequence that ends (stop
token, token limit, context limit) leaves the batch at once and its slot and pages are given back;
the others go on in a smaller batch.  Requests beyond what one batch may hold run in further
batches, one after another, which reuse the slots.

Rules taken from the reference's session (pkg/runtime/session.go:50-81, :133-159): the default
limit is 128 new tokens; a sampled stop token ends the sequence and is neither appended to the
output nor fed to the model; a sampler result below 0 ends it too; the `on_token` callback may end
it by returning False; a sequence whose next position would reach the context length ends (the
reference returns an error for its single sequence, session.go:69-72; in a batch the sequence ends
with reason "length" and the others go on).  Stop *strings* need a tokenizer and are out of scope.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple

from ..sampling.sampler import SamplerConfig, make_sampler
from .step import StepEntry


@dataclass
class GenerateParams:
    """pkg/runtime GenerateParams as used by session.go:133-159."""
    max_tokens: int = 128
    sampler: object = field(default_factory=SamplerConfig)   # a SamplerConfig, or a function of a row's logits
    repeat_penalty: float = 1.0
    repeat_last_n: int = 64
    stop_token_ids: Optional[Sequence[int]] = None     # None: the model's own (eos_token_id)
    on_token: Optional[Callable[[int, int], bool]] = None   # (request index, token) -> go on?
    keep_logits: bool = False      # results carry the float32 logits every sampled token was drawn from (host copies)


@dataclass
class GenerationResult:
    tokens: List[int]
    finish_reason: str        # "stop" | "length" | "callback"
    prompt_tokens: int
    logits: Optional[list] = None     # with GenerateParams.keep_logits: one [vocab] float32 row per sampling step, the
                                      # one that ended the sequence with a stop token included


def plan_batches(prompt_lens: Sequence[int], max_new: int, max_batch: int, capacity_tokens: int,
                 page_size: int, context: int) -> List[List[int]]:
    """Split requests, in order, into batches that fit: at most `max_batch` sequences, and pages for
    every sequence's prompt plus its new tokens (bounded by the context) within the cache."""
    if max_batch <= 0:
        raise ValueError("max_batch must be positive")
    batches: List[List[int]] = []
    cur: List[int] = []
    used = 0
    for i, n in enumerate(prompt_lens):
        if n <= 0:
            raise ValueError(f"request {i}: empty prompt")
        if n > context:
            raise ValueError(f"request {i}: prompt of {n} tokens exceeds the context of {context}")
        need_tokens = min(n + max(max_new, 0), context)
        need = -(-need_tokens // page_size) * page_size
        if need > capacity_tokens:
            raise ValueError(f"request {i}: needs room for {need} tokens but the cache holds {capacity_tokens}")
        if cur and (len(cur) >= max_batch or used + need > capacity_tokens):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


class Generator:
    """Runs batches of requests on a stepper (anything with `.step(entries)` and `.cache`)."""

    def __init__(self, stepper, vocab_size: int, context: int, default_stop: Sequence[int] = (),
                 max_batch: int = 64, prefill_tokens: int = 16384):
        self.stepper = stepper
        self.cache = stepper.cache
        self.vocab_size = vocab_size
        self.context = context
        self.default_stop = tuple(default_stop)
        self.max_batch = max_batch
        # The prompts of a batch run in as few steps as hold this many tokens each (a longer prompt is cut):
        # the activations of a step grow with its tokens, the time of a token does not shrink beyond this.
        self.prefill_tokens = prefill_tokens
        self.timer = None            # a PhaseTimer (engine.timing) when per-phase timing was asked for

    def _tic(self, phase: str, tokens: int = 0) -> None:
        if self.timer is not None:
            self.timer.begin(phase, tokens)

    def _toc(self) -> None:
        if self.timer is not None:
            self.timer.end()

    def _prefill(self, live: List[int], prompts, slots, cached=None):
        """The prompts of the batch, in order; returns the logits of their last tokens, one row per request.
        `cached[i]` tokens of request i are in its slot already (a conversation's earlier turns): only the
        rest of its prompt runs.  A step holds at most `prefill_tokens` tokens: the prompts are packed into
        steps in order, and a prompt that does not fit what is left of a step goes on in the next one (its
        later tokens read its earlier ones from the cache, as a decode step does)."""
        cached = cached or {}
        steps: List[List[Tuple[int, int, int]]] = [[]]      # per step: (request, first token, one past the last)
        room = self.prefill_tokens
        for i in live:
            a, n = cached.get(i, 0), len(prompts[i])
            while a < n:
                if room == 0:
                    steps.append([])
                    room = self.prefill_tokens
                take = min(n - a, room)
                steps[-1].append((i, a, a + take))
                a += take
                room -= take
        outs = {}
        for st in steps:
            entries = [StepEntry(slots[i], list(prompts[i][a:e]), want=[e - a - 1] if e == len(prompts[i]) else [])
                       for i, a, e in st]
            self._tic("prefill", sum(e - a for _, a, e in st))
            logits = self.stepper.step(entries)
            self._toc()
            ends = [i for i, a, e in st if e == len(prompts[i])]
            if len(steps) == 1:
                return logits
            for r, i in enumerate(ends):                     # a step's logits live until the next step
                outs[i] = logits[r:r + 1].clone()
        import torch
        return torch.cat([outs[i] for i in live], dim=0)

    def generate(self, prompts: Sequence[Sequence[int]], params: Optional[GenerateParams] = None,
                 held: Optional[dict] = None) -> List[GenerationResult]:
        """`held` maps a request's index to a slot that is open already and holds the first tokens of its
        prompt (as many as the cache says): only the rest of the prompt is run, and when the request ends
        the slot stays open, cut back to the tokens of prompt + result that it holds (a conversation,
        pkg/runtime/conversation.go:87-133).  A prompt that is wholly in its slot gives its last token
        back first, so that there are logits to sample from (conversation.go:120-126)."""
        params = params or GenerateParams()
        max_new = params.max_tokens if params.max_tokens > 0 else 128      # session.go:134-137
        results: List[Optional[GenerationResult]] = [None] * len(prompts)
        batches = plan_batches([len(p) for p in prompts], max_new, self.max_batch,
                               self._room(held), self.cache.page_size, self.context)
        for batch in batches:
            self._run_batch(batch, prompts, params, max_new, results, held or {})
        return [r for r in results if r is not None]

    def _room(self, held: Optional[dict] = None) -> int:
        """Tokens this call may plan with: what is free now plus what its own held slots already hold.
        Pages of other open slots (another conversation, an open session) are not this call's to use, so a
        request that cannot fit beside them is refused before the first step instead of failing in the
        middle of decoding."""
        cache = self.cache
        ps = cache.page_size
        own = sum(-(-cache.length(s) // ps) * ps for s in (held or {}).values())
        return min(cache.max_tokens, cache.free_tokens() + own)

    def _let_go(self, i: int, slots, held, prompts, generated) -> None:
        """Request i has ended: its slot goes back, unless its owner holds it; then it keeps the tokens of
        prompt + result that are in it and loses what a step ahead of the host put beyond them."""
        s = slots.pop(i)
        if i not in held:
            self.cache.close(s)
            return
        keep = min(self.cache.length(s), len(prompts[i]) + len(generated[i]))
        if not self.cache.truncate(s, keep):
            self.cache.restart(s)            # the owner runs the whole history again at its next turn

    def _finish_reason(self, i: int, t: int, prompts, generated, params: GenerateParams, max_new: int,
                       stop) -> Optional[str]:
        """Take the sampled token `t` of request i: append it unless it stops the sequence, and say why the
        sequence ends, if it does (pkg/runtime/session.go:58-72, :143-151)."""
        if t < 0 or t in stop:
            return "stop"
        generated[i].append(int(t))
        if params.on_token is not None and not params.on_token(i, int(t)):
            return "callback"
        if len(generated[i]) >= max_new:
            return "length"
        if len(prompts[i]) + len(generated[i]) > self.context:
            return "length"          # the token's own position would lie outside the context
        return None

    def _run_batch(self, batch: List[int], prompts, params: GenerateParams, max_new: int, results,
                   held=None) -> None:
        held = held or {}
        stop = set(self.default_stop if params.stop_token_ids is None else params.stop_token_ids)
        sampler = make_sampler(params.sampler, params.repeat_penalty, params.repeat_last_n, self.vocab_size)
        cache = self.cache
        slots, cached = {}, {}
        generated = {i: [] for i in batch}
        live: List[int] = list(batch)
        try:
            for i in batch:
                if i in held:
                    slots[i] = held[i]
                    have = min(cache.length(held[i]), len(prompts[i]) - 1)
                    if not cache.truncate(held[i], have):
                        cache.restart(held[i])
                        have = 0
                    cached[i] = have
                else:
                    slots[i] = cache.open()
            logits = self._prefill(live, prompts, slots, cached)
            # a step ahead of the host needs a stepper that replays captured decode steps
            # (and no copies of every step's logits to the host, which the loop below makes)
            ahead = (hasattr(self.stepper, "decode_from_device") and getattr(self.stepper, "capturable", True)
                     and getattr(logits, "is_cuda", False) and len(live) <= 256 and not params.keep_logits)
            kept = {i: [] for i in batch} if params.keep_logits else None
            if ahead:
                sampler.begin(live, [prompts[i] for i in live], logits.device)     # rings for a repeat penalty
            if ahead and sampler.device_only:
                self._decode_one_ahead(live, logits, sampler, slots, generated, prompts, params, max_new, stop, results,
                                       held)
                return
            while live:
                hist = [list(prompts[i]) + generated[i] for i in live] if sampler.penalised else None
                self._tic("sample", len(live))
                nxt = sampler.sample(logits, streams=live, steps=[len(generated[i]) for i in live],
                                     histories=hist)
                self._toc()
                if kept is not None:
                    host = logits[:len(live)].float().cpu()
                    for r, i in enumerate(live):
                        kept[i].append(host[r])
                go_on: List[int] = []
                for i, t in zip(live, nxt):
                    reason = self._finish_reason(i, t, prompts, generated, params, max_new, stop)
                    if reason is None:
                        go_on.append(i)
                    else:
                        results[i] = GenerationResult(generated[i], reason, len(prompts[i]),
                                                      kept[i] if kept is not None else None)
                        self._let_go(i, slots, held, prompts, generated)
                live = go_on
                if not live:
                    break
                entries = [StepEntry(slots[i], [generated[i][-1]], want=[0]) for i in live]
                self._tic("decode", len(live))
                logits = self.stepper.step(entries)
                self._toc()
        finally:
            for i in list(slots):
                self._let_go(i, slots, held, prompts, generated)

    def _decode_one_ahead(self, live, logits, sampler, slots, generated, prompts, params, max_new, stop, results,
                          held=None):
        """The same loop with the device kept busy: while the host reads the ids of step k, step k + 1 is
        already running on the ids that the sampling kernel left on the device.  A sequence whose id turns
        out to be a stop token (or whose callback says stop) was then run one step too far; its extra row
        is dropped and its slot is given back, and nobody else's result depends on it."""
        rows = list(live)                                   # requests whose ids are on their way
        self._tic("sample", len(rows))
        pending = sampler.sample_async(logits, rows, [len(generated[i]) for i in rows])
        self._toc()
        dev_row = {i: r for r, i in enumerate(rows)}        # where each request's id sits in the device buffer
        while rows:
            # who certainly goes on after the id that is on its way (its value is not needed for this)?
            cont = [i for i in rows
                    if len(generated[i]) + 1 < max_new and len(prompts[i]) + len(generated[i]) + 1 <= self.context]
            nxt_pending = None
            if cont:
                src = [dev_row[i] for i in cont]
                self._tic("decode", len(cont))
                logits = self.stepper.decode_from_device([slots[i] for i in cont], pending.device_tokens, src)
                self._toc()
                self._tic("sample")
                nxt_pending = sampler.sample_async(logits, cont, [len(generated[i]) + 1 for i in cont])
                self._toc()
            ids = pending.tokens()                           # the host catches up with the previous step
            stopped = set()
            for i, t in zip(rows, ids):
                reason = self._finish_reason(i, t, prompts, generated, params, max_new, stop)
                if reason is not None:
                    results[i] = GenerationResult(generated[i], reason, len(prompts[i]))
                    self._let_go(i, slots, held or {}, prompts, generated)
                    stopped.add(i)
            if nxt_pending is None:
                break
            dev_row = {i: r for r, i in enumerate(cont)}
            if stopped & set(cont):
                # rows of sequences that have ended are still in the step that is running: take the ids of
                # the others from their places
                keep = [i for i in cont if i not in stopped]
                nxt_pending = _SubsetSample(nxt_pending, [cont.index(i) for i in keep])
                cont = keep
            rows, pending = cont, nxt_pending


class _SubsetSample:
    """Some rows of a pending sample: ids of sequences that ended meanwhile are left out."""

    def __init__(self, base, keep_rows):
        self._base, self._keep = base, list(keep_rows)
        self.device_tokens = base.device_tokens
        self.rows = len(self._keep)
        self.row_map = self._keep

    def tokens(self):
        ids = self._base.tokens()
        return [ids[r] for r in self._keep]


class GenerationSession:
    """Step-by-step generation after a prefill (GenerationSession, pkg/runtime/session.go:11-81): the
    caller asks for one token at a time and may change the sampling between steps.

    `start` runs the prompts of a batch in one step (StartGeneration, session.go:19-41) and keeps the
    logits of their last tokens; `decode_step` samples one token per live sequence from the kept logits,
    with the repeat penalty over prompt + generated (session.go:83-103), ends the sequences whose token
    is a stop token or below 0 (neither appended nor run, session.go:58-65) or whose next position lies
    outside the context (session.go:69-72: an error there, the end of that sequence here, since others
    may go on), runs the new tokens of the others as one step and keeps their logits.  A sequence that
    has ended gives -1 from then on and its slot is free at once."""

    def __init__(self, generator: "Generator", prompts: Sequence[Sequence[int]],
                 stop_token_ids: Optional[Sequence[int]] = None):
        self._gen = generator
        self.prompts = [list(p) for p in prompts]
        n = len(self.prompts)
        if n == 0 or n > generator.max_batch:
            raise ValueError(f"a session takes 1 to {generator.max_batch} prompts, not {n}")
        plan = plan_batches([len(p) for p in self.prompts], 1, generator.max_batch, generator._room(),
                            generator.cache.page_size, generator.context)
        if len(plan) != 1:
            raise ValueError("the prompts of a session must fit the cache together")
        self.stop = set(generator.default_stop if stop_token_ids is None else stop_token_ids)
        self.generated: List[List[int]] = [[] for _ in range(n)]
        self.finish_reason: List[Optional[str]] = [None] * n
        self._slots = {}
        self._samplers = {}
        self._live: List[int] = list(range(n))
        try:
            for i in range(n):
                self._slots[i] = generator.cache.open()
            self._logits = generator._prefill(self._live, self.prompts, self._slots)
        except Exception:
            self.close()
            raise

    @property
    def live(self) -> List[int]:
        """Indices of the requests that have not ended."""
        return list(self._live)

    def decode_step(self, params: Optional[GenerateParams] = None) -> List[int]:
        """DecodeStepWith (session.go:50-81) for every request: its next token, or -1 if it has ended."""
        params = params or GenerateParams()
        out = [-1] * len(self.prompts)
        if not self._live:
            return out
        key = (params.sampler, params.repeat_penalty, params.repeat_last_n)
        sampler = self._samplers.get(key)
        if sampler is None:
            sampler = self._samplers[key] = make_sampler(params.sampler, params.repeat_penalty, params.repeat_last_n,
                                                         self._gen.vocab_size)
        live = self._live
        hist = [self.prompts[i] + self.generated[i] for i in live] if sampler.penalised else None
        nxt = sampler.sample(self._logits, streams=live, steps=[len(self.generated[i]) for i in live], histories=hist)
        go_on: List[int] = []
        for i, t in zip(live, nxt):
            t = int(t)
            if t < 0 or t in self.stop:
                self._end(i, "stop")
                continue
            self.generated[i].append(t)
            out[i] = t
            if len(self.prompts[i]) + len(self.generated[i]) > self._gen.context:
                self._end(i, "length")           # the token's own position would lie outside the context
                continue
            go_on.append(i)
        self._live = go_on
        if go_on:
            entries = [StepEntry(self._slots[i], [self.generated[i][-1]], want=[0]) for i in go_on]
            self._logits = self._gen.stepper.step(entries)
        return out

    def _end(self, i: int, reason: str) -> None:
        self.finish_reason[i] = reason
        self._gen.cache.close(self._slots.pop(i))

    def generated_tokens(self, i: int = 0) -> List[int]:
        """GeneratedTokens (session.go:106-110)."""
        return list(self.generated[i])

    def generated_count(self, i: int = 0) -> int:
        """GeneratedCount (session.go:118-120)."""
        return len(self.generated[i])

    def prompt_token_count(self, i: int = 0) -> int:
        """PromptTokenCount (session.go:123-125)."""
        return len(self.prompts[i])

    def close(self) -> None:
        """Give back the slots of the requests that are still live."""
        for i in list(self._slots):
            self._gen.cache.close(self._slots.pop(i))
        self._live = []

    def __enter__(self) -> "GenerationSession":
        return self

    def __exit__(self, *exc) -> None:
        self.close()
