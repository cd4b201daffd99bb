"""The library's entry point, in the manner of the reference's facade (gogguf.go:14-82):

    engine = gogguf_b200.load(folder, LoadOptions(dtype="bfloat16"))
    ctx = engine.new_context()
    results = ctx.generate([[1, 2, 3], [4, 5]], GenerateParams(max_tokens=16,
                           sampler=SamplerConfig(temp=0.8, seed=7)))

`load` reads a model folder (config.json + model.safetensors), `Engine.new_context` makes a cache
and a stepper (runtime.Engine.NewContext, pkg/runtime/context.go:29-38), `Context.generate` runs the
generation loop (Context.Generate, context.go:100-130) and `Context.forward_token_ids` is the raw
hook (Engine.ForwardTokenIDs, pkg/runtime/engine.go:79-81).  Prompts are token ids: the tokenizer
and chat templates of the reference are outside this library.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Union

import torch

from .engine.generate import GenerateParams, GenerationResult, GenerationSession, Generator
from .engine.model import Model
from .engine.step import StepEntry, Stepper
from .sampling.sampler import Sampler, SamplerConfig, greedy as Greedy  # noqa: N812


@dataclass
class LoadOptions:
    """Where the reference has NGL and GPUMaxSeq (pkg/runtime/options.go:6-9) this library has the
    compute dtype and the cache size: the whole model always runs on the GPU."""
    dtype: str = "bfloat16"
    device: str = "cuda:0"
    max_tokens: int = 0           # cache capacity in tokens; 0: the model's context length
    max_batch: int = 64
    fast: bool = True             # False: plain kernels only (for comparisons)
    graphs: bool = True           # replay captured decode steps where possible
    timing: bool = False          # bracket prefill, decode steps and sampling with CUDA events (Context.last_timing)


class Engine:
    def __init__(self, model: Model, options: LoadOptions):
        self.model = model
        self.options = options

    def context_length(self) -> int:
        """pkg/runtime/engine.go: ContextLength from the model's metadata."""
        return self.model.spec.max_positions

    def new_context(self, max_tokens: Optional[int] = None, max_batch: Optional[int] = None) -> "Context":
        mt = max_tokens or self.options.max_tokens or self.context_length()
        return Context(self, mt, max_batch or self.options.max_batch)

    def close(self) -> None:
        self.model = None


class Context:
    def __init__(self, engine: Engine, max_tokens: int, max_batch: int):
        self.engine = engine
        model = engine.model
        self.cache = model.new_cache(max_tokens)
        if engine.options.graphs and model.rt.device.type == "cuda":
            from .engine.graphs import GraphStepper
            self.stepper = GraphStepper(model, self.cache)
        else:
            self.stepper = Stepper(model, self.cache)
        self.generator = Generator(self.stepper, model.spec.vocab_size, model.spec.max_positions,
                                   default_stop=model.spec.stop_token_ids, max_batch=max_batch)
        if engine.options.timing:
            from .engine.timing import PhaseTimer
            self.generator.timer = PhaseTimer(model.rt.device)

    def generate(self, prompts: Union[Sequence[int], Sequence[Sequence[int]]],
                 params: Optional[GenerateParams] = None) -> Union[GenerationResult, List[GenerationResult]]:
        """One prompt (a list of ids) gives one result; a list of prompts gives a list."""
        single = len(prompts) > 0 and isinstance(prompts[0], int)
        if self.generator.timer is not None:
            self.generator.timer.reset()
        res = self.generator.generate([list(prompts)] if single else [list(p) for p in prompts], params)
        return res[0] if single else res

    def last_timing(self):
        """The `PhaseReport` of the last `generate` call (LoadOptions(timing=True)): prefill, time to the first
        token, decode split into model steps and sampling, on the device (cmd/tools/bench.go:302-364)."""
        if self.generator.timer is None:
            raise ValueError("this context was not made with LoadOptions(timing=True)")
        return self.generator.timer.report()

    def start_generation(self, prompts: Union[Sequence[int], Sequence[Sequence[int]]],
                         stop_token_ids: Optional[Sequence[int]] = None) -> GenerationSession:
        """Context.StartGeneration (pkg/runtime/session.go:19-41): the prompts run in one step, then the
        caller takes one token per `decode_step`.  One prompt (a list of ids) or a batch of them."""
        single = len(prompts) > 0 and isinstance(prompts[0], int)
        return GenerationSession(self.generator, [list(prompts)] if single else [list(p) for p in prompts],
                                 stop_token_ids)

    def new_conversation(self) -> "Conversation":
        """Context.NewConversation (pkg/runtime/conversation.go:15-17)."""
        return Conversation(self)

    def forward_token_ids(self, tokens: Sequence[int]) -> torch.Tensor:
        """Logits [len(tokens), vocab] of one fresh sequence (float32, on the device)."""
        slot = self.cache.open()
        try:
            out = self.stepper.step([StepEntry(slot, list(tokens), want=list(range(len(tokens))))])
            return out.clone()
        finally:
            self.cache.close(slot)


class Conversation:
    """Several turns in one cache slot (Conversation, pkg/runtime/conversation.go:9-151).

    Every call of `generate` brings the whole conversation so far as token ids, as the reference's
    takes the whole rendered prompt.  If it goes on from the tokens that the slot holds, only the new
    ones are run (conversation.go:107-117); if it is shorter or differs somewhere, the slot starts
    again (`should_reset`, conversation.go:135-137).  After a turn the history is the prompt plus the
    tokens that were made (`Commit`, conversation.go:36-38); a turn that raises leaves the history as
    it was (conversation.go:67-70)."""

    def __init__(self, ctx: "Context"):
        self.ctx = ctx
        self.tokens: List[int] = []
        self._slot: Optional[int] = None

    @staticmethod
    def should_reset(held: Sequence[int], prompt: Sequence[int]) -> bool:
        """conversation.go:135-151: the held tokens must be a prefix of the prompt."""
        n = len(held)
        return n > len(prompt) or list(prompt[:n]) != list(held)

    def token_count(self) -> int:
        """TokenCount (conversation.go:26-28): prompt and made tokens of the turns so far."""
        return len(self.tokens)

    def reset(self) -> None:
        """Reset (conversation.go:20-23): no history, an empty slot."""
        self.tokens = []
        if self._slot is not None:
            self.ctx.cache.restart(self._slot)

    def rollback(self, token_count: int) -> None:
        """Rollback (conversation.go:40-58): back to the first `token_count` tokens.  The reference runs
        them again from an empty cache; here the slot is cut where its groups allow it, and only
        otherwise emptied, in which case the next turn runs the history again."""
        if token_count < 0 or token_count > len(self.tokens):
            raise ValueError(f"the conversation holds {len(self.tokens)} tokens, cannot go back to {token_count}")
        self.tokens = self.tokens[:token_count]
        if self._slot is not None:
            cache = self.ctx.cache
            if not cache.truncate(self._slot, min(cache.length(self._slot), token_count)):
                cache.restart(self._slot)

    def generate(self, prompt: Sequence[int], params: Optional[GenerateParams] = None) -> GenerationResult:
        """Generate (conversation.go:60-74)."""
        prompt = list(prompt)
        if not prompt:
            raise ValueError("empty prompt")            # conversation.go:118-119
        if self._slot is None:
            self._slot = self.ctx.cache.open()
        if self.should_reset(self.tokens, prompt):
            self.reset()
        cache = self.ctx.cache
        # the slot may hold fewer tokens than the history (the last made token is not run until it is
        # needed), never other ones
        if cache.length(self._slot) > len(self.tokens):
            if not cache.truncate(self._slot, len(self.tokens)):
                cache.restart(self._slot)
        snap = len(self.tokens)
        try:
            res = self.ctx.generator.generate([prompt], params, held={0: self._slot})[0]
        except Exception:
            self.rollback(snap)
            raise
        self.tokens = prompt + list(res.tokens)
        return res

    def close(self) -> None:
        if self._slot is not None:
            self.ctx.cache.close(self._slot)
            self._slot = None
        self.tokens = []


def load(path: str, options: Optional[LoadOptions] = None) -> Engine:
    """gogguf.Load (gogguf.go:52-55): model folder -> engine."""
    options = options or LoadOptions()
    if not torch.cuda.is_available():
        raise RuntimeError("gogguf_b200 needs a CUDA device (B200); there is no CPU path")
    model = Model.load(path, dtype=options.dtype, device=options.device, fast=options.fast)
    return Engine(model, options)


def load_random(config, seed: int = 0, options: Optional[LoadOptions] = None, std: Optional[float] = None,
                norm_std: float = 0.0) -> Engine:
    """An engine over random weights made on the device from a configuration (a config.json path or its
    dictionary) and a seed: the random-weights mode without a folder in between.  The values come from the
    device's generator, so a seed names another model here than in a folder written by `random` (which draws
    on the host); the same seed gives the same model every time."""
    import json
    from .config import config_from_dict
    options = options or LoadOptions()
    if not torch.cuda.is_available():
        raise RuntimeError("gogguf_b200 needs a CUDA device (B200); there is no CPU path")
    if not isinstance(config, dict):
        with open(config) as f:
            config = json.load(f)
    model = Model.random(config_from_dict(config), seed=seed, dtype=options.dtype, device=options.device,
                         fast=options.fast, std=std, norm_std=norm_std)
    return Engine(model, options)


def new_sampler(cfg: SamplerConfig) -> Sampler:
    """gogguf.NewSampler (gogguf.go:63-66)."""
    return Sampler(cfg)
