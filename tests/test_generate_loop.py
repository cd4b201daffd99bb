"""The generation loop's decisions, with a scripted model on the CPU (no GPU)."""
import pytest
import torch

from gogguf_b200.cache import KVRequest, SequenceCache
from gogguf_b200.engine.generate import GenerateParams, Generator, plan_batches
from gogguf_b200.sampling import SamplerConfig

V = 16


class ScriptedStepper:
    """Stands in for the stepper: the next token of a sequence is (last token + 1) % V."""

    def __init__(self, max_tokens=64 * 8, max_slots=None):
        self.cache = SequenceCache([KVRequest(1, 4)], [None], max_tokens, dtype=torch.float32, device="cpu",
                                   max_slots=max_slots)
        self.steps = []

    def step(self, entries):
        slots = [e.slot for e in entries]
        counts = [len(e.tokens) for e in entries]
        self.cache.plan(slots, counts)
        self.steps.append([(e.slot, len(e.tokens)) for e in entries])
        rows = []
        for e in entries:
            for w in e.want:
                row = torch.zeros(V)
                row[(e.tokens[w] + 1) % V] = 5.0
                rows.append(row)
        self.cache.commit(slots, counts)
        self.cache.check()
        return torch.stack(rows) if rows else None


def gen(stepper, context=1000, **kw):
    return Generator(stepper, V, context, **kw)


def test_plan_batches():
    assert plan_batches([5, 3, 9], 4, max_batch=2, capacity_tokens=640, page_size=64, context=100) == [[0, 1], [2]]
    # capacity: each needs 2 pages (70+20=90 -> 128), 3 pages in all -> one per batch
    assert plan_batches([70, 70], 20, 8, 192, 64, 1000) == [[0], [1]]
    # the context bounds what a sequence can hold
    assert plan_batches([60, 60], 500, 8, 128, 64, context=64) == [[0, 1]]
    with pytest.raises(ValueError):
        plan_batches([0], 4, 2, 640, 64, 100)
    with pytest.raises(ValueError):
        plan_batches([200], 4, 2, 640, 64, 100)
    with pytest.raises(ValueError):
        plan_batches([100], 100, 2, 128, 64, 1000)


def test_unequal_prompts_and_token_limit():
    st = ScriptedStepper()
    out = gen(st).generate([[1, 2, 3], [7]], GenerateParams(max_tokens=3))
    assert [r.tokens for r in out] == [[4, 5, 6], [8, 9, 10]]
    assert all(r.finish_reason == "length" for r in out)
    assert st.steps[0] == [(st.steps[0][0][0], 3), (st.steps[0][1][0], 1)]      # prompts in one step
    assert all(n == 1 for step in st.steps[1:] for _, n in step)                # then one token each
    assert len(st.steps) == 3            # the third token is sampled but never fed
    assert st.cache.live_slots == 0


def test_stop_token_is_neither_kept_nor_fed_and_others_go_on():
    st = ScriptedStepper()
    out = gen(st).generate([[1], [9]], GenerateParams(max_tokens=6, stop_token_ids=[4]))
    assert out[0].tokens == [2, 3] and out[0].finish_reason == "stop"           # 4 is not appended
    assert out[1].tokens == [10, 11, 12, 13, 14, 15] and out[1].finish_reason == "length"
    sizes = [len(s) for s in st.steps]
    assert sizes == [2, 2, 2, 1, 1, 1]   # the batch shrinks when the first sequence ends
    fed = sum(n for s in st.steps for _, n in s)
    assert fed == 2 + 2 + 2 + 1 + 1 + 1  # the stop token itself was never fed
    st.cache.check()


def test_results_can_carry_the_logits_each_token_was_drawn_from():
    st = ScriptedStepper()
    out = gen(st).generate([[1], [9]], GenerateParams(max_tokens=4, stop_token_ids=[4], keep_logits=True))
    assert out[0].tokens == [2, 3] and out[1].tokens == [10, 11, 12, 13]
    # one row per sampling step: the step whose token was the stop token is there too
    assert len(out[0].logits) == 3 and len(out[1].logits) == 4
    for r in out:
        assert all(row.shape == (V,) and row.dtype == torch.float32 for row in r.logits)
    assert [int(row.argmax()) for row in out[0].logits] == [2, 3, 4]
    assert [int(row.argmax()) for row in out[1].logits] == [10, 11, 12, 13]
    assert gen(ScriptedStepper()).generate([[1]], GenerateParams(max_tokens=2))[0].logits is None


def test_default_stop_tokens_come_from_the_model():
    st = ScriptedStepper()
    out = gen(st, default_stop=(3,)).generate([[1]], GenerateParams(max_tokens=9))
    assert out[0].tokens == [2] and out[0].finish_reason == "stop"
    out = gen(st, default_stop=(3,)).generate([[1]], GenerateParams(max_tokens=4, stop_token_ids=[]))
    assert out[0].tokens == [2, 3, 4, 5]


def test_batches_follow_one_another_and_reuse_slots():
    st = ScriptedStepper(max_slots=2)
    prompts = [[i] for i in range(5)]
    out = gen(st, max_batch=2).generate(prompts, GenerateParams(max_tokens=2))
    assert [r.tokens for r in out] == [[i + 1, i + 2] for i in range(5)]
    prefills = [s for s in st.steps if any(n >= 1 for _, n in s)][::2]
    used = {slot for s in st.steps for slot, _ in s}
    assert used <= {0, 1} and st.cache.live_slots == 0


def test_context_limit_ends_one_sequence_only():
    st = ScriptedStepper()
    out = gen(st, context=6).generate([[1, 2, 3, 4], [1]], GenerateParams(max_tokens=5))
    # 4 prompt tokens: positions 4 and 5 can be fed, the token that would sit at 6 cannot
    assert out[0].tokens == [5, 6, 7] and out[0].finish_reason == "length"
    assert out[1].tokens == [2, 3, 4, 5, 6]
    assert max(st.cache.lengths) == 0 and st.cache.live_slots == 0


def test_callback_can_end_a_sequence():
    st = ScriptedStepper()
    seen = []

    def cb(i, t):
        seen.append((i, t))
        return not (i == 0 and t == 3)

    out = gen(st).generate([[1], [5]], GenerateParams(max_tokens=4, on_token=cb))
    assert out[0].tokens == [2, 3] and out[0].finish_reason == "callback"
    assert out[1].tokens == [6, 7, 8, 9]


def test_max_tokens_zero_means_128():
    st = ScriptedStepper(max_tokens=64 * 4)
    out = gen(st).generate([[1]], GenerateParams(max_tokens=0))
    assert len(out[0].tokens) == 128       # session.go:134-137


def test_temperature_draws_do_not_depend_on_the_batch():
    p = GenerateParams(max_tokens=4, sampler=SamplerConfig(temp=1.5, seed=11))

    class Flat(ScriptedStepper):
        def step(self, entries):
            super().step(entries)
            return torch.zeros(sum(len(e.want) for e in entries), V)     # uniform distribution

    alone = gen(Flat()).generate([[3]], p)[0].tokens
    both = gen(Flat()).generate([[3], [9, 9]], p)
    assert both[0].tokens == alone and both[1].tokens != alone


def test_prompts_of_a_large_batch_run_in_several_steps():
    """The prompts of a batch start together but need not share one step: a step holds at most `prefill_tokens`
    tokens (a longer prompt is cut and goes on from the cache), the results are those of one step, and decoding
    begins after the last."""
    prompts = [[1, 2, 3, 4, 5], [7, 8], [2] * 6, [9], [4, 4, 4]]
    one = ScriptedStepper()
    want = gen(one).generate(prompts, GenerateParams(max_tokens=3))
    st = ScriptedStepper()
    out = gen(st, prefill_tokens=7).generate(prompts, GenerateParams(max_tokens=3))
    assert [r.tokens for r in out] == [r.tokens for r in want]
    assert [[n for _, n in step] for step in st.steps[:3]] == [[5, 2], [6, 1], [3]]      # 7, 7 and 3 tokens
    assert all(n == 1 for step in st.steps[3:] for _, n in step) and len(st.steps[3]) == 5
    assert one.steps[0] == [(s, n) for s, n in one.steps[0]] and len(one.steps[0]) == 5  # by default: one step
    st.cache.check()
    assert st.cache.live_slots == 0
    # prompts longer than a step: 10 and 3 tokens in steps of 4 -> 4 | 4 | 2 + 2 | 1, the logits of each
    # request taken from the step that holds its last token
    prompts = [list(range(1, 11)), [5, 6, 7]]
    st = ScriptedStepper()
    out = gen(st, prefill_tokens=4).generate(prompts, GenerateParams(max_tokens=2))
    assert [r.tokens for r in out] == [[11, 12], [8, 9]]
    assert [[n for _, n in step] for step in st.steps[:4]] == [[4], [4], [2, 2], [1]]
    assert st.steps[2][0][0] == st.steps[0][0][0] and st.steps[3][0][0] == st.steps[2][1][0]
    assert [n for _, n in st.steps[4]] == [1, 1]
    st.cache.check()


# ----------------------------------------------------------------------------- conversations
class _Ctx:
    """What a Conversation needs of a context: a cache and a generator."""

    def __init__(self, stepper, context=1000):
        self.stepper = stepper
        self.cache = stepper.cache
        self.generator = gen(stepper, context)


def test_conversation_runs_only_what_is_new():
    from gogguf_b200.api import Conversation
    st = ScriptedStepper()
    conv = Conversation(_Ctx(st))
    r1 = conv.generate([1, 2, 3], GenerateParams(max_tokens=3))
    assert r1.tokens == [4, 5, 6]
    assert conv.token_count() == 6 and conv.tokens == [1, 2, 3, 4, 5, 6]
    assert st.cache.live_slots == 1 and st.cache.length(conv._slot) == 5       # 6 was sampled, not run
    n_before = len(st.steps)
    # the next turn brings the whole conversation plus two new tokens: 6 (not yet run), 9 and 10 are run
    r2 = conv.generate(conv.tokens + [9, 10], GenerateParams(max_tokens=2))
    assert r2.tokens == [11, 12] and r2.prompt_tokens == 8
    assert st.steps[n_before] == [(conv._slot, 3)]
    assert conv.tokens == [1, 2, 3, 4, 5, 6, 9, 10, 11, 12]
    # a prompt that is wholly in the slot gives its last token back to have logits (conversation.go:120-126)
    conv.rollback(8)
    assert st.cache.length(conv._slot) == 8
    n_before = len(st.steps)
    r3 = conv.generate(conv.tokens, GenerateParams(max_tokens=1))
    assert r3.tokens == [11] and st.steps[n_before] == [(conv._slot, 1)]
    st.cache.check()
    conv.close()
    assert st.cache.live_slots == 0
    st.cache.check()


def test_conversation_starts_again_when_the_prompt_does_not_go_on_from_it():
    from gogguf_b200.api import Conversation
    assert Conversation.should_reset([1, 2, 3, 4, 5], [9, 9])                   # shorter (conversation_test.go:24-26)
    assert not Conversation.should_reset([1, 2, 3, 4, 5], [1, 2, 3, 4, 5, 6])   # goes on (:28-30)
    assert Conversation.should_reset([1, 2, 3, 4, 5], [1, 2, 9, 4, 5])          # differs (:32-34)
    st = ScriptedStepper()
    conv = Conversation(_Ctx(st))
    conv.generate([1, 2, 3], GenerateParams(max_tokens=2))
    n_before = len(st.steps)
    r = conv.generate([7, 8], GenerateParams(max_tokens=2))
    assert r.tokens == [9, 10] and st.steps[n_before] == [(conv._slot, 2)]
    assert conv.tokens == [7, 8, 9, 10] and st.cache.length(conv._slot) == 3
    conv.reset()
    assert conv.token_count() == 0 and st.cache.length(conv._slot) == 0
    st.cache.check()


def test_conversation_keeps_its_history_when_a_turn_fails():
    from gogguf_b200.api import Conversation
    st = ScriptedStepper(max_tokens=64 * 2)
    conv = Conversation(_Ctx(st))
    conv.generate([1, 2, 3], GenerateParams(max_tokens=2))
    held = list(conv.tokens)
    with pytest.raises(ValueError):
        conv.generate(held + [5] * 200, GenerateParams(max_tokens=2))          # more than the cache holds
    assert conv.tokens == held
    r = conv.generate(held + [1], GenerateParams(max_tokens=1))
    assert r.tokens == [2]
    st.cache.check()


def test_conversation_stop_token_is_not_in_the_slot():
    from gogguf_b200.api import Conversation
    st = ScriptedStepper()
    conv = Conversation(_Ctx(st))
    r = conv.generate([1], GenerateParams(max_tokens=8, stop_token_ids=[4]))
    assert r.tokens == [2, 3] and r.finish_reason == "stop"
    assert conv.tokens == [1, 2, 3] and st.cache.length(conv._slot) == 3       # 3 was run, 4 was not


# ----------------------------------------------------------------------------- step-by-step sessions
def test_session_gives_one_token_per_step_and_minus_one_after_the_end():
    from gogguf_b200.engine.generate import GenerationSession
    st = ScriptedStepper()
    sess = GenerationSession(gen(st), [[1, 2], [9]], stop_token_ids=[4])
    assert st.steps == [[(sess._slots[0], 2), (sess._slots[1], 1)]] and sess.live == [0, 1]
    assert sess.decode_step() == [3, 10]
    assert sess.decode_step() == [-1, 11]                  # 4 stops the first: not kept, not run
    assert sess.finish_reason == ["stop", None] and sess.live == [1]
    assert st.cache.live_slots == 1 and st.steps[-1] == [(sess._slots[1], 1)]
    assert sess.decode_step(GenerateParams(sampler=SamplerConfig(temp=0.5, seed=3))) == [-1, 12]   # one-hot logits
    assert sess.generated_tokens(0) == [3] and sess.generated_tokens(1) == [10, 11, 12]
    assert sess.generated_count(1) == 3 and sess.prompt_token_count(0) == 2
    sess.close()
    assert st.cache.live_slots == 0 and sess.decode_step() == [-1, -1]
    st.cache.check()


def test_session_ends_a_sequence_at_the_context_and_frees_slots_on_errors():
    from gogguf_b200.engine.generate import GenerationSession
    st = ScriptedStepper()
    with GenerationSession(gen(st, context=4), [[1, 2, 3]], stop_token_ids=[]) as sess:
        assert sess.decode_step() == [4]                   # position 3 is the last one
        assert sess.decode_step() == [5] and sess.finish_reason == ["length"]     # 5 is given, cannot be run
        assert sess.decode_step() == [-1]
    assert st.cache.live_slots == 0
    with pytest.raises(ValueError):
        GenerationSession(gen(st, context=4), [[1, 2, 3, 4, 5]])
    with pytest.raises(ValueError):
        GenerationSession(gen(ScriptedStepper(max_tokens=64)), [[1] * 40, [2] * 40])      # two pages needed, one there
    assert st.cache.live_slots == 0


# ----------------------------------------------------------------------------- a caller's own sampler
def test_a_function_can_take_the_samplers_place():
    """GenerateParams.sampler may be a function of a row's logits (sampler.Func of the reference): it is
    called once per live sequence and step, after the repeat penalty, and an id below 0 ends the sequence."""
    import numpy as np
    import gogguf_b200 as gg
    seen = []

    def second_best(row):
        assert isinstance(row, np.ndarray) and row.dtype == np.float32 and row.shape == (V,)
        seen.append(int(np.argmax(row)))
        return int(np.argsort(row)[-2])             # some id whose logit is 0

    st = ScriptedStepper()
    out = gen(st).generate([[1], [9]], GenerateParams(max_tokens=3, sampler=second_best, stop_token_ids=[]))
    assert seen[:2] == [2, 10] and len(seen) == 6
    assert all(len(r.tokens) == 3 for r in out)
    # gg.Greedy is such a function (gogguf.Greedy)
    out = gen(ScriptedStepper()).generate([[1]], GenerateParams(max_tokens=3, sampler=gg.Greedy, stop_token_ids=[]))
    assert out[0].tokens == [2, 3, 4]
    # the repeat penalty reaches the function's logits: token 2's logit 5.0 is divided by 2.5
    def look(row):
        look.row = row.copy()
        return 7
    gen(ScriptedStepper()).generate([[3, 1]], GenerateParams(max_tokens=1, sampler=look, repeat_penalty=2.5,
                                                             stop_token_ids=[]))
    assert look.row[2] == 5.0                       # 2 is not in the history
    gen(ScriptedStepper()).generate([[2, 1]], GenerateParams(max_tokens=1, sampler=look, repeat_penalty=2.5,
                                                             stop_token_ids=[]))
    assert look.row[2] == 2.0
    # an id below 0 ends the sequence (session.go:58-60)
    out = gen(ScriptedStepper()).generate([[1]], GenerateParams(max_tokens=5, sampler=lambda row: -1))
    assert out[0].tokens == [] and out[0].finish_reason == "stop"
    with pytest.raises(TypeError):
        gen(ScriptedStepper()).generate([[1]], GenerateParams(sampler="greedy"))


def test_interactive_mode_is_one_conversation_with_a_line_of_ids_per_turn():
    import io
    from gogguf_b200.api import Conversation
    from gogguf_b200.cli import run_interactive
    st = ScriptedStepper()

    class Ctx(_Ctx):
        def new_conversation(self):
            return Conversation(self)

    ctx = Ctx(st)
    out = io.StringIO()
    inp = io.StringIO("9 10\n/clear\n5\n\n7\n")          # the empty line ends it: "7" is never read
    rc = run_interactive(ctx, GenerateParams(max_tokens=2, stop_token_ids=[]), [[1, 2, 3]], inp, out)
    assert rc == 0
    assert out.getvalue().splitlines() == ["4 5", "11 12", "6 7"]
    # first turn: the prompt; second: 5 (made, not yet run), 9 and 10; after /clear the slot starts again
    assert [n for step in st.steps for _, n in step] == [3, 1, 3, 1, 1, 1]
    assert st.cache.live_slots == 0
    st.cache.check()


def test_two_conversations_share_one_cache_and_a_request_that_cannot_fit_beside_them_is_refused():
    """Batches are planned against what is free now plus what the call's own slot holds, not against the
    whole cache: pages held by another conversation are not this call's to use."""
    from gogguf_b200.api import Conversation
    st = ScriptedStepper(max_tokens=64 * 4)
    a, b = Conversation(_Ctx(st)), Conversation(_Ctx(st))
    a.generate(list(range(1, 11)) * 10, GenerateParams(max_tokens=20))       # 100 + 20 tokens: 2 pages held
    assert st.cache.free_tokens() == 64 * 2
    # b asks for 3 pages: the whole cache would hold them, what is free does not -> refused before any step
    n_before = len(st.steps)
    with pytest.raises(ValueError, match="needs room"):
        b.generate([1] * 100, GenerateParams(max_tokens=60))
    assert len(st.steps) == n_before
    st.cache.check()
    # what fits beside a runs, and a's slot is untouched by it
    r = b.generate([1, 2, 3], GenerateParams(max_tokens=4))
    assert r.tokens == [4, 5, 6, 7] and st.cache.length(a._slot) == 119
    # a may grow into its own pages and the free ones
    r = a.generate(a.tokens + [5], GenerateParams(max_tokens=3))
    assert r.tokens == [6, 7, 8]
    a.close(); b.close()
    st.cache.check()
    assert st.cache.free_tokens() == 64 * 4 and st.cache.live_slots == 0
