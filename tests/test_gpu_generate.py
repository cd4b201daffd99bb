"""Generation through the entry point against the plain implementation; long decoding; first tokens."""
import pytest
import torch

import plain_qwen3 as plain
from helpers import TOL_BF16, TOL_F32, make_folder, random_tokens, read_folder, rel_err

pytestmark = pytest.mark.gpu


def test_greedy_generation_through_the_entry_point(tmp_path_factory):
    import gogguf_b200 as gg
    folder = make_folder(tmp_path_factory.getbasetemp(), "A", "float32")
    cfg, w = read_folder(folder)
    prompts = [random_tokens(cfg["vocab_size"], 5, 1), random_tokens(cfg["vocab_size"], 3, 2)]
    engine = gg.load(folder, gg.LoadOptions(dtype="float32", max_tokens=1024))
    ctx = engine.new_context()
    out = ctx.generate(prompts, gg.GenerateParams(max_tokens=4, stop_token_ids=[]))
    for p, r in zip(prompts, out):
        assert r.tokens == plain.generate_greedy(cfg, w, p, 4, wide=True)
        assert r.finish_reason == "length" and r.prompt_tokens == len(p)
    # a stop token ends one sequence early; the other goes on and its tokens do not change
    ref0 = plain.generate_greedy(cfg, w, prompts[0], 12, wide=True)
    ref1 = plain.generate_greedy(cfg, w, prompts[1], 12, wide=True)
    stop = next(t for t in ref0[2:] if t not in ref1)
    out = ctx.generate(prompts, gg.GenerateParams(max_tokens=12, stop_token_ids=[stop]))
    assert out[0].tokens == ref0[:ref0.index(stop)] and out[0].finish_reason == "stop"
    assert out[1].tokens == ref1
    # a single prompt gives a single result
    one = ctx.generate(prompts[0], gg.GenerateParams(max_tokens=3, stop_token_ids=[]))
    assert one.tokens == ref0[:3]
    ctx.cache.check()
    assert ctx.cache.live_slots == 0


def test_temperature_sampling_follows_the_plain_sampler(tmp_path_factory):
    import gogguf_b200 as gg
    folder = make_folder(tmp_path_factory.getbasetemp(), "B", "float32", scale=8.0)
    cfg, w = read_folder(folder)
    prompts = [random_tokens(cfg["vocab_size"], n, 20 + n) for n in (7, 1, 4)]
    engine = gg.load(folder, gg.LoadOptions(dtype="float32", max_tokens=1024))
    params = gg.GenerateParams(max_tokens=5, sampler=gg.SamplerConfig(temp=0.8, seed=123), stop_token_ids=[])
    out = engine.new_context().generate(prompts, params)
    for i, (p, r) in enumerate(zip(prompts, out)):
        seq = list(p)
        for k, tok in enumerate(r.tokens):
            logits = plain.forward(cfg, w, seq, wide=True)[-1].float().tolist()
            assert tok == plain.sample(logits, 0.8, 0, 1.0, 0.0, plain.uniform01(123, i, k)), (i, k)
            seq.append(tok)
    # a top-k chain runs on the device too (one step ahead of the host, like greedy)
    sc = gg.SamplerConfig(temp=0.7, top_k=6, top_p=0.85, min_p=0.02, seed=9)
    assert sc.on_device and sc.device_chain
    out = engine.new_context().generate(prompts, gg.GenerateParams(max_tokens=5, sampler=sc, stop_token_ids=[]))
    for i, (p, r) in enumerate(zip(prompts, out)):
        seq = list(p)
        for k, tok in enumerate(r.tokens):
            logits = plain.forward(cfg, w, seq, wide=True)[-1].float().tolist()
            assert tok == plain.sample(logits, 0.7, 6, 0.85, 0.02, plain.uniform01(9, i, k)), (i, k)
            seq.append(tok)
    # with a repeat penalty: the last ids of every sequence live in a ring on the device (here a short one, so
    # that it wraps), the penalty and the append are kernels, and the loop still runs one step ahead
    for sc, last_n in ((gg.SamplerConfig(temp=0.9, top_k=7, top_p=0.9, seed=5), 64), (gg.SamplerConfig(), 4),
                       (gg.SamplerConfig(temp=1.1, seed=2), 3)):
        params = gg.GenerateParams(max_tokens=9, sampler=sc, repeat_penalty=1.3, repeat_last_n=last_n, stop_token_ids=[])
        out = engine.new_context().generate(prompts, params)
        for i, (p, r) in enumerate(zip(prompts, out)):
            seq = list(p)
            for k, tok in enumerate(r.tokens):
                logits = plain.forward(cfg, w, seq, wide=True)[-1].float().tolist()
                plain.repeat_penalty(logits, seq, 1.3, last_n)
                assert tok == plain.sample(logits, sc.temp, sc.top_k, sc.top_p, sc.min_p, plain.uniform01(sc.seed, i, k)), (i, k)
                seq.append(tok)
    # top-p without a top-k has no kernel: the host chain, with the penalty, on the same logits
    params = gg.GenerateParams(max_tokens=4, sampler=gg.SamplerConfig(temp=0.9, top_p=0.9, seed=5),
                               repeat_penalty=1.3, stop_token_ids=[])
    out = engine.new_context().generate(prompts[:1], params)
    seq = list(prompts[0])
    for k, tok in enumerate(out[0].tokens):
        logits = plain.forward(cfg, w, seq, wide=True)[-1].float().tolist()
        plain.repeat_penalty(logits, seq, 1.3, 64)
        assert tok == plain.sample(logits, 0.9, 0, 0.9, 0.0, plain.uniform01(5, 0, k))
        seq.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(tmp_path_factory, dtype):
    from gogguf_b200.engine import Model, StepEntry, Stepper
    name = "W"
    folder = make_folder(tmp_path_factory.getbasetemp(), name, dtype, scale=1.0 if dtype == "float32" else 4.0)
    cfg, w = read_folder(folder)
    toks = random_tokens(cfg["vocab_size"], 330, 4)
    oracle = plain.forward(cfg, w, toks, wide=True)
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    model = Model.load(folder, dtype=dtype)
    cache = model.new_cache(512)
    st = Stepper(model, cache)
    s = cache.open()
    # the first tokens of a sequence, one by one from position 0, then hundreds of single steps
    for i, t in enumerate(toks):
        got = st.step([StepEntry(s, [t], want=[0])])
        if i < 4 or i % 37 == 0 or i > 320:
            assert rel_err(got, oracle[i:i + 1]) < tol, i
    cache.close(s)
    cache.check()


def test_one_step_ahead_loop_equals_the_plain_loop(tmp_path_factory):
    """The entry point keeps the device one step ahead of the host (the next step starts from ids that are
    still on the device).  Sequences that end on a stop token, on a callback or on the token limit while
    the step after theirs is already running must give the same tokens as the step-by-step loop."""
    import gogguf_b200 as gg
    from gogguf_b200.engine import Model, Stepper
    from gogguf_b200.engine.generate import Generator
    folder = make_folder(tmp_path_factory.getbasetemp(), "B", "float32", scale=6.0)
    cfg, w = read_folder(folder)
    prompts = [random_tokens(cfg["vocab_size"], n, 40 + n) for n in (9, 2, 17, 5)]
    refs = [plain.generate_greedy(cfg, w, p, 14, wide=True) for p in prompts]
    stop_tok = refs[0][5]
    engine = gg.load(folder, gg.LoadOptions(dtype="float32", max_tokens=2048))
    seen = []

    def cb(i, t):
        seen.append((i, t))
        return not (i == 2 and len([1 for j, _ in seen if j == 2]) == 4)      # request 2 ends after 4 tokens

    params = gg.GenerateParams(max_tokens=14, stop_token_ids=[stop_tok], on_token=cb)
    ahead = engine.new_context().generate(prompts, params)
    # the same requests through the eager stepper, which has no device-side token feed: the plain loop
    model = engine.model
    cache = model.new_cache(2048)
    seen.clear()
    slow = Generator(Stepper(model, cache), model.spec.vocab_size, model.spec.max_positions).generate(prompts, params)
    for a, b in zip(ahead, slow):
        assert a.tokens == b.tokens and a.finish_reason == b.finish_reason
    # and against the plain implementation
    def expected(i):
        out = []
        for k, t in enumerate(refs[i]):
            if t == stop_tok:
                return out, "stop"
            out.append(t)
            if i == 2 and len(out) == 4:
                return out, "callback"
        return out, "length"
    for i, r in enumerate(ahead):
        toks, why = expected(i)
        assert r.tokens == toks and r.finish_reason == why, i
    assert cache.live_slots == 0
