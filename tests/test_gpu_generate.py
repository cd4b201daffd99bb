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
    # a function of the row's logits in the sampler's place (gogguf.Greedy is one)
    out = ctx.generate(prompts, gg.GenerateParams(max_tokens=4, stop_token_ids=[], sampler=gg.Greedy))
    assert [r.tokens for r in out] == [ref0[:4], ref1[:4]]
    # the logits every token was drawn from, on request
    out = ctx.generate(prompts, gg.GenerateParams(max_tokens=3, stop_token_ids=[], keep_logits=True))
    for p, r in zip(prompts, out):
        assert len(r.logits) == 3
        whole = plain.forward(cfg, w, list(p) + r.tokens[:2], wide=True)
        for k, row in enumerate(r.logits):
            assert rel_err(row, whole[len(p) - 1 + k]) < TOL_F32
            assert int(row.argmax()) == r.tokens[k]
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


@pytest.mark.parametrize("name,first,back", [("A", 70, 3), ("B", 70, 3), ("W", 130, 50)])
def test_conversation_turns_equal_whole_histories(tmp_path_factory, name, first, back):
    """Several turns in one slot: every turn's tokens are those of the plain implementation on the whole
    history, although only the new tokens are run; a stop token that the device ran one step ahead of the
    host is cut out of the slot again; a rollback cuts the slot and the next turn goes on from there (with
    windows, "W", the rollback reaches behind a page that the window has already given back: the slot
    starts again and the next turn runs the whole history)."""
    import gogguf_b200 as gg
    folder = make_folder(tmp_path_factory.getbasetemp(), name, "float32")
    cfg, w = read_folder(folder)
    V = cfg["vocab_size"]
    engine = gg.load(folder, gg.LoadOptions(dtype="float32", max_tokens=2048))
    ctx = engine.new_context()
    conv = ctx.new_conversation()
    p1 = random_tokens(V, first, 5)                            # more than a page
    r1 = conv.generate(p1, gg.GenerateParams(max_tokens=6, stop_token_ids=[]))
    assert r1.tokens == plain.generate_greedy(cfg, w, p1, 6, wide=True)
    assert ctx.cache.length(conv._slot) <= len(p1) + 6 and conv.token_count() == len(p1) + 6
    # second turn: the history and some new tokens; ends on a stop token, which the device had already run
    p2 = conv.tokens + random_tokens(V, 9, 6)
    ref2 = plain.generate_greedy(cfg, w, p2, 10, wide=True)
    stop = ref2[4] if ref2[4] not in ref2[:4] else None
    r2 = conv.generate(p2, gg.GenerateParams(max_tokens=10, stop_token_ids=[stop] if stop is not None else []))
    want2 = ref2[:4] if stop is not None else ref2
    assert r2.tokens == want2 and r2.prompt_tokens == len(p2)
    assert conv.tokens == p2 + want2
    assert ctx.cache.length(conv._slot) <= len(conv.tokens)
    # third turn after a rollback into the middle of the second
    conv.rollback(len(p2) - back)
    assert ctx.cache.length(conv._slot) == (len(p2) - back if name != "W" else 0)
    p3 = conv.tokens + random_tokens(V, 2, 7)
    r3 = conv.generate(p3, gg.GenerateParams(max_tokens=5, stop_token_ids=[]))
    assert r3.tokens == plain.generate_greedy(cfg, w, p3, 5, wide=True)
    # a prompt that does not go on from the history starts the slot again; other requests run beside it
    p4 = random_tokens(V, 11, 8)
    r4 = conv.generate(p4, gg.GenerateParams(max_tokens=4, stop_token_ids=[]))
    other = ctx.generate([p1[:5]], gg.GenerateParams(max_tokens=4, stop_token_ids=[]))
    assert r4.tokens == plain.generate_greedy(cfg, w, p4, 4, wide=True)
    assert other[0].tokens == plain.generate_greedy(cfg, w, p1[:5], 4, wide=True)
    r5 = conv.generate(conv.tokens + [3], gg.GenerateParams(max_tokens=3, stop_token_ids=[]))
    assert r5.tokens == plain.generate_greedy(cfg, w, p4 + r4.tokens + [3], 3, wide=True)
    ctx.cache.check()
    conv.close()
    assert ctx.cache.live_slots == 0
    ctx.cache.check()


def test_step_by_step_session_equals_the_loop(tmp_path_factory):
    """Context.start_generation + decode_step: the tokens of the plain implementation, a stop token that
    ends one sequence while the other goes on, sampling changed between steps, slots given back."""
    import gogguf_b200 as gg
    folder = make_folder(tmp_path_factory.getbasetemp(), "B", "float32", scale=8.0)
    cfg, w = read_folder(folder)
    V = cfg["vocab_size"]
    prompts = [random_tokens(V, 9, 31), random_tokens(V, 4, 32)]
    engine = gg.load(folder, gg.LoadOptions(dtype="float32", max_tokens=1024))
    ctx = engine.new_context()
    ref = [plain.generate_greedy(cfg, w, p, 6, wide=True) for p in prompts]
    stop = next(t for t in ref[0][1:] if t not in ref[1])
    with ctx.start_generation(prompts, stop_token_ids=[stop]) as sess:
        got = [sess.decode_step() for _ in range(6)]
    k = ref[0].index(stop)
    assert [g[0] for g in got] == ref[0][:k] + [-1] * (6 - k)
    assert [g[1] for g in got] == ref[1]
    assert sess.finish_reason[0] == "stop" and ctx.cache.live_slots == 0
    # one prompt; greedy for two steps, then seeded temperature sampling with a repeat penalty
    sess = ctx.start_generation(prompts[0], stop_token_ids=[])
    seq = list(prompts[0])
    for step in range(5):
        if step < 2:
            params, want = gg.GenerateParams(), None
        else:
            params = gg.GenerateParams(sampler=gg.SamplerConfig(temp=0.8, top_k=5, seed=11), repeat_penalty=1.2)
        (tok,) = sess.decode_step(params)
        logits = plain.forward(cfg, w, seq, wide=True)[-1].float().tolist()
        if step < 2:
            assert tok == plain.greedy(logits)
        else:
            plain.repeat_penalty(logits, seq, 1.2, 64)
            assert tok == plain.sample(logits, 0.8, 5, 1.0, 0.0, plain.uniform01(11, 0, step))
        seq.append(tok)
    assert sess.generated_tokens() == seq[len(prompts[0]):] and sess.prompt_token_count() == 9
    sess.close()
    ctx.cache.check()
    assert ctx.cache.live_slots == 0


@pytest.mark.parametrize("name", ["L", "M"])
def test_bfloat16_one_step_ahead_loop_on_the_tensor_core_path(tmp_path_factory, name, monkeypatch):
    """bfloat16 through `Context.generate`: captured decode steps, padded batch buckets, ids fed from the
    device, sampling kernels.  The ids equal those of the plain loop over the eager stepper on the same model,
    and the logits the loop sampled from, at every fed position, lie within the bfloat16 bound of the plain
    implementation on the sequence that was generated."""
    import gogguf_b200 as gg
    from gogguf_b200.engine import Stepper
    from gogguf_b200.engine.generate import Generator
    from gogguf_b200.sampling.sampler import Sampler
    folder = make_folder(tmp_path_factory.getbasetemp(), name, "bfloat16", scale=4.0)
    cfg, w = read_folder(folder)
    V = cfg["vocab_size"]
    prompts = [random_tokens(V, n, 70 + n) for n in (140, 3, 66, 31, 9)]       # five rows in a bucket of eight
    engine = gg.load(folder, gg.LoadOptions(dtype="bfloat16", max_tokens=4096))
    seen = []
    real = Sampler.sample_async

    def spy(self, logits, streams, steps):
        seen.append((list(streams), list(steps), logits[:len(streams)].clone()))
        return real(self, logits, streams, steps)

    monkeypatch.setattr(Sampler, "sample_async", spy)
    n_new = 40
    params = gg.GenerateParams(max_tokens=n_new, stop_token_ids=[])
    ctx = engine.new_context()
    ahead = ctx.generate(prompts, params)
    assert ctx.stepper.replays >= n_new - 1 and len(seen) == n_new
    monkeypatch.setattr(Sampler, "sample_async", real)
    model = engine.model
    slow = Generator(Stepper(model, model.new_cache(4096)), V, model.spec.max_positions).generate(prompts, params)
    oracle = [plain.forward(cfg, w, p + r.tokens, wide=True) for p, r in zip(prompts, ahead)]
    for streams, steps, logits in seen:
        for row, (i, k) in enumerate(zip(streams, steps)):
            at = len(prompts[i]) - 1 + k              # the position whose logits the k-th new token was sampled from
            assert rel_err(logits[row:row + 1], oracle[i][at:at + 1]) < TOL_BF16, (i, k)
            assert ahead[i].tokens[k] == int(logits[row].argmax()), (i, k)
    # The eager loop runs the same kernels on batches that are not padded and with the true lengths as the bound
    # of the attention's splits, so its bfloat16 logits differ from the captured steps' in the last bits.  The ids
    # are the same until two candidates lie that close together; from there the sequences are different texts.
    for i, (a, b) in enumerate(zip(ahead, slow)):
        k = next((k for k in range(n_new) if a.tokens[k] != b.tokens[k]), None)
        if k is None:
            continue
        row = oracle[i][len(prompts[i]) - 1 + k]
        top = float(row.abs().max())
        assert abs(float(row[a.tokens[k]] - row[b.tokens[k]])) < TOL_BF16 * top, (i, k)
        assert float(row.max() - row[a.tokens[k]]) < TOL_BF16 * top, (i, k)
    assert sum(a.tokens == b.tokens for a, b in zip(ahead, slow)) >= 2
    # a seeded top-k chain with a repeat penalty, all on the device and a step ahead: every id is what the plain
    # sampler draws from the very logits the kernels saw
    seen.clear()
    monkeypatch.setattr(Sampler, "sample_async", spy)
    sc = gg.SamplerConfig(temp=0.8, top_k=12, top_p=0.9, seed=4)
    params = gg.GenerateParams(max_tokens=12, stop_token_ids=[], repeat_penalty=1.2, sampler=sc)
    out = engine.new_context().generate(prompts, params)
    monkeypatch.setattr(Sampler, "sample_async", real)
    assert len(seen) == 12
    for streams, steps, logits in seen:
        for row, (i, k) in enumerate(zip(streams, steps)):
            lg = logits[row].float().tolist()
            plain.repeat_penalty(lg, prompts[i] + out[i].tokens[:k], 1.2, 64)
            assert out[i].tokens[k] == plain.sample(lg, 0.8, 12, 0.9, 0.0, plain.uniform01(4, i, k)), (i, k)


def test_top_k_beyond_the_kernels_shared_memory_falls_back_to_the_host_chain():
    """top-k 1,024 over more than 163,840 ids does not fit the top-k kernel: the sampler answers from the host
    chain instead of raising, id for id what the plain sampler gives."""
    from gogguf_b200.sampling import Sampler, SamplerConfig
    V = 170000
    logits = torch.randn(3, V, generator=torch.Generator().manual_seed(1)) * 3
    cfg = SamplerConfig(temp=0.9, top_k=1024, top_p=0.95, seed=3)
    s = Sampler(cfg, vocab_size=V)
    assert not s.device_chain and not s.device_only
    got = s.sample(logits.cuda(), [0, 1, 2], [5, 5, 5])
    for r in range(3):
        assert got[r] == plain.sample(logits[r].tolist(), 0.9, 1024, 0.95, 0.0, plain.uniform01(3, r, 5))
    # and within the limit the kernel gives the same ids as the host chain
    V2 = 163840
    s2 = Sampler(cfg, vocab_size=V2)
    assert s2.device_chain
    l2 = logits[:, :V2].contiguous()
    assert s2.sample(l2.cuda(), [0, 1, 2], [5, 5, 5]) == Sampler(cfg).sample(l2, [0, 1, 2], [5, 5, 5])


def test_per_phase_timing_behind_a_flag(tmp_path_factory, capsys):
    """LoadOptions(timing=True): prefill, time to the first token and decode (model steps and sampling apart)
    from CUDA events around the loop's phases; `run --timing` prints the reference's bench lines."""
    import gogguf_b200 as gg
    from gogguf_b200 import cli
    folder = make_folder(tmp_path_factory.getbasetemp(), "L", "bfloat16", scale=4.0)
    cfg, _ = read_folder(folder)
    prompts = [random_tokens(cfg["vocab_size"], n, 90 + n) for n in (200, 31, 7)]
    plain_ctx = gg.load(folder, gg.LoadOptions(max_tokens=4096)).new_context()
    with pytest.raises(ValueError):
        plain_ctx.last_timing()
    want = plain_ctx.generate(prompts, gg.GenerateParams(max_tokens=9, stop_token_ids=[]))
    for sampler in (gg.SamplerConfig(), gg.SamplerConfig(temp=0.8, top_p=0.9, seed=1)):       # a step ahead / host chain
        ctx = gg.load(folder, gg.LoadOptions(max_tokens=4096, timing=True)).new_context()
        out = ctx.generate(prompts, gg.GenerateParams(max_tokens=9, stop_token_ids=[], sampler=sampler))
        if sampler.greedy:
            assert [r.tokens for r in out] == [r.tokens for r in want]          # timing changes no result
        t = ctx.last_timing()
        assert t.prompt_tokens == 238 and t.decode_tokens == 27 and t.prefill_steps == 1 and t.decode_steps == 8
        assert 0 < t.prefill_ms <= t.ttft_ms <= t.total_ms and 0 < t.step_ms < t.decode_ms < t.total_ms
        assert t.sampling_ms > 0 and t.decode_tps > 0 and t.prefill_tps > 0 and t.host_ms > 0
        assert len(t.lines()) == 4 and t.lines()[0].startswith("Prefill (238 tok, 1 step)")
        # a second call starts from zero
        ctx.generate(prompts[:1], gg.GenerateParams(max_tokens=2, stop_token_ids=[]))
        assert ctx.last_timing().prompt_tokens == 200 and ctx.last_timing().decode_tokens == 2
    ids = " ".join(map(str, prompts[2]))
    assert cli.main(["run", "-m", folder, "-p", ids, "-n", "5", "--timing", "--stop-ids", ""]) == 0
    err = capsys.readouterr().err
    assert "Load: " in err and "Prefill (7 tok" in err and "TTFT: " in err and "Decode (5 tok, 4 steps)" in err


def test_random_weights_without_a_folder(tmp_path_factory, capsys):
    """`load_random` makes a model on the device from a configuration and a seed, without a folder;
    `run --random CONFIG.json` is its command line."""
    import os
    import gogguf_b200 as gg
    from gogguf_b200 import cli
    from helpers import TINY
    cfg, seed, std, nstd = TINY["B"]
    folder = make_folder(tmp_path_factory.getbasetemp(), "B", "float32")
    prompts = [random_tokens(cfg["vocab_size"], n, 40 + n) for n in (6, 2)]
    params = gg.GenerateParams(max_tokens=6, stop_token_ids=[])
    opts = gg.LoadOptions(dtype="float32", max_tokens=1024)
    first = gg.load_random(dict(cfg), seed, opts, std=std, norm_std=nstd)
    got = first.new_context().generate(prompts, params)
    again = gg.load_random(dict(cfg), seed, opts, std=std, norm_std=nstd).new_context().generate(prompts, params)
    assert [r.tokens for r in got] == [r.tokens for r in again]                 # a seed names one model
    other = gg.load_random(dict(cfg), seed + 1, opts, std=std, norm_std=nstd).new_context().generate(prompts, params)
    assert [r.tokens for r in other] != [r.tokens for r in got]
    ids = " ".join(map(str, prompts[0]))
    assert cli.main(["run", "--random", os.path.join(folder, "config.json"), "--weights-seed", "3", "-p", ids, "-n", "4",
                     "--dtype", "float32", "--stop-ids", ""]) == 0
    assert len(capsys.readouterr().out.split()) == 4
