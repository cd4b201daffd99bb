"""Each request alone and whole: the engine's logits at every position against the plain implementation."""
import os

import pytest
import torch

import plain_qwen3 as plain
from helpers import TINY, TOL_BF16, TOL_F32, make_folder, random_tokens, read_folder, rel_err

pytestmark = pytest.mark.gpu


def engine_whole(folder, dtype, tokens, fast=True, fold_norms=None):
    from gogguf_b200.engine import Model, StepEntry, Stepper
    model = Model.load(folder, dtype=dtype, fast=fast, fold_norms=fold_norms)
    cache = model.new_cache(max_tokens=1024)
    st = Stepper(model, cache)
    slot = cache.open()
    logits = st.step([StepEntry(slot, tokens, want=list(range(len(tokens))))]).clone()
    cache.close(slot)
    cache.check()
    return logits


@pytest.mark.parametrize("name", ["A", "B", "W"])
@pytest.mark.parametrize("n", [1, 7, 100])
def test_whole_f32(tmp_path_factory, name, n):
    folder = make_folder(tmp_path_factory.getbasetemp(), name, "float32")
    cfg, w = read_folder(folder)
    tokens = random_tokens(cfg["vocab_size"], n, seed=n)
    want = plain.forward(cfg, w, tokens, wide=True)
    got = engine_whole(folder, "float32", tokens)
    assert rel_err(got, want) < TOL_F32


@pytest.mark.parametrize("name", ["B", "L"])
def test_float16_folder_is_exact_on_the_32_bit_path(tmp_path, name):
    """A checkpoint stored in float16: the 32-bit path runs the stored values themselves (float32 holds
    every float16 exactly), not their bfloat16 rounding; the bfloat16 path rounds them once."""
    from gogguf_b200.weights.safetensors_io import write_safetensors
    folder = make_folder(tmp_path, name, "float32", scale=4.0)
    cfg, w = read_folder(folder)
    w16 = {k: v.to(torch.float16) for k, v in w.items()}
    write_safetensors(os.path.join(folder, "model.safetensors"), w16)
    tokens = random_tokens(cfg["vocab_size"], 90, seed=8)
    want = plain.forward(cfg, {k: v.float() for k, v in w16.items()}, tokens, wide=True)
    got = engine_whole(folder, "float32", tokens)
    assert rel_err(got, want) < TOL_F32
    rounded = plain.forward(cfg, {k: v.to(torch.bfloat16).float() for k, v in w16.items()}, tokens, wide=True)
    assert rel_err(rounded, want) > 20 * TOL_F32        # the test can tell the two apart
    assert rel_err(engine_whole(folder, "bfloat16", tokens), rounded) < TOL_BF16


@pytest.mark.parametrize("name", ["A", "B", "W", "M", "L"])
def test_whole_bf16(tmp_path_factory, name):
    folder = make_folder(tmp_path_factory.getbasetemp(), name, "bfloat16", scale=4.0)
    cfg, w = read_folder(folder)
    tokens = random_tokens(cfg["vocab_size"], 200, seed=3)
    want = plain.forward(cfg, w, tokens, wide=True)
    got = engine_whole(folder, "bfloat16", tokens)
    # These weights are four times the usual size, so that the logits are not flat; rounding the activations to
    # bfloat16 then costs 1.0e-2 to 2.5e-2 of the largest logit whatever the kernels (measured: the twins' error).
    tight = 3e-2
    assert rel_err(got, want) < tight
    # the plain kernels on the same bfloat16 weights (the twins of the tensor-core kernels) agree too
    twin = engine_whole(folder, "bfloat16", tokens, fast=False)
    assert rel_err(twin, want) < tight
    # the fast path differs from the twin in its kernels only: it may not add to the twin's own error
    assert rel_err(got, want) < 1.5 * rel_err(twin, want) + 5e-3
    # and the tensor-core path with every norm as a kernel of its own instead of folded into the products
    unfolded = engine_whole(folder, "bfloat16", tokens, fold_norms=False)
    assert rel_err(unfolded, want) < tight
    assert rel_err(unfolded, want) < 1.5 * rel_err(twin, want) + 5e-3
    if os.environ.get("GOGGUF_B200_FOLD_NORMS", "1") != "0":
        assert not torch.equal(unfolded, got)    # the two really are different routes


def test_norms_are_folded_into_the_products_on_the_fast_path(tmp_path_factory):
    from gogguf_b200.csrc import build
    from gogguf_b200.engine import Model, StepEntry, Stepper
    folder = make_folder(tmp_path_factory.getbasetemp(), "M", "bfloat16", scale=4.0)
    counts = {}
    for fold in (True, False):
        model = Model.load(folder, dtype="bfloat16", fold_norms=fold)
        assert all(b.mixer_folded == fold and b.feed_forward_folded == fold for b in model.blocks)
        cache = model.new_cache(256)
        st = Stepper(model, cache)
        slot = cache.open()
        st.step([StepEntry(slot, [1, 2, 3], want=[2])])
        n0 = build.launch_count()
        st.step([StepEntry(slot, [4], want=[0])])
        counts[fold] = build.launch_count() - n0
        cache.close(slot)
    layers = len(model.blocks)
    assert counts[False] - counts[True] == 2 * layers - 1      # two norms a layer less, one statistics kernel more


@pytest.mark.parametrize("name,dtype", [("L", "bfloat16"), ("M", "bfloat16"), ("B", "float32")])
def test_captured_decode_steps_equal_eager_steps(tmp_path_factory, name, dtype):
    """The generation path replays decode steps as CUDA graphs, padded to a batch bucket; it must give what
    the eager stepper gives, for batches that shrink and for sequences that cross page edges."""
    from gogguf_b200.engine import Model, StepEntry, Stepper
    from gogguf_b200.engine.graphs import GraphStepper
    folder = make_folder(tmp_path_factory.getbasetemp(), name, dtype, scale=1.0 if dtype == "float32" else 3.0)
    cfg, w = read_folder(folder)
    model = Model.load(folder, dtype=dtype)
    reqs = [random_tokens(cfg["vocab_size"], n, n) for n in (150, 9, 70)]
    oracle = [plain.forward(cfg, w, t, wide=True) for t in reqs]
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    results = {}
    for kind in (Stepper, GraphStepper):
        cache = model.new_cache(1024)
        st = kind(model, cache)
        slots = [cache.open() for _ in reqs]
        pre = [len(t) - 25 if len(t) > 30 else 2 for t in reqs]
        st.step([StepEntry(s, t[:p], want=[p - 1]) for s, t, p in zip(slots, reqs, pre)])
        pos, live, got = list(pre), [0, 1, 2], {}
        while live:
            out = st.step([StepEntry(slots[i], [reqs[i][pos[i]]], want=[0]) for i in live]).clone()
            for j, i in enumerate(live):
                got[(i, pos[i])] = out[j]
                assert rel_err(out[j:j + 1], oracle[i][pos[i]:pos[i] + 1]) < tol, (kind.__name__, i, pos[i])
                pos[i] += 1
            live = [i for i in live if pos[i] < len(reqs[i])]
        results[kind.__name__] = got
        if kind is GraphStepper:
            assert st.replays > 20 and len(st._graphs) >= 2       # batch 3 (bucket 4, one padding row), then smaller
    for key, v in results["Stepper"].items():
        assert rel_err(results["GraphStepper"][key][None], v[None]) < (1e-6 if dtype == "float32" else 2e-2), key


def test_bfloat16_run_of_a_folder_stored_in_32_bit(tmp_path_factory):
    """A tensor stored in 32-bit stays 32-bit: under dtype=bfloat16 the activations are bfloat16 and the
    products with such matrices run on the mixed-operand kernel.  The result must be as close to the plain
    implementation as any bfloat16 run."""
    folder = make_folder(tmp_path_factory.getbasetemp(), "M", "float32")
    cfg, w = read_folder(folder)
    tokens = random_tokens(cfg["vocab_size"], 150, seed=8)
    want = plain.forward(cfg, w, tokens, wide=True)
    got = engine_whole(folder, "bfloat16", tokens)
    assert rel_err(got, want) < TOL_BF16
    from gogguf_b200.engine import Model
    m = Model.load(folder, dtype="bfloat16")
    assert m.blocks[0].mixer.qkv.weight.dtype == torch.float32 and m.blocks[0].mixer.qkv._fast is None


def test_decode_projection_does_the_per_head_work_when_the_head_size_is_128(tmp_path_factory, monkeypatch):
    from gogguf_b200.csrc import build
    from gogguf_b200.engine import Model, StepEntry, Stepper
    folder = make_folder(tmp_path_factory.getbasetemp(), "L", "bfloat16", scale=4.0)
    counts, logits = {}, {}
    for fuse in ("1", "0"):
        monkeypatch.setenv("GOGGUF_B200_FUSE_QKV_ROPE", fuse)
        model = Model.load(folder, dtype="bfloat16")
        cache = model.new_cache(256)
        st = Stepper(model, cache)
        slot = cache.open()
        st.step([StepEntry(slot, list(range(1, 70)), want=[68])])
        n0 = build.launch_count()
        logits[fuse] = st.step([StepEntry(slot, [4], want=[0])]).clone()
        counts[fuse] = build.launch_count() - n0
        cache.close(slot)
    assert counts["0"] - counts["1"] == len(model.blocks)       # one kernel a layer less
    assert rel_err(logits["1"], logits["0"]) < 2e-2


def test_prefill_projection_does_the_per_head_work_too(tmp_path_factory, monkeypatch):
    """More than 128 tokens: the CTA-pair form of the q/k/v product has the same epilogue, so a layer of a
    prompt is five kernels as well; the logits of every position agree with the separate kernel's."""
    from gogguf_b200.csrc import build
    from gogguf_b200.engine import Model, StepEntry, Stepper
    if os.environ.get("GOGGUF_B200_GEMM_PAIR", "1") == "0":
        pytest.skip("the single-CTA prefill form has no q/k/v epilogue")
    folder = make_folder(tmp_path_factory.getbasetemp(), "L", "bfloat16", scale=4.0)
    cfg, w = read_folder(folder)
    prompts = [random_tokens(cfg["vocab_size"], n, 60 + n) for n in (300, 131)]
    counts, logits = {}, {}
    for fuse in ("1", "0"):
        monkeypatch.setenv("GOGGUF_B200_FUSE_QKV_ROPE", fuse)
        model = Model.load(folder, dtype="bfloat16")
        cache = model.new_cache(1024)
        st = Stepper(model, cache)
        slots = [cache.open(), cache.open()]
        st.step([StepEntry(slots[0], prompts[0][:5], want=[4])])        # position 0 is not where the prompt's rest starts
        n0 = build.launch_count()
        logits[fuse] = st.step([StepEntry(slots[0], prompts[0][5:], want=list(range(295))),
                                StepEntry(slots[1], prompts[1], want=list(range(131)))]).clone()
        counts[fuse] = build.launch_count() - n0
        for s_ in slots:
            cache.close(s_)
    assert counts["0"] - counts["1"] == len(model.blocks)       # one kernel a layer less
    assert rel_err(logits["1"], logits["0"]) < 2e-2
    want = torch.cat([plain.forward(cfg, w, prompts[0], wide=True)[5:], plain.forward(cfg, w, prompts[1], wide=True)])
    assert rel_err(logits["1"], want) < TOL_BF16


def test_a_stored_head_of_a_tied_model_is_named_and_not_used(tmp_path):
    from gogguf_b200.weights.safetensors_io import write_safetensors
    folder = make_folder(tmp_path, "A", "float32")
    cfg, w = read_folder(folder)
    tokens = random_tokens(cfg["vocab_size"], 12, seed=2)
    want = engine_whole(folder, "float32", tokens)
    w["lm_head.weight"] = torch.randn_like(w["model.embed_tokens.weight"])       # another matrix altogether
    write_safetensors(os.path.join(folder, "model.safetensors"), w)
    with pytest.warns(UserWarning, match="ties the head"):
        got = engine_whole(folder, "float32", tokens)
    assert torch.equal(got, want)


@pytest.mark.parametrize("graphs", [False, True])
def test_a_status_per_entry_and_the_good_entries_still_run(tmp_path_factory, graphs):
    """try_step on the device: bad entries are named and change nothing, the others give the logits they give
    alone, for prompts and (through captured graphs too) for decode steps."""
    from gogguf_b200.engine import Model, StepEntry, Stepper
    from gogguf_b200.engine.graphs import GraphStepper
    folder = make_folder(tmp_path_factory.getbasetemp(), "B", "float32")
    cfg, w = read_folder(folder)
    V = cfg["vocab_size"]
    a, b = random_tokens(V, 21, 1), random_tokens(V, 9, 2)
    wa, wb = plain.forward(cfg, w, a, wide=True), plain.forward(cfg, w, b, wide=True)
    model = Model.load(folder, dtype="float32")
    cache = model.new_cache(64 * 4)
    st = (GraphStepper if graphs else Stepper)(model, cache)
    sa, sb, sc = cache.open(), cache.open(), cache.open()
    out = st.try_step([StepEntry(sa, a[:-1], want=[19]), StepEntry(sc, [1, V], want=[0]), StepEntry(sb, b[:-1], want=[0, 7]),
                       StepEntry(99, [1])])
    assert [s.code if s else None for s in out.status] == [None, "bad_token", None, "unknown_slot"]
    assert rel_err(out.logits, torch.cat([wa[19:20], wb[[0, 7]]])) < TOL_F32
    assert cache.length(sc) == 0 and cache.length(sa) == 20
    # a decode step: one entry would pass the context's end, the others go on
    cache.lengths[sc] = cfg["max_position_embeddings"]            # as if slot c were full
    out = st.try_step([StepEntry(sa, a[-1:], want=[0]), StepEntry(sc, [3], want=[0]), StepEntry(sb, b[-1:], want=[0])])
    assert [s.code if s else None for s in out.status] == [None, "context_overflow", None]
    assert rel_err(out.logits, torch.cat([wa[-1:], wb[-1:]])) < TOL_F32
    if graphs:
        assert st.replays == 1
    cache.lengths[sc] = 0
    assert st.try_step([StepEntry(sc, [], want=[])]).logits is None
    for s in (sa, sb, sc):
        cache.close(s)
    cache.check()
