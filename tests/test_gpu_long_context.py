"""Long contexts, for correctness: decode attention over thousands of cached keys (the path that puts sixteen
splits of one sequence into a cluster), prompts that the generation loop cuts into several steps, and one step
of more than 65,535 tokens.  The models are tiny (one layer) so that the plain implementation can follow; the
q-norm weights are scaled up so that the softmax is peaked and a page that is skipped or counted twice shows."""
import math
import os

import pytest
import torch

import plain_qwen3 as plain
from helpers import TOL_BF16, TOL_F32, random_tokens, read_folder, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

LONG_128 = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=1, hidden_size=256, num_attention_heads=4, num_key_value_heads=1, head_dim=128,
    intermediate_size=320, vocab_size=777, rope_theta=1000000.0, rms_norm_eps=1e-6,
    tie_word_embeddings=True, max_position_embeddings=70016,
)
LONG_64 = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=1, hidden_size=136, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
    intermediate_size=200, vocab_size=523, rope_theta=500000.0, rms_norm_eps=2e-6,
    tie_word_embeddings=False, max_position_embeddings=70016,
)


def long_folder(tmp, cfg, dtype, seed):
    """A one-layer model with q-norm weights of about 3: scores up to 3 * sqrt(head_dim), a peaked softmax."""
    from gogguf_b200.config import config_from_dict
    from gogguf_b200.engine.model import write_random_model
    from gogguf_b200.weights.safetensors_io import write_safetensors
    folder = os.path.join(str(tmp), f"long_{cfg['head_dim']}_{dtype}")
    if not os.path.isdir(folder):
        write_random_model(config_from_dict(cfg), seed, folder, dtype=dtype, std=0.08, norm_std=0.05)
        _, w = read_folder(folder)
        w["model.layers.0.self_attn.q_norm.weight"] = w["model.layers.0.self_attn.q_norm.weight"] * 3
        write_safetensors(os.path.join(folder, "model.safetensors"), w)
    return folder


@pytest.mark.parametrize("cfg,dtype", [(LONG_128, "bfloat16"), (LONG_64, "bfloat16"), (LONG_128, "float32")])
def test_decode_over_thousands_of_keys(tmp_path_factory, cfg, dtype):
    """Three sequences of 5,000, 9,000 and 20,000 keys decode together, then the longest alone (one sequence
    with a long context: sixteen splits in a cluster), eight steps each through captured graphs."""
    from gogguf_b200.engine import Model, StepEntry
    from gogguf_b200.engine.graphs import GraphStepper
    folder = long_folder(tmp_path_factory.getbasetemp(), cfg, dtype, seed=31)
    c, w = read_folder(folder)
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    lens = [5000, 9000, 20000] if dtype == "bfloat16" else [5000, 9000]
    n_dec = 8
    seqs = [random_tokens(c["vocab_size"], n, seed=n) for n in lens]
    rows = [list(range(n - n_dec - 1, n)) for n in lens]
    oracle = [plain.forward(c, w, t, wide=dtype == "float32", rows=r) for t, r in zip(seqs, rows)]
    model = Model.load(folder, dtype=dtype)
    cache = model.new_cache(sum(lens) + 64 * 4)
    st = GraphStepper(model, cache)
    for group in ([0, 1, 2][:len(lens)], [len(lens) - 1]):
        slots = {i: cache.open() for i in group}
        got = st.step([StepEntry(slots[i], seqs[i][:lens[i] - n_dec], want=[lens[i] - n_dec - 1]) for i in group])
        for j, i in enumerate(group):
            assert rel_err(got[j:j + 1], oracle[i][0:1]) < tol, ("prompt", i)
        before = st.replays
        for k in range(n_dec):
            got = st.step([StepEntry(slots[i], [seqs[i][lens[i] - n_dec + k]], want=[0]) for i in group])
            for j, i in enumerate(group):
                assert rel_err(got[j:j + 1], oracle[i][k + 1:k + 2]) < tol, ("decode", i, k)
        assert st.replays == before + n_dec
        for s in slots.values():
            cache.close(s)
        cache.check()


@pytest.mark.parametrize("cfg", [LONG_128, LONG_64])
def test_a_long_prompt_cut_by_the_generation_loop(tmp_path_factory, cfg):
    """A 20,000-token prompt and a 3,000-token one: in one step, and cut by the loop into steps of at most
    16,384 tokens (the later part of the long prompt reads its earlier part from the cache).  The same
    logits, hence the same tokens, and those of the plain implementation."""
    import gogguf_b200 as gg
    from gogguf_b200.engine import StepEntry
    folder = long_folder(tmp_path_factory.getbasetemp(), cfg, "bfloat16", seed=31)
    c, w = read_folder(folder)
    prompts = [random_tokens(c["vocab_size"], 20000, 1), random_tokens(c["vocab_size"], 3000, 2)]
    engine = gg.load(folder, gg.LoadOptions(dtype="bfloat16", max_tokens=32768))
    ctx = engine.new_context()
    assert ctx.generator.prefill_tokens == 16384
    seen = []
    real = ctx.stepper.step
    ctx.stepper.step = lambda entries, taps=None: (seen.append([len(e.tokens) for e in entries]), real(entries, taps))[1]
    cut_logits = ctx.generator._prefill([0, 1], prompts, {0: ctx.cache.open(), 1: ctx.cache.open()}).clone()
    assert seen == [[16384], [3616, 3000]]
    for s in [i for i in range(ctx.cache.max_slots) if ctx.cache.slots.is_held(i)]:
        ctx.cache.close(s)
    slots = [ctx.cache.open(), ctx.cache.open()]
    whole = real([StepEntry(s, p, want=[len(p) - 1]) for s, p in zip(slots, prompts)]).clone()
    for s in slots:
        ctx.cache.close(s)
    want = torch.cat([plain.forward(c, w, p, rows=[len(p) - 1]) for p in prompts])
    assert rel_err(whole, want) < TOL_BF16 and rel_err(cut_logits, want) < TOL_BF16
    assert rel_err(cut_logits, whole) < 1e-2
    ctx.stepper.step = real
    out = ctx.generate(prompts, gg.GenerateParams(max_tokens=4, stop_token_ids=[]))
    assert [len(r.tokens) for r in out] == [4, 4] and ctx.cache.live_slots == 0
    ctx.cache.check()


def test_one_step_of_more_than_65535_tokens(tmp_path_factory):
    """66,000 tokens in one step, one sequence of 40,000 and one of 26,000: grids whose second and third
    dimensions stop at 65,535 must not be indexed by the token."""
    from gogguf_b200.engine import Model, StepEntry, Stepper
    folder = long_folder(tmp_path_factory.getbasetemp(), LONG_128, "bfloat16", seed=31)
    c, w = read_folder(folder)
    lens = [40000, 26000]
    seqs = [random_tokens(c["vocab_size"], n, seed=n + 1) for n in lens]
    wants = [[0, 1000, 39999], [7, 25535, 25536, 25999]]       # rows on both sides of 65,535 in the packed step
    model = Model.load(folder, dtype="bfloat16")
    cache = model.new_cache(sum(lens) + 128)
    st = Stepper(model, cache)
    slots = [cache.open(), cache.open()]
    got = st.step([StepEntry(s, t, want=wt) for s, t, wt in zip(slots, seqs, wants)])
    want = torch.cat([plain.forward(c, w, t, rows=wt) for t, wt in zip(seqs, wants)])
    for r in range(want.shape[0]):
        assert rel_err(got[r:r + 1], want[r:r + 1]) < TOL_BF16, r
    for s in slots:
        cache.close(s)
    cache.check()
