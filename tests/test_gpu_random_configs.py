"""Configurations drawn from a seeded generator: head sizes in steps of 16 up to 256, any number of heads and
groups, widths and vocabularies that are no power of two, one to three layers, windows on some layers, tied or
separate heads.  Each is checked whole, then token by token, in 32-bit and in bfloat16, against the plain
implementation, like the fixed tiny configurations elsewhere: what differs here is that nobody chose the sizes."""
import json
import os
import random

import pytest
import torch

import plain_qwen3 as plain
from helpers import TOL_BF16, TOL_F32, random_tokens, read_folder, rel_err

pytestmark = pytest.mark.gpu


def draw_config(seed: int) -> dict:
    r = random.Random(seed)
    d = r.choice([16, 32, 48, 64, 80, 96, 112, 128, 160, 256])
    nkv = r.choice([1, 2, 3, 5])
    group = r.choice([1, 2, 3, 4, 7])
    layers = r.choice([1, 2, 3])
    hidden = r.choice([8, 16, 24]) * r.choice([3, 5, 7, 9, 11])            # multiples of 8, none a power of two
    cfg = dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=layers, hidden_size=hidden,
        num_attention_heads=nkv * group, num_key_value_heads=nkv, head_dim=d,
        intermediate_size=r.choice([8, 64]) * r.choice([3, 5, 7]), vocab_size=r.choice([97, 331, 1000, 2053]),
        rope_theta=r.choice([1e4, 5e4, 1e6]), rms_norm_eps=r.choice([1e-6, 3e-6, 1e-5]),
        tie_word_embeddings=r.random() < 0.5, max_position_embeddings=512,
    )
    if r.random() < 0.5:
        cfg["sliding_window"] = r.choice([5, 37, 64, 100])
        cfg["layer_types"] = [r.choice(["full_attention", "sliding_attention"]) for _ in range(layers)]
        if "sliding_attention" not in cfg["layer_types"]:
            cfg["layer_types"][0] = "sliding_attention"
    return cfg


@pytest.mark.parametrize("seed", list(range(10)))
def test_a_configuration_nobody_chose(tmp_path, seed):
    check_configuration(draw_config(seed), seed, tmp_path)


def edge_config(d, hidden, inter, vocab, nq=4, nkv=2):
    return dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=hidden,
                num_attention_heads=nq, num_key_value_heads=nkv, head_dim=d, intermediate_size=inter, vocab_size=vocab,
                rope_theta=1e4, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=512)


@pytest.mark.parametrize("cfg", [
    edge_config(2, 64, 96, 331), edge_config(24, 64, 96, 331), edge_config(100, 64, 96, 331),
    edge_config(200, 64, 96, 331),                       # head sizes that are no multiple of 16
    edge_config(32, 50, 37, 101), edge_config(32, 4, 2, 3), edge_config(32, 1000, 1001, 999),    # widths no multiple of 8
    edge_config(128, 72, 96, 331, nq=17, nkv=1),         # more query heads per kv head than an MMA tile has rows
    edge_config(64, 72, 96, 331, nq=33, nkv=11),
], ids=lambda c: f"d{c['head_dim']}-h{c['hidden_size']}-i{c['intermediate_size']}-v{c['vocab_size']}-q{c['num_attention_heads']}")
def test_sizes_at_the_edges_of_what_the_kernels_take(tmp_path, cfg):
    """What the configuration allows and no fast kernel was written for goes to the general kernels, with the
    same results."""
    check_configuration(cfg, 3, tmp_path)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_head_size_beyond_the_kernels_is_refused_when_the_model_is_built(tmp_path, dtype):
    from gogguf_b200.config import config_from_dict
    from gogguf_b200.engine import Model
    from gogguf_b200.engine.model import write_random_model
    folder = os.path.join(str(tmp_path), "m")
    write_random_model(config_from_dict(edge_config(272, 64, 96, 331)), 0, folder, dtype=dtype)
    with pytest.raises(ValueError, match="head_dim=272 is not supported"):
        Model.load(folder, dtype=dtype)


def check_configuration(cfg, seed, tmp_path):
    from gogguf_b200.config import config_from_dict
    from gogguf_b200.engine import Model, StepEntry, Stepper
    from gogguf_b200.engine.graphs import GraphStepper
    from gogguf_b200.engine.model import write_random_model
    n = 150
    tokens = random_tokens(cfg["vocab_size"], n, seed)
    for dtype, tol, std in (("float32", TOL_F32, 0.05), ("bfloat16", TOL_BF16, 0.08)):
        folder = os.path.join(str(tmp_path), dtype)
        write_random_model(config_from_dict(cfg), seed, folder, dtype=dtype, std=std, norm_std=0.05)
        c, w = read_folder(folder)
        want = plain.forward(c, w, tokens, wide=True)
        model = Model.load(folder, dtype=dtype)
        cache = model.new_cache(1024)
        # whole
        st = Stepper(model, cache)
        slot = cache.open()
        got = st.step([StepEntry(slot, tokens, want=list(range(n)))]).clone()
        assert rel_err(got, want) < tol, (json.dumps(cfg), dtype)
        cache.close(slot)
        # a prompt, then the rest one by one, as captured graphs, beside a second shorter sequence
        gs = GraphStepper(model, cache)
        a, b = cache.open(), cache.open()
        cut = n - 40
        gs.step([StepEntry(a, tokens[:cut], want=[cut - 1]), StepEntry(b, tokens[:9], want=[8])])
        for k in range(cut, n):
            ents = [StepEntry(a, [tokens[k]], want=[0])]
            if 9 + k - cut < 30:
                ents.append(StepEntry(b, [tokens[9 + k - cut]], want=[0]))
            out = gs.step(ents)
            assert rel_err(out[0:1], want[k:k + 1]) < tol, (json.dumps(cfg), dtype, k)
            if len(ents) == 2:
                assert rel_err(out[1:2], want[9 + k - cut:10 + k - cut]) < tol, (json.dumps(cfg), dtype, "b", k)
        cache.close(a)
        cache.close(b)
        cache.check()
