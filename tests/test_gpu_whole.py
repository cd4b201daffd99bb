"""Each request alone and whole: the engine's logits at every position against the plain implementation."""
import pytest
import torch

import plain_qwen3 as plain
from helpers import TINY, TOL_BF16, TOL_F32, make_folder, random_tokens, read_folder, rel_err

pytestmark = pytest.mark.gpu


def engine_whole(folder, dtype, tokens, fast=True):
    from gogguf_b200.engine import Model, StepEntry, Stepper
    model = Model.load(folder, dtype=dtype, fast=fast)
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


@pytest.mark.parametrize("name", ["A", "B", "W", "M"])
def test_whole_bf16(tmp_path_factory, name):
    folder = make_folder(tmp_path_factory.getbasetemp(), name, "bfloat16", scale=4.0)
    cfg, w = read_folder(folder)
    tokens = random_tokens(cfg["vocab_size"], 200, seed=3)
    want = plain.forward(cfg, w, tokens, wide=True)
    got = engine_whole(folder, "bfloat16", tokens)
    assert rel_err(got, want) < TOL_BF16
    # the plain kernels on the same bfloat16 weights (the twins of the tensor-core kernels) agree too
    twin = engine_whole(folder, "bfloat16", tokens, fast=False)
    assert rel_err(twin, want) < TOL_BF16
