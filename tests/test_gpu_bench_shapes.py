"""Whole-model parity at the layer sizes that the measurements run: two layers of the 8B shape and one of
the 14B shape (full widths, heads and vocabulary; only the depth is cut), in bfloat16.  These sizes select
kernel variants that no tiny configuration reaches: the decode products' deeper ring and their cluster of
eight K splits, the head with more than a thousand CTAs, the CTA-pair product with hundreds of tiles, the
q/k/v epilogue with 32 or 40 query heads.  Ragged prompts in one step, then 40 decode steps at batch 8 through
`Context.generate` (captured graphs, ids fed from the device, one step ahead of the host) and again, fed the
same tokens, through the stepper; logits at sampled rows against the plain implementation on the CPU."""
import pytest
import torch

import plain_qwen3 as plain
from helpers import random_tokens

pytestmark = pytest.mark.gpu

SHAPES = {
    "8b": dict(num_hidden_layers=2, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               intermediate_size=12288),
    "14b": dict(num_hidden_layers=1, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, head_dim=128,
                intermediate_size=17408),
}
# Measured on B200: at worst 1.1e-2 (8B sizes) and 9e-3 (14B sizes) of a row's largest logit over all checked
# rows.  A dropped K split, a head or a page left out moves a row by several times this bound (tried once by
# editing the kernel so that the owner of a token leaves out the partial sums of the cluster's last rank: the
# test fails at the first checked row).
TOL_ROW = 1.5e-2


def row_err(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.double().cpu(), want.double().cpu()
    return float(((got - want).abs().max(dim=-1).values / want.abs().max(dim=-1).values).max())


def plain_rows(cfg, w, tokens, rows):
    """plain.forward(..., rows=rows) with the head applied in slices, so that a vocabulary of 151,936 by
    4,096 or 5,120 never exists in float32 on the host."""
    c = plain.plain_config(cfg)
    x = plain.embed(w["model.embed_tokens.weight"], tokens).float()
    pos = list(range(len(tokens)))
    for layer in range(c["layers"]):
        x = plain.block(x, w, layer, c, pos, rows=rows if layer == c["layers"] - 1 else None)
    h = plain.rms_norm(x, w["model.norm.weight"], c["eps"])
    head = w["lm_head.weight"]
    return torch.cat([h @ head[a:a + 16384].float().T for a in range(0, head.shape[0], 16384)], dim=1)


@pytest.mark.parametrize("shape", ["8b", "14b"])
def test_whole_model_at_the_measured_layer_sizes(shape, monkeypatch):
    import gogguf_b200 as gg
    from gogguf_b200.api import Engine
    from gogguf_b200.config import config_from_dict
    from gogguf_b200.engine import Model, StepEntry
    from gogguf_b200.engine.model import expected_tensors
    from gogguf_b200.sampling.sampler import Sampler
    from gogguf_b200.weights import random_tensors
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, rope_theta=1000000.0,
               rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096, **SHAPES[shape])
    config = config_from_dict(cfg)
    spec = config.to_spec()
    tensors = random_tensors(expected_tensors(spec), seed=7, std=0.02, norm_std=0.05, dtype=torch.bfloat16,
                             device="cuda:0")
    w = {k: v.cpu() for k, v in tensors.items()}              # bfloat16 on the host; widened slice by slice
    model = Model(spec, tensors, dtype="bfloat16", config=config, consume=True)
    del tensors
    V = cfg["vocab_size"]
    n_new = 40 if shape == "8b" else 12
    lens = [320, 131, 40, 17, 64, 5, 33, 1]                   # one prompt of more than 300 tokens, shorter ones beside it
    prompts = [random_tokens(V, n, seed=100 + n) for n in lens]
    ctx = Engine(model, gg.LoadOptions(dtype="bfloat16", max_tokens=8 * 512)).new_context()
    seen = []
    real = Sampler.sample_async

    def spy(self, logits, streams, steps):
        seen.append((list(streams), list(steps), logits[:len(streams)].clone()))
        return real(self, logits, streams, steps)

    monkeypatch.setattr(Sampler, "sample_async", spy)
    out = ctx.generate(prompts, gg.GenerateParams(max_tokens=n_new, stop_token_ids=[]))
    monkeypatch.setattr(Sampler, "sample_async", real)
    assert len(seen) == n_new and ctx.stepper.replays >= n_new - 1 and all(len(r.tokens) == n_new for r in out)
    full = [p + r.tokens for p, r in zip(prompts, out)]
    # rows to check: the prompt's last token (the prefill step), the first decode steps, every fifth, the last
    ks = sorted(set([0, 1, 2] + list(range(5, n_new, 5)) + [n_new - 1]))
    rows = [[len(p) - 1 + k for k in ks] for p in prompts]
    oracle = [plain_rows(cfg, w, t[:-1], r) for t, r in zip(full, rows)]
    worst = 0.0
    for streams, steps, logits in seen:
        for row, (i, k) in enumerate(zip(streams, steps)):
            if k in ks:
                e = row_err(logits[row:row + 1], oracle[i][ks.index(k):ks.index(k) + 1])
                worst = max(worst, e)
                assert e < TOL_ROW, ("one step ahead", i, k, e)
    # the same tokens through the stepper: ragged prompts in one step with several wanted rows, then decode
    # steps one by one (captured graphs), the batch shrinking at the end as sequences are let go
    st, cache = ctx.stepper, ctx.cache
    slots = [cache.open() for _ in prompts]
    got = st.step([StepEntry(s, p, want=[0, len(p) - 1]) for s, p in zip(slots, prompts)]).clone()
    first = [plain_rows(cfg, w, p, [0]) for p in prompts[:2]]
    for i in range(len(prompts)):
        assert row_err(got[2 * i + 1:2 * i + 2], oracle[i][0:1]) < TOL_ROW, ("prefill", i)
    for i in range(2):
        assert row_err(got[2 * i:2 * i + 1], first[i]) < TOL_ROW, ("first row", i)
    live = list(range(len(prompts)))
    for k in range(1, n_new):
        if k == n_new - 3:
            for i in live[5:]:
                cache.close(slots[i])
            live = live[:5]
        got = st.step([StepEntry(slots[i], [full[i][len(prompts[i]) + k - 1]], want=[0]) for i in live])
        if k in ks:
            for j, i in enumerate(live):
                e = row_err(got[j:j + 1], oracle[i][ks.index(k):ks.index(k) + 1])
                worst = max(worst, e)
                assert e < TOL_ROW, ("stepper", i, k, e)
    for i in live:
        cache.close(slots[i])
    cache.check()
    print(f"{shape}: worst row error {worst:.2e}")
