"""The host sampling chain against the plain restatement of the reference's sampler (no GPU)."""
import numpy as np
import pytest

import plain_qwen3 as plain
from gogguf_b200.sampling import SamplerConfig, apply_repeat_penalty, greedy, sample_host, uniform01


def test_greedy_takes_the_first_maximum():
    assert greedy([0.5, 2.0, 2.0, -1.0]) == 1 == plain.greedy([0.5, 2.0, 2.0, -1.0])
    assert greedy([]) == -1
    assert SamplerConfig().greedy and SamplerConfig(temp=0, top_p=1.0).greedy
    assert not SamplerConfig(temp=0, top_k=2).greedy        # chain.go:19


def test_uniform_matches_its_restatement_and_is_a_pure_function():
    for args in [(0, 0, 0), (7, 3, 11), (2 ** 63 + 5, 2 ** 40, 9)]:
        u = uniform01(*args)
        assert u == plain.uniform01(*args) and 0.0 <= u < 1.0
    us = [uniform01(1, s, k) for s in range(20) for k in range(20)]
    assert len(set(us)) == len(us) and 0.35 < np.mean(us) < 0.65


@pytest.mark.parametrize("cfg", [
    SamplerConfig(temp=0.8, seed=1), SamplerConfig(temp=1.0, seed=2), SamplerConfig(temp=0.0, top_k=3),
    SamplerConfig(temp=1.3, top_k=5), SamplerConfig(temp=0.7, top_p=0.6), SamplerConfig(temp=0.9, min_p=0.2),
    SamplerConfig(temp=1.1, top_k=8, top_p=0.8, min_p=0.05),
])
def test_chain_equals_the_plain_sampler(cfg):
    rng = np.random.default_rng(0)
    for trial in range(40):
        logits = (rng.standard_normal(50) * 3).astype(np.float32)
        u = uniform01(cfg.seed, trial, 0)
        got = sample_host(logits, cfg, u)
        want = plain.sample(logits.tolist(), cfg.temp, cfg.top_k, cfg.top_p, cfg.min_p, u)
        assert got == want


def test_reference_sampler_facts():
    # top-k = 2 never leaves the two largest (pkg/sampler/chain_test.go)
    logits = np.array([1.0, 5.0, 4.0, -2.0], dtype=np.float32)
    for k in range(50):
        assert sample_host(logits, SamplerConfig(temp=1.0, top_k=2), uniform01(0, 0, k)) in (1, 2)
    # top-p keeps {.4,.4} of {.4,.4,.1,.1} at 0.79
    lp = np.log(np.array([0.4, 0.4, 0.1, 0.1], dtype=np.float32))
    for k in range(50):
        assert sample_host(lp, SamplerConfig(temp=1.0, top_p=0.79), uniform01(0, 0, k)) in (0, 1)
    # u = 0 returns the first allowed id; u close to 1 the last
    assert sample_host(lp, SamplerConfig(temp=1.0), 0.0) == 0
    assert sample_host(lp, SamplerConfig(temp=1.0), 0.999999) == 3


def test_repeat_penalty():
    x = np.array([2.0, -2.0, 1.0, 3.0], dtype=np.float32)
    y = x.copy()
    apply_repeat_penalty(y, [0, 1, 1, 9, -1], 2.0, 64)
    assert y.tolist() == [1.0, -4.0, 1.0, 3.0]        # each distinct id once; unknown ids ignored
    z = x.copy()
    apply_repeat_penalty(z, [0, 3], 2.0, 1)           # only the last id counts
    assert z.tolist() == [2.0, -2.0, 1.0, 1.5]
    w = x.copy()
    apply_repeat_penalty(w, [0, 1], 1.0, 64)
    assert w.tolist() == x.tolist()
    p = x.tolist()
    plain.repeat_penalty(p, [0, 1, 1, 9, -1], 2.0, 64)
    assert p == y.tolist()


def test_a_top_k_chain_too_wide_for_the_kernel_goes_to_the_host_chain():
    """The top-k kernel keeps k candidates per 8,192-logit slice in 160 KB of shared memory: top-k 1,024 fits a
    vocabulary of up to 163,840 ids.  Beyond that the sampler must not ask the kernel (which refuses) but run
    the host chain, and say so before the loop decides to stay a step ahead."""
    from gogguf_b200.sampling import Sampler, SamplerConfig
    cfg = SamplerConfig(temp=0.7, top_k=1024, seed=1)
    assert Sampler(cfg, vocab_size=151936).device_chain and Sampler(cfg, vocab_size=151936).device_only
    wide = Sampler(cfg, vocab_size=163841)
    assert not wide.device_chain and not wide.on_device and not wide.device_only
    assert Sampler(SamplerConfig(temp=0.7, top_k=40), vocab_size=400000).device_chain      # 49 slices x 40 fit
    assert Sampler(SamplerConfig(temp=0.7), vocab_size=400000).on_device                   # plain temperature
    # on the CPU the host chain answers whatever the sizes
    import torch
    logits = torch.randn(2, 300)
    assert Sampler(cfg, vocab_size=300).sample(logits, [0, 1], [0, 0]) == Sampler(cfg).sample(logits, [0, 1], [0, 0])
