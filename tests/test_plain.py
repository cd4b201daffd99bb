"""The plain implementation checked against facts the reference's own unit tests state (no GPU)."""
import math

import torch

import plain_qwen3 as plain
from helpers import make_folder, read_folder, random_tokens, rel_err


def test_rmsnorm_of_1_2_3_has_unit_rms():
    # pkg/ops/ops_test.go:24-41
    out = plain.rms_norm(torch.tensor([[1.0, 2.0, 3.0]]), torch.ones(3), 1e-6)
    assert abs(float(out.pow(2).mean().sqrt()) - 1.0) < 1e-4
    wide = plain.rms_norm(torch.tensor([[1.0, 2.0, 3.0]]), torch.ones(3), 1e-6, wide=True)
    assert rel_err(out, wide) < 1e-6


def test_attention_with_one_key_returns_v():
    # pkg/ops/rope_test.go:53-69, two query heads on one kv head
    q = torch.randn(1, 2, 4)
    k = torch.randn(1, 1, 4)
    v = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]])
    out = plain.attention(q, k, v)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 1], v[0, 0])


def test_rope_is_identity_at_position_zero_and_pairs_are_neox():
    x = torch.randn(1, 2, 8)
    cos, sin = plain.rope_tables([0], 8, 10000.0)
    assert torch.equal(plain.rope_neox(x, cos, sin), x)
    # one pair (i, i + d/2) rotates by pos * theta^(-2i/d): element 1 pairs with element 5
    cos, sin = plain.rope_tables([3], 8, 10000.0)
    e = torch.zeros(1, 1, 8); e[0, 0, 1] = 1.0
    out = plain.rope_neox(e, cos, sin)
    ang = 3 * 10000.0 ** (-2 * 1 / 8)
    assert abs(float(out[0, 0, 1]) - math.cos(ang)) < 1e-6 and abs(float(out[0, 0, 5]) - math.sin(ang)) < 1e-6
    assert float(out[0, 0, 2].abs() + out[0, 0, 0].abs()) == 0.0     # not the adjacent-pair form


def test_softmax_rows_sum_to_one_and_window_masks():
    s = torch.randn(5, 7)
    assert torch.allclose(plain.softmax_rows(s).sum(-1), torch.ones(5), atol=1e-6)
    # window 2: token 3 sees keys 2 and 3 only; make key 0 huge and check it is ignored
    q = torch.zeros(4, 1, 2); q[3, 0, 0] = 1.0
    k = torch.zeros(4, 1, 2); k[0, 0, 0] = 100.0
    v = torch.arange(8, dtype=torch.float32).reshape(4, 1, 2)
    full = plain.attention(q, k, v)
    win = plain.attention(q, k, v, window=2)
    assert torch.allclose(full[3, 0], v[0, 0], atol=1e-4)
    assert torch.allclose(win[3, 0], (v[2, 0] + v[3, 0]) / 2, atol=1e-6)


def test_silu_and_matvec_facts():
    assert abs(float(plain.silu(torch.tensor(1.0))) - 1.0 / (1.0 + math.exp(-1.0))) < 1e-7
    w = torch.tensor([[1.0, 2.0], [3.0, 4.0]])
    assert (torch.tensor([[1.0, 0.0]]) @ w.T).tolist() == [[1.0, 3.0]]      # pkg/ops/ops_test.go:11-22


def test_float32_form_tracks_the_wide_form_and_prefixes_agree(tmp_path):
    folder = make_folder(tmp_path, "B", "float32")
    cfg, w = read_folder(folder)
    toks = random_tokens(cfg["vocab_size"], 24, 0)
    a = plain.forward(cfg, w, toks)
    b = plain.forward(cfg, w, toks, wide=True)
    assert rel_err(a, b) < 5e-6
    assert rel_err(plain.forward(cfg, w, toks[:9], wide=True), b[:9]) < 1e-12     # causal: a prefix stands alone
    taps = []
    plain.forward(cfg, w, toks, taps=taps)
    assert len(taps) == cfg["num_hidden_layers"] + 1


def test_greedy_generation_stops_on_a_stop_token(tmp_path):
    folder = make_folder(tmp_path, "A", "float32")
    cfg, w = read_folder(folder)
    toks = plain.generate_greedy(cfg, w, [1, 2, 3], 6)
    assert len(toks) == 6
    cut = plain.generate_greedy(cfg, w, [1, 2, 3], 6, stop=[toks[2]])
    assert cut == toks[:toks.index(toks[2])]
