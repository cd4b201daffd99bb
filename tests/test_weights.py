"""Weights: container round trip, one error for all disagreements, storage policy, random mode (no GPU)."""
import json
import os
import struct

import pytest
import torch

from gogguf_b200.config import config_from_dict
from gogguf_b200.engine.model import expected_tensors, write_random_model
from gogguf_b200.weights import (SafetensorsError, SafetensorsFile, WeightsError, load_tensors, write_safetensors)
from helpers import TINY_A, TINY_B, make_folder, read_folder


def test_container_round_trip_against_the_safetensors_package(tmp_path):
    t = {"a.weight": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int64),
         "c": torch.randn(2, 2, 2), "empty": torch.zeros(0, 4)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t)
    from safetensors import safe_open
    with safe_open(p, framework="pt") as f:
        for k in t:
            assert torch.equal(f.get_tensor(k), t[k])
    mine = SafetensorsFile(p)
    for k in t:
        assert torch.equal(mine.tensor(k), t[k])
    mine.close()
    from safetensors.torch import save_file
    q = str(tmp_path / "y.safetensors")
    save_file({k: v.contiguous() for k, v in t.items()}, q)
    theirs = SafetensorsFile(q)
    for k in t:
        assert torch.equal(theirs.tensor(k), t[k])
    theirs.close()


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = make_folder(tmp_path, "B", "float32")
    cfg, w = read_folder(folder)
    del w["model.layers.1.self_attn.q_norm.weight"]
    del w["model.norm.weight"]
    w["model.layers.0.mlp.extra.weight"] = torch.zeros(2)
    w["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(16, 96)
    write_safetensors(os.path.join(folder, "model.safetensors"), w)
    exp = expected_tensors(config_from_dict(cfg).to_spec())
    with pytest.raises(WeightsError) as e:
        load_tensors(folder, exp)
    err = e.value
    assert err.missing == ["model.layers.1.self_attn.q_norm.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.mlp.extra.weight"]
    assert err.wrong_shape == [("model.layers.2.self_attn.k_proj.weight", (16, 96), (32, 96))]
    msg = str(err)
    for word in ("missing", "unexpected", "wrong shape", "model.norm.weight", "extra.weight", "[16, 96]", "[32, 96]"):
        assert word in msg


def test_tied_head_may_be_present_or_absent(tmp_path):
    folder = make_folder(tmp_path, "A", "float32")
    cfg, w = read_folder(folder)
    assert "lm_head.weight" not in w
    exp = expected_tensors(config_from_dict(cfg).to_spec())
    assert "lm_head.weight" not in load_tensors(folder, exp)
    w["lm_head.weight"] = w["model.embed_tokens.weight"].clone()
    write_safetensors(os.path.join(folder, "model.safetensors"), w)
    assert "lm_head.weight" in load_tensors(folder, exp)


def test_storage_policy(tmp_path):
    cfg = config_from_dict(TINY_A)
    folder = str(tmp_path / "m")
    write_random_model(cfg, 1, folder, dtype="bfloat16")
    _, w = read_folder(folder)
    w["model.norm.weight"] = w["model.norm.weight"].float()                     # stored in 32-bit: stays so
    w["model.layers.0.mlp.up_proj.weight"] = w["model.layers.0.mlp.up_proj.weight"].to(torch.float16)
    write_safetensors(os.path.join(folder, "model.safetensors"), w)
    got = load_tensors(folder, expected_tensors(cfg.to_spec()))
    assert got["model.norm.weight"].dtype == torch.float32
    assert got["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert got["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16
    # float16 has no kernels of its own: rounded to bfloat16 for the bfloat16 path, but widened exactly
    # for the 32-bit path, whose results must be those of the stored values
    got32 = load_tensors(folder, expected_tensors(cfg.to_spec()), compute_dtype=torch.float32)
    up = got32["model.layers.0.mlp.up_proj.weight"]
    assert up.dtype == torch.float32
    assert torch.equal(up, w["model.layers.0.mlp.up_proj.weight"].float())
    assert got32["model.embed_tokens.weight"].dtype == torch.bfloat16


def test_truncated_and_broken_files(tmp_path):
    folder = make_folder(tmp_path, "A", "float32")
    p = os.path.join(folder, "model.safetensors")
    data = open(p, "rb").read()
    with open(p, "wb") as f:
        f.write(data[:len(data) - 100])
    with pytest.raises(SafetensorsError) as e:
        SafetensorsFile(p)
    assert "truncated" in str(e.value)
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", 10 ** 12) + b"{}")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)
    os.remove(p)
    with pytest.raises(WeightsError):
        load_tensors(folder, {})


def test_random_mode_is_seeded_and_shaped(tmp_path):
    cfg = config_from_dict(TINY_B)
    write_random_model(cfg, 7, str(tmp_path / "a"), dtype="float32", std=0.03, norm_std=0.05)
    write_random_model(cfg, 7, str(tmp_path / "b"), dtype="float32", std=0.03, norm_std=0.05)
    write_random_model(cfg, 8, str(tmp_path / "c"), dtype="bfloat16", std=0.03, norm_std=0.05)
    ca, wa = read_folder(str(tmp_path / "a"))
    _, wb = read_folder(str(tmp_path / "b"))
    _, wc = read_folder(str(tmp_path / "c"))
    assert config_from_dict(ca) == cfg
    assert set(wa) == set(n for n, d in expected_tensors(cfg.to_spec()).items() if not d.optional)
    for k in wa:
        assert torch.equal(wa[k], wb[k])
    assert not torch.equal(wa["lm_head.weight"], wc["lm_head.weight"].float())
    assert wc["lm_head.weight"].dtype == torch.bfloat16
    q = wa["model.layers.0.self_attn.q_proj.weight"]
    assert abs(q.std().item() - 0.03) < 0.003 and abs(q.mean().item()) < 0.003
    n = wa["model.layers.1.input_layernorm.weight"]
    assert abs(n.mean().item() - 1.0) < 0.03


def test_gguf_style_names_and_sharded_folders(tmp_path):
    """A folder may name its tensors as the reference's GGUF files do, and may be split into shards."""
    cfg = config_from_dict(TINY_B)
    folder = str(tmp_path / "m")
    write_random_model(cfg, 3, folder, dtype="float32")
    _, w = read_folder(folder)
    back = {v: k for k, v in cfg.tensor_aliases().items()}
    renamed = {back[k]: v for k, v in w.items()}
    assert "blk.2.attn_q_norm.weight" in renamed and "token_embd.weight" in renamed and "output.weight" in renamed
    os.remove(os.path.join(folder, "model.safetensors"))
    names = sorted(renamed)
    half = len(names) // 2
    write_safetensors(os.path.join(folder, "model-00001-of-00002.safetensors"), {n: renamed[n] for n in names[:half]})
    write_safetensors(os.path.join(folder, "model-00002-of-00002.safetensors"), {n: renamed[n] for n in names[half:]})
    with open(os.path.join(folder, "model.safetensors.index.json"), "w") as f:
        json.dump({"weight_map": {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                                  for i, n in enumerate(names)}}, f)
    got = load_tensors(folder, expected_tensors(cfg.to_spec()), aliases=cfg.tensor_aliases())
    assert set(got) == set(w)
    for k in w:
        assert torch.equal(got[k], w[k])


def test_compare_command(tmp_path, capsys):
    import numpy as np
    from gogguf_b200.cli import main
    a = np.arange(12, dtype="<f4").reshape(3, 4)
    b = a.copy()
    b[1, 2] += 0.5
    a.tofile(tmp_path / "a.f32")
    b.tofile(tmp_path / "b.f32")
    assert main(["compare", str(tmp_path / "a.f32"), str(tmp_path / "a.f32")]) == 0
    assert main(["compare", str(tmp_path / "a.f32"), str(tmp_path / "b.f32"), "--vocab", "4"]) == 2
    out = capsys.readouterr().out
    assert "max abs diff: 0.5" in out and "over tolerance 0.0001: 1" in out and "same arg-max: 3 of 3" in out
