"""The measurement script's contract that needs no GPU: what it answers for more than one GPU and for the
reference arm, and the bytes and flops it divides by."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=120)


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_more_than_one_gpu_is_one_line_and_exit_code_2():
    r = run_bench("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert r.returncode == 2
    assert len(r.stdout.strip().splitlines()) == 1 and "one GPU" in r.stdout


def test_reference_arm_says_why_it_is_unavailable():
    r = run_bench("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and line["unavailable"]


def test_bytes_and_flops_of_the_8b_shape():
    b = load_bench()
    c = dict(b.QWEN3_8B)
    layers = c["num_hidden_layers"]
    # every weight once: 36 layers of q/k/v, O, gate, up, down (bf16) + norms, the head, the final norm, B rows
    per_layer = ((32 + 16) * 128 * 4096 + 4096 * 4096 + 3 * 4096 * 12288) * 2 + (2 * 4096 + 2 * 128) * 4
    assert b.layer_weight_bytes(c) == per_layer
    kv_per_token = 2 * layers * 8 * 128 * 2
    assert kv_per_token == 147456
    for batch in (1, 8, 64):
        want = layers * per_layer + 151936 * 4096 * 2 + 4096 * 4 + batch * 4096 * 2 + batch * 2048 * kv_per_token
        assert b.decode_bytes(c, layers, batch, 2048) == want
    assert abs(b.decode_bytes(c, layers, 8, 2048) / 1e9 - (15.14 + 8 * 0.302)) < 0.02
    # a 2,048-token prompt: 2 flops per weight and token in the layers, the head for one row, causal attention
    fl = b.prefill_flops(c, layers, 2048)
    mats = (6144 * 4096 + 4096 * 4096 + 3 * 4096 * 12288) * layers
    attn = layers * 4 * 32 * 128 * (2048 * 2049 / 2)
    assert fl == 2 * 2048 * mats + 2 * 151936 * 4096 + attn
    assert 29.0e12 < fl < 30.5e12


def test_peaks_come_from_the_measured_file_when_it_is_there(tmp_path, monkeypatch):
    b = load_bench()
    assert b.peaks()["source"] in ("fallback", "measured")
    monkeypatch.setattr(b, "ROOT", str(tmp_path))
    assert b.peaks() == dict(b.FALLBACK_PEAKS, source="fallback")
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 7000.0, "bf16_tflops": 1600, "clocks": {"sm": 1900}}))
    p = b.peaks()
    assert p["source"] == "measured" and p["hbm_gbs"] == 7000.0 and p["bf16_tflops"] == 1600.0
    assert p["bf16_tflops_sustained"] == b.FALLBACK_PEAKS["bf16_tflops_sustained"]
    (tmp_path / "MEASURED_PEAKS.json").write_text("not json")
    assert b.peaks()["source"] == "fallback"


def test_kernel_microbenchmarks_name_their_cases_and_need_a_gpu():
    """`python -m gogguf_b200.csrc.microbench` is the script that the per-kernel figures under profiles/ were made
    with: its cases are listed by --help, and without a CUDA device it ends with an error, never with numbers."""
    import torch
    mb = [sys.executable, "-m", "gogguf_b200.csrc.microbench"]
    r = subprocess.run(mb + ["--help"], capture_output=True, text=True, timeout=120, cwd=ROOT)
    assert r.returncode == 0
    for case in ("gemm", "gemm_layer", "attn", "prefill_attn", "sample"):
        assert case in r.stdout
    r = subprocess.run(mb + ["nonsense"], capture_output=True, text=True, timeout=120, cwd=ROOT)
    assert r.returncode != 0 and "invalid choice" in r.stderr
    if not torch.cuda.is_available():
        r = subprocess.run(mb + ["sample", "--m", "1"], capture_output=True, text=True, timeout=300, cwd=ROOT)
        assert r.returncode != 0 and "us" not in r.stdout
