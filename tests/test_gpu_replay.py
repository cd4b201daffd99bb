"""Trace replay through bin/trace_run, the program a user runs: the same requests whole, with the last
32 tokens one by one, and in batches of unequal lengths whose shorter requests end earlier, one batch
after another so that slots and pages are used again - in 32-bit and in bfloat16, against the plain
implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import TOL_BF16, TOL_F32, make_folder, random_tokens, read_folder, rel_err

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class Trace:
    def __init__(self, folder, dtype, out, max_tokens, extra=()):
        self.out = str(out)
        self.p = subprocess.Popen(
            [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
             "--out", self.out, "--max-tokens", str(max_tokens), *extra],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
        self.n = 0

    def step(self, entries, end=()):
        s = self.n
        self.n += 1
        self.p.stdin.write(json.dumps({"step": s, "entries": entries, "end": list(end)}) + "\n")
        self.p.stdin.flush()
        line = self.p.stdout.readline().strip()
        assert line == f"done {s}", f"trace_run answered {line!r} (exit {self.p.poll()})"
        path = os.path.join(self.out, f"{s}.f32")
        wanted = sum(len(e.get("want", [])) for e in entries)
        if not wanted:
            assert not os.path.exists(path)
            return None
        return np.fromfile(path, dtype="<f4").reshape(wanted, -1)

    def close(self):
        self.p.stdin.close()
        assert self.p.wait(timeout=60) == 0


# By default replay steps through generation's own stepper, which replays plain decode steps as captured CUDA
# graphs (padded to a batch bucket, integer inputs in a fixed device buffer); --no-graphs runs every step eagerly.
@pytest.mark.parametrize("name,dtype,extra", [
    ("A", "float32", ()), ("B", "float32", ()), ("W", "float32", ()),
    ("A", "bfloat16", ()), ("B", "bfloat16", ()), ("W", "bfloat16", ()),
    ("M", "bfloat16", ()), ("M", "float32", ()), ("L", "bfloat16", ()),
    ("B", "float32", ("--no-graphs",)), ("W", "bfloat16", ("--no-graphs",)), ("L", "bfloat16", ("--no-graphs",))])
def test_replay_shapes(tmp_path_factory, tmp_path, name, dtype, extra):
    store = "float32" if dtype == "float32" else "bfloat16"
    folder = make_folder(tmp_path_factory.getbasetemp(), name, store, scale=1.0 if dtype == "float32" else 4.0)
    cfg, w = read_folder(folder)
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    V = cfg["vocab_size"]
    lens = [150, 33, 97, 64, 5, 129]
    reqs = {f"r{i}": random_tokens(V, n, seed=10 + i) for i, n in enumerate(lens)}
    oracle = {k: plain.forward(cfg, w, t, wide=True) for k, t in reqs.items()}
    # the cache holds two batches' worth at most: slots and pages must be reused
    tr = Trace(folder, dtype, tmp_path / "out", max_tokens=3 * 64 + 2 * 64 + 64, extra=extra)
    try:
        # (1) each request alone and whole, every position wanted
        for k, t in reqs.items():
            got = tr.step([{"id": k + "w", "tokens": t, "want": list(range(len(t)))}], end=[k + "w"])
            assert rel_err(torch.from_numpy(got), oracle[k]) < tol, (k, "whole")
        # (2) the last 32 tokens one by one after a whole prefill of the rest
        for k in ("r0", "r3", "r2"):
            t = reqs[k]
            cut = len(t) - 32
            got = tr.step([{"id": k + "d", "tokens": t[:cut], "want": [cut - 1]}])
            assert rel_err(torch.from_numpy(got), oracle[k][cut - 1:cut]) < tol
            for i in range(cut, len(t)):
                last = i == len(t) - 1
                got = tr.step([{"id": k + "d", "tokens": [t[i]], "want": [0]}], end=[k + "d"] if last else [])
                assert rel_err(torch.from_numpy(got), oracle[k][i:i + 1]) < tol, (k, "decode", i)
        # (3) batches of unequal lengths; shorter requests end earlier; one batch after another
        for batch in (["r1", "r4", "r3"], ["r5", "r2"], ["r0", "r4"]):
            pre = {k: len(reqs[k]) - 6 if len(reqs[k]) > 8 else 2 for k in batch}
            entries = [{"id": k + "b", "tokens": reqs[k][:pre[k]], "want": [0, pre[k] - 1]} for k in batch]
            got = tr.step(entries)
            for j, k in enumerate(batch):
                want = oracle[k][[0, pre[k] - 1]]
                assert rel_err(torch.from_numpy(got[2 * j:2 * j + 2]), want) < tol, (k, "batch prefill")
            pos = dict(pre)
            live = list(batch)
            while live:
                entries = [{"id": k + "b", "tokens": [reqs[k][pos[k]]], "want": [0]} for k in live]
                ending = [k for k in live if pos[k] + 1 == len(reqs[k])]
                got = tr.step(entries, end=[k + "b" for k in ending])
                for j, k in enumerate(live):
                    assert rel_err(torch.from_numpy(got[j:j + 1]), oracle[k][pos[k]:pos[k] + 1]) < tol, (k, pos[k])
                    pos[k] += 1
                live = [k for k in live if k not in ending]
        # a step that wants nothing writes no file
        assert tr.step([{"id": "q", "tokens": reqs["r4"], "want": []}], end=["q"]) is None
    finally:
        tr.close()


def test_replay_refuses_what_does_not_fit(tmp_path_factory, tmp_path):
    folder = make_folder(tmp_path_factory.getbasetemp(), "A", "float32")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype",
                        "float32", "--out", str(tmp_path / "o"), "--max-tokens", "64"],
                       input=json.dumps({"step": 0, "entries": [{"id": "a", "tokens": [1] * 65, "want": [0]}],
                                         "end": []}) + "\n", capture_output=True, text=True)
    assert p.returncode != 0 and "pages" in p.stderr


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("M", "bfloat16")])
def test_replay_writes_the_layers_of_the_wanted_places(tmp_path_factory, tmp_path, name, dtype):
    """--layers: hidden states after the embedding and after every block, beside the logits, for prompts and
    for decode steps (which then run eagerly), against the plain implementation's taps."""
    sys.path.insert(0, ROOT)
    from gogguf_b200.engine.layers_dump import read_layers
    store = "float32" if dtype == "float32" else "bfloat16"
    folder = make_folder(tmp_path_factory.getbasetemp(), name, store, scale=1.0 if dtype == "float32" else 4.0)
    cfg, w = read_folder(folder)
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    toks = {k: random_tokens(cfg["vocab_size"], n, seed=60 + n) for k, n in (("a", 70), ("b", 12))}
    taps = {}
    for k, t in toks.items():
        taps[k] = []
        plain.forward(cfg, w, t, wide=True, taps=taps[k])
    tr = Trace(folder, dtype, tmp_path / "out", max_tokens=256, extra=("--layers",))
    try:
        tr.step([{"id": "a", "tokens": toks["a"][:-1], "want": [0, 40]}, {"id": "b", "tokens": toks["b"][:-1], "want": [10]}])
        d = read_layers(os.path.join(tr.out, "0.layers.bin"))
        assert d.layers.shape == (cfg["num_hidden_layers"], 3, cfg["hidden_size"]) and d.embed.shape == d.layers.shape[1:]
        for layer in range(-1, cfg["num_hidden_layers"]):
            got = torch.from_numpy(d.embed if layer < 0 else d.layers[layer])
            want = torch.stack([taps["a"][layer + 1][0], taps["a"][layer + 1][40], taps["b"][layer + 1][10]])
            assert rel_err(got, want) < tol, layer
        tr.step([{"id": "a", "tokens": toks["a"][-1:], "want": [0]}, {"id": "b", "tokens": toks["b"][-1:], "want": [0]}],
                end=["a", "b"])
        d = read_layers(os.path.join(tr.out, "1.layers.bin"))
        for layer in range(cfg["num_hidden_layers"]):
            want = torch.stack([taps["a"][layer + 1][-1], taps["b"][layer + 1][-1]])
            assert rel_err(torch.from_numpy(d.layers[layer]), want) < tol, layer
    finally:
        tr.close()
