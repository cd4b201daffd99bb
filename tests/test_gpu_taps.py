"""Layer taps of the step function and the layer tools of the command line: the hidden states after the
embedding and after every block, against the plain implementation's."""
import io
import json
import os
from contextlib import redirect_stdout

import pytest
import torch

import plain_qwen3 as plain
from helpers import TOL_BF16, TOL_F32, make_folder, random_tokens, read_folder, rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("A", "bfloat16"), ("L", "bfloat16")])
def test_every_tap_equals_the_plain_implementation(tmp_path_factory, name, dtype):
    from gogguf_b200.engine import Model, StepEntry, Stepper
    from gogguf_b200.engine.graphs import GraphStepper
    from gogguf_b200.engine.layers_dump import LayerCollector
    store = "float32" if dtype == "float32" else "bfloat16"
    folder = make_folder(tmp_path_factory.getbasetemp(), name, store, scale=1.0 if dtype == "float32" else 4.0)
    cfg, w = read_folder(folder)
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    L = cfg["num_hidden_layers"]
    a, b = random_tokens(cfg["vocab_size"], 75, 1), random_tokens(cfg["vocab_size"], 20, 2)
    want_taps = {}
    for k, t in (("a", a), ("b", b)):
        want_taps[k] = []
        want_taps[k + "logits"] = plain.forward(cfg, w, t, wide=True, taps=want_taps[k])
    model = Model.load(folder, dtype=dtype)
    cache = model.new_cache(512)
    st = GraphStepper(model, cache)
    sa, sb = cache.open(), cache.open()
    taps = LayerCollector(logits=True)
    wa, wb = [0, 30, 73], [18]
    logits = st.step([StepEntry(sa, a[:-1], want=wa), StepEntry(sb, b[:-1], want=wb)], taps).clone()
    assert len(taps.layers) == L and len(taps.layer_logits) == L and taps.embed.shape == (4, cfg["hidden_size"])
    pick = lambda i: torch.cat([want_taps["a"][i][wa], want_taps["b"][i][wb]])      # noqa: E731
    assert rel_err(taps.embed, pick(0)) < (1e-7 if dtype == "float32" else 1e-2)
    for i in range(L):
        assert rel_err(taps.layers[i], pick(i + 1)) < tol, i
    # the head after the last layer is the step's own result; after an earlier layer it is the plain head on that tap
    assert torch.equal(taps.layer_logits[-1], logits) and torch.equal(taps.final_logits, logits)
    c = plain.plain_config(cfg)
    head = w["model.embed_tokens.weight"] if c["tied"] else w["lm_head.weight"]
    early = plain.rms_norm(pick(1), w["model.norm.weight"], c["eps"], wide=True) @ head.double().T
    assert rel_err(taps.layer_logits[0], early) < tol
    # a decode step with taps runs eagerly (no graph is captured or replayed for it) and gives the same rows
    taps = LayerCollector()
    logits = st.step([StepEntry(sa, a[-1:], want=[0]), StepEntry(sb, b[-1:], want=[0])], taps)
    assert st.replays == 0
    for i in range(L):
        want = torch.stack([want_taps["a"][i + 1][-1], want_taps["b"][i + 1][-1]])
        assert rel_err(taps.layers[i], want) < tol, i
    assert rel_err(logits, torch.stack([want_taps["alogits"][-1], want_taps["blogits"][-1]])) < tol
    # without taps the step is unchanged: nothing is handed out, nothing extra runs
    cache.close(sa); cache.close(sb)
    cache.check()


def test_layer_tools_of_the_command_line(tmp_path_factory, tmp_path):
    from gogguf_b200 import cli
    from gogguf_b200.engine.layers_dump import read_layers
    folder = make_folder(tmp_path_factory.getbasetemp(), "B", "float32")
    cfg, w = read_folder(folder)
    toks = random_tokens(cfg["vocab_size"], 23, 5)
    ids = " ".join(map(str, toks))
    want_taps = []
    want = plain.forward(cfg, w, toks, wide=True, taps=want_taps)
    pa, pb = str(tmp_path / "f32"), str(tmp_path / "bf16")
    assert cli.main(["dumplayers", "-m", folder, "-p", ids, "-o", pa]) == 0
    assert cli.main(["dumplayers", "-m", folder, "-p", ids, "-o", pb, "--dtype", "bfloat16"]) == 0
    d = read_layers(pa + ".bin")
    assert d.rows == 1 and d.layers.shape[0] == cfg["num_hidden_layers"]
    for i in range(cfg["num_hidden_layers"]):
        assert rel_err(torch.from_numpy(d.layers[i]), want_taps[i + 1][-1:]) < TOL_F32
    meta = json.load(open(pa + ".json"))
    assert meta["greedy"] == int(want[-1].argmax()) and meta["tokens"] == toks and len(meta["layer_rms"]) == d.layers.shape[0]
    assert abs(meta["layer_rms"][-1] - float(want_taps[-1][-1].pow(2).mean().sqrt())) < 1e-4
    # float32 against bfloat16 of the same weights: within a tolerance above their largest difference, not
    # within one below it; the difference itself is small against the hidden states
    from gogguf_b200.engine.layers_dump import diff_layers
    dd = diff_layers(d, read_layers(pb + ".bin"), 0.0)
    worst = max(st.max_abs for st in dd.layers)
    assert 0 < worst < 0.05 * float(abs(d.layers).max())
    out = io.StringIO()
    with redirect_stdout(out):
        assert cli.main(["comparelayers", "-a", pa + ".bin", "-b", pb + ".bin", "--tol", str(2 * worst)]) == 0
        assert cli.main(["comparelayers", "-a", pa + ".bin", "-b", pb + ".bin", "--tol", "1e-6"]) == 2
        assert cli.main(["comparelayers", "-m", folder, "-p", ids, "--tol", str(2 * worst), "-v"]) == 0
    text = out.getvalue()
    assert "OK: hidden states" in text and "FAIL" in text and "first at layer 0" in text and "layer[2]:" in text
    out = io.StringIO()
    with redirect_stdout(out):
        assert cli.main(["layerlogits", "-m", folder, "-p", ids, "--top", "3"]) == 0
    case = json.loads(out.getvalue())["cases"][0]
    assert len(case["layer_greedy"]) == cfg["num_hidden_layers"] and case["layer_greedy"][-1] == int(want[-1].argmax())
    top = case["layer_top_logits"][-1]
    assert [t["id"] for t in top] == want[-1].topk(3).indices.tolist()
    assert abs(top[0]["logit"] - float(want[-1].max())) < 1e-4
