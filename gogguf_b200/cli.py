"""Command line, in the manner of the reference's `gogguf` (cmd/gogguf/main.go:21-51):

    gogguf_b200 run (-m DIR | --random CONFIG.json [--weights-seed 0]) -p "1 2 3" [-p "4 5"] [-n 128] [--temp 0]
                    [--top-k 0] [--top-p 1] [--min-p 0] [--repeat-penalty 1] [--repeat-last-n 64] [--seed 0]
                    [--dtype bfloat16] [-i]
    gogguf_b200 info -m DIR
    gogguf_b200 inspect DIR
    gogguf_b200 random -c CONFIG.json -o DIR [--seed 0] [--dtype bfloat16] [--std S] [--norm-std S]
    gogguf_b200 compare A.f32 B.f32 [--tol 1e-4] [--vocab V]
    gogguf_b200 dumplayers -m DIR -p "1 2 3" -o PREFIX [--dtype float32] [--all]
    gogguf_b200 comparelayers -a A.bin -b B.bin [--tol 1e-4]   |   -m DIR -p "1 2 3" (float32 against bfloat16)
    gogguf_b200 layerlogits -m DIR -p "1 2 3" [--top 5] [--dtype float32]

`run` keeps the reference's option names and defaults (cmd/gogguf/run.go:17-34).  A prompt is a list
of token ids (the tokenizer is outside this library); several -p make a batch.  Dropped: -hf
(network), --chat/--thinking (text templates), -ngl (the whole model is always on the GPU).  -i is the
reference's REPL on token ids: one conversation, a line of new ids per turn.
`info` prints what the reference's info prints (cmd/gogguf/info.go:27-44), `inspect` every
configuration key and tensor (cmd/gogguf/inspect.go:13-41).  `random` is the random-weights mode.
`dumplayers`, `comparelayers` and `layerlogits` are the reference's layer tools (cmd/tools/dumplayers.go,
comparelayers.go, layerlogits.go) on the engine's layer taps: hidden states after the embedding and after
every block, two such dumps compared layer by layer, and the head applied after every layer.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys
import time
from typing import List, Optional


def _ids(text: str) -> List[int]:
    parts = [p for p in re.split(r"[\s,]+", text.strip()) if p]
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise SystemExit(f"prompt must be token ids separated by spaces or commas, got {text!r}")


def cmd_run(a) -> int:
    import gogguf_b200 as gg
    if not a.m and not a.random:
        raise SystemExit("usage: gogguf_b200 run (-m DIR | --random CONFIG.json [--weights-seed S]) -p \"token ids\" [-n 128]")
    if a.m and a.random:
        raise SystemExit("give a model folder (-m) or a configuration for random weights (--random), not both")
    prompts: List[List[int]] = [_ids(p) for p in (a.p or [])]
    if a.prompt_file:
        with open(a.prompt_file) as f:
            prompts += [_ids(line) for line in f if line.strip()]
    if not prompts and not a.i:
        raise SystemExit("give a prompt with -p (token ids) or --prompt-file, or use -i")
    t_load = time.perf_counter()
    options = gg.LoadOptions(dtype=a.dtype, max_tokens=a.cache_tokens, max_batch=a.max_batch, timing=a.timing)
    engine = gg.load(a.m, options) if a.m else gg.load_random(a.random, a.weights_seed, options)
    ctx = engine.new_context()
    t_load = (time.perf_counter() - t_load) * 1e3
    params = gg.GenerateParams(
        max_tokens=a.n,
        sampler=gg.SamplerConfig(temp=a.temp, top_k=a.top_k, top_p=a.top_p, min_p=a.min_p, seed=a.seed),
        repeat_penalty=a.repeat_penalty, repeat_last_n=a.repeat_last_n,
        stop_token_ids=None if a.stop_ids is None else _ids(a.stop_ids))
    if a.i:
        return run_interactive(ctx, params, prompts, sys.stdin, sys.stdout)
    for r in ctx.generate(prompts, params):
        print(" ".join(str(t) for t in r.tokens))
        print(f"# prompt {r.prompt_tokens} tokens, generated {len(r.tokens)}, finish: {r.finish_reason}",
              file=sys.stderr)
    if a.timing:
        # the reference's bench lines (cmd/tools/bench.go:296-299) for this run
        print(f"Load: {t_load:.1f} ms", file=sys.stderr)
        for line in ctx.last_timing().lines():
            print(line, file=sys.stderr)
    return 0


def run_interactive(ctx, params, first: List[List[int]], inp, out) -> int:
    """The reference's REPL (runInteractive, cmd/gogguf/run.go:115-175) on token ids: every line is the new
    ids of a turn; they are added to the conversation so far (ids given and ids made), only they are run, and
    the turn's ids are printed.  An empty line or the end of the input ends it; `/clear` starts the
    conversation again (run.go:135-140).  A prompt given with -p is the first turn."""
    print("interactive: a line of token ids per turn; an empty line ends, /clear starts again", file=sys.stderr)
    conv = ctx.new_conversation()
    turns = list(first[:1])
    try:
        while True:
            if turns:
                new = turns.pop(0)
            else:
                print("> ", end="", file=sys.stderr, flush=True)
                line = inp.readline()
                if not line or not line.strip():
                    break
                if line.strip() == "/clear":
                    conv.reset()
                    print("conversation cleared", file=sys.stderr)
                    continue
                new = _ids(line)
            r = conv.generate(conv.tokens + new, params)
            print(" ".join(str(t) for t in r.tokens), file=out, flush=True)
            print(f"# conversation {conv.token_count()} tokens, generated {len(r.tokens)}, finish: {r.finish_reason}",
                  file=sys.stderr)
    finally:
        conv.close()
    return 0


def _folder_summary(folder: str):
    from .config.registry import load_config
    from .weights.safetensors_io import open_model_files
    cfg = load_config(folder)
    files = open_model_files(folder)
    tensors = []
    for f in files:
        for n in f.names():
            dt, shape = f.info(n)
            numel = 1
            for s in shape:
                numel *= s
            tensors.append((n, dt, shape, numel * (8 if "64" in str(dt) else 4 if "32" in str(dt) else
                                                   2 if "16" in str(dt) else 1)))
        f.close()
    return cfg, tensors


def cmd_info(a) -> int:
    if not a.m:
        raise SystemExit("usage: gogguf_b200 info -m DIR")
    cfg, tensors = _folder_summary(a.m)
    d = cfg.to_dict()
    print(f"Folder: {a.m}")
    print(f"Architecture: {d.get('architectures', ['?'])[0]}")
    print(f"Tensors: {len(tensors)}")
    print(f"Weights size: {sum(t[3] for t in tensors) / 1e6:.1f} MB")
    if hasattr(cfg, "parameter_count"):
        print(f"Parameters: {cfg.parameter_count():,}")
    if hasattr(cfg, "kv_bytes_per_token"):
        print(f"Cache per token (bfloat16): {cfg.kv_bytes_per_token(2)} bytes")
    print(f"Context: {cfg.to_spec().max_positions} tokens")
    return 0


def cmd_inspect(a) -> int:
    cfg, tensors = _folder_summary(a.folder)
    for k, v in cfg.to_dict().items():
        print(f"{k} = {json.dumps(v)}")
    for n, dt, shape, nbytes in sorted(tensors):
        print(f"{n}\t{str(dt).replace('torch.', '')}\t{list(shape)}\t{nbytes}")
    return 0


def cmd_random(a) -> int:
    from .config.registry import load_config
    from .engine.model import write_random_model
    cfg = load_config(a.c)
    write_random_model(cfg, a.seed, a.o, dtype=a.dtype, std=a.std, norm_std=a.norm_std)
    print(f"wrote {os.path.join(a.o, 'config.json')} and model.safetensors (seed {a.seed}, {a.dtype})")
    return 0


def cmd_compare(a) -> int:
    """Difference of two logits dumps (files of little-endian float32, as trace_run writes them): the
    figures of the reference's DiffLogits (pkg/debug/diff.go:17-48): max abs, mean abs, rmse, count over
    a tolerance, and whether the arg-max rows agree."""
    import numpy as np
    x = np.fromfile(a.a, dtype="<f4")
    y = np.fromfile(a.b, dtype="<f4")
    if x.size != y.size:
        print(f"sizes differ: {x.size} and {y.size} values", file=sys.stderr)
        return 1
    d = np.abs(x.astype(np.float64) - y.astype(np.float64))
    print(f"values: {x.size}")
    print(f"max abs diff: {d.max() if d.size else 0.0:.6g}")
    print(f"mean abs diff: {d.mean() if d.size else 0.0:.6g}")
    print(f"rmse: {float(np.sqrt((d * d).mean())) if d.size else 0.0:.6g}")
    print(f"over tolerance {a.tol:g}: {int((d > a.tol).sum())}")
    if a.vocab and x.size % a.vocab == 0:
        same = (x.reshape(-1, a.vocab).argmax(1) == y.reshape(-1, a.vocab).argmax(1))
        print(f"rows with the same arg-max: {int(same.sum())} of {same.size}")
    return 0 if (d <= a.tol).all() else 2


def _collect_layers(folder: str, dtype: str, prompt: List[int], all_rows: bool, logits: bool = False):
    """One prompt through an eager step with layer taps (collectLayersDump, cmd/tools/dumplayers.go:55-108):
    the last token's rows as the reference dumps them, or every token's with `all_rows`."""
    import gogguf_b200 as gg
    from .engine.layers_dump import LayerCollector
    from .engine.step import StepEntry
    engine = gg.load(folder, gg.LoadOptions(dtype=dtype, max_tokens=len(prompt) + 64, graphs=False))
    ctx = engine.new_context()
    taps = LayerCollector(logits=logits)
    slot = ctx.cache.open()
    try:
        want = list(range(len(prompt))) if all_rows else [len(prompt) - 1]
        ctx.stepper.step([StepEntry(slot, prompt, want=want)], taps)
    finally:
        ctx.cache.close(slot)
    return taps


def cmd_dumplayers(a) -> int:
    """runDumpLayers (cmd/tools/dumplayers.go:16-53): PREFIX.bin and PREFIX.json."""
    from .engine.layers_dump import save_layers
    from .sampling.sampler import greedy as greedy_host
    prompt = _ids(a.p)
    taps = _collect_layers(a.m, a.dtype, prompt, a.all)
    dump = taps.dump()
    save_layers(a.o, dump, model=os.path.basename(os.path.normpath(a.m)), tokens=prompt, dtype=a.dtype,
                greedy=greedy_host(taps.final_logits[-1].tolist()))
    print(f"wrote {a.o}.bin / {a.o}.json (embd={dump.hidden} layers={dump.layers.shape[0]} rows={dump.rows})")
    return 0


def cmd_comparelayers(a) -> int:
    """runCompareLayers (cmd/tools/comparelayers.go:11-84): two dumps, or one model in float32 against
    bfloat16 (where the reference compares its CPU path with its GPU path).  Prints the reference's lines
    and, beyond them, rmse per layer and the first layer over the tolerance."""
    from .engine.layers_dump import diff_layers, read_layers
    if a.m:
        prompt = _ids(a.p)
        x = _collect_layers(a.m, "float32", prompt, a.all).dump()
        y = _collect_layers(a.m, "bfloat16", prompt, a.all).dump()
    elif a.a and a.b:
        x, y = read_layers(a.a), read_layers(a.b)
    else:
        raise SystemExit("usage: gogguf_b200 comparelayers -a A.bin -b B.bin | -m DIR -p \"token ids\"")
    d = diff_layers(x, y, a.tol)
    e = d.embed
    print(f"embed: max_abs={e.max_abs:.6g}@{e.max_abs_idx} mean={e.mean_abs:.6g} rmse={e.rmse:.6g} over={e.over_tol}")
    for i, st in enumerate(d.layers):
        if st.over_tol > 0 or a.verbose:
            print(f"layer[{i}]: max_abs={st.max_abs:.6g}@{st.max_abs_idx} rmse={st.rmse:.6g} over={st.over_tol}")
    w = d.worst_layer
    total = sum(st.over_tol for st in d.layers)
    print(f"layers: n={len(d.layers)} worst_max_abs={d.layers[w].max_abs if w >= 0 else 0.0:.6g}@layer{w} "
          f"total_over_tol={total} (tol={a.tol:g})")
    if e.over_tol or total:
        first = d.first_over
        print(f"FAIL: hidden states differ by more than the tolerance, first at "
              f"{'the embedding' if first == -1 else f'layer {first}'}")
        return 2
    print("OK: hidden states of every layer are within the tolerance")
    return 0


def cmd_layerlogits(a) -> int:
    """runLayerLogits (cmd/tools/layerlogits.go:31-114): the arg-max and the `--top` largest logits of the
    last token with the final norm and head applied after every layer, as JSON."""
    from .sampling.sampler import greedy as greedy_host
    prompt = _ids(a.p)
    taps = _collect_layers(a.m, a.dtype, prompt, False, logits=True)
    case = dict(name="layer_greedy", input=prompt,
                layer_greedy=[greedy_host(lg[-1].tolist()) for lg in taps.layer_logits])
    if a.top > 0:
        tops = []
        for lg in taps.layer_logits:
            v, i = lg[-1].topk(min(a.top, lg.shape[-1]))
            tops.append([dict(id=int(t), logit=float(x)) for x, t in zip(v.tolist(), i.tolist())])
        case["layer_top_logits"] = tops
    json.dump(dict(model=os.path.basename(os.path.normpath(a.m)), cases=[case]), sys.stdout, indent=2)
    print()
    return 0


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="gogguf_b200", description="Qwen3 inference on B200")
    sub = ap.add_subparsers(dest="cmd")
    r = sub.add_parser("run", help="generate tokens")
    r.add_argument("-m", help="model folder (config.json + model.safetensors)")
    r.add_argument("--random", metavar="CONFIG.json", help="instead of -m: random weights made on the device from this configuration")
    r.add_argument("--weights-seed", type=int, default=0, help="seed of the random weights (--random)")
    r.add_argument("-p", action="append", help="prompt as token ids; repeat for a batch")
    r.add_argument("--prompt-file", help="one prompt of token ids per line")
    r.add_argument("-i", action="store_true", help="interactive: a conversation, one line of token ids per turn")
    r.add_argument("-n", type=int, default=128, help="most new tokens")
    r.add_argument("--temp", type=float, default=0.0, help="temperature (0 = greedy)")
    r.add_argument("--top-k", type=int, default=0, help="top-k sampling (0 = off)")
    r.add_argument("--top-p", type=float, default=1.0, help="nucleus sampling (1 = off)")
    r.add_argument("--min-p", type=float, default=0.0, help="min-p sampling (0 = off)")
    r.add_argument("--repeat-penalty", type=float, default=1.0, help="penalty for repeated tokens (1 = off)")
    r.add_argument("--repeat-last-n", type=int, default=64, help="history window of the repeat penalty")
    r.add_argument("--seed", type=int, default=0, help="seed of the sampling draws")
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.add_argument("--stop-ids", default=None, help="stop token ids (default: the model's eos_token_id)")
    r.add_argument("--cache-tokens", type=int, default=0, help="cache capacity in tokens (0 = context length)")
    r.add_argument("--max-batch", type=int, default=64)
    r.add_argument("--timing", action="store_true",
                   help="print load, prefill, time to first token, decode (model steps / sampling) timed on the device")
    r.set_defaults(fn=cmd_run)
    i = sub.add_parser("info", help="short summary of a model folder")
    i.add_argument("-m")
    i.set_defaults(fn=cmd_info)
    s = sub.add_parser("inspect", help="every configuration key and tensor")
    s.add_argument("folder")
    s.set_defaults(fn=cmd_inspect)
    g = sub.add_parser("random", help="write a model folder with random weights")
    g.add_argument("-c", required=True, help="config.json (or a folder holding one)")
    g.add_argument("-o", required=True, help="output folder")
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--std", type=float, default=None, help="std of matrices (default: initializer_range)")
    g.add_argument("--norm-std", type=float, default=0.02, help="std of norm weights around 1")
    g.set_defaults(fn=cmd_random)
    c = sub.add_parser("compare", help="difference of two logits dumps (.f32 files)")
    c.add_argument("a")
    c.add_argument("b")
    c.add_argument("--tol", type=float, default=1e-4)
    c.add_argument("--vocab", type=int, default=0, help="row length, to compare arg-max per row")
    c.set_defaults(fn=cmd_compare)
    d = sub.add_parser("dumplayers", help="hidden states after the embedding and after every layer")
    d.add_argument("-m", required=True)
    d.add_argument("-p", required=True, help="prompt as token ids")
    d.add_argument("-o", required=True, help="output prefix: PREFIX.bin and PREFIX.json")
    d.add_argument("--dtype", default="float32", choices=["bfloat16", "float32"])
    d.add_argument("--all", action="store_true", help="every token's rows, not the last token's only")
    d.set_defaults(fn=cmd_dumplayers)
    cl = sub.add_parser("comparelayers", help="two layer dumps, or float32 against bfloat16 of one model")
    cl.add_argument("-a", help="dump A (.bin)")
    cl.add_argument("-b", help="dump B (.bin)")
    cl.add_argument("-m", help="model folder: float32 against bfloat16")
    cl.add_argument("-p", default="1", help="prompt as token ids, for -m")
    cl.add_argument("--all", action="store_true", help="every token's rows, for -m")
    cl.add_argument("--tol", type=float, default=1e-4)
    cl.add_argument("-v", "--verbose", action="store_true", help="print every layer, not only those over the tolerance")
    cl.set_defaults(fn=cmd_comparelayers)
    ll = sub.add_parser("layerlogits", help="arg-max and top logits of the last token after every layer")
    ll.add_argument("-m", required=True)
    ll.add_argument("-p", required=True, help="prompt as token ids")
    ll.add_argument("--top", type=int, default=5, help="largest logits per layer (0: arg-max only)")
    ll.add_argument("--dtype", default="float32", choices=["bfloat16", "float32"])
    ll.set_defaults(fn=cmd_layerlogits)
    return ap


def main(argv: Optional[List[str]] = None) -> int:
    ap = build_parser()
    a = ap.parse_args(argv)
    if not getattr(a, "fn", None):
        ap.print_help()
        return 1
    try:
        return a.fn(a)
    except (ValueError, RuntimeError, OSError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
