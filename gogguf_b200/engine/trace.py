"""Trace replay: feed given token ids through a model step by step and write the logits.

Nothing is sampled and nothing here computes: every step goes through the same `Stepper.step`,
cache and kernels that generation uses.  The nearest things in the reference are
Engine.ForwardTokenIDs (pkg/runtime/engine.go:79-81) and `tools dumplogits`
(cmd/tools/dumplogits.go), both for one sequence and one call.

Input: one JSON object per line,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
A request's first appearance opens a slot for it; `end` lists requests that are finished after the
step, whose slot and pages are given back.  For a step in which something is wanted the logits at
the wanted places are written to ``<out>/<step>.f32`` as little-endian float32 [wanted, vocab], in
the order of the entries and of `want`.  After every step the line ``done <step>`` is printed and
flushed.

By default the steps go through the stepper that generation uses, which replays plain decode steps
as captured CUDA graphs (`--no-graphs`: every step eagerly).  With `--layers` the hidden states of the
wanted places after the embedding and after every block are written to ``<out>/<step>.layers.bin``
(`engine.layers_dump`), which makes such a step run eagerly.
"""
from __future__ import annotations

import json
import os
import sys
from typing import Dict, IO, Iterable, Optional

import torch

from .model import Model
from .step import StepEntry, Stepper


class TraceError(ValueError):
    pass


class TraceRunner:
    def __init__(self, model: Model, max_tokens: int, out_dir: str, graphs: bool = True, layers: bool = False):
        self.model = model
        self.cache = model.new_cache(max_tokens)
        if graphs and model.rt.device.type == "cuda":
            from .graphs import GraphStepper
            self.stepper: Stepper = GraphStepper(model, self.cache)
        else:
            self.stepper = Stepper(model, self.cache)
        self.layers = layers
        self.out_dir = out_dir
        os.makedirs(out_dir, exist_ok=True)
        self.slot_of: Dict[str, int] = {}

    def run_step(self, obj: dict) -> None:
        if "step" not in obj or "entries" not in obj:
            raise TraceError("a step needs 'step' and 'entries'")
        step_id = obj["step"]
        entries = []
        opened = []
        try:
            for e in obj["entries"]:
                rid = str(e["id"])
                if rid not in self.slot_of:
                    self.slot_of[rid] = self.cache.open()
                    opened.append(rid)
                entries.append(StepEntry(slot=self.slot_of[rid], tokens=[int(t) for t in e["tokens"]],
                                         want=[int(w) for w in e.get("want", [])]))
            taps = None
            if self.layers and any(e.want for e in entries):
                from .layers_dump import LayerCollector
                taps = LayerCollector()
            logits = self.stepper.step(entries, taps) if entries else None
        except Exception:
            for rid in opened:       # a refused step leaves no half-opened request behind
                self.cache.close(self.slot_of.pop(rid))
            raise
        if logits is not None:
            arr = logits.detach().to("cpu", torch.float32).contiguous().numpy()
            path = os.path.join(self.out_dir, f"{step_id}.f32")
            with open(path + ".tmp", "wb") as f:
                f.write(arr.astype("<f4", copy=False).tobytes())
            os.replace(path + ".tmp", path)
            if taps is not None:
                from .layers_dump import write_layers
                write_layers(os.path.join(self.out_dir, f"{step_id}.layers.bin"), taps.dump())
        else:
            torch.cuda.synchronize(self.model.rt.device) if self.model.rt.device.type == "cuda" else None
        for rid in obj.get("end", []) or []:
            rid = str(rid)
            if rid not in self.slot_of:
                raise TraceError(f"step {step_id}: request {rid!r} ends but was never started")
            self.cache.close(self.slot_of.pop(rid))

    def run(self, lines: Iterable[str], out: IO[str] = sys.stdout) -> None:
        for line in lines:
            line = line.strip()
            if not line:
                continue
            try:
                obj = json.loads(line)
            except json.JSONDecodeError as e:
                raise TraceError(f"not a JSON line: {e}") from None
            self.run_step(obj)
            out.write(f"done {obj['step']}\n")
            out.flush()


def main(argv: Optional[list] = None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description="replay a token trace and write logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--graphs", dest="graphs", action="store_true", default=True,
                    help="replay plain decode steps as captured CUDA graphs, as generation does (default)")
    ap.add_argument("--no-graphs", dest="graphs", action="store_false", help="run every step eagerly")
    ap.add_argument("--layers", action="store_true",
                    help="also write <step>.layers.bin: hidden states of the wanted places after every block")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("trace_run: no CUDA device is available; this library has no CPU path", file=sys.stderr)
        return 1
    model = Model.load(args.model, dtype=args.dtype, device=args.device)
    runner = TraceRunner(model, args.max_tokens, args.out, graphs=args.graphs, layers=args.layers)
    # readline, not iteration: a step must be answered before the next line arrives
    runner.run(iter(sys.stdin.readline, ""))
    return 0
