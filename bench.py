#!/usr/bin/env python3
"""Measurement: Qwen3-8B-shaped random-weight model, bfloat16, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl ours|reference]
                    [--shape 8b|14b|32b] [--workload] [--prefill-lengths 256,1024] [--decode-contexts 16384,32768]

A "step" is one decode step of a batch: every sequence goes on by one token, sampled greedily on the
device.  The timed region is exactly K steps after W warm-up steps, timed with CUDA events on the
launching stream.  One JSON line is printed:

  value        decoded tokens per second (batch * K / time), device timed, CUDA-graph replay per step
  e2e          the same through the Python entry point (Context.generate): host token ids in, host
               token ids out, every step copies its inputs from pinned host memory and reads the
               sampled ids back
  prefill      one 2,048-token prompt: tokens per second, and flops / time / measured bf16 peak
  roofline     bytes a decode step must read (every weight once + the cache of the live sequences)
               / time, against the measured HBM copy bandwidth
  points       decode tokens per second at batch 1 and 64
  config       every size, flat
  workload     (--workload) the shape's own request mix through Context.generate: prefill and decode rates
  prefill_sweep_ms  (--prefill-lengths) one prefill step per listed prompt length
  decode_by_context (--decode-contexts) decode steps of sequences that already hold that many tokens

Peaks come from MEASURED_PEAKS.json beside this file when the driver wrote it, else from the
fallback figures of an earlier measurement on this pool.  The weights (16 GB) are far larger than
the 126 MB L2, so consecutive steps cannot be served from cache.  The reference cannot be installed
here (it is a Go program; there is no Go toolchain and no network): `--impl reference` says so.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the headline configuration: Qwen3-8B shape
QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
    intermediate_size=12288, vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6,
    tie_word_embeddings=False, max_position_embeddings=4096, initializer_range=0.02,
)
# the layer sizes of the 14B and 32B shapes (same vocabulary and rotary base)
SHAPES = {
    "8b": {},
    "14b": dict(num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, intermediate_size=17408),
    "32b": dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, intermediate_size=25600,
                max_position_embeddings=8192),      # its request mix has prompts of 4,096 tokens
}
PROMPT_LEN = 2048
CONTEXT = 4096
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            with open(p) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if k in d and d[k]:
                    out[k] = float(d[k])
            out["source"] = "measured"
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def layer_weight_bytes(c, itemsize=2):
    qw = c["num_attention_heads"] * c["head_dim"]
    kvw = c["num_key_value_heads"] * c["head_dim"]
    h, i = c["hidden_size"], c["intermediate_size"]
    mats = (qw + 2 * kvw) * h + h * qw + 3 * h * i
    return mats * itemsize + (2 * h + 2 * c["head_dim"]) * 4      # norm weights are float32


def decode_bytes(c, layers, batch, ctx_len):
    """Bytes one decode step has to read: every weight it uses once, and the cache of the live requests."""
    h, v = c["hidden_size"], c["vocab_size"]
    w = layers * layer_weight_bytes(c) + v * h * 2 + h * 4 + batch * h * 2     # head, final norm, B embedding rows
    kv = batch * ctx_len * 2 * layers * c["num_key_value_heads"] * c["head_dim"] * 2
    return w + kv


def prefill_flops(c, layers, t):
    qw = c["num_attention_heads"] * c["head_dim"]
    kvw = c["num_key_value_heads"] * c["head_dim"]
    h, i, v = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    gemm = 2 * t * ((qw + 2 * kvw) * h + h * qw + 3 * h * i) * layers + 2 * 1 * v * h
    attn = layers * 2 * 2 * c["num_attention_heads"] * c["head_dim"] * (t * (t + 1) / 2)
    return gemm + attn


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="layer sizes: the 8B shape is the contract's")
    ap.add_argument("--layers", type=int, default=0,
                    help="fewer layers than the configuration has (same layer sizes); named in config")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end run (for short profiling runs)")
    ap.add_argument("--workload", action="store_true",
                    help="also run the shape's own request mix through the entry point (14b: 16 prompts of 128 to 2,048 "
                    "tokens and 256 new tokens each; 32b: 8 prompts of 4,096 tokens and 128 new tokens; 8b: 8 prompts "
                    "of 2,048 tokens and 64 new tokens); added to the line as workload")
    ap.add_argument("--decode-contexts", default="", help="comma separated context lengths: time decode steps of batch "
                    "--batch (and of one sequence) whose sequences already hold that many tokens (added to the line as "
                    "decode_by_context)")
    ap.add_argument("--prefill-lengths", default="", help="comma separated prompt lengths: time one prefill step of each "
                    "(printed on stderr, added to the line as prefill_sweep)")
    a = ap.parse_args()

    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "magomedcoder/gogguf is a Go program; no Go toolchain and no network here, pip cannot install it"}))
        return 0
    if a.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {a.gpus} is not built (this library runs on a single B200)")
        return 2
    if a.warmup < 3:
        a.warmup = 3

    import torch
    from gogguf_b200.config import config_from_dict
    from gogguf_b200.csrc import build
    from gogguf_b200.engine import Model, StepEntry
    from gogguf_b200.engine.graphs import GraphStepper
    from gogguf_b200.csrc import tcgen05_gemm
    from gogguf_b200.sampling import Sampler, SamplerConfig

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    base = dict(QWEN3_8B, **SHAPES[a.shape])
    if a.layers <= 0:
        a.layers = base["num_hidden_layers"]
    cdict = dict(base, num_hidden_layers=a.layers)
    long_ctx = [int(x) for x in a.decode_contexts.split(",") if x.strip()]
    longest = max(long_ctx + [int(x) for x in a.prefill_lengths.split(",") if x.strip()] + [0])
    if longest:         # the rotary tables are computed per step, so the context length is only a bound
        cdict["max_position_embeddings"] = max(cdict["max_position_embeddings"], longest + 128)
    cfg = config_from_dict(cdict)
    pk = peaks()
    t0 = time.time()
    model = Model.random(cfg, seed=2, dtype="bfloat16", device=dev, std=0.02, norm_std=0.0)
    torch.cuda.synchronize()
    print(f"[bench] model built in {time.time() - t0:.1f} s ({cfg.parameter_count() / 1e9:.2f} B parameters)", file=sys.stderr)

    g = torch.Generator().manual_seed(0)
    V = cfg.vocab_size

    def rand_tokens(n):
        return torch.randint(0, V, (n,), generator=g).tolist()

    def decode_run(batch, steps, warmup, sampler_cfg=None, prompt_len=PROMPT_LEN):
        """Prefill `batch` prompts of `prompt_len` tokens, then time `steps` greedy decode steps on the device."""
        PROMPT_LEN = prompt_len
        room = PROMPT_LEN + warmup + steps + 8
        cache = model.new_cache(batch * (-(-room // 64) * 64))
        st = GraphStepper(model, cache)
        slots = [cache.open() for _ in range(batch)]
        chunk = max(1, 8192 // PROMPT_LEN)       # prompts per prefill step, bounds the workspace
        logits_last = []
        for i in range(0, batch, chunk):
            ents = [StepEntry(s, rand_tokens(PROMPT_LEN), want=[PROMPT_LEN - 1]) for s in slots[i:i + chunk]]
            logits_last.append(st.step(ents).clone())
        # greedy sampling on the device; each step takes its input ids from the device buffer the previous
        # step's sampling kernel wrote, and the host reads every step's ids (one step behind the device)
        sampler = Sampler(sampler_cfg if sampler_cfg is not None else SamplerConfig())
        rows = list(range(batch))
        pending = sampler.sample_async(torch.cat(logits_last), rows, [0] * batch)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        clock_sampler = None
        n_launch0 = 0
        produced = []
        for it in range(warmup + steps):
            if it == warmup:
                produced.append(pending.tokens())
                torch.cuda.synchronize()
                clock_sampler = ClockSampler()
                clock_sampler.start()
                time.sleep(0.25)
                n_launch0 = build.launch_count()
                replay0 = st.replays
                ev0.record()
            logits = st.decode_from_device(slots, pending.device_tokens, rows)
            nxt_pending = sampler.sample_async(logits, rows, [it + 1] * batch)
            produced.append(pending.tokens())      # device-to-host read of the step's result, every step
            pending = nxt_pending
        ev1.record()
        torch.cuda.synchronize()
        tcgen05_gemm.check_status(dev)       # a bounded wait that ran out inside a kernel would invalidate the run
        clocks = clock_sampler.stop()
        ms = ev0.elapsed_time(ev1)
        direct = build.launch_count() - n_launch0
        launches = direct + (st.replays - replay0) * getattr(st, "last_graph_kernels", 0)
        ctx_len = PROMPT_LEN + warmup + steps // 2
        for s in slots:
            cache.close(s)
        del st, cache
        torch.cuda.empty_cache()
        return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "clocks": clocks,
                "launches": launches, "bytes": decode_bytes(cdict, a.layers, batch, ctx_len)}

    def e2e_run(batch, steps, warmup):
        """The same through the generation loop of the entry point: host ids in, host ids out."""
        import gogguf_b200 as gg
        engine = gg.Engine(model, gg.LoadOptions(dtype="bfloat16", max_batch=batch))
        # The prompts of the whole batch are prefilled in one step right before decoding starts, and the
        # first decode steps after that burst run at a lower clock (under the power cap) for some tens of
        # milliseconds; they are warm-up here, so that the timed steps are steady-state decoding as in
        # `decode_run`, which pauses between its prefill and its timed region.
        warmup = max(warmup, 32)
        room = PROMPT_LEN + warmup + steps + 8
        ctx = engine.new_context(max_tokens=batch * (-(-room // 64) * 64), max_batch=batch)
        prompts = [rand_tokens(PROMPT_LEN) for _ in range(batch)]
        stamps = []

        def on_token(i, t):
            if i == 0:
                stamps.append(time.perf_counter())     # the id has just arrived on the host
            return True

        ctx.generate(prompts, gg.GenerateParams(max_tokens=warmup + steps + 1, stop_token_ids=[], on_token=on_token))
        # stamps[k] is taken when token k of request 0 has reached the host; steps between stamps are decode steps
        dt = stamps[warmup + steps] - stamps[warmup]
        # bytes per decode step: the packed integer inputs (tokens, positions, slots, lengths, page tables)
        # copied from pinned host memory, and the sampled ids read back
        return {"tok_s": batch * steps / dt, "h2d": getattr(ctx.stepper, "last_h2d_bytes", None), "d2h": batch * 4,
                "warmup": warmup}

    def workload_run():
        """The request mix named for this shape, through Context.generate: host ids in, host ids out.

        Times the batch's prefill (until every request's first id is on the host) and the decoding after it."""
        import gogguf_b200 as gg
        if a.shape == "14b":
            lens = torch.randint(128, 2049, (16,), generator=torch.Generator().manual_seed(3)).tolist()
            new = 256
        elif a.shape == "32b":
            lens, new = [4096] * 8, 128
        else:
            lens, new = [PROMPT_LEN] * 8, 64
        batch = len(lens)
        engine = gg.Engine(model, gg.LoadOptions(dtype="bfloat16", max_batch=batch))
        ctx = engine.new_context(max_tokens=sum(-(-(n + new + 8) // 64) * 64 for n in lens), max_batch=batch)
        out = None
        for rep in range(2):                       # the first pass captures the graphs
            prompts = [rand_tokens(n) for n in lens]
            first = {}

            def on_token(i, t):
                if i not in first:
                    first[i] = time.perf_counter()
                return True

            torch.cuda.synchronize()
            t_start = time.perf_counter()
            res = ctx.generate(prompts, gg.GenerateParams(max_tokens=new, stop_token_ids=[], on_token=on_token))
            t_end = time.perf_counter()
            t_first = max(first.values())
            made = sum(len(r.tokens) for r in res)
            out = {"requests": batch, "prompt_tokens": sum(lens), "new_tokens": made,
                   "prefill_ms": (t_first - t_start) * 1e3, "prefill_tok_s": sum(lens) / (t_first - t_start),
                   "decode_tok_s": (made - batch) / (t_end - t_first), "decode_ms_per_step": (t_end - t_first) * 1e3 / (new - 1),
                   "total_s": t_end - t_start}
        return out

    def prefill_run(prompt_len=PROMPT_LEN):
        cache = model.new_cache(prompt_len + 64)
        st = GraphStepper(model, cache)
        times = []
        torch.cuda.synchronize()
        time.sleep(0.5)            # as before the timed decode region: start from an idle GPU, not from the previous run's heat
        for it in range(4):
            s = cache.open()
            toks = rand_tokens(prompt_len)
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            ev0.record()
            st.step([StepEntry(s, toks, want=[prompt_len - 1])])
            ev1.record()
            torch.cuda.synchronize()
            times.append(ev0.elapsed_time(ev1))
            cache.close(s)
        ms = sorted(times[1:])[len(times[1:]) // 2]
        fl = prefill_flops(cdict, a.layers, prompt_len)
        return {"value": prompt_len / (ms / 1e3), "tokens": prompt_len, "ms": ms,
                "frac": fl / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), "tflops": fl / (ms / 1e3) / 1e12}

    main_run = decode_run(a.batch, a.steps, a.warmup)
    print(f"[bench] decode batch {a.batch}: {main_run['tok_s']:.1f} tok/s, {main_run['ms_per_step']:.3f} ms/step", file=sys.stderr)
    if a.no_e2e:
        e2e = {"tok_s": None, "h2d": None, "d2h": None, "warmup": None}
    else:
        e2e = e2e_run(a.batch, a.steps, a.warmup)
        print(f"[bench] e2e batch {a.batch}: {e2e['tok_s']:.1f} tok/s", file=sys.stderr)
    points, prefill = {}, None
    if not a.no_points:
        prefill = prefill_run()
        print(f"[bench] prefill: {prefill['value']:.0f} tok/s, {prefill['ms']:.2f} ms, {prefill['tflops']:.0f} TFLOP/s", file=sys.stderr)
        for b in (1, 64):
            r = decode_run(b, max(8, min(a.steps, 32)), 3)
            points[f"decode_b{b}"] = r["tok_s"]
            points[f"decode_b{b}_hbm_frac"] = r["bytes"] / (r["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"]
            print(f"[bench] decode batch {b}: {r['tok_s']:.1f} tok/s, {r['ms_per_step']:.3f} ms/step", file=sys.stderr)

    if not a.no_points:
        # the same steps with the sampling chain a chat deployment of this architecture uses, all of it on the device
        r = decode_run(a.batch, max(8, min(a.steps, 32)), 3, SamplerConfig(temp=0.6, top_k=20, top_p=0.95, seed=1))
        points[f"decode_b{a.batch}_temp0.6_top_k20_top_p0.95"] = r["tok_s"]
        print(f"[bench] decode batch {a.batch}, temp 0.6 / top-k 20 / top-p 0.95 on the device: {r['tok_s']:.1f} tok/s, "
              f"{r['ms_per_step']:.3f} ms/step", file=sys.stderr)

    sweep = {}
    for t in [int(x) for x in a.prefill_lengths.split(",") if x.strip()]:
        r = prefill_run(t)
        sweep[str(t)] = round(r["ms"], 3)
        print(f"[bench] prefill of {t} tokens: {r['ms']:.3f} ms, {r['value']:.0f} tok/s, {r['tflops']:.0f} TFLOP/s", file=sys.stderr)

    by_context = {}
    for c in long_ctx:
        for b in sorted({1, a.batch}):
            r = decode_run(b, 16, 3, prompt_len=c)
            frac = r["bytes"] / (r["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"]
            by_context[f"ctx{c}_b{b}"] = {"tok_s": round(r["tok_s"], 1), "ms_per_step": round(r["ms_per_step"], 3),
                                          "hbm_frac": round(frac, 3)}
            print(f"[bench] decode at context {c}, batch {b}: {r['tok_s']:.1f} tok/s, {r['ms_per_step']:.3f} ms/step, "
                  f"{frac:.3f} of the HBM roofline", file=sys.stderr)

    workload = None
    if a.workload:
        workload = workload_run()
        print(f"[bench] workload: {workload}", file=sys.stderr)

    achieved = main_run["bytes"] / (main_run["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": f"Qwen3-{a.shape.upper()} bf16 decode tok/s @ batch {a.batch} (points: batch 1/64; prefill tok/s @ 2,048 tokens)",
        "value": main_run["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": main_run["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded uniform token ids, random weights N(0, 0.02), norm weights 1",
        "impl": "ours",
        "config": {
            "model": f"Qwen3-{a.shape.upper()} shape", "layers": a.layers, "layers_of_config": base["num_hidden_layers"],
            "hidden": cdict["hidden_size"], "q_heads": cdict["num_attention_heads"],
            "kv_heads": cdict["num_key_value_heads"], "head_dim": cdict["head_dim"],
            "intermediate": cdict["intermediate_size"], "vocab": cdict["vocab_size"],
            "rope_theta": cdict["rope_theta"], "rms_norm_eps": cdict["rms_norm_eps"], "tied": False,
            "global_batch": a.batch, "prompt_len": PROMPT_LEN, "seq_len": CONTEXT, "parallelism": "single GPU",
            "sampling": "greedy on device", "l2": "inputs>L2 (16 GB of weights per step)",
            "peaks": pk["source"],
        },
        "e2e": {"value": e2e["tok_s"], "unit": "tokens/s", "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                "warmup": e2e["warmup"]},       # untimed decode steps of this arm (at least 32, see e2e_run)
        "gpu_launches": main_run["launches"],
        "clocks": main_run["clocks"],
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "of": pk["source"]},
    }
    if prefill is not None:
        line["prefill"] = {k: prefill[k] for k in ("value", "tokens", "ms", "frac")}
        line["points"] = points
    if sweep:
        line["prefill_sweep_ms"] = sweep
    if by_context:
        line["decode_by_context"] = by_context
    if workload is not None:
        line["workload"] = workload
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
