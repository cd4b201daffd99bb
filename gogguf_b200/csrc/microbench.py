"""Kernel micro-benchmarks: python -m gogguf_b200.csrc.microbench [gemm|gemm_layer|attn|prefill_attn|sample] [--m 1,8,64] [--ctx 2048,8192]

Times single kernels the way a decode step runs them: forty launches captured in a CUDA graph and
replayed, so that host launch cost is out of the picture and dependent launches overlap as they do
in a step.  Weights rotate over more than 400 MB so that the 126 MB L2 cannot serve them.  Prints
one line per (shape, M) with microseconds per launch and the achieved weight or cache bandwidth.
"""
from __future__ import annotations

import argparse
import math

import torch

SHAPES = {"qkv": (6144, 4096), "o": (4096, 4096), "gateup": (24576, 4096), "down": (4096, 12288),
          "head": (151936, 4096)}


def _time_graph(fn, reps: int = 40) -> float:
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(reps):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps * 1e3


def gemm(ms) -> None:
    from . import tcgen05_gemm as tc
    dev = "cuda:0"
    for name, (N, K) in SHAPES.items():
        nbuf = max(2, int(400e6 // (N * K * 2)) + 1)
        ws = [torch.randn(N, K, device=dev).to(torch.bfloat16) for _ in range(nbuf)]
        for M in ms:
            x = torch.randn(M, K, device=dev).to(torch.bfloat16)
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            us = _time_graph(lambda i: tc.gemm_tc(x, ws[i % nbuf], out, cluster=True))
            print(f"gemm {name:7s} M={M:4d} splits={tc.splits_for(M, N, K, True):2d} {us:8.1f} us "
                  f"{N * K * 2 / us / 1e6:6.2f} TB/s", flush=True)
        del ws
        torch.cuda.empty_cache()


def gemm_layer(ms) -> None:
    """The four products of a layer as the layer runs them: q/k/v and gate-up (+ SwiGLU) with the folded norm on
    the way in, O and down adding into the residual and writing the next product's row statistics."""
    from . import tcgen05_gemm as tc
    dev = "cuda:0"
    H, QKV, I = 4096, 6144, 12288
    for M in ms:
        resid = torch.randn(M, H, device=dev)
        xh = resid.to(torch.bfloat16)
        ssq = torch.rand(M, H // 128, device=dev) * 128
        oss = torch.empty(M, H // 128, device=dev)
        oxh = torch.empty(M, H, device=dev, dtype=torch.bfloat16)
        act = torch.randn(M, I, device=dev).to(torch.bfloat16)
        attn_out = torch.randn(M, H, device=dev).to(torch.bfloat16)
        cases = (
            ("qkv    norm in", QKV, H, lambda w, o: tc.gemm_tc_norm(xh, w, o, in_ssq=ssq, eps=1e-6),
             torch.empty(M, QKV, device=dev, dtype=torch.bfloat16)),
            ("o      add+stats", H, H, lambda w, o: tc.gemm_tc_norm(attn_out, w, o, accumulate=True, out_ssq=oss, out_xhat=oxh), resid),
            ("gateup norm in, swiglu", 2 * I, H, lambda w, o: tc.gemm_tc_norm(xh, w, o, swiglu=True, in_ssq=ssq, eps=1e-6),
             torch.empty(M, I, device=dev, dtype=torch.bfloat16)),
            ("down   add+stats", H, I, lambda w, o: tc.gemm_tc_norm(act, w, o, accumulate=True, out_ssq=oss, out_xhat=oxh), resid),
        )
        for name, N, K, fn, out in cases:
            nbuf = max(2, int(400e6 // (N * K * 2)) + 1)
            ws = [(torch.randn(N, K, device=dev) * 0.01).to(torch.bfloat16) for _ in range(nbuf)]
            us = _time_graph(lambda i: fn(ws[i % nbuf], out))
            print(f"gemm_layer {name:24s} M={M:5d} {us:8.1f} us {2.0 * M * N * K / us / 1e6:7.1f} TFLOP/s "
                  f"{N * K * 2 / us / 1e6:6.2f} TB/s", flush=True)
            del ws
            torch.cuda.empty_cache()
        tc.check_status(torch.device(dev))


def attn(ms, ctx_len: int = 2048, nq: int = 32, nkv: int = 8, d: int = 128, cluster: bool = True) -> None:
    from . import fast_attention as fa
    dev = "cuda:0"
    for B in ms:
        pages_per = (ctx_len + 63) // 64
        layers = max(2, int(400e6 // (B * pages_per * nkv * 64 * d * 2 * 2)) + 1)     # rotate over layers' pools
        kp = [torch.randn(B * pages_per, nkv, 64, d, device=dev).to(torch.bfloat16) for _ in range(layers)]
        vp = [torch.randn(B * pages_per, nkv, 64, d, device=dev).to(torch.bfloat16) for _ in range(layers)]
        table = torch.arange(B * pages_per, dtype=torch.int32, device=dev).view(B, pages_per)
        pos = torch.full((B,), ctx_len - 1, dtype=torch.int32, device=dev)
        sot = torch.arange(B, dtype=torch.int32, device=dev)
        q = torch.randn(B, nq, d, device=dev).to(torch.bfloat16)
        out = torch.empty_like(q)
        splits = fa.decode_tma_splits(B, nkv, ctx_len, cluster=cluster)
        po = torch.empty(B * nq * splits * d, device=dev) if not cluster else None
        pm = torch.empty(B * nq * splits * 2, device=dev) if not cluster else None
        us = _time_graph(lambda i: fa.attn_decode_tma(q, kp[i % layers], vp[i % layers], out, pos, sot, table, 64, B,
                                                      nq, nkv, d, 1.0 / math.sqrt(d), 0, splits, po, pm, cluster=cluster))
        nbytes = B * ctx_len * nkv * d * 2 * 2
        form = f"cluster of {splits}" if cluster else f"{splits} splits + combine"
        print(f"attn decode B={B:4d} ctx={ctx_len:6d} {form:22s} {us:8.1f} us {nbytes / us / 1e6:6.2f} TB/s", flush=True)
        del kp, vp
        torch.cuda.empty_cache()


def prefill_attn(lens, nq: int = 32, nkv: int = 8, d: int = 128) -> None:
    """One sequence of T new tokens from position 0, both prefill kernels."""
    from . import fast_attention as fa
    dev = "cuda:0"
    for T in lens:
        pages = (T + 63) // 64
        kp = torch.randn(pages, nkv, 64, d, device=dev).to(torch.bfloat16)
        vp = torch.randn(pages, nkv, 64, d, device=dev).to(torch.bfloat16)
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages)
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        cl = torch.tensor([T], dtype=torch.int32, device=dev)
        sot = torch.zeros(T, dtype=torch.int32, device=dev)
        q = torch.randn(T, nq, d, device=dev).to(torch.bfloat16)
        out = torch.empty_like(q)
        flops = 4.0 * nq * d * (T * (T + 1) / 2)
        us = _time_graph(lambda i: fa.attn_prefill(q, kp, vp, out, cu, cl, sot, table, 64, 1, T // 64 + 1, nq, nkv, d,
                                                   1.0 / math.sqrt(d), 0), reps=10)
        print(f"attn prefill mma.sync T={T:6d} {us:9.1f} us {flops / us / 1e6:7.1f} TFLOP/s", flush=True)
        us = _time_graph(lambda i: fa.attn_prefill_tc(q, kp, vp, out, cu, cl, sot, table, 64, T, 1, T // 128 + 1, nq, nkv,
                                                      d, 1.0 / math.sqrt(d), 0), reps=10)
        print(f"attn prefill tcgen05  T={T:6d} {us:9.1f} us {flops / us / 1e6:7.1f} TFLOP/s", flush=True)


def sample(ms, V: int = 151936) -> None:
    """The sampling kernels on [batch, vocabulary] float32 logits: greedy, temperature, and the top-k chain."""
    from . import kernels as K
    dev = "cuda:0"
    for B in ms:
        logits = torch.randn(B, V, device=dev) * 3
        out = torch.empty(B, dtype=torch.int32, device=dev)
        u = torch.rand(B, dtype=torch.float64, device=dev)
        temps = torch.full((B,), 0.6, device=dev)
        for name, fn in (("greedy", lambda i: K.argmax(logits, out, B)),
                         ("temperature 0.6", lambda i: K.sample(logits, temps, u, out, B)),
                         ("temp 0.6, top-k 20, top-p 0.95", lambda i: K.sample_topk(logits, 0.6, 20, 0.95, 0.0, u, out, B)),
                         ("temp 0.6, top-k 1000, top-p 0.95", lambda i: K.sample_topk(logits, 0.6, 1000, 0.95, 0.0, u, out, B))):
            us = _time_graph(fn, reps=10)
            print(f"sample B={B:4d} V={V} {name:34s} {us:8.1f} us", flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "gemm_layer", "attn", "prefill_attn", "sample"])
    ap.add_argument("--m", default="1,8,64", help="token counts (gemm), batch sizes (attn) or prompt lengths (prefill_attn)")
    ap.add_argument("--ctx", default="2048", help="attn: cached positions per sequence (comma separated)")
    ap.add_argument("--scratch", action="store_true", help="attn: splits merged by a second kernel instead of inside clusters")
    a = ap.parse_args()
    ms = [int(x) for x in a.m.split(",")]
    if a.what == "attn":
        for c in a.ctx.split(","):
            attn(ms, ctx_len=int(c), cluster=not a.scratch)
    else:
        {"gemm": gemm, "gemm_layer": gemm_layer, "prefill_attn": prefill_attn, "sample": sample}[a.what](ms)


if __name__ == "__main__":
    main()
