"""Run by tests/test_gpu_kernels.py in a process of its own with GOGGUF_B200_DEBUG=1 (the build flags are read
when the package is imported).  Every attention kernel is given a page table with one page id beyond the pool
and, separately, a context that needs more table entries than the table has; the debug build must record its
code in the status word and read page 0 instead.  The pools are views of larger buffers, so that even a kernel
without the check would stay inside allocated memory."""
import math
import sys
from types import SimpleNamespace

import torch

sys.path.insert(0, sys.argv[1])
from gogguf_b200.csrc import build, fast_attention as fa, kernels as K, tcgen05_gemm as tc   # noqa: E402

assert build.DEBUG
DEV = "cuda:0"
assert build.module("attention_fast").lib.gg_attention_fast_checked() == 1
assert build.module("attention_plain").lib.gg_attention_plain_checked() == 1
nq, nkv, d, n_pages, spare = 8, 2, 128, 12, 6
scale = 1.0 / math.sqrt(d)
g = torch.Generator(device=DEV).manual_seed(1)
status = tc.status_word(DEV)


def read_status():
    v = int(status.item())
    status.zero_()
    return v


def run(kind, dt, table, ctx_len, n_new):
    big_k = torch.randn(n_pages + spare, nkv, 64, d, device=DEV, generator=g).to(dt)
    big_v = torch.randn(n_pages + spare, nkv, 64, d, device=DEV, generator=g).to(dt)
    kp, vp = big_k[:n_pages], big_v[:n_pages]
    T = n_new
    mk = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)      # noqa: E731
    pos, sot = mk(list(range(ctx_len - n_new, ctx_len))), mk([0] * T)
    cu, cl = mk([0, T]), mk([ctx_len])
    q = torch.randn(T, nq, d, device=DEV, generator=g).to(dt)
    out = torch.full((T, nq, d), float("nan"), device=DEV, dtype=dt)
    if kind == "plain":
        K.attention_plain(q, kp, vp, out, pos, sot, table, 64, T, nq, nkv, d, scale, 0)
    elif kind == "decode":
        po = torch.empty(T * nq * 2 * d, device=DEV); pm = torch.empty(T * nq * 2 * 2, device=DEV)
        fa.attn_decode(q, kp, vp, out, pos, sot, table, 64, T, nq, nkv, d, scale, 0, 2, po, pm)
    elif kind == "decode_tma":
        fa.attn_decode_tma(q, kp, vp, out, pos, sot, table, 64, T, nq, nkv, d, scale, 0, 2, cluster=True)
    elif kind == "prefill":
        fa.attn_prefill(q, kp, vp, out, cu, cl, sot, table, 64, 1, T // 64 + 1, nq, nkv, d, scale, 0)
    elif kind == "prefill_tc":
        fa.attn_prefill_tc(q, kp, vp, out, cu, cl, sot, table, 64, T, 1, T // 128 + 1, nq, nkv, d, scale, 0)
    torch.cuda.synchronize()
    return out


codes = {"plain": 41, "decode": 42, "prefill": 43, "decode_tma": 44, "prefill_tc": 45}
ctx_len = 5 * 64 + 9
good = torch.tensor([[3, 7, 1, 11, 0, 5, 2, 2]], dtype=torch.int32, device=DEV)
for kind, code in codes.items():
    for dt in ((torch.float32, torch.bfloat16) if kind == "plain" else (torch.bfloat16,)):
        n_new = 1 if kind.startswith("decode") else 70
        out = run(kind, dt, good, ctx_len, n_new)
        assert read_status() == 0, (kind, "a good table must leave the status word alone")
        assert bool(torch.isfinite(out.float()).all())
        bad = good.clone()
        bad[0, 2] = n_pages + 3                       # a page id beyond the pool (inside the larger buffer)
        out = run(kind, dt, bad, ctx_len, n_new)
        assert read_status() == code, (kind, "page id out of range")
        assert bool(torch.isfinite(out.float()).all())
        bad[0, 2] = -4
        run(kind, dt, bad, ctx_len, n_new)
        assert read_status() == code, (kind, "negative page id")
        short = good[:, :4].contiguous()              # the context needs six table entries, the table has four
        run(kind, dt, short, ctx_len, n_new)
        assert read_status() == code, (kind, "table index out of range")
# The cache writers: a bad page id or a table that is too short makes them write nothing at all for that token
# (every byte of the larger buffers keeps its sentinel), a good table makes them write exactly one row per head.
assert build.module("elementwise").lib.gg_elementwise_checked() == 1


def write_run(kind, dt, table, pos_list):
    big_k = torch.full((n_pages + spare, nkv, 64, d), 7.0, device=DEV, dtype=dt)
    big_v = torch.full((n_pages + spare, nkv, 64, d), 7.0, device=DEV, dtype=dt)
    kp, vp = big_k[:n_pages], big_v[:n_pages]
    T = len(pos_list)
    mk = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)      # noqa: E731
    pos, sot = mk(pos_list), mk([0] * T)
    cos = torch.ones(T, d // 2, device=DEV); sin = torch.zeros(T, d // 2, device=DEV)
    q_out = torch.empty(T, nq * d, device=DEV, dtype=dt)
    if kind == "plain":
        qkv = torch.randn(T, (nq + 2 * nkv) * d, device=DEV, generator=g).to(dt)
        K.qk_norm_rope_cache(qkv, q_out, None, None, 1e-6, cos, sin, pos, sot, table, 64, kp, vp, T, nq, nkv, d, d)
    else:
        Kd = 256
        x = torch.randn(T, Kd, device=DEV, generator=g).to(dt)
        w = (torch.randn((nq + 2 * nkv) * d, Kd, device=DEV, generator=g) * 0.1).to(dt)
        tc.gemm_tc_qkv_rope(x, w, T, q_out=q_out, qw=None, kw=None, eps=1e-6, cos=cos, sin=sin, positions=pos,
                            seq_of_token=sot, page_table=table, page_size=64, k_pool=kp, v_pool=vp, nq=nq, nkv=nkv)
    torch.cuda.synchronize()
    changed = int((big_k != 7.0).any(-1).sum()) + int((big_v != 7.0).any(-1).sum())
    return changed


for kind, dt, code, T in (("plain", torch.float32, 46, 5), ("plain", torch.bfloat16, 47, 5), ("product", torch.bfloat16, 48, 5),
                          ("product", torch.bfloat16, 48, 300)):
    pos_list = list(range(64 * 2 + 3, 64 * 2 + 3 + T)) if T < 64 else list(range(T))
    changed = write_run(kind, dt, good, pos_list)
    assert read_status() == 0 and changed == 2 * nkv * T, (kind, dt, changed)
    bad = good.clone()
    bad[0, :] = n_pages + 2                                   # every page id beyond the pool
    changed = write_run(kind, dt, bad, pos_list)
    assert read_status() == code and changed == 0, (kind, dt, T, changed)
    short = good[:, :2].contiguous()
    changed = write_run(kind, dt, short, [64 * 2 + 3 + i for i in range(min(T, 5))])     # page index 2: beyond the table
    assert read_status() == code and changed == 0, (kind, dt, "short table", changed)

# the host raises with the kernel's name when it next checks the word
bad = good.clone(); bad[0, 1] = 99
run("decode_tma", torch.bfloat16, bad, ctx_len, 1)
try:
    tc.check_status(DEV)
    raise SystemExit("check_status did not raise")
except build.KernelError as e:
    assert "attn_decode_tma" in str(e) and "page" in str(e), str(e)
assert int(status.item()) == 0
print("debug bounds ok")
