"""Each kernel alone against a plain float32/float64 PyTorch reference of the same op, at sizes other
than the engine's (odd widths, head sizes in steps of 16, vocabularies that are no power of two)."""
import math
import os

from types import SimpleNamespace

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def K():
    from gogguf_b200.csrc import kernels
    return kernels


def rel(a, b):
    a, b = a.double(), b.double()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


# ------------------------------------------------------------------------------------------ elementwise
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_embed_gather(dt):
    g = torch.Generator(device=DEV).manual_seed(0)
    table = torch.randn(331, 72, device=DEV, generator=g).to(dt)
    toks = torch.tensor([5, 330, -1, 0, 17], dtype=torch.int32, device=DEV)
    out = torch.full((5, 72), 9.0, device=DEV)
    K().embed_gather(table, toks, out)
    want = table[toks.clamp_min(0).long()].float()
    want[2] = 0
    assert torch.equal(out, want)


@pytest.mark.parametrize("H,eps", [(72, 1e-6), (1000, 1e-5), (4096, 3e-6), (5120 + 8, 1e-6)])
@pytest.mark.parametrize("odt", [torch.float32, torch.bfloat16])
def test_rmsnorm(H, eps, odt):
    g = torch.Generator(device=DEV).manual_seed(1)
    x = torch.randn(7, H, device=DEV, generator=g) * 3
    w = 1 + 0.1 * torch.randn(H, device=DEV, generator=g)
    out = torch.empty(7, H, device=DEV, dtype=odt)
    K().rmsnorm(x, w, eps, out)
    xd = x.double()
    want = xd / torch.sqrt((xd * xd).mean(-1, keepdim=True) + eps) * w.double()
    assert rel(out, want) < (2e-6 if odt == torch.float32 else 5e-3)
    rows = torch.tensor([6, -1, 0], dtype=torch.int32, device=DEV)
    out2 = torch.empty(3, H, device=DEV, dtype=odt)
    K().rmsnorm(x, w, eps, out2, rows)
    assert torch.equal(out2[0], out[6]) and torch.equal(out2[2], out[0]) and float(out2[1].abs().sum()) == 0


def test_rope_tables_in_float64():
    pos = torch.tensor([0, 1, 777, 40000, -1], dtype=torch.int32, device=DEV)
    d, theta = 48, 50000.0
    inv = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * torch.arange(d // 2, dtype=torch.float64) / d).to(DEV)
    cos = torch.empty(5, d // 2, device=DEV)
    sin = torch.empty(5, d // 2, device=DEV)
    K().rope_tables(pos, inv, cos, sin)
    ang = pos.clamp_min(0).double()[:, None] * inv[None, :]
    assert float((cos.double() - torch.cos(ang)).abs().max()) < 1e-7
    assert float((sin.double() - torch.sin(ang)).abs().max()) < 1e-7


def plain_norm_rope(x, w, eps, cos, sin, rot):
    xd = x.double()
    if w is not None:
        xd = xd / torch.sqrt((xd * xd).mean(-1, keepdim=True) + eps) * w.double()
    half = rot // 2
    x0, x1, rest = xd[..., :half], xd[..., half:rot], xd[..., rot:]
    c, s = cos.double()[:, None, :], sin.double()[:, None, :]
    return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c, rest], -1)


@pytest.mark.parametrize("nq,nkv,d,rot,norm", [(4, 2, 16, 16, True), (6, 1, 32, 32, True), (3, 3, 48, 48, True),
                                               (5, 5, 80, 64, False), (8, 2, 128, 128, True), (2, 1, 256, 256, True)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_qk_norm_rope_cache(nq, nkv, d, rot, norm, dt):
    g = torch.Generator(device=DEV).manual_seed(2)
    ps, n_pages, B = 64, 6, 2
    # two sequences: 70 new tokens from position 60 (crosses a page edge), and 3 tokens from 0; one padding row
    starts, counts = [60, 0], [70, 3]
    T = sum(counts) + 1
    qkv = (torch.randn(T, (nq + 2 * nkv) * d, device=DEV, generator=g)).to(dt)
    qw = (1 + 0.1 * torch.randn(d, device=DEV, generator=g)) if norm else None
    kw = (1 + 0.1 * torch.randn(d, device=DEV, generator=g)) if norm else None
    positions = torch.tensor(list(range(60, 130)) + [0, 1, 2] + [0], dtype=torch.int32, device=DEV)
    sot = torch.tensor([0] * 70 + [1] * 3 + [-1], dtype=torch.int32, device=DEV)
    table = torch.tensor([[4, 1, 5], [2, 0, 0]], dtype=torch.int32, device=DEV)
    inv = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot).to(DEV)
    cos = torch.empty(T, rot // 2, device=DEV); sin = torch.empty(T, rot // 2, device=DEV)
    K().rope_tables(positions, inv, cos, sin)
    kp = torch.full((n_pages, nkv, ps, d), 7.0, device=DEV, dtype=dt)
    vp = torch.full((n_pages, nkv, ps, d), 7.0, device=DEV, dtype=dt)
    q = torch.empty(T, nq * d, device=DEV, dtype=dt)
    K().qk_norm_rope_cache(qkv, q, qw, kw, 1e-5, cos, sin, positions, sot, table, ps, kp, vp, T, nq, nkv, d, rot)
    x = qkv.float().reshape(T, nq + 2 * nkv, d)
    wq = plain_norm_rope(x[:, :nq], qw, 1e-5, cos, sin, rot)
    wk = plain_norm_rope(x[:, nq:nq + nkv], kw, 1e-5, cos, sin, rot)
    wv = x[:, nq + nkv:].double()
    tol = 3e-6 if dt == torch.float32 else 6e-3
    assert rel(q.reshape(T, nq, d), wq) < tol
    written = torch.zeros(n_pages, ps, dtype=torch.bool)
    for t in range(T - 1):
        b, p = int(sot[t]), int(positions[t])
        page = int(table[b, p // ps])
        written[page, p % ps] = True
        assert rel(kp[page, :, p % ps], wk[t]) < tol
        assert rel(vp[page, :, p % ps].double(), wv[t]) < (1e-7 if dt == torch.float32 else 1e-9) or torch.equal(vp[page, :, p % ps].float(), x[t, nq + nkv:])
    # nothing else was touched (the padding row writes nothing)
    untouched = ~written.to(DEV)
    assert bool((kp.float()[untouched.nonzero(as_tuple=True)[0], :, untouched.nonzero(as_tuple=True)[1]] == 7.0).all())
    # a layer that reads another layer's cache writes none
    kp2 = kp.clone()
    K().qk_norm_rope_cache(qkv * 2, q, qw, kw, 1e-5, cos, sin, positions, sot, table, ps, None, None, T, nq, nkv, d, rot)
    assert torch.equal(kp, kp2)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_swiglu_and_residual_add(dt):
    g = torch.Generator(device=DEV).manual_seed(3)
    T, I = 5, 104
    gu = (torch.randn(T, 2 * I, device=DEV, generator=g) * 4).to(dt)
    out = torch.empty(T, I, device=DEV, dtype=dt)
    K().swiglu(gu, out, T, I)
    gd, ud = gu[:, :I].double(), gu[:, I:].double()
    assert rel(out, gd / (1 + torch.exp(-gd)) * ud) < (2e-6 if dt == torch.float32 else 5e-3)
    x = torch.randn(T, I, device=DEV, generator=g)
    x0 = x.clone()
    K().residual_add(x, out)
    assert torch.equal(x, x0 + out.float())


# ------------------------------------------------------------------------------------------ products
@pytest.mark.parametrize("M,N,K_", [(1, 7, 5), (3, 64, 64), (70, 130, 257), (129, 96, 72), (5, 331, 104)])
@pytest.mark.parametrize("xdt,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                     (torch.bfloat16, torch.float32)])
def test_gemm_plain(M, N, K_, xdt, wdt):
    g = torch.Generator(device=DEV).manual_seed(4)
    x = torch.randn(M, K_, device=DEV, generator=g).to(xdt)
    w = torch.randn(N, K_, device=DEV, generator=g).to(wdt)
    want = x.double() @ w.double().T
    out = torch.empty(M, N, device=DEV)
    K().gemm_plain(x, w, out)
    assert rel(out, want) < 2e-6
    res = torch.randn(M, N, device=DEV, generator=g)
    acc = res.clone()
    K().gemm_plain(x, w, acc, accumulate=True)
    assert rel(acc, res.double() + want) < 2e-6
    if xdt == torch.bfloat16:
        ob = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
        K().gemm_plain(x, w, ob)
        assert rel(ob, want) < 5e-3
    # batch invariance: a row's result does not depend on the other rows (bitwise)
    one = torch.empty(1, N, device=DEV)
    K().gemm_plain(x[M // 2:M // 2 + 1].contiguous(), w, one)
    assert torch.equal(one[0], out[M // 2])


TC_SHAPES = [(1, 128, 64), (8, 256, 512), (16, 4096, 4096), (17, 384, 1024), (64, 1000, 520), (128, 768, 2048),
             (129, 256, 64), (300, 520, 264), (2048, 1024, 4096), (70, 96, 72), (5, 331, 104), (1000, 72, 48)]


@pytest.mark.parametrize("M,N,K_", TC_SHAPES)
def test_gemm_tcgen05(M, N, K_):
    from gogguf_b200.csrc import tcgen05_gemm as tc
    g = torch.Generator(device=DEV).manual_seed(5)
    x = torch.randn(M, K_, device=DEV, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K_, device=DEV, generator=g).to(torch.bfloat16)
    want = x.double() @ w.double().T
    # float32 accumulation over K terms: the rounding error grows like sqrt(K) * 2^-24
    tol = 2e-6 + 2e-7 * math.sqrt(K_)
    splits = tc.splits_for(M, N, K_)
    scratch = torch.empty(max(1, splits * M * N), device=DEV) if splits > 1 else None
    out = torch.full((M, N), float("nan"), device=DEV)
    tc.gemm_tc(x, w, out, scratch=scratch)
    tc.check_status(DEV)
    assert rel(out, want) < tol, (splits,)
    res = torch.randn(M, N, device=DEV, generator=g)
    acc = res.clone()
    tc.gemm_tc(x, w, acc, accumulate=True, scratch=scratch)
    assert rel(acc, res.double() + want) < tol
    ob = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    tc.gemm_tc(x, w, ob, scratch=scratch)
    tc.check_status(DEV)
    assert rel(ob, want) < 5e-3
    # the cluster form (partial sums added through distributed shared memory, no scratch)
    oc = torch.full((M, N), float("nan"), device=DEV)
    tc.gemm_tc(x, w, oc, cluster=True)
    tc.check_status(DEV)
    assert rel(oc, want) < tol, (tc.splits_for(M, N, K_, True),)
    accc = res.clone()
    tc.gemm_tc(x, w, accc, accumulate=True, cluster=True)
    assert rel(accc, res.double() + want) < tol
    obc = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    tc.gemm_tc(x, w, obc, cluster=True)
    assert rel(obc, want) < 5e-3
    again = torch.empty(M, N, device=DEV)
    tc.gemm_tc(x, w, again, cluster=True)
    assert torch.equal(again, oc)            # the order of the additions is fixed: same bits every time
    # the plain twin agrees
    twin = torch.empty(M, N, device=DEV)
    K().gemm_plain(x, w, twin)
    assert rel(out, twin) < tol


@pytest.mark.parametrize("M,I,K_", [(1, 128, 64), (8, 192, 256), (64, 12288, 512), (100, 640, 136), (129, 128, 72),
                                    (300, 448, 264), (2048, 1024, 1024)])
def test_gemm_tcgen05_fused_swiglu(M, I, K_):
    from gogguf_b200.csrc import tcgen05_gemm as tc
    g = torch.Generator(device=DEV).manual_seed(15)
    x = torch.randn(M, K_, device=DEV, generator=g).to(torch.bfloat16)
    wg = (torch.randn(I, K_, device=DEV, generator=g) / math.sqrt(K_)).to(torch.bfloat16)
    wu = (torch.randn(I, K_, device=DEV, generator=g) / math.sqrt(K_)).to(torch.bfloat16)
    w = tc.interleave_gate_up(wg, wu)
    out = torch.full((M, I), float("nan"), device=DEV, dtype=torch.bfloat16)
    tc.gemm_tc(x, w, out, cluster=True, swiglu=True)
    tc.check_status(DEV)
    gd, ud = x.double() @ wg.double().T, x.double() @ wu.double().T
    want = gd / (1 + torch.exp(-gd)) * ud
    assert rel(out, want) < 6e-3
    # the unfused pair of kernels gives the same to bfloat16 rounding
    gu = torch.empty(M, 2 * I, device=DEV, dtype=torch.bfloat16)
    tc.gemm_tc(x, torch.cat([wg, wu]), gu, cluster=True)
    twin = torch.empty(M, I, device=DEV, dtype=torch.bfloat16)
    K().swiglu(gu, twin, M, I)
    assert rel(out, twin) < 1.2e-2


def test_gemm_tcgen05_strided_rows_and_padding_rows():
    from gogguf_b200.csrc import tcgen05_gemm as tc
    g = torch.Generator(device=DEV).manual_seed(6)
    big = torch.randn(40, 512, device=DEV, generator=g).to(torch.bfloat16)
    x = big[:, :256]                       # row stride 512, K = 256
    w = torch.randn(200, 256, device=DEV, generator=g).to(torch.bfloat16)
    outbig = torch.zeros(40, 300, device=DEV)
    out = outbig[:, :200]
    splits = tc.splits_for(24, 200, 256)
    scratch = torch.empty(max(1, splits * 24 * 200), device=DEV)
    tc.gemm_tc(x, w, out, m=24, scratch=scratch)      # only the first 24 rows are computed
    tc.check_status(DEV)
    assert rel(out[:24], x[:24].double() @ w.double().T) < 3e-6
    assert float(outbig[24:].abs().sum()) == 0 and float(outbig[:, 200:].abs().sum()) == 0


def plain_row_stats(x):
    """bfloat16 copy and per-128-column sums of squares of float32 rows (the plain statement of row_stats)."""
    T, H = x.shape
    parts = (H + 127) // 128
    pad = torch.zeros(T, parts * 128, dtype=torch.float64, device=x.device)
    pad[:, :H] = x.double()
    return x.to(torch.bfloat16), (pad * pad).view(T, parts, 128).sum(-1)


@pytest.mark.parametrize("T,H", [(1, 128), (5, 200), (64, 4096), (300, 1000), (3, 5128)])
def test_row_stats(T, H):
    g = torch.Generator(device=DEV).manual_seed(31)
    x = torch.randn(T, H, device=DEV, generator=g) * 3
    xh = torch.empty(T, H, device=DEV, dtype=torch.bfloat16)
    ssq = torch.full((T, (H + 127) // 128), float("nan"), device=DEV)
    K().row_stats(x, xh, ssq)
    wh, ws = plain_row_stats(x)
    assert torch.equal(xh, wh)
    assert rel(ssq, ws) < 1e-6


NORM_SHAPES = [(1, 128, 128), (8, 256, 512), (8, 4096, 4096), (17, 384, 1000), (64, 1000, 520), (128, 768, 2048),
               (129, 256, 136), (300, 520, 264), (1024, 1024, 4096), (70, 96, 72), (5, 331, 104), (1000, 72, 48),
               (260, 200, 64),
               # owners that pull: from two, three and eight ranks, up to six tokens per warp
               (48, 24576, 256), (100, 16384, 512), (64, 4096, 4096), (128, 4096, 1024)]


@pytest.mark.parametrize("M,N,K_", NORM_SHAPES)
def test_gemm_tcgen05_with_folded_norm(M, N, K_):
    """The product that reads raw rows and applies 1/rms in its epilogue, and the accumulating product that
    also writes the next product's inputs; against the plain statement in float64."""
    from gogguf_b200.csrc import tcgen05_gemm as tc
    g = torch.Generator(device=DEV).manual_seed(33)
    eps = 3e-5
    resid = torch.randn(M, K_, device=DEV, generator=g) * torch.linspace(0.2, 5.0, M, device=DEV)[:, None]
    w = (torch.randn(N, K_, device=DEV, generator=g) / math.sqrt(K_)).to(torch.bfloat16)
    xh, ssq = plain_row_stats(resid)
    ssq = ssq.float().contiguous()
    factor = 1.0 / torch.sqrt((resid.double() ** 2).mean(-1, keepdim=True) + eps)
    want = (xh.double() @ w.double().T) * factor
    tol = 3e-6 + 2e-7 * math.sqrt(K_)
    # (1) factor on the way in, each output mode
    out = torch.full((M, N), float("nan"), device=DEV)
    tc.gemm_tc_norm(xh, w, out, in_ssq=ssq, eps=eps)
    tc.check_status(DEV)
    assert rel(out, want) < tol
    ob = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    tc.gemm_tc_norm(xh, w, ob, in_ssq=ssq, eps=eps)
    assert rel(ob, want) < 5e-3
    # (2) accumulate and emit the statistics of the updated rows
    res = torch.randn(M, N, device=DEV, generator=g)
    acc = res.clone()
    oh = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    oss = torch.full((M, (N + 127) // 128), float("nan"), device=DEV)
    tc.gemm_tc_norm(xh, w, acc, accumulate=True, in_ssq=ssq, eps=eps, out_ssq=oss, out_xhat=oh)
    tc.check_status(DEV)
    assert rel(acc, res.double() + want) < tol
    wh, ws = plain_row_stats(acc)
    assert torch.equal(oh, wh)
    assert rel(oss, ws) < 1e-6
    # (3) emit without a factor on the way in (the projection after attention)
    acc2 = res.clone()
    oh.fill_(float("nan")); oss.fill_(float("nan"))
    tc.gemm_tc_norm(xh, w, acc2, accumulate=True, out_ssq=oss, out_xhat=oh)
    assert rel(acc2, res.double() + xh.double() @ w.double().T) < tol
    wh, ws = plain_row_stats(acc2)
    assert torch.equal(oh, wh) and rel(oss, ws) < 1e-6
    # same bits on a second call
    again = torch.empty(M, N, device=DEV)
    tc.gemm_tc_norm(xh, w, again, in_ssq=ssq, eps=eps)
    assert torch.equal(again, out)


@pytest.mark.parametrize("M,I,K_", [(1, 128, 128), (8, 12288, 512), (100, 640, 136), (300, 448, 264), (520, 1024, 1024),
                                    (64, 12288, 512), (128, 6144, 1024), (40, 12288, 256), (33, 12288, 4096)])
def test_gemm_tcgen05_fused_swiglu_with_folded_norm(M, I, K_):
    from gogguf_b200.csrc import tcgen05_gemm as tc
    g = torch.Generator(device=DEV).manual_seed(35)
    eps = 1e-6
    resid = torch.randn(M, K_, device=DEV, generator=g) * 4
    wg = (torch.randn(I, K_, device=DEV, generator=g) / math.sqrt(K_)).to(torch.bfloat16)
    wu = (torch.randn(I, K_, device=DEV, generator=g) / math.sqrt(K_)).to(torch.bfloat16)
    w = tc.interleave_gate_up(wg, wu)
    xh, ssq = plain_row_stats(resid)
    factor = 1.0 / torch.sqrt((resid.double() ** 2).mean(-1, keepdim=True) + eps)
    out = torch.full((M, I), float("nan"), device=DEV, dtype=torch.bfloat16)
    tc.gemm_tc_norm(xh, w, out, swiglu=True, in_ssq=ssq.float().contiguous(), eps=eps)
    tc.check_status(DEV)
    gd, ud = (xh.double() @ wg.double().T) * factor, (xh.double() @ wu.double().T) * factor
    assert rel(out, gd / (1 + torch.exp(-gd)) * ud) < 6e-3


@pytest.mark.parametrize("M,nq,nkv,K_,norm,fold", [(1, 2, 1, 128, True, False), (8, 8, 2, 512, True, True),
                                                   (37, 3, 3, 264, False, True), (128, 4, 1, 1024, True, False),
                                                   (300, 8, 2, 512, True, True), (1000, 5, 5, 136, False, False),
                                                   (129, 3, 1, 264, True, False), (600, 2, 1, 2048, True, True),
                                                   (256, 32, 8, 4096, True, True), (384, 4, 4, 1024, False, False)])
def test_gemm_tcgen05_qkv_with_norm_rope_and_cache_write(M, nq, nkv, K_, norm, fold):
    """The q/k/v product with the per-head work in its epilogue (decode form up to 128 tokens, CTA-pair form
    above), against the unfused pair (product, then the qk_norm_rope_cache kernel), and against the plain
    statement."""
    from gogguf_b200.csrc import tcgen05_gemm as tc
    if M > 128 and not tc.qkv_rope_takes(M):
        pytest.skip("the single-CTA prefill form has no q/k/v epilogue")
    d, ps = 128, 64
    UNWRITTEN = 2.0 ** 100
    g = torch.Generator(device=DEV).manual_seed(41)
    resid = torch.randn(M, K_, device=DEV, generator=g) * 2
    w = (torch.randn((nq + 2 * nkv) * d, K_, device=DEV, generator=g) / math.sqrt(K_)).to(torch.bfloat16)
    xh, ssq = plain_row_stats(resid)
    ssq = ssq.float().contiguous()
    eps_in, eps = 2e-6, 1e-5
    qw = (1 + 0.2 * torch.randn(d, device=DEV, generator=g)) if norm else None
    kw = (1 + 0.2 * torch.randn(d, device=DEV, generator=g)) if norm else None
    # tokens: sequence b holds a few tokens at positions that cross a page edge; one padding token at the end
    nseq = max(1, M // 5)
    seq_of = torch.tensor([min(t % nseq, nseq - 1) for t in range(M)], dtype=torch.int32)
    pos = torch.tensor([60 + t // nseq for t in range(M)], dtype=torch.int32)
    if M > 1:
        seq_of[-1] = -1
    pages_per = 3
    table = torch.randperm(nseq * pages_per, generator=torch.Generator().manual_seed(1)).to(torch.int32).view(nseq, pages_per)
    seq_of, pos, table = seq_of.to(DEV), pos.to(DEV), table.to(DEV)
    inv = torch.pow(torch.tensor(1e4, dtype=torch.float64), -2.0 * torch.arange(64, dtype=torch.float64) / d).to(DEV)
    cos, sin = torch.empty(M, 64, device=DEV), torch.empty(M, 64, device=DEV)
    K().rope_tables(pos, inv, cos, sin)
    npages = nseq * pages_per

    def pools():
        # a value no product reaches marks the rows that nobody wrote
        return (torch.full((npages, nkv, ps, d), UNWRITTEN, device=DEV, dtype=torch.bfloat16),
                torch.full((npages, nkv, ps, d), UNWRITTEN, device=DEV, dtype=torch.bfloat16))

    # unfused twin
    qkv = torch.empty(M, (nq + 2 * nkv) * d, device=DEV, dtype=torch.bfloat16)
    if fold:
        tc.gemm_tc_norm(xh, w, qkv, in_ssq=ssq, eps=eps_in)
    else:
        tc.gemm_tc(xh, w, qkv, cluster=True)
    q1 = torch.empty(M, nq * d, device=DEV, dtype=torch.bfloat16)
    k1, v1 = pools()
    K().qk_norm_rope_cache(qkv, q1, qw, kw, eps, cos, sin, pos, seq_of, table, ps, k1, v1, M, nq, nkv, d, d)
    # fused
    q2 = torch.full((M, nq * d), float("nan"), device=DEV, dtype=torch.bfloat16)
    k2, v2 = pools()
    tc.gemm_tc_qkv_rope(xh, w, M, q2, qw, kw, eps, cos, sin, pos, seq_of, table, ps, k2, v2, nq, nkv,
                        in_ssq=ssq if fold else None, in_eps=eps_in)
    tc.check_status(DEV)
    # the same cache rows were written, and no others
    assert torch.equal(k2 == UNWRITTEN, k1 == UNWRITTEN) and torch.equal(v2 == UNWRITTEN, v1 == UNWRITTEN)
    wk, wv = k1 != UNWRITTEN, v1 != UNWRITTEN
    assert wk.any() or M == 1
    assert rel(q2, q1) < 1e-2 and rel(k2[wk], k1[wk]) < 1e-2 and rel(v2[wv], v1[wv]) < 1e-2
    # plain statement in float64 (the fused epilogue does not round q/k/v to bfloat16 before the norm)
    factor = 1.0 / torch.sqrt((resid.double() ** 2).mean(-1, keepdim=True) + eps_in) if fold else 1.0
    full = (xh.double() @ w.double().T) * factor
    qd = full[:, :nq * d].view(M, nq, d)
    if norm:
        qd = qd / torch.sqrt((qd ** 2).mean(-1, keepdim=True) + eps) * qw.double()
    c, s_ = cos.double()[:, None, :], sin.double()[:, None, :]
    want = torch.cat([qd[..., :64] * c - qd[..., 64:] * s_, qd[..., :64] * s_ + qd[..., 64:] * c], dim=-1).view(M, nq * d)
    assert rel(q2, want) < 6e-3
    # writes_cache False: only q is written
    q3 = torch.empty_like(q2)
    tc.gemm_tc_qkv_rope(xh, w, M, q3, qw, kw, eps, cos, sin, pos, seq_of, table, ps, None, None, nq, nkv,
                        in_ssq=ssq if fold else None, in_eps=eps_in)
    assert torch.equal(q3, q2)
    # with room for partial tiles a product of a few hundred tokens splits K over the CTA pairs, and the kernel
    # that adds the partial tiles does the per-head work
    need = tc.pair_scratch_elems(M, w.shape[0], K_) if M > 128 else 0
    if need:
        scratch = torch.full((need,), float("nan"), device=DEV)
        q4 = torch.full((M, nq * d), float("nan"), device=DEV, dtype=torch.bfloat16)
        k4, v4 = pools()
        tc.gemm_tc_qkv_rope(xh, w, M, q4, qw, kw, eps, cos, sin, pos, seq_of, table, ps, k4, v4, nq, nkv,
                            in_ssq=ssq if fold else None, in_eps=eps_in, scratch=scratch)
        tc.check_status(DEV)
        assert torch.equal(k4 == UNWRITTEN, k1 == UNWRITTEN) and torch.equal(v4 == UNWRITTEN, v1 == UNWRITTEN)
        assert rel(q4, want) < 6e-3 and rel(q4, q2) < 6e-3
        assert rel(k4[wk], k2[wk]) < 6e-3 and rel(v4[wv], v2[wv]) < 6e-3
    if (M, K_) in ((600, 2048), (256, 4096)):
        assert need > 0              # these shapes are here because they split


@pytest.mark.parametrize("M,N,K_", [(256, 4096, 4096), (300, 520, 2048), (512, 1024, 8192), (200, 264, 1024),
                                    (1024, 768, 4096),
                                    # more tiles than CTA pairs: the full wave whole, the tiles of the last wave split
                                    (1280, 4096, 4096), (1100, 4200, 4096), (1536, 4096, 4096), (2560, 4096, 4096)])
def test_gemm_tcgen05_prefill_form_splits_k_when_it_has_few_tiles(M, N, K_):
    """A few hundred tokens give the CTA-pair form fewer tiles than there are pairs, or a last wave that is nearly
    empty; with scratch it splits K (of all tiles, or of the last wave's), leaves float32 partial tiles and a second
    kernel applies the output mode.  Every mode, against float64."""
    from gogguf_b200.csrc import tcgen05_gemm as tc
    g = torch.Generator(device=DEV).manual_seed(43)
    need = tc.pair_scratch_elems(M, N, K_)
    assert need > 0 and need % M == 0, "these shapes are meant to split"
    tiles = -(-M // 256) * -(-N // 256)
    assert (need % (M * N) == 0) == (tiles <= 74), "every tile is split where there are few, else only some tile columns"
    scratch = torch.full((need,), float("nan"), device=DEV)
    resid = torch.randn(M, K_, device=DEV, generator=g) * 2
    w = (torch.randn(N, K_, device=DEV, generator=g) / math.sqrt(K_)).to(torch.bfloat16)
    xh, ssq = plain_row_stats(resid)
    ssq = ssq.float().contiguous()
    eps = 1e-6
    factor = 1.0 / torch.sqrt((resid.double() ** 2).mean(-1, keepdim=True) + eps)
    plain_prod = xh.double() @ w.double().T
    tol = 3e-6 + 2e-7 * math.sqrt(K_)
    # plain float32 and bfloat16 stores, split against unsplit
    out = torch.full((M, N), float("nan"), device=DEV)
    tc.gemm_tc(xh, w, out, scratch=scratch, cluster=True)
    tc.check_status(DEV)
    assert rel(out, plain_prod) < tol
    unsplit = torch.empty(M, N, device=DEV)
    tc.gemm_tc(xh, w, unsplit, cluster=True)
    assert rel(out, unsplit) < tol
    if os.environ.get("GOGGUF_B200_GEMM_PAIR", "1") != "0":      # (the single-CTA form has no K split)
        assert not torch.equal(out, unsplit)
    ob = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    tc.gemm_tc(xh, w, ob, scratch=scratch, cluster=True)
    assert rel(ob, plain_prod) < 5e-3
    # folded norm in, residual add with row statistics out
    res = torch.randn(M, N, device=DEV, generator=g)
    acc = res.clone()
    oh = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    oss = torch.full((M, (N + 127) // 128), float("nan"), device=DEV)
    tc.gemm_tc_norm(xh, w, acc, accumulate=True, in_ssq=ssq, eps=eps, out_ssq=oss, out_xhat=oh, scratch=scratch)
    tc.check_status(DEV)
    assert rel(acc, res.double() + plain_prod * factor) < tol
    wh, ws_ = plain_row_stats(acc)
    assert torch.equal(oh, wh) and rel(oss, ws_) < 1e-6
    # fused SwiGLU
    if N % 128 == 0 and N >= 256:
        out_s = torch.full((M, N // 2), float("nan"), device=DEV, dtype=torch.bfloat16)
        tc.gemm_tc_norm(xh, w, out_s, swiglu=True, in_ssq=ssq, eps=eps, scratch=scratch)
        prod = (plain_prod * factor).view(M, N // 128, 2, 64)
        gd, ud = prod[:, :, 0], prod[:, :, 1]
        want = (gd / (1 + torch.exp(-gd)) * ud).reshape(M, N // 2)
        assert rel(out_s, want) < 6e-3


def test_linear_takes_the_split_scratch_from_the_workspace():
    from gogguf_b200.csrc import tcgen05_gemm as tc
    from gogguf_b200.parts.base import Linear, Runtime, Workspace
    g = torch.Generator(device=DEV).manual_seed(47)
    M, N, K_ = 300, 4096, 2048
    w = (torch.randn(N, K_, device=DEV, generator=g) / math.sqrt(K_)).to(torch.bfloat16)
    x = torch.randn(M, K_, device=DEV, generator=g).to(torch.bfloat16)
    lin = Linear(w, Runtime(dtype=torch.bfloat16, device=torch.device(DEV), fast=True))
    ws = Workspace(DEV)
    out = torch.empty(M, N, device=DEV)
    lin(x, out, ws=ws)
    tc.check_status(DEV)
    assert ("gemm_partial_tiles", torch.float32) in ws._bufs and tc.pair_scratch_elems(M, N, K_) > 0
    assert rel(out, x.double() @ w.double().T) < 3e-6 + 2e-7 * math.sqrt(K_)
    # without a workspace the same product runs unsplit
    out2 = torch.empty(M, N, device=DEV)
    lin(x, out2)
    assert rel(out2, out) < 1e-5


# ------------------------------------------------------------------------------------------ attention
def make_paged(seqs, nkv, d, dt, seed, n_pages=None, ps=64):
    """seqs: list of (context length after the step, new tokens).  Returns pools, table and per-sequence K, V."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    need = sum((c + ps - 1) // ps for c, _ in seqs)
    n_pages = n_pages or need + 3
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    width = max((c + ps - 1) // ps for c, _ in seqs) + 1
    kp = torch.randn(n_pages, nkv, ps, d, device=DEV, generator=g).to(dt)
    vp = torch.randn(n_pages, nkv, ps, d, device=DEV, generator=g).to(dt)
    table = torch.zeros(len(seqs), width, dtype=torch.int32)
    ks, vs = [], []
    for b, (c, _) in enumerate(seqs):
        pages = [perm.pop() for _ in range((c + ps - 1) // ps)]
        table[b, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
        k = torch.cat([kp[p] for p in pages], dim=1)[:, :c]        # [nkv, c, d]
        v = torch.cat([vp[p] for p in pages], dim=1)[:, :c]
        ks.append(k)
        vs.append(v)
    return kp, vp, table.to(DEV), ks, vs


def attention_reference(q, ks, vs, seqs, nq, nkv, scale, window):
    outs = []
    r = 0
    G = nq // nkv
    for b, (c, n) in enumerate(seqs):
        for i in range(n):
            pos = c - n + i
            lo = max(0, pos - window + 1) if window else 0
            for h in range(nq):
                k = ks[b][h // G, lo:pos + 1].double()
                v = vs[b][h // G, lo:pos + 1].double()
                s = (k @ q[r, h].double()) * scale
                outs.append(torch.softmax(s, 0) @ v)
            r += 1
    return torch.stack(outs).reshape(r, nq, -1)


def step_meta(seqs):
    pos, sot, cu, cl = [], [], [0], []
    for b, (c, n) in enumerate(seqs):
        pos += list(range(c - n, c))
        sot += [b] * n
        cu.append(cu[-1] + n)
        cl.append(c)
    mk = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return mk(pos), mk(sot), mk(cu), mk(cl)


ATT_CASES = [
    # nq, nkv, d, window, seqs [(context after the step, new tokens)]
    (4, 2, 16, 0, [(5, 5), (70, 3)]),
    (6, 1, 32, 0, [(130, 130), (1, 1), (64, 64)]),
    (3, 3, 48, 37, [(100, 100), (200, 1)]),
    (8, 2, 128, 0, [(300, 300), (65, 1), (129, 2)]),
    (8, 2, 64, 70, [(257, 257), (500, 7)]),
    (32, 8, 128, 0, [(1, 1), (200, 72)]),
]


@pytest.mark.parametrize("nq,nkv,d,window,seqs", ATT_CASES)
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_attention_plain(nq, nkv, d, window, seqs, dt):
    kp, vp, table, ks, vs = make_paged(seqs, nkv, d, dt, seed=7)
    pos, sot, cu, cl = step_meta(seqs)
    T = pos.numel()
    q = torch.randn(T, nq, d, device=DEV, generator=torch.Generator(device=DEV).manual_seed(8)).to(dt)
    out = torch.empty(T, nq, d, device=DEV, dtype=dt)
    scale = 1.0 / math.sqrt(d)
    K().attention_plain(q, kp, vp, out, pos, sot, table, 64, T, nq, nkv, d, scale, window)
    want = attention_reference(q, ks, vs, seqs, nq, nkv, scale, window)
    assert rel(out, want) < (3e-6 if dt == torch.float32 else 6e-3)


@pytest.mark.parametrize("nq,nkv,d,window,seqs", [c for c in ATT_CASES if c[2] in (64, 128)] + [
    (4, 1, 128, 0, [(2048, 2048)]), (16, 1, 64, 100, [(700, 330), (90, 90)])])
def test_attention_prefill_tensor_cores(nq, nkv, d, window, seqs):
    from gogguf_b200.csrc import fast_attention as fa
    dt = torch.bfloat16
    kp, vp, table, ks, vs = make_paged(seqs, nkv, d, dt, seed=9)
    pos, sot, cu, cl = step_meta(seqs)
    T = pos.numel()
    q = torch.randn(T, nq, d, device=DEV, generator=torch.Generator(device=DEV).manual_seed(10)).to(dt)
    out = torch.full((T, nq, d), float("nan"), device=DEV, dtype=dt)
    scale = 1.0 / math.sqrt(d)
    fa.attn_prefill(q, kp, vp, out, cu, cl, sot, table, 64, len(seqs), T // 64 + len(seqs), nq, nkv, d, scale, window)
    twin = torch.empty_like(out)
    K().attention_plain(q, kp, vp, twin, pos, sot, table, 64, T, nq, nkv, d, scale, window)
    want = attention_reference(q, ks, vs, seqs, nq, nkv, scale, window) if T <= 400 else twin
    assert rel(out, want) < 8e-3
    assert rel(out, twin) < 8e-3
    # the tcgen05 form (S and O in tensor memory)
    from gogguf_b200.csrc import tcgen05_gemm as tc
    out2 = torch.full((T, nq, d), float("nan"), device=DEV, dtype=dt)
    fa.attn_prefill_tc(q, kp, vp, out2, cu, cl, sot, table, 64, T, len(seqs), T // 128 + len(seqs), nq, nkv, d, scale, window)
    tc.check_status(DEV)
    assert rel(out2, want) < 8e-3
    assert rel(out2, twin) < 8e-3


@pytest.mark.parametrize("step", [5.0, 30.0, 140.0])
@pytest.mark.parametrize("window", [0, 150])
def test_attention_prefill_scores_that_grow_from_page_to_page(step, window):
    """The tensor-core prefill kernel computes a page with the maximum of the pages before it and looks for the
    page's own maximum only when the page's sum says that it must.  Here every page's scores lie `step` powers of
    two above those of the page before: within the margin that needs no rescaling (5), far beyond it but still
    representable (30), and beyond what a float holds (140), where the page has to be computed again."""
    from gogguf_b200.csrc import fast_attention as fa
    from gogguf_b200.csrc import tcgen05_gemm as tc
    dt = torch.bfloat16
    nq, nkv, d, n = 4, 1, 128, 384
    seqs = [(n, n)]
    kp, vp, table, _, vs = make_paged(seqs, nkv, d, dt, seed=31)
    pos, sot, cu, cl = step_meta(seqs)
    scale = 1.0 / math.sqrt(d)
    q = torch.randn(n, nq, d, device=DEV, generator=torch.Generator(device=DEV).manual_seed(32)).to(dt)
    q[:, :, 0] = 16.0
    # key t has (t // 64) * c in its first component: score * scale * log2(e) grows by `step` per page
    c = step / (16.0 * scale * 1.4426950408889634)
    pages = table[0].tolist()
    for t in range(n):
        kp[pages[t // 64], :, t % 64, 0] = (t // 64) * c
    ks = [torch.cat([kp[pg] for pg in pages[:n // 64]], dim=1)[:, :n]]
    want = attention_reference(q, ks, vs, seqs, nq, nkv, scale, window)
    out = torch.full((n, nq, d), float("nan"), device=DEV, dtype=dt)
    fa.attn_prefill_tc(q, kp, vp, out, cu, cl, sot, table, 64, n, 1, n // 128 + 1, nq, nkv, d, scale, window)
    tc.check_status(DEV)
    assert rel(out, want) < 8e-3


@pytest.mark.parametrize("nq,nkv,d,window,ctxs", [
    (8, 2, 128, 0, [1, 64, 65, 300, 2049]), (32, 8, 128, 0, [2048] * 3 + [17]), (8, 8, 64, 0, [100, 1000]),
    (16, 1, 64, 90, [500, 89, 90, 91]), (12, 2, 128, 33, [4000, 5])])
def test_attention_decode_tensor_cores(nq, nkv, d, window, ctxs):
    from gogguf_b200.csrc import fast_attention as fa
    dt = torch.bfloat16
    seqs = [(c, 1) for c in ctxs]
    kp, vp, table, ks, vs = make_paged(seqs, nkv, d, dt, seed=11)
    pos, sot, cu, cl = step_meta(seqs)
    # a padding row in the middle must change nothing and give zeros
    pos = torch.cat([pos[:1], torch.zeros(1, dtype=torch.int32, device=DEV), pos[1:]])
    sot = torch.cat([sot[:1], torch.full((1,), -1, dtype=torch.int32, device=DEV), sot[1:]])
    T = pos.numel()
    q = torch.randn(T, nq, d, device=DEV, generator=torch.Generator(device=DEV).manual_seed(12)).to(dt)
    scale = 1.0 / math.sqrt(d)
    qr = torch.cat([q[:1], q[2:]])
    want = attention_reference(qr, ks, vs, seqs, nq, nkv, scale, window)
    from gogguf_b200.csrc import tcgen05_gemm as tc
    for max_ctx in (max(ctxs), 8192):
        for form in ("direct", "tma", "tma_cluster"):
            if form == "direct":
                splits = fa.decode_splits(T, nkv, max_ctx)
            else:
                splits = fa.decode_tma_splits(T, nkv, max_ctx, cluster=form == "tma_cluster")
            po = torch.empty(T * nq * splits * d, device=DEV)
            pm = torch.empty(T * nq * splits * 2, device=DEV)
            out = torch.full((T, nq, d), float("nan"), device=DEV, dtype=dt)
            if form == "direct":
                fa.attn_decode(q, kp, vp, out, pos, sot, table, 64, T, nq, nkv, d, scale, window, splits, po, pm)
            elif form == "tma":
                fa.attn_decode_tma(q, kp, vp, out, pos, sot, table, 64, T, nq, nkv, d, scale, window, splits, po, pm)
            else:
                fa.attn_decode_tma(q, kp, vp, out, pos, sot, table, 64, T, nq, nkv, d, scale, window, splits, cluster=True)
            tc.check_status(DEV)
            got = torch.cat([out[:1], out[2:]])
            assert rel(got, want) < 8e-3, (form, splits)
            assert float(out[1].float().abs().sum()) == 0.0


@pytest.mark.parametrize("kind", ["plain_f32", "plain_bf16", "decode", "decode_tma", "prefill"])
def test_attention_finds_a_far_key_and_respects_the_window_edge(kind):
    """Random numbers hide a key that is skipped among hundreds.  Here one far key (and, for the
    window, the keys just inside and just outside its edge) is scaled so that it takes all the weight."""
    from gogguf_b200.csrc import fast_attention as fa
    dt = torch.float32 if kind == "plain_f32" else torch.bfloat16
    nq, nkv, d, ctx = 8, 2, 128, 900
    n_new = 1 if kind.startswith("decode") else 130
    seqs = [(ctx, n_new)]
    scale = 1.0 / math.sqrt(d)
    for window, hot in ((0, 3), (0, 447), (200, ctx - 200), (200, ctx - 201)):
        kp, vp, table, ks, vs = make_paged(seqs, nkv, d, dt, seed=13)
        pos, sot, cu, cl = step_meta(seqs)
        T = pos.numel()
        q = torch.randn(T, nq, d, device=DEV, generator=torch.Generator(device=DEV).manual_seed(14)).to(dt)
        # the last query token and the key at `hot` point the same way, strongly
        page, off = int(table[0, hot // 64]), hot % 64
        kp[page, :, off] = 0
        kp[page, :, off, 0] = 30.0
        q[-1, :, 0] = 30.0
        vp[page, :, off] = 5.0
        out = torch.empty(T, nq, d, device=DEV, dtype=dt)
        if kind.startswith("plain"):
            K().attention_plain(q, kp, vp, out, pos, sot, table, 64, T, nq, nkv, d, scale, window)
        elif kind == "decode":
            splits = fa.decode_splits(T, nkv, 1024)
            po = torch.empty(T * nq * splits * d, device=DEV); pm = torch.empty(T * nq * splits * 2, device=DEV)
            fa.attn_decode(q, kp, vp, out, pos, sot, table, 64, T, nq, nkv, d, scale, window, splits, po, pm)
        elif kind == "decode_tma":
            splits = fa.decode_tma_splits(T, nkv, 1024, cluster=True)
            assert splits > 1
            fa.attn_decode_tma(q, kp, vp, out, pos, sot, table, 64, T, nq, nkv, d, scale, window, splits, cluster=True)
        else:
            fa.attn_prefill(q, kp, vp, out, cu, cl, sot, table, 64, 1, T // 64 + 1, nq, nkv, d, scale, window)
        last = out[-1].float()
        inside = window == 0 or hot >= (ctx - 1) - window + 1
        if inside:
            assert float((last - 5.0).abs().max()) < 0.05, (window, hot)     # all weight on the hot key
        else:
            assert float(last.abs().max()) < 4.0, (window, hot)              # the hot key is outside the window


@pytest.mark.parametrize("nq,nkv,d,ctxs", [(8, 2, 128, [20000]), (8, 2, 128, [5000, 9000, 333]), (16, 4, 64, [9000]),
                                          (32, 8, 128, [20000, 70, 5000]), (4, 1, 128, [40000])])
def test_attention_decode_reads_every_page_of_a_long_context(nq, nkv, d, ctxs):
    """Among thousands of random keys a page that is skipped, or read twice, changes the output by less than
    the bfloat16 bound.  So every query head is given one key that takes all the weight (the key points where
    the head's query points, sixty times as long), each head its own, and from launch to launch these keys
    move on so that every page of every sequence is, once, the page that holds a head's only key.  The head's
    output must then be that position's value row.  Both through the sizes an eager step passes and through
    the bound a captured step passes (the page-table width rounded up to a power of two)."""
    from gogguf_b200.csrc import fast_attention as fa
    from gogguf_b200.csrc import tcgen05_gemm as tc
    dt = torch.bfloat16
    seqs = [(c, 1) for c in ctxs]
    kp, vp, table, ks, vs = make_paged(seqs, nkv, d, dt, seed=21)
    pos, sot, cu, cl = step_meta(seqs)
    T, G = len(ctxs), nq // nkv
    scale = 1.0 / math.sqrt(d)
    q = torch.randn(T, nq, d, device=DEV, generator=torch.Generator(device=DEV).manual_seed(22)).to(dt)
    run = fa.try_make(nq, nkv, d, scale, 0)
    n_pages = [(c + 63) // 64 for c in ctxs]
    width_bound = 64 * (1 << (max(n_pages) - 1).bit_length())
    rng = torch.Generator().manual_seed(23)
    launches = (max(n_pages) + nq - 1) // nq
    for r in range(launches):
        saved, expect = [], {}
        for b, c in enumerate(ctxs):
            for h in range(nq):
                pg = (r * nq + h) % n_pages[b]
                off = int(torch.randint(0, min(64, c - pg * 64), (1,), generator=rng))
                page = int(table[b, pg])
                if any(sv[0] == page and sv[1] == h // G and sv[2] == off for sv in saved):
                    continue                                   # two heads of a group drew the same place: the first keeps it
                saved.append((page, h // G, off, kp[page, h // G, off].clone()))
                qh = q[b, h].float()
                kp[page, h // G, off] = (60.0 * qh / qh.norm()).to(dt)
                expect[(b, h)] = vp[page, h // G, off].float()
        for max_ctx in (max(ctxs), width_bound):
            ctx = SimpleNamespace(n_tokens=T, n_seqs=T, decode=True, max_ctx=max_ctx, max_new=1, positions=pos,
                                  seq_of_token=sot, cu_seqlens=cu, ctx_lens=cl)
            out = torch.full((T, nq, d), float("nan"), device=DEV, dtype=dt)
            run(q, kp, vp, out, ctx, table, 64)
            tc.check_status(DEV)
            for (b, h), v in expect.items():
                err = float((out[b, h].float() - v).abs().max())
                assert err < 0.05, (r, b, h, max_ctx, err)
        for page, g, off, old in saved:
            kp[page, g, off] = old


def test_a_bounded_wait_that_runs_out_leaves_its_code_and_ends_the_kernel():
    """The time-out path of the kernels' mbarrier waits, run for its own sake: a barrier nothing arrives at, a
    limit of a millisecond.  The wait returns false, its code is in the status word, the abort flag is up, the
    second role left because of the flag long before its own limit, and the host's check raises."""
    from gogguf_b200.csrc import tcgen05_gemm as tc
    from gogguf_b200.csrc.build import KernelError
    word = torch.zeros(1, dtype=torch.int32, device=DEV)
    limit = 2_000_000
    rep = K().wait_probe(limit, 7, word).cpu().tolist()
    assert rep[0] == 0 and rep[1] == 0 and rep[4] == 1
    assert int(word.item()) == 7                               # the first code stays; the second role adds none
    assert limit // 1024 <= rep[2] < 50 * (limit // 1024)
    assert rep[3] < 100 * (limit // 1024)                      # not its own limit of a thousand times that
    word.fill_(3)
    K().wait_probe(limit, 7, word)
    assert int(word.item()) == 3                               # an earlier code is never overwritten
    K().wait_probe(limit, 2, tc.status_word(DEV))
    with pytest.raises(KernelError, match="code 2"):
        tc.check_status(DEV)
    tc.check_status(DEV)                                       # the word is clear again


def test_debug_build_checks_page_tables_instead_of_reading_out_of_range():
    """GOGGUF_B200_DEBUG=1 builds the kernels with checked page tables: the stand-in for a memory checker."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, GOGGUF_B200_DEBUG="1")
    env.pop("GOGGUF_B200_GEMM_PAIR", None)        # the script drives the CTA-pair q/k/v epilogue, whatever this run's switches
    p = subprocess.run([sys.executable, os.path.join(root, "tests", "debug_bounds_script.py"), root], env=env,
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and "debug bounds ok" in p.stdout, p.stdout[-2000:] + p.stderr[-4000:]


# ------------------------------------------------------------------------------------------ sampling chain
@pytest.mark.parametrize("temp,top_k,top_p,min_p", [(0.8, 20, 0.95, 0.0), (0.0, 3, 1.0, 0.0), (1.0, 1, 0.5, 0.0),
                                                     (1.3, 40, 0.6, 0.1), (0.6, 1000, 0.9, 0.0), (2.5, 64, 1.0, 0.3),
                                                     (0.7, 5000, 0.8, 0.0)])
def test_sampling_chain_with_top_k_on_device(temp, top_k, top_p, min_p):
    """The device chain against the host chain (which tests/test_sampling.py holds to the plain sampler),
    on rows with distinct values and on rows made of a few values only, so that the k-th place falls among
    equal logits and the lower ids must win."""
    import numpy as np
    from gogguf_b200.sampling.sampler import SamplerConfig, sample_host, uniform01
    V = (20011 if top_k in (20, 40) else 4099) if top_k <= 1024 else 600     # 20011: three slices in stage one
    if top_k > 1024:
        top_k = 1024                                   # with V = 600: every id survives the top-k
    rows = 16
    g = torch.Generator().manual_seed(7)
    logits = torch.randn(rows, V, generator=g) * 4
    logits[4:8] = torch.round(logits[4:8] * 2) / 2      # many ties
    logits[8:10] = torch.round(logits[8:10])            # a handful of values
    logits[10] = 1.5                                    # all equal
    logits[11, ::7] = 30.0                              # equal maxima
    cfg = SamplerConfig(temp=temp, top_k=top_k, top_p=top_p, min_p=min_p, seed=3)
    assert cfg.device_chain
    for step in range(3):
        us = [uniform01(3, r, step) for r in range(rows)]
        out = torch.full((rows,), -7, dtype=torch.int32, device=DEV)
        K().sample_topk(logits.to(DEV), temp, top_k, top_p, min_p, torch.tensor(us, dtype=torch.float64, device=DEV), out)
        want = [sample_host(logits[r].numpy(), cfg, us[r]) for r in range(rows)]
        assert out.cpu().tolist() == want, step


@pytest.mark.parametrize("V", [331, 5000, 40000])
def test_temperature_sampling_and_argmax_on_device(V):
    """One block per row for short rows, several blocks per row from 16,384 ids on; both against the host chain.
    A row with temperature 0 is greedy: the first maximum."""
    from gogguf_b200.sampling.sampler import SamplerConfig, sample_host, uniform01
    rows = 9
    g = torch.Generator().manual_seed(11)
    logits = torch.randn(rows, V, generator=g) * 3
    logits[3, V // 2] = logits[3, V - 5] = 25.0            # equal maxima: greedy takes the first
    temps = [0.7, 1.0, 1.9, 0.0, 0.3, 5.0, 0.0, 1.2, 0.05]
    for step in range(4):
        us = [uniform01(5, r, step) for r in range(rows)]
        out = torch.full((rows,), -7, dtype=torch.int32, device=DEV)
        K().sample(logits.to(DEV), torch.tensor(temps, device=DEV), torch.tensor(us, dtype=torch.float64, device=DEV), out)
        want = [sample_host(logits[r].numpy(), SamplerConfig(temp=temps[r]), us[r]) for r in range(rows)]
        assert out.cpu().tolist() == want, step
    am = torch.empty(rows, dtype=torch.int32, device=DEV)
    K().argmax(logits.to(DEV), am)
    assert am.cpu().tolist() == logits.argmax(dim=1).tolist() and am[3].item() == V // 2


@pytest.mark.parametrize("temp,top_p,min_p", [(0.8, 0.9, 0.0), (1.0, 0.5, 0.0), (0.7, 1.0, 0.05), (1.2, 0.95, 0.02),
                                              (40.0, 0.9, 0.0), (30.0, 1.0, 0.5)])
def test_top_p_and_min_p_without_top_k_on_device(temp, top_p, min_p):
    """The kernel answers from the 1,024 largest logits of a row and flags the rows whose answer may lie beyond
    them (a flat distribution: the last two cases); unflagged rows equal the host chain, and through the sampler
    every row does."""
    from gogguf_b200.sampling.sampler import Sampler, SamplerConfig, sample_host, uniform01
    V, rows = 20011, 12
    g = torch.Generator().manual_seed(17)
    logits = torch.randn(rows, V, generator=g) * 3
    logits[5] = torch.round(logits[5])                  # ties
    logits[6, 100:140] = 9.0                            # a plateau at the top
    cfg = SamplerConfig(temp=temp, top_p=top_p, min_p=min_p, seed=8)
    assert not cfg.on_device
    dl = logits.to(DEV)
    for step in range(3):
        us = [uniform01(8, r, step) for r in range(rows)]
        out = torch.full((rows,), -7, dtype=torch.int32, device=DEV)
        flags = torch.full((rows,), -7, dtype=torch.int32, device=DEV)
        K().sample_nucleus(dl, temp, top_p, min_p, torch.tensor(us, dtype=torch.float64, device=DEV), out, flags)
        want = [sample_host(logits[r].numpy(), cfg, us[r]) for r in range(rows)]
        got, fl = out.cpu().tolist(), flags.cpu().tolist()
        assert all(f in (0, 1) for f in fl)
        assert all(g_ == w for g_, w, f in zip(got, want, fl) if not f), step
        if temp >= 30:
            assert sum(fl) == rows          # nothing is certain from 1,024 of 20,011 nearly equal probabilities
        else:
            assert sum(fl) == 0
        assert Sampler(cfg).sample(dl, streams=list(range(rows)), steps=[step] * rows) == want
