"""Each part alone against the plain implementation, and a toy mixer with state of its own that is
defined here, registered, built into a model and stepped without any change to the package."""
import math
from dataclasses import replace
from types import SimpleNamespace

import pytest
import torch

import plain_qwen3 as plain
from helpers import TINY_B, TINY_M, TOL_BF16, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def runtime(dtype):
    from gogguf_b200.parts.base import Runtime
    return Runtime(dtype=dtype, device=torch.device(DEV), fast=True)


def part_context(rt, cache, entries):
    """A step context for parts run outside a model: the stepper's own packing, with a bare model."""
    from gogguf_b200.engine.step import Stepper
    st = Stepper(SimpleNamespace(rt=rt, spec=None), cache)
    cache.plan([e.slot for e in entries], [len(e.tokens) for e in entries])
    ctx, lay, rows = st.build_context(entries)
    return ctx, st


def rand(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_position_embedding_head_alone(dtype):
    from gogguf_b200.config import PartSpec
    from gogguf_b200.parts import registry as R
    rt = runtime(dtype)
    tol = 3e-6 if dtype == torch.float32 else 6e-3
    # norm
    w = 1 + rand((72,), 1, 0.1)
    norm = R.NORMS["rmsnorm"](PartSpec("rmsnorm", dict(size=72, eps=3e-6)), {"weight": w}, rt)
    x = rand((9, 72), 2, 2.0).to(DEV)
    out = torch.empty(9, 72, device=DEV, dtype=dtype)
    norm.forward(x, out)
    assert rel_err(out, plain.rms_norm(x.cpu(), w, 3e-6, wide=True)) < tol
    # position tables
    rope = R.POSITIONS["rope_neox"](dict(theta=50000.0, rotary_dim=48), rt)
    from gogguf_b200.parts.base import StepContext, Workspace
    pos = torch.tensor([0, 5, 900], dtype=torch.int32, device=DEV)
    ctx = SimpleNamespace(ws=Workspace(DEV), n_tokens=3, positions=pos, shared={})
    cos, sin = rope.tables(ctx)
    pc, ps_ = plain.rope_tables([0, 5, 900], 48, 50000.0)
    assert float((cos.cpu().double() - pc).abs().max()) < 1e-7 and float((sin.cpu().double() - ps_).abs().max()) < 1e-7
    assert rope.tables(ctx)[0] is cos        # computed once per step
    # embedding and head (tied)
    table = rand((331, 72), 3, 0.5)
    emb = R.EMBEDDINGS["embedding"](PartSpec("embedding", dict(vocab_size=331, hidden_size=72)), {"weight": table.to(dtype)}, rt)
    toks = torch.tensor([3, 330, 0], dtype=torch.int32, device=DEV)
    xe = torch.empty(3, 72, device=DEV)
    emb.forward(toks, xe)
    assert torch.equal(xe.cpu(), plain.embed(table.to(dtype).float(), [3, 330, 0]))
    head = R.HEADS["linear_head"](PartSpec("linear_head", dict(vocab_size=331, hidden_size=72, tied_to="x")), {}, rt, tied=emb.weight)
    hin = rand((3, 72), 4).to(DEV).to(dtype)
    logits = torch.empty(3, 331, device=DEV)
    head.forward(hin, logits, SimpleNamespace(ws=Workspace(DEV)))
    assert rel_err(logits, hin.cpu().double() @ table.to(dtype).double().T) < (3e-6 if dtype == torch.float32 else 1e-5)


@pytest.mark.parametrize("dtype,cfg", [(torch.float32, TINY_B), (torch.bfloat16, TINY_M)])
def test_mixer_feed_forward_and_block_alone(dtype, cfg):
    from gogguf_b200.cache import SequenceCache
    from gogguf_b200.config import config_from_dict
    from gogguf_b200.engine.step import StepEntry
    from gogguf_b200.parts import registry as R
    rt = runtime(dtype)
    tol = 2e-5 if dtype == torch.float32 else TOL_BF16
    spec = config_from_dict(cfg).to_spec()
    c = plain.plain_config(cfg)
    layer = 1
    b = spec.blocks[layer]
    H = cfg["hidden_size"]
    mcls, fcls = R.MIXERS[b.mixer.kind], R.FEED_FORWARDS[b.feed_forward.kind]
    mw = {k: (rand(d.shape, 10 + i, 0.08) if d.init == "normal" else 1 + rand(d.shape, 10 + i, 0.05)).to(dtype)
          for i, (k, d) in enumerate(mcls.tensors(b.mixer).items())}
    fw = {k: rand(d.shape, 30 + i, 0.08).to(dtype) for i, (k, d) in enumerate(fcls.tensors(b.feed_forward).items())}
    nw = {"weight": (1 + rand((H,), 40, 0.05)).to(dtype)}
    mixer, ffn = mcls(b.mixer, mw, rt), fcls(b.feed_forward, fw, rt)
    norm1 = R.NORMS["rmsnorm"](b.mixer_norm, nw, rt)
    norm2 = R.NORMS["rmsnorm"](b.feed_forward_norm, nw, rt)

    cache = SequenceCache([mcls.cache_request(b.mixer)], [None], 1024, dtype=dtype, device=DEV)
    lens = [70, 3]
    slots = [cache.open() for _ in lens]
    entries = [StepEntry(s, [0] * n) for s, n in zip(slots, lens)]
    ctx, st = part_context(rt, cache, entries)
    T = sum(lens)
    h = rand((T, H), 50).to(dtype)
    x0 = rand((T, H), 51)
    pw = {("P." + k): v.float() for k, v in mw.items()}
    window = b.mixer.get("window")
    # mixer alone: adds its output into the residual
    res = x0.clone().to(DEV)
    mixer.prepare(ctx)
    mixer.forward(h.to(DEV), res, ctx, cache.view(0), True)
    want, r = [], 0
    for n in lens:
        want.append(plain.attention_mixer(h[r:r + n].float(), pw, "P.", c, list(range(n)), window, wide=True))
        r += n
    assert rel_err(res.cpu().double() - x0.double(), torch.cat(want)) < tol
    # feed-forward alone
    res = x0.clone().to(DEV)
    ffn.forward(h.to(DEV), res, ctx)
    wantf = plain.swiglu_ffn(h.float(), fw["gate_proj.weight"].float(), fw["up_proj.weight"].float(),
                             fw["down_proj.weight"].float(), wide=True)
    assert rel_err(res.cpu().double() - x0.double(), wantf) < tol
    # the whole block (same positions, so the cache rows are simply written again); on the fast path the
    # arrangement hands its norms to the parts, which from then on read the raw rows and their statistics
    block = R.ARRANGEMENTS[b.arrangement](b, dict(mixer=mixer, feed_forward=ffn, mixer_norm=norm1, feed_forward_norm=norm2), rt)
    assert block.mixer_folded == block.feed_forward_folded == (dtype == torch.bfloat16)
    xb = x0.clone().to(DEV)
    block.forward(xb, ctx, cache.view(0), True)
    allw = {f"model.layers.{layer}.self_attn.{k}": v.float() for k, v in mw.items()}
    allw.update({f"model.layers.{layer}.mlp.{k}": v.float() for k, v in fw.items()})
    allw[f"model.layers.{layer}.input_layernorm.weight"] = nw["weight"].float()
    allw[f"model.layers.{layer}.post_attention_layernorm.weight"] = nw["weight"].float()
    wantb, r = [], 0
    for n in lens:
        wantb.append(plain.block(x0[r:r + n].double(), allw, layer, c, list(range(n)), wide=True))
        r += n
    assert rel_err(xb, torch.cat(wantb)) < tol


# --------------------------------------------------------------------------------------------- toy mixer
def register_toy():
    """A mixer with a fixed-size state per sequence: the running sum of its inputs and their count.
    Output for a token = W . mean(inputs of its sequence so far, itself included).  Written with
    torch ops; it exists only in this test."""
    from gogguf_b200.cache import StateRequest
    from gogguf_b200.parts import registry as R
    from gogguf_b200.weights import TensorDecl
    if "toy_running_mean" in R.MIXERS:
        return R.MIXERS["toy_running_mean"]

    @R.register_mixer("toy_running_mean")
    class RunningMean:
        @classmethod
        def tensors(cls, spec):
            return {"mix.weight": TensorDecl(shape=(spec["hidden_size"], spec["hidden_size"]))}

        @classmethod
        def cache_request(cls, spec):
            return StateRequest(shape=(spec["hidden_size"] + 1,), dtype=torch.float32)

        def __init__(self, spec, weights, rt):
            self.w = weights["mix.weight"].to(rt.device).float()

        def forward(self, h, residual, ctx, cache, writes_cache=True):
            cu = ctx.cu_seqlens.cpu().tolist()
            slots = ctx.slots.cpu().tolist()
            sot = ctx.seq_of_token.cpu().tolist()
            hf = h.float()
            for b in range(ctx.n_seqs):
                a, e = cu[b], cu[b + 1]
                if sot[a] < 0:
                    continue
                st = cache.state[slots[b]]
                sums = st[:-1] + torch.cumsum(hf[a:e], 0)
                counts = st[-1] + torch.arange(1, e - a + 1, device=h.device, dtype=torch.float32)
                residual[a:e] += (sums / counts[:, None]) @ self.w.T
                if writes_cache:
                    st[:-1] = sums[-1]
                    st[-1] = counts[-1]

    return RunningMean


def toy_spec():
    from gogguf_b200.config import PartSpec, ScheduleEntry, config_from_dict
    spec = config_from_dict(TINY_B).to_spec()
    H = TINY_B["hidden_size"]
    blocks = list(spec.blocks)
    blocks[1] = blocks[1].with_part("mixer", PartSpec("toy_running_mean", dict(hidden_size=H), prefix="model.layers.1.toy."))
    # order as data: layer 0, the toy layer, layer 2, then layer 0 again reading the cache its first run wrote
    schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2), ScheduleEntry(0, cache_of=0))
    return replace(spec, blocks=tuple(blocks), schedule=schedule)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_is_registered_built_and_stepped(dtype):
    from gogguf_b200.cache import StateView
    from gogguf_b200.engine import Model, StepEntry, Stepper
    from gogguf_b200.engine.model import expected_tensors
    from gogguf_b200.weights import random_tensors
    register_toy()
    spec = toy_spec()
    exp = expected_tensors(spec)
    assert "model.layers.1.toy.mix.weight" in exp and "model.layers.1.self_attn.q_proj.weight" not in exp
    tensors = random_tensors(exp, seed=3, std=0.05, norm_std=0.05, dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    model = Model(spec, tensors, dtype=dtype)
    cache = model.new_cache(max_tokens=64 * 6, max_slots=3)
    assert isinstance(cache.view(1), StateView) and cache.view(3) is cache.view(0) and len(cache.groups) == 1
    assert cache.groups[0].k.shape[0] == 2          # layers 0 and 2 own storage; the second run of layer 0 does not
    st = Stepper(model, cache)
    V = spec.vocab_size
    g = torch.Generator().manual_seed(5)
    seqs = [torch.randint(0, V, (n,), generator=g).tolist() for n in (40, 9, 23)]
    tol = 2e-5 if dtype == "float32" else TOL_BF16

    def whole(t):
        s = cache.open()
        out = st.step([StepEntry(s, t, want=list(range(len(t))))]).clone()
        cache.close(s)
        return out

    ref = [whole(t) for t in seqs]
    # token by token: the state carries the sequence from step to step
    s = cache.open()
    for i, tok in enumerate(seqs[0]):
        got = st.step([StepEntry(s, [tok], want=[0])])
        assert rel_err(got, ref[0][i:i + 1]) < tol, i
    cache.close(s)
    # unequal batch, shorter ones end earlier, then the slots are used again: the state must start from zero
    for rnd in range(2):
        slots = [cache.open() for _ in seqs]
        pre = [len(t) - 5 for t in seqs]
        got = st.step([StepEntry(sl, t[:p], want=[p - 1]) for sl, t, p in zip(slots, seqs, pre)])
        for j in range(3):
            assert rel_err(got[j:j + 1], ref[j][pre[j] - 1:pre[j]]) < tol
        for k in range(5):
            got = st.step([StepEntry(sl, [t[p + k]], want=[0]) for sl, t, p in zip(slots, seqs, pre)])
            for j in range(3):
                assert rel_err(got[j:j + 1], ref[j][pre[j] + k:pre[j] + k + 1]) < tol, (rnd, j, k)
        for sl in slots:
            cache.close(sl)
        cache.check()
    # the toy mixer itself against a direct computation
    x = torch.randn(7, TINY_B["hidden_size"], generator=g)
    w = tensors["model.layers.1.toy.mix.weight"].float()
    want = (torch.cumsum(x, 0) / torch.arange(1, 8)[:, None]) @ w.T
    mixer = model.blocks[1].mixer
    s = cache.open()
    from gogguf_b200.engine.step import StepEntry as SE
    cache.plan([s], [7])
    ctx, _, _ = st.build_context([SE(s, [0] * 7)])
    res = torch.zeros(7, TINY_B["hidden_size"], device=DEV)
    mixer.forward(x.to(DEV), res, ctx, cache.view(1), True)
    assert rel_err(res, want) < 1e-5
    cache.close(s)


# --------------------------------------------------------------------------------------------- more toy parts
def register_toy_router_and_position():
    """A feed-forward with routing (router logits in float32, top-2 of 4 small experts, weights renormalised)
    and a position encoding that is not rotary (a learned-free sinusoid added to q and k before the scores),
    both defined here only, to show that the registries take parts the package has never seen."""
    from gogguf_b200.parts import registry as R
    from gogguf_b200.weights import TensorDecl
    if "toy_routed" in R.FEED_FORWARDS:
        return

    @R.register_feed_forward("toy_routed")
    class Routed:
        @classmethod
        def tensors(cls, spec):
            h, e, i = spec["hidden_size"], spec["experts"], spec["expert_size"]
            t = {"router.weight": TensorDecl(shape=(e, h))}
            for k in range(e):
                t[f"experts.{k}.up.weight"] = TensorDecl(shape=(i, h))
                t[f"experts.{k}.down.weight"] = TensorDecl(shape=(h, i))
            return t

        def __init__(self, spec, weights, rt):
            self.e, self.k = spec["experts"], spec["top_k"]
            self.router = weights["router.weight"].to(rt.device).float()
            self.up = [weights[f"experts.{j}.up.weight"].to(rt.device).float() for j in range(self.e)]
            self.down = [weights[f"experts.{j}.down.weight"].to(rt.device).float() for j in range(self.e)]

        def forward(self, h, residual, ctx):
            x = h.float()
            logits = x @ self.router.T                                  # router logits in float32
            top, idx = torch.topk(logits, self.k, dim=-1)
            gate = torch.softmax(top, dim=-1)
            out = torch.zeros_like(x)
            for j in range(self.e):
                for slot in range(self.k):
                    m = idx[:, slot] == j
                    if bool(m.any()):
                        out[m] += gate[m, slot, None] * (torch.relu(x[m] @ self.up[j].T) @ self.down[j].T)
            pad = (ctx.seq_of_token < 0)
            out[pad] = 0
            residual += out

    @R.register_position("toy_additive_sinusoid")
    class AdditiveSinusoid:
        """tables(ctx) returns (cos, sin) as the attention mixer expects, but built so that the 'rotation'
        is the identity and nothing depends on the position: with it the model is permutation-blind within
        the causal mask, which the test checks."""

        def __init__(self, params, rt):
            self.rotary_dim = int(params["rotary_dim"])
            self.key = ("toy_additive_sinusoid", self.rotary_dim)

        def tables(self, ctx):
            got = ctx.shared.get(self.key)
            if got is None:
                half = self.rotary_dim // 2
                cos = ctx.ws.get("toy_cos", (ctx.n_tokens, half), torch.float32)
                sin = ctx.ws.get("toy_sin", (ctx.n_tokens, half), torch.float32)
                cos.fill_(1.0)
                sin.zero_()
                got = ctx.shared[self.key] = (cos, sin)
            return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_routed_feed_forward_and_other_position_encoding(dtype):
    from gogguf_b200.config import PartSpec, config_from_dict
    from gogguf_b200.engine import Model, StepEntry, Stepper
    from gogguf_b200.engine.model import expected_tensors
    from gogguf_b200.weights import random_tensors
    register_toy_router_and_position()
    spec = config_from_dict(TINY_B).to_spec()
    H = TINY_B["hidden_size"]
    blocks = list(spec.blocks)
    blocks[0] = blocks[0].with_part("feed_forward", PartSpec(
        "toy_routed", dict(hidden_size=H, experts=4, top_k=2, expert_size=40), prefix="model.layers.0.moe."))
    mixer2 = blocks[2].mixer
    blocks[2] = blocks[2].with_part("mixer", PartSpec(
        mixer2.kind, {**mixer2.params, "position": {"kind": "toy_additive_sinusoid", "rotary_dim": TINY_B["head_dim"]}},
        prefix=mixer2.prefix))
    spec = replace(spec, blocks=tuple(blocks))
    exp = expected_tensors(spec)
    assert "model.layers.0.moe.router.weight" in exp and "model.layers.0.mlp.gate_proj.weight" not in exp
    tensors = random_tensors(exp, seed=4, std=0.08, norm_std=0.05,
                             dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    model = Model(spec, tensors, dtype=dtype)
    cache = model.new_cache(512)
    st = Stepper(model, cache)
    g = torch.Generator().manual_seed(6)
    toks = torch.randint(0, spec.vocab_size, (50,), generator=g).tolist()
    s = cache.open()
    whole = st.step([StepEntry(s, toks, want=list(range(len(toks))))]).clone()
    cache.close(s)
    # whole == chunked == token by token, through the toy parts as through the built-in ones
    tol = 2e-5 if dtype == "float32" else TOL_BF16
    s = cache.open()
    got = [st.step([StepEntry(s, toks[:20], want=list(range(20)))]).clone()]
    got.append(st.step([StepEntry(s, toks[20:37], want=list(range(17)))]).clone())
    for t in toks[37:]:
        got.append(st.step([StepEntry(s, [t], want=[0])]).clone())
    cache.close(s)
    got = torch.cat(got)
    for i in range(len(toks)):
        assert rel_err(got[i:i + 1], whole[i:i + 1]) < tol, i
    cache.check()
