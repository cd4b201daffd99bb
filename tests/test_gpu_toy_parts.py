"""How far the description of a model as data reaches, shown with toy parts that exist only in this file:
an arrangement with four norms per layer, an arrangement without a feed-forward, a per-token cache that is
not a key/value pair (its request class and store are registered here), a mixer that cannot be captured in
a CUDA graph going through the entry point's generation loop, and a position encoding that is a scaled,
partial rotation.  Nothing in the package is changed for any of them, and none of them is a model of
anyone's: each is checked against a few lines of plain arithmetic written beside it."""
from dataclasses import dataclass, replace

import pytest
import torch

import plain_qwen3 as plain
from helpers import TINY_B, TINY_L, TOL_BF16, TOL_F32, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


# ------------------------------------------------------------------------------------------------ toy parts
def register_toys():
    from gogguf_b200.cache import PagedStore, register_cache_store
    from gogguf_b200.parts import registry as R
    from gogguf_b200.weights import TensorDecl
    if "toy_sandwich" in R.ARRANGEMENTS:
        return

    @R.register_arrangement("toy_sandwich")
    class Sandwich:
        """x += norm_out(part(norm_in(x))) for the mixer and for the feed-forward: four norms a layer.
        A part adds into the float32 buffer it is given, so it is handed a zeroed one."""
        roles = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "mixer_out_norm": "norm",
                 "feed_forward_norm": "norm", "feed_forward_out_norm": "norm"}

        def __init__(self, spec, parts, rt):
            self.parts, self.rt = dict(parts), rt

        def _around(self, x, ctx, norm_in, norm_out, run):
            T, H = x.shape
            h = ctx.ws.get("toy_h", (T, H), self.rt.dtype)
            tmp = ctx.ws.get("toy_tmp", (T, H), torch.float32)
            o = ctx.ws.get("toy_o", (T, H), self.rt.dtype)
            norm_in.forward(x, h)
            tmp.zero_()
            run(h, tmp)
            norm_out.forward(tmp, o)
            x += o.float()

        def forward(self, x, ctx, cache, writes_cache):
            p = self.parts
            self._around(x, ctx, p["mixer_norm"], p["mixer_out_norm"],
                         lambda h, out: p["mixer"].forward(h, out, ctx, cache, writes_cache))
            self._around(x, ctx, p["feed_forward_norm"], p["feed_forward_out_norm"],
                         lambda h, out: p["feed_forward"].forward(h, out, ctx))

    @R.register_arrangement("toy_mixer_only")
    class MixerOnly:
        """x += mixer(norm(x)): a layer without a feed-forward."""
        roles = {"mixer": "mixer", "mixer_norm": "norm"}

        def __init__(self, spec, parts, rt):
            self.parts, self.rt = dict(parts), rt

        def forward(self, x, ctx, cache, writes_cache):
            h = ctx.ws.get("toy_h", tuple(x.shape), self.rt.dtype)
            self.parts["mixer_norm"].forward(x, h)
            self.parts["mixer"].forward(h, x, ctx, cache, writes_cache)

    @dataclass(frozen=True)
    class LatentRequest:
        dim: int

    @dataclass
    class LatentView:
        group: int
        lat: torch.Tensor          # [page][page_size][dim]
        page_size: int

    @register_cache_store(LatentRequest)
    class LatentStore(PagedStore):
        """One float32 vector of `dim` numbers per token and layer, in pages: not keys and values."""

        @staticmethod
        def group_key(request):
            return request

        def __init__(self, request, entries, n_pages, page_size, dtype, device, max_slots=0):
            super().__init__(request, entries, n_pages, page_size)
            self.lat = torch.zeros(len(entries), n_pages, page_size, request.dim, dtype=torch.float32, device=device)

        def view(self, entry):
            return LatentView(self.index, self.lat[self.entries.index(entry)], self.page_size)

    @R.register_mixer("toy_latent_mean")
    class LatentMean:
        """Caches c_t = Wc h_t per token; output for a token = Wo mean(c_0..c_t).  It reads sizes back to
        the host, so it says that it cannot be captured."""
        capturable = False
        request_cls = LatentRequest

        @classmethod
        def tensors(cls, spec):
            h, c = spec["hidden_size"], spec["latent"]
            return {"down.weight": TensorDecl(shape=(c, h)), "up.weight": TensorDecl(shape=(h, c))}

        @classmethod
        def cache_request(cls, spec):
            return LatentRequest(dim=int(spec["latent"]))

        def __init__(self, spec, weights, rt):
            self.wc = weights["down.weight"].to(rt.device).float()
            self.wo = weights["up.weight"].to(rt.device).float()

        def forward(self, h, residual, ctx, cache, writes_cache=True):
            ps = cache.page_size
            table = ctx.page_tables[cache.group].long()
            pos, sot = ctx.positions.long(), ctx.seq_of_token.long()
            live = sot >= 0
            c = h.float() @ self.wc.T
            if writes_cache:
                page = table[sot.clamp_min(0), pos // ps]
                cache.lat[page[live], (pos % ps)[live]] = c[live]
            cu, lens = ctx.cu_seqlens.cpu().tolist(), ctx.ctx_lens.cpu().tolist()
            for b in range(ctx.n_seqs):
                a, e, n = cu[b], cu[b + 1], lens[b]
                if n == 0:
                    continue
                held = cache.lat[table[b, :(n + ps - 1) // ps]].reshape(-1, c.shape[1])[:n]
                means = torch.cumsum(held, 0) / torch.arange(1, n + 1, device=h.device)[:, None]
                residual[a:e] += means[pos[a:e]] @ self.wo.T

    @R.register_position("toy_scaled_partial_rope")
    class ScaledPartialRope:
        """Rotation of the first `rotary_dim` elements of a head by angle (pos / factor) * theta^(-2i/rotary_dim),
        with cos and sin multiplied by `magnitude`: positions are interpolated and q, k grow a little.  It keeps
        the contract of a position part: per-step tables of [tokens, rotary_dim / 2] for a rotation of pairs
        (i, i + rotary_dim/2)."""

        def __init__(self, params, rt):
            self.rot, self.theta = int(params["rotary_dim"]), float(params["theta"])
            self.factor, self.magnitude = float(params["factor"]), float(params["magnitude"])
            self.key = ("toy_scaled_partial_rope", self.rot, self.theta, self.factor, self.magnitude)

        def tables(self, ctx):
            got = ctx.shared.get(self.key)
            if got is None:
                half = self.rot // 2
                inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64),
                                -2.0 * torch.arange(half, dtype=torch.float64) / self.rot).to(ctx.positions.device)
                ang = (ctx.positions.double() / self.factor)[:, None] * inv[None, :]
                cos = ctx.ws.get("toy_spr_cos", (ctx.n_tokens, half), torch.float32)
                sin = ctx.ws.get("toy_spr_sin", (ctx.n_tokens, half), torch.float32)
                cos.copy_(torch.cos(ang) * self.magnitude)
                sin.copy_(torch.sin(ang) * self.magnitude)
                got = ctx.shared[self.key] = (cos, sin)
            return got


def build(spec, dtype, seed, std=0.06):
    from gogguf_b200.engine import Model
    from gogguf_b200.engine.model import expected_tensors
    from gogguf_b200.weights import random_tensors
    exp = expected_tensors(spec)
    tensors = random_tensors(exp, seed=seed, std=std, norm_std=0.05,
                             dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    host = {k: v.float().cpu() for k, v in tensors.items()}
    return Model(spec, tensors, dtype=dtype), host, exp


def whole_chunked_decoded(model, toks, tol):
    """The same tokens whole, in chunks and one by one, with a slot that is used again in between."""
    from gogguf_b200.engine import StepEntry, Stepper
    cache = model.new_cache(64 * 4, max_slots=2)
    st = Stepper(model, cache)
    s = cache.open()
    whole = st.step([StepEntry(s, toks, want=list(range(len(toks))))]).clone()
    cache.close(s)
    s = cache.open()
    a, b = len(toks) // 3, 2 * len(toks) // 3
    got = [st.step([StepEntry(s, toks[:a], want=list(range(a)))]).clone(),
           st.step([StepEntry(s, toks[a:b], want=list(range(b - a)))]).clone()]
    for t in toks[b:]:
        got.append(st.step([StepEntry(s, [t], want=[0])]).clone())
    cache.close(s)
    cache.check()
    got = torch.cat(got)
    for i in range(len(toks)):
        assert rel_err(got[i:i + 1], whole[i:i + 1]) < tol, i
    return whole


def head_of(x, w, c):
    h = plain.rms_norm(x, w["model.norm.weight"], c["eps"], wide=True)
    return h @ w["lm_head.weight"].double().T


def tokens(vocab, n, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


# ------------------------------------------------------------------------------------------------ tests
def test_blocks_with_four_norms_and_without_a_feed_forward_are_data():
    from gogguf_b200.config import BlockSpec, PartSpec, config_from_dict
    from gogguf_b200.engine.model import expected_tensors
    register_toys()
    spec = config_from_dict(TINY_B).to_spec()
    H, eps = TINY_B["hidden_size"], TINY_B["rms_norm_eps"]
    blocks = list(spec.blocks)
    norm = lambda name: PartSpec("rmsnorm", dict(size=H, eps=eps), prefix=f"model.layers.0.{name}.")   # noqa: E731
    blocks[0] = (blocks[0].with_arrangement("toy_sandwich")
                 .with_part("mixer_out_norm", norm("after_attention"))
                 .with_part("feed_forward_out_norm", norm("after_mlp")))
    blocks[2] = BlockSpec("toy_mixer_only", mixer=blocks[2].mixer, mixer_norm=blocks[2].mixer_norm)
    spec = replace(spec, blocks=tuple(blocks))
    model, w, exp = build(spec, "float32", seed=21)
    assert "model.layers.0.after_mlp.weight" in exp and "model.layers.2.mlp.down_proj.weight" not in exp
    assert "model.layers.2.post_attention_layernorm.weight" not in exp
    toks = tokens(spec.vocab_size, 45, 1)
    got = whole_chunked_decoded(model, toks, TOL_F32)
    # the same three layers from the plain parts
    c = plain.plain_config(TINY_B)
    pos = list(range(len(toks)))
    x = plain.embed(w["model.embed_tokens.weight"], toks).double()
    p = "model.layers.0."
    a = plain.attention_mixer(plain.rms_norm(x, w[p + "input_layernorm.weight"], eps, True), w, p + "self_attn.", c,
                              pos, None, wide=True)
    x = x + plain.rms_norm(a, w[p + "after_attention.weight"], eps, True)
    f = plain.swiglu_ffn(plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], eps, True),
                         w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"], True)
    x = x + plain.rms_norm(f, w[p + "after_mlp.weight"], eps, True)
    x = plain.block(x, w, 1, c, pos, wide=True)
    p = "model.layers.2."
    x = x + plain.attention_mixer(plain.rms_norm(x, w[p + "input_layernorm.weight"], eps, True), w, p + "self_attn.",
                                  c, pos, None, wide=True)
    assert rel_err(got, head_of(x, w, c)) < TOL_F32
    # a block spec that does not fit its arrangement is refused with the roles named
    bad = replace(spec, blocks=(blocks[1].with_part("feed_forward", None),) + tuple(blocks[1:]))
    with pytest.raises(ValueError, match="missing.*feed_forward"):
        expected_tensors(bad)
    bad = replace(spec, blocks=(blocks[2].with_part("spare_norm", norm("spare")),) + tuple(blocks[1:]))
    with pytest.raises(ValueError, match="not known to it.*spare_norm"):
        expected_tensors(bad)


def toy_latent_spec():
    from gogguf_b200.config import PartSpec, config_from_dict
    spec = config_from_dict(TINY_B).to_spec()
    blocks = list(spec.blocks)
    blocks[1] = blocks[1].with_part("mixer", PartSpec("toy_latent_mean", dict(hidden_size=TINY_B["hidden_size"], latent=24),
                                                      prefix="model.layers.1.latent."))
    return replace(spec, blocks=tuple(blocks))


def test_a_cache_kind_of_its_own_is_registered_paged_and_reused():
    from gogguf_b200.cache import KVGroup
    from gogguf_b200.engine import StepEntry, Stepper
    register_toys()
    spec = toy_latent_spec()
    model, w, _ = build(spec, "float32", seed=22)
    cache = model.new_cache(64 * 5, max_slots=3)
    kinds = [type(g).__name__ for g in cache.groups]
    assert kinds == ["KVGroup", "LatentStore"] and isinstance(cache.groups[0], KVGroup)
    assert cache.groups[0].k.shape[0] == 2 and cache.groups[1].lat.shape[:2] == (1, 5)
    toks = tokens(spec.vocab_size, 150, 2)           # three pages of latents
    got = whole_chunked_decoded(model, toks, TOL_F32)
    c = plain.plain_config(TINY_B)
    pos = list(range(len(toks)))
    x = plain.embed(w["model.embed_tokens.weight"], toks).double()
    x = plain.block(x, w, 0, c, pos, wide=True)
    p = "model.layers.1."
    h = plain.rms_norm(x, w[p + "input_layernorm.weight"], c["eps"], True)
    lat = h @ w[p + "latent.down.weight"].double().T
    means = torch.cumsum(lat, 0) / torch.arange(1, len(toks) + 1, dtype=torch.float64)[:, None]
    x = x + means @ w[p + "latent.up.weight"].double().T
    h = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], c["eps"], True)
    x = x + plain.swiglu_ffn(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                             w[p + "mlp.down_proj.weight"], True)
    x = plain.block(x, w, 2, c, pos, wide=True)
    assert rel_err(got, head_of(x, w, c)) < TOL_F32
    # unequal batch in a cache that cannot hold all three at once: pages of both kinds go round
    st = Stepper(model, cache)
    seqs = [toks[:100], toks[:30], toks[:70]]
    for rnd in range(2):
        slots = [cache.open() for _ in range(2)]
        out = st.step([StepEntry(s, q, want=[len(q) - 1]) for s, q in zip(slots, seqs[rnd:rnd + 2])])
        for j, q in enumerate(seqs[rnd:rnd + 2]):
            assert rel_err(out[j:j + 1], got[len(q) - 1:len(q)]) < TOL_F32
        for s in slots:
            cache.close(s)
        cache.check()
    assert all(g.pages.held_count == 0 for g in cache.groups)


def test_a_part_that_cannot_be_captured_goes_through_the_entry_point_eagerly():
    import gogguf_b200 as gg
    from gogguf_b200.api import Engine
    from gogguf_b200.engine.graphs import GraphStepper
    register_toys()
    model, w, _ = build(toy_latent_spec(), "float32", seed=23)
    ctx = Engine(model, gg.LoadOptions(dtype="float32", max_tokens=64 * 8)).new_context()
    assert isinstance(ctx.stepper, GraphStepper) and not ctx.stepper.capturable
    prompts = [tokens(model.vocab_size, n, 30 + n) for n in (9, 3, 14)]
    out = ctx.generate(prompts, gg.GenerateParams(max_tokens=6, stop_token_ids=[]))
    assert ctx.stepper.replays == 0 and not ctx.stepper._graphs
    for p, r in zip(prompts, out):
        seq = list(p)
        for t in r.tokens:                           # greedy: every token is the arg-max of the whole sequence so far
            assert int(ctx.forward_token_ids(seq)[-1].argmax()) == t
            seq.append(t)
    ctx.cache.check()
    assert ctx.cache.live_slots == 0


@pytest.mark.parametrize("dtype,cfg", [("float32", TINY_B), ("bfloat16", TINY_L)])
def test_a_position_encoding_that_is_a_scaled_partial_rotation(dtype, cfg):
    from gogguf_b200.config import PartSpec, config_from_dict
    register_toys()
    spec = config_from_dict(cfg).to_spec()
    d = cfg["head_dim"]
    rot, theta, factor, mag = d // 2, 777.0, 4.0, 1.25
    blocks = list(spec.blocks)
    m = blocks[1].mixer
    blocks[1] = blocks[1].with_part("mixer", PartSpec(m.kind, {**m.params, "position": dict(
        kind="toy_scaled_partial_rope", rotary_dim=rot, theta=theta, factor=factor, magnitude=mag)}, prefix=m.prefix))
    spec = replace(spec, blocks=tuple(blocks))
    model, w, _ = build(spec, dtype, seed=24, std=0.06 if dtype == "float32" else 0.1)
    toks = tokens(spec.vocab_size, 120, 3)
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    got = whole_chunked_decoded(model, toks, tol)
    c = plain.plain_config(cfg)
    T = len(toks)
    pos = list(range(T))
    x = plain.embed(w["model.embed_tokens.weight"], toks).double()
    x = plain.block(x, w, 0, c, pos, wide=True)
    p = "model.layers.1.self_attn."
    h = plain.rms_norm(x, w["model.layers.1.input_layernorm.weight"], c["eps"], True)
    q = (h @ w[p + "q_proj.weight"].double().T).reshape(T, c["heads"], d)
    k = (h @ w[p + "k_proj.weight"].double().T).reshape(T, c["kv_heads"], d)
    v = (h @ w[p + "v_proj.weight"].double().T).reshape(T, c["kv_heads"], d)
    q = plain.rms_norm(q, w[p + "q_norm.weight"], c["eps"], True)
    k = plain.rms_norm(k, w[p + "k_norm.weight"], c["eps"], True)
    ang = (torch.arange(T, dtype=torch.float64) / factor)[:, None] * torch.pow(
        torch.tensor(theta, dtype=torch.float64), -2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)[None, :]
    cs, sn = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]

    def turn(t):
        a, b, rest = t[..., :rot // 2], t[..., rot // 2:rot], t[..., rot:]
        return torch.cat([a * cs - b * sn, a * sn + b * cs, rest], dim=-1)

    o = plain.attention(turn(q), turn(k), v, None, wide=True).reshape(T, c["heads"] * d)
    x = x + o @ w[p + "o_proj.weight"].double().T
    h = plain.rms_norm(x, w["model.layers.1.post_attention_layernorm.weight"], c["eps"], True)
    q_ = "model.layers.1.mlp."
    x = x + plain.swiglu_ffn(h, w[q_ + "gate_proj.weight"], w[q_ + "up_proj.weight"], w[q_ + "down_proj.weight"], True)
    for layer in range(2, c["layers"]):
        x = plain.block(x, w, layer, c, pos, wide=True)
    assert rel_err(got, head_of(x, w, c)) < tol
    # and it is not the model's own encoding in disguise
    assert rel_err(plain.forward(cfg, w, toks, wide=True), head_of(x, w, c)) > 0.2
