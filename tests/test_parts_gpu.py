"""Each part alone against the plain implementation, and parts that the framework
does not have - a mixer with per-request state, a routed feed-forward, another
position encoding - defined here, registered, built and stepped without touching
the framework's files."""
import math

import numpy as np
import pytest
import torch

import helpers
from plain import plain_qwen2

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class _Ctx:
    def __init__(self, kernels, dtype):
        self.kernels, self.dtype = kernels, dtype


def _rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_norm_ffn_embedding_head_alone(cuda_kernels, dtype, tol):
    from inferflux_b200.config import PartSpec
    from inferflux_b200.parts import build_part
    ctx = _Ctx(cuda_kernels, dtype)
    H, I, V, T = 72, 200, 333, 19
    x = _rnd(T, H, seed=1)
    # norm (with and without a pending delta)
    norm = build_part("norm", PartSpec("rmsnorm", {"size": H, "eps": 1e-3}))
    w = 1 + _rnd(H, seed=2, scale=0.2)
    norm.load({"weight": w}, dtype, DEV)
    got = norm.forward(x.to(DEV), None, ctx).float().cpu()
    assert float((got - plain_qwen2.rmsnorm(x, w, 1e-3)).abs().max()) < tol * 4
    delta = _rnd(T, H, seed=3).to(dtype)
    xs = x.to(DEV).clone()
    got = norm.forward(xs, delta.to(DEV), ctx).float().cpu()
    assert float((got - plain_qwen2.rmsnorm(x + delta.float(), w, 1e-3)).abs().max()) < tol * 4
    assert torch.allclose(xs.cpu(), x + delta.float())
    # feed-forward
    ffn = build_part("ffn", PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I}))
    wg, wu, wd = (_rnd(I, H, seed=4, scale=0.1).to(dtype), _rnd(I, H, seed=5, scale=0.1).to(dtype),
                  _rnd(H, I, seed=6, scale=0.1).to(dtype))
    ffn.load({"gate_proj.weight": wg, "up_proj.weight": wu, "down_proj.weight": wd}, dtype, DEV)
    h = x.to(dtype)
    got = cuda_kernels.materialize(ffn.forward(h.to(DEV), ctx)).float().cpu()
    want = plain_qwen2.swiglu_mlp(h.double(), wg.double(), wu.double(), wd.double())
    assert float((got - want).abs().max()) < tol * max(1.0, float(want.abs().max()))
    # embedding and head (tied)
    emb = build_part("embedding", PartSpec("embedding", {"vocab_size": V, "hidden_size": H}))
    table = _rnd(V, H, seed=7).to(dtype)
    emb.load({"weight": table}, dtype, DEV)
    ctx.token_ids = torch.tensor([5, 0, V - 1, 17], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(ctx).cpu(), table[[5, 0, V - 1, 17]].float())
    head = build_part("lm_head", PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "tied": True}))
    head.load({}, dtype, DEV, tied_table=emb.table)
    got = head.forward(h.to(DEV), ctx)
    assert got.dtype == torch.float32
    want = h.double() @ table.double().t()
    assert float((got.cpu() - want).abs().max()) < tol * float(want.abs().max())


def test_rope_part_tables():
    from inferflux_b200.config import PartSpec
    from inferflux_b200.parts import build_part
    rope = build_part("position", PartSpec("rope", {"theta": 1e6, "rotary_dim": 32, "pairing": "split_half"}))
    t = rope.rotary(DEV)
    want = 1.0 / (1e6 ** (torch.arange(0, 32, 2, dtype=torch.float32) / 32))
    assert torch.equal(t.inv_freq.cpu(), want) and t.rotary_dim == 32 and not t.interleaved
    assert build_part("position", PartSpec("none")).rotary(DEV) is None
    with pytest.raises(ValueError):
        build_part("position", PartSpec("rope", {"theta": 1e4, "rotary_dim": 7}))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
def test_attention_part_alone(cuda_kernels, dtype, tol):
    """The attention mixer over its own cache, whole and in two portions."""
    from inferflux_b200.cache import CacheManager
    from inferflux_b200.config import PartSpec, ScheduleEntry
    from inferflux_b200.engine.batch import StepContext, StepEntry
    from inferflux_b200.parts import build_part
    H, nq, nkv, d, T = 80, 6, 3, 16, 37
    spec = PartSpec("attention", {"hidden_size": H, "num_heads": nq, "num_kv_heads": nkv, "head_dim": d,
                                  "window": 9, "qkv_bias": True, "scale": None,
                                  "position": PartSpec("rope", {"theta": 1e4, "rotary_dim": d})})
    mixer = build_part("mixer", spec)
    tensors = {n: _rnd(*s.shape, seed=10 + i, scale=0.3).to(dtype) for i, (n, s) in enumerate(mixer.param_specs().items())}
    mixer.load(tensors, dtype, DEV)
    h = _rnd(T, H, seed=30).to(dtype)
    cfg = {"num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": d, "hidden_size": H, "rope_theta": 1e4,
           "use_sliding_window": True, "sliding_window": 9, "max_window_layers": 0}
    W = {"model.layers.0.self_attn." + n: t.double() for n, t in tensors.items()}
    want = plain_qwen2.attention_block(h.double(), W, cfg, 0, torch.arange(T))
    for cuts in ([T], [20, 17], [5, 1, 1, 30]):
        cache = CacheManager([(mixer.cache_spec(), None)], page_size=4, num_pages=12, max_seqs=2, max_seq_len=64,
                             dtype=dtype, device=DEV)
        cache.add_request("r")
        outs, pos = [], 0
        for n in cuts:
            cache.reserve("r", pos + n)
            # the mixer's own step arrays travel with the step's metadata (or, for the 17, are made when first used)
            ctx = StepContext.build(cuda_kernels, dtype, DEV, [StepEntry("r", [0] * n, [])], [pos], [cache.slot("r")],
                                    cache.drain_table_updates(), providers=[mixer] if n != 17 else [])
            for g, (idx, page) in zip(cache.groups, ctx.table_updates):
                cuda_kernels.scatter_i32(g.table, idx, page)
            outs.append(cuda_kernels.materialize(mixer.forward(h[pos:pos + n].to(DEV).contiguous(), ctx,
                                                               cache.view(ScheduleEntry(0, 0)))))
            cache.commit("r", pos + n)
            pos += n
        got = torch.cat(outs).float().cpu()
        assert float((got - want).abs().max()) < tol * max(1.0, float(want.abs().max())), f"cuts {cuts}"


# ------------------------------------------------------------- parts of the test's own

def _register_toys():
    from inferflux_b200.parts import (FeedForward, Mixer, PositionEncoding, RotaryTable, StateSpec, register_part)
    from inferflux_b200.weights import TensorSpec

    @register_part("mixer", "toy_decay")
    class DecayMixer(Mixer):
        """s <- a * s + h[t];  y[t] = s . Wo^T, with s kept per request between steps."""
        graph_safe = False                                   # walks the spans on the host

        def __init__(self, spec):
            super().__init__(spec)
            self.hidden = spec.params["hidden_size"]

        def state_spec(self):
            return StateSpec((self.hidden,), torch.float32)

        def param_specs(self):
            return {"decay": TensorSpec((self.hidden,), init="ones"), "out.weight": TensorSpec((self.hidden, self.hidden))}

        def load(self, tensors, dtype, device):
            self.decay = torch.sigmoid(tensors["decay"].to(device=device, dtype=torch.float32))
            self.w = tensors["out.weight"].to(device=device, dtype=dtype).contiguous()

        def forward(self, h, ctx, cache):
            assert cache.kv is None and cache.state is not None
            out = torch.empty_like(h, dtype=torch.float32)
            base = 0
            for (start, n), slot in zip(ctx.spans, ctx.slots_host):
                s = cache.state[slot]
                if start == 0:
                    assert float(s.abs().sum()) == 0.0, "a fresh request did not get a zeroed state"
                for t in range(base, base + n):
                    s = self.decay * s + h[t].float()
                    out[t] = s
                cache.state[slot] = s
                base += n
            return ctx.kernels.linear(out.to(h.dtype), self.w)

    @register_part("ffn", "toy_routed")
    class RoutedFFN(FeedForward):
        """Two experts, each token goes to the one its float32 router logit prefers."""
        graph_safe = False

        def __init__(self, spec):
            super().__init__(spec)
            self.hidden, self.inter = spec.params["hidden_size"], spec.params["intermediate_size"]

        def param_specs(self):
            s = {"router.weight": TensorSpec((2, self.hidden))}
            for e in range(2):
                s[f"experts.{e}.up.weight"] = TensorSpec((self.inter, self.hidden))
                s[f"experts.{e}.down.weight"] = TensorSpec((self.hidden, self.inter))
            return s

        def load(self, tensors, dtype, device):
            self.t = {n: v.to(device=device, dtype=torch.float32 if "router" in n else dtype).contiguous()
                      for n, v in tensors.items()}

        def forward(self, h, ctx):
            choice = (h.float() @ self.t["router.weight"].t()).argmax(-1)
            out = torch.zeros_like(h)
            for e in range(2):
                idx = (choice == e).nonzero().flatten()
                if idx.numel():
                    up = ctx.kernels.linear(h[idx].contiguous(), self.t[f"experts.{e}.up.weight"])
                    out[idx] = ctx.kernels.linear(torch.relu(up), self.t[f"experts.{e}.down.weight"])
            return out

    @register_part("position", "toy_scaled_rope")
    class ScaledRope(PositionEncoding):
        """Interleaved pairs, only part of the head, frequencies divided by a factor."""

        def rotary(self, device):
            p = self.spec.params
            inv = 1.0 / (p["theta"] ** (torch.arange(0, p["rotary_dim"], 2, dtype=torch.float32) / p["rotary_dim"]))
            return RotaryTable((inv / p["factor"]).to(device), p["rotary_dim"], True)


def _toy_plan(H, V, I):
    from inferflux_b200.config import ModelPlan, PartSpec, ScheduleEntry, prenorm_layer
    norm = PartSpec("rmsnorm", {"size": H, "eps": 1e-5})
    attn = PartSpec("attention", {"hidden_size": H, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16, "window": None,
                                  "qkv_bias": "if_present", "scale": 0.3,
                                  "position": PartSpec("toy_scaled_rope", {"theta": 1e4, "rotary_dim": 8, "factor": 4.0})})
    swiglu = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I})
    layers = [
        prenorm_layer("model.layers.0.", attn, swiglu, norm, norm),
        prenorm_layer("model.layers.1.", PartSpec("toy_decay", {"hidden_size": H}),
                      PartSpec("toy_routed", {"hidden_size": H, "intermediate_size": I}), norm, norm),
    ]
    # layer 0 runs twice (second time on a cache of its own), then the toy layer
    schedule = [ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2)]
    return ModelPlan("ToyHybrid", H, V, 256, PartSpec("embedding", {"vocab_size": V, "hidden_size": H}), layers,
                     schedule, norm, PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "tied": False}))


def _toy_oracle(W, toks, H):
    """Whole-sequence statement of the toy model, float64."""
    W = {k: v.double() for k, v in W.items()}
    T = len(toks)
    pos = torch.arange(T)
    x = W["model.embed_tokens.weight"][torch.tensor(toks)]

    def attn_layer(x):
        p = "model.layers.0."
        h = plain_qwen2.rmsnorm(x, W[p + "input_layernorm.weight"], 1e-5)
        q = plain_qwen2.linear(h, W[p + "self_attn.q_proj.weight"], W[p + "self_attn.q_proj.bias"]).view(T, 4, 16)
        k = plain_qwen2.linear(h, W[p + "self_attn.k_proj.weight"], W[p + "self_attn.k_proj.bias"]).view(T, 2, 16)
        v = plain_qwen2.linear(h, W[p + "self_attn.v_proj.weight"], W[p + "self_attn.v_proj.bias"]).view(T, 2, 16)
        inv = (1.0 / (1e4 ** (torch.arange(0, 8, 2, dtype=torch.float32) / 8)) / 4.0)
        ang = pos.float()[:, None] * inv[None, :]
        cos, sin = torch.cos(ang).double()[:, None, :], torch.sin(ang).double()[:, None, :]

        def turn(z):
            a, b = z[..., 0:8:2], z[..., 1:8:2]
            z = z.clone()
            z[..., 0:8:2], z[..., 1:8:2] = a * cos - b * sin, a * sin + b * cos
            return z
        q, k = turn(q), turn(k)
        out = torch.zeros(T, 4, 16, dtype=torch.float64)
        for hd in range(4):
            s = (q[:, hd] @ k[:, hd // 2].t()) * 0.3
            s = s.masked_fill(pos[None, :] > pos[:, None], float("-inf"))
            out[:, hd] = torch.softmax(s, -1) @ v[:, hd // 2]
        x = x + out.reshape(T, 64) @ W[p + "self_attn.o_proj.weight"].t()
        m = plain_qwen2.rmsnorm(x, W[p + "post_attention_layernorm.weight"], 1e-5)
        return x + plain_qwen2.swiglu_mlp(m, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"],
                                          W[p + "mlp.down_proj.weight"])

    def toy_layer(x):
        p = "model.layers.1."
        h = plain_qwen2.rmsnorm(x, W[p + "input_layernorm.weight"], 1e-5)
        a = torch.sigmoid(W[p + "self_attn.decay"].float()).double()
        s, ys = torch.zeros(H, dtype=torch.float64), []
        for t in range(T):
            s = a * s + h[t]
            ys.append(s)
        x = x + torch.stack(ys) @ W[p + "self_attn.out.weight"].t()
        m = plain_qwen2.rmsnorm(x, W[p + "post_attention_layernorm.weight"], 1e-5)
        choice = (m @ W[p + "mlp.router.weight"].t()).argmax(-1)
        f = torch.zeros_like(m)
        for e in range(2):
            idx = (choice == e).nonzero().flatten()
            f[idx] = torch.relu(m[idx] @ W[p + f"mlp.experts.{e}.up.weight"].t()) @ W[p + f"mlp.experts.{e}.down.weight"].t()
        return x + f

    x = attn_layer(x)
    x = toy_layer(x)
    x = attn_layer(x)
    return plain_qwen2.rmsnorm(x, W["model.norm.weight"], 1e-5) @ W["lm_head.weight"].t()


def test_toy_parts_register_build_and_step(cuda_kernels):
    """A model made of the framework's attention, run twice, around a layer whose
    mixer keeps per-request state and whose feed-forward routes tokens: built from a
    plan, random weights by the parts' own declarations, stepped under every cutting."""
    from inferflux_b200.engine import ModelRunner
    from inferflux_b200.models import Model
    from inferflux_b200.weights import random_tensors
    _register_toys()
    H, V, I = 64, 300, 96
    plan = _toy_plan(H, V, I)
    model = Model(plan)
    expected = model.expected_tensors()
    assert "model.layers.1.self_attn.decay" in expected and "model.layers.1.mlp.experts.1.down.weight" in expected
    tensors = random_tensors(expected, seed=3, dtype=torch.float32, std=0.08, norm_jitter=0.1)
    tensors["model.embed_tokens.weight"] *= 10
    model.load(tensors, torch.float32, DEV)
    specs = model.cache_specs()
    assert specs[0][0] is not None and specs[1][0] is None and specs[1][1].shape == (H,) and specs[2][0] is not None
    reqs = {f"r{i}": helpers.random_tokens(V, n, 200 + i) for i, n in enumerate([40, 33, 50, 60, 21])}
    want = {rid: _toy_oracle(tensors, toks, H).numpy() for rid, toks in reqs.items()}
    for make in (helpers.trace_whole, helpers.trace_portions, lambda r: helpers.trace_mixed(r, 192)):
        runner = ModelRunner(model, cuda_kernels, page_size=8, num_pages=192 // 8, max_seqs=4, cuda_graphs=True)
        assert not runner.cuda_graphs                      # a part said it cannot be captured
        steps = make(reqs)
        got = helpers.collect(steps, helpers.run_steps_in_process(runner, steps), V)
        bad = helpers.first_bad(got, want, 2e-4)
        assert bad is None, f"first wrong row (request, position, diff): {bad}"


def test_a_block_kind_of_the_tests_own_with_four_norms_and_no_feed_forward(cuda_kernels):
    """A block arrangement defined here, with parts under names of its own (four norms around a
    mixer, no feed-forward), becomes a model without a change to the framework's files: the plan
    names the parts, the block kind says which it arranges, weights are declared and made by them."""
    from inferflux_b200.config import LayerSpec, ModelPlan, PartSpec, SubPart, default_schedule
    from inferflux_b200.engine import ModelRunner
    from inferflux_b200.models import Model
    from inferflux_b200.parts import Block, register_part
    from inferflux_b200.weights import random_tensors
    _register_toys()

    @register_part("block", "toy_sandwich")
    class SandwichBlock(Block):
        """x += post(mixer(pre(x)));  x += outer(inner(x))."""
        sub_parts = {"pre": "norm", "mixer": "mixer", "post": "norm", "inner": "norm", "outer": "norm"}

        def forward(self, x, pending, ctx, cache):
            k = ctx.kernels
            if pending is not None:
                k.residual_add(x, pending)
            a = k.materialize(self.mixer.forward(self.pre.forward(x, None, ctx), ctx, cache))
            k.residual_add(x, self.post.forward(a.float(), None, ctx))
            g = self.outer.forward(self.inner.forward(x, None, ctx).float(), None, ctx)
            return x, g                                   # handed on unadded, like any block's last delta

    H, V = 48, 200
    attn = PartSpec("attention", {"hidden_size": H, "num_heads": 3, "num_kv_heads": 1, "head_dim": 16, "window": None,
                                  "qkv_bias": False, "scale": None,
                                  "position": PartSpec("rope", {"theta": 1e4, "rotary_dim": 16})})
    def norm(eps):
        return PartSpec("rmsnorm", {"size": H, "eps": eps})
    layers = []
    for i, mixer in enumerate((attn, PartSpec("toy_decay", {"hidden_size": H}))):
        layers.append(LayerSpec(f"blocks.{i}.", PartSpec("toy_sandwich"), {
            "pre": SubPart("norm", norm(1e-5), "n1."), "mixer": SubPart("mixer", mixer, "mix."),
            "post": SubPart("norm", norm(1e-4), "n2."), "inner": SubPart("norm", norm(1e-3), "n3."),
            "outer": SubPart("norm", norm(1e-2), "n4.")}))
    with pytest.raises(ValueError, match="lacks"):           # a layer that does not bring what the block arranges
        Model(ModelPlan("Bad", H, V, 128, PartSpec("embedding", {"vocab_size": V, "hidden_size": H}),
                        [LayerSpec("blocks.0.", PartSpec("toy_sandwich"), {"mixer": SubPart("mixer", attn, "mix.")})],
                        default_schedule(1), norm(1e-5), PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "tied": True})))
    plan = ModelPlan("ToySandwich", H, V, 128, PartSpec("embedding", {"vocab_size": V, "hidden_size": H}), layers,
                     default_schedule(2), norm(1e-5), PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "tied": True}))
    model = Model(plan)
    expected = model.expected_tensors()
    assert "blocks.0.n4.weight" in expected and "blocks.1.mix.decay" in expected and not any("mlp" in n for n in expected)
    W = random_tensors(expected, seed=8, dtype=torch.float32, std=0.1, norm_jitter=0.2)
    W["model.embed_tokens.weight"] *= 8
    model.load(W, torch.float32, DEV)

    def oracle(toks):
        Wd = {k: v.double() for k, v in W.items()}
        T = len(toks)
        x = Wd["model.embed_tokens.weight"][torch.tensor(toks)]
        for i in range(2):
            p = f"blocks.{i}."
            h = plain_qwen2.rmsnorm(x, Wd[p + "n1.weight"], 1e-5)
            if i == 0:
                q = plain_qwen2.rope_neox(plain_qwen2.linear(h, Wd[p + "mix.q_proj.weight"]).view(T, 3, 16), torch.arange(T), 1e4)
                k = plain_qwen2.rope_neox(plain_qwen2.linear(h, Wd[p + "mix.k_proj.weight"]).view(T, 1, 16), torch.arange(T), 1e4)
                v = plain_qwen2.linear(h, Wd[p + "mix.v_proj.weight"]).view(T, 1, 16)
                a = plain_qwen2.attention_gqa_causal(q, k, v).reshape(T, 48) @ Wd[p + "mix.o_proj.weight"].t()
            else:
                decay, s, ys = torch.sigmoid(W[p + "mix.decay"].float()).double(), torch.zeros(H, dtype=torch.float64), []
                for t in range(T):
                    s = decay * s + h[t]
                    ys.append(s)
                a = torch.stack(ys) @ Wd[p + "mix.out.weight"].t()
            x = x + plain_qwen2.rmsnorm(a, Wd[p + "n2.weight"], 1e-4)
            x = x + plain_qwen2.rmsnorm(plain_qwen2.rmsnorm(x, Wd[p + "n3.weight"], 1e-3), Wd[p + "n4.weight"], 1e-2)
        return plain_qwen2.rmsnorm(x, Wd["model.norm.weight"], 1e-5) @ Wd["model.embed_tokens.weight"].t()

    reqs = {f"r{i}": helpers.random_tokens(V, n, 300 + i) for i, n in enumerate([35, 50, 21])}
    want = {rid: oracle(toks).numpy() for rid, toks in reqs.items()}
    for make in (helpers.trace_whole, helpers.trace_portions, lambda r: helpers.trace_mixed(r, 128)):
        runner = ModelRunner(model, cuda_kernels, page_size=8, num_pages=128 // 8, max_seqs=4)
        steps = make(reqs)
        got = helpers.collect(steps, helpers.run_steps_in_process(runner, steps), V)
        bad = helpers.first_bad(got, want, 2e-4)
        assert bad is None, f"first wrong row (request, position, diff): {bad}"
