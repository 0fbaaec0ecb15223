"""Each part alone against the plain implementation's function for it, and a toy mixer with state
of its own that is registered, built and stepped from this file without touching the framework."""

from types import SimpleNamespace

import pytest
import torch

import helpers as H
import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = [pytest.param(torch.float32, id="f32"), pytest.param(torch.bfloat16, id="bf16")]


def tol(dtype):
    return 2e-5 if dtype == torch.float32 else 3e-2


def getter(weights, dtype):
    from llm_pipeline_b200.weights import stored_dtype_policy

    def get(name, role):
        t = weights[name]
        return t.to(device=DEV, dtype=stored_dtype_policy(role, t.dtype, dtype))
    return get


def context_for(dtype, cache_specs, chunks, page_size=8, num_pages=32, vocab=1000):
    """A runner over a model stand-in, so that parts can be stepped with real step contexts."""
    from llm_pipeline_b200.cache import CacheManager
    from llm_pipeline_b200.engine import ModelRunner

    cache = CacheManager(cache_specs, page_size=page_size, num_pages=num_pages, max_requests=4,
                         max_request_tokens=512, device=DEV, dtype=dtype)
    model = SimpleNamespace(device=DEV, dtype=dtype, spec=SimpleNamespace(vocab_size=vocab))
    return ModelRunner(model, cache), cache


@pytest.mark.parametrize("dtype", DTYPES)
def test_rms_norm_part(dtype):
    from llm_pipeline_b200.parts import ResidualStream, lookup
    w = {"n.weight": 1 + 0.1 * torch.randn(200)}
    norm = lookup("norm", "rms_norm")("n", size=200, eps=1e-5)
    assert set(norm.param_specs()) == {"n.weight"}
    norm.load(getter(w, dtype))
    x = torch.randn(5, 200, device=DEV)
    delta = torch.randn(5, 200, device=DEV).to(dtype)
    stream = ResidualStream(x.clone())
    stream.add(delta)
    out = norm.add_norm(stream, SimpleNamespace(dtype=dtype))
    want = plain.rms_norm(x + delta.float(), w["n.weight"].to(DEV).to(dtype).float(), 1e-5)
    assert stream.pending is None and torch.allclose(stream.residual, x + delta.float(), atol=1e-6)
    assert torch.allclose(out.float(), want, atol=tol(dtype), rtol=1e-2 if dtype == torch.bfloat16 else 1e-5)


def test_rotary_part_tables():
    from llm_pipeline_b200.parts import lookup
    rope = lookup("position", "rotary")("", rotary_dim=48, theta=50000.0)
    ctx = SimpleNamespace(device=DEV, num_tokens=4, positions=torch.tensor([0, 5, 6, 2000], dtype=torch.int32, device=DEV))
    cos, sin = rope.tables(ctx)
    want_cos, want_sin = plain.rope_cos_sin(ctx.positions.cpu(), 48, 50000.0)
    assert torch.allclose(cos.cpu(), want_cos[:, :24], atol=2e-6) and torch.allclose(sin.cpu(), want_sin[:, :24], atol=2e-6)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part(dtype):
    from llm_pipeline_b200.parts import lookup
    cfg = plain.TINY_C
    w = {k.replace("model.layers.0.mlp", "ff"): v for k, v in plain.random_weights(cfg, 3, std=0.1).items() if ".layers.0.mlp." in k}
    if dtype == torch.bfloat16:
        w = {k: v.to(dtype).float() for k, v in w.items()}
    ff = lookup("feed_forward", "swiglu")("ff", hidden_size=cfg["hidden_size"], intermediate_size=cfg["intermediate_size"])
    ff.load(getter(w, dtype))
    x = torch.randn(6, cfg["hidden_size"], device=DEV).to(dtype)
    out, bias = ff.forward(x, SimpleNamespace(dtype=dtype))
    want = plain.mlp(x.float().cpu(), w, "ff")
    assert bias is None and torch.allclose(out.float().cpu(), want, atol=tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    from llm_pipeline_b200.parts import lookup
    w = {"e.weight": torch.randn(300, 40).to(dtype).float(), "h.weight": torch.randn(300, 40).to(dtype).float()}
    emb = lookup("embedding", "token_embedding")("e", vocab_size=300, hidden_size=40)
    emb.load(getter(w, dtype))
    ids = torch.tensor([1, 299, 17], dtype=torch.int32, device=DEV)
    out = emb.forward(SimpleNamespace(device=DEV, num_tokens=3, token_ids=ids))
    assert out.dtype == torch.float32 and torch.equal(out.cpu(), w["e.weight"][ids.cpu().long()])
    for tied, name in ((None, "h.weight"), ("e", "e.weight")):
        head = lookup("head", "linear_head")("h", vocab_size=300, hidden_size=40, tied_to=tied)
        head.load(getter(w, dtype))
        x = torch.randn(3, 40, device=DEV).to(dtype)
        logits = head.forward(x, None)
        assert logits.dtype == torch.float32
        assert torch.allclose(logits.cpu(), x.float().cpu() @ w[name].t(), atol=1e-4 if dtype == torch.float32 else 5e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tiny", [plain.TINY_B, plain.TINY_C], ids=["b", "c"])
def test_attention_part_alone_in_two_portions(dtype, tiny):
    """The mixer on a sequence cut in two steps equals the plain attention on the whole sequence."""
    from llm_pipeline_b200.config import resolve_config
    from llm_pipeline_b200.engine import StepEntry
    from llm_pipeline_b200.parts import LayerCache, lookup
    cfg = resolve_config(tiny)
    spec = cfg.model_spec()
    part = spec.layers[1].mixer
    weights = {k: v for k, v in plain.random_weights(tiny, 4, std=0.08).items()}
    if dtype == torch.bfloat16:
        weights = {k: v.to(dtype).float() for k, v in weights.items()}
    mixer = lookup("mixer", part.kind)(part.prefix, **part.args)
    mixer.load(getter(weights, dtype))
    rope = lookup("position", "rotary")("", **spec.positions["rope"].args)
    runner, cache = context_for(dtype, [(mixer.cache_spec(), None)], None)
    T, cutat = 29, 18
    x = torch.randn(T, tiny["hidden_size"])
    if dtype == torch.bfloat16:
        x = x.to(dtype).float()
    cos, sin = plain.rope_cos_sin(torch.arange(T), tiny["head_dim"], tiny["rope_theta"])
    want = plain.attention(x, weights, part.prefix, tiny, cos, sin)
    got = []
    for lo, hi in ((0, cutat), (cutat, T)):
        ctx = runner._prepare([StepEntry("r", [1] * (hi - lo), [])])
        ctx.position_tables = {"rope": rope.tables(ctx)}
        out, bias = mixer.forward(x[lo:hi].to(DEV).to(dtype), ctx, LayerCache(cache.pages_tensor(0), 0, None, True))
        out = out.float() + (bias.float() if bias is not None else 0)
        got.append(out.cpu())
        cache.commit("r", hi)
    assert torch.allclose(torch.cat(got), want, atol=tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_part(dtype):
    from llm_pipeline_b200.config import resolve_config
    from llm_pipeline_b200.engine import StepEntry
    from llm_pipeline_b200.parts import LayerCache, ResidualStream, lookup
    tiny = plain.TINY_A
    spec = resolve_config(tiny).model_spec()
    layer = spec.layers[1]
    weights = plain.random_weights(tiny, 5, std=0.08)
    if dtype == torch.bfloat16:
        weights = {k: v.to(dtype).float() for k, v in weights.items()}
    make = lambda family, p: lookup(family, p.kind)(p.prefix, **p.args)   # noqa: E731
    block = lookup("block", layer.block)(make("mixer", layer.mixer), make("feed_forward", layer.feed_forward),
                                         make("norm", layer.mixer_norm), make("norm", layer.feed_forward_norm))
    for part in block.parts():
        part.load(getter(weights, dtype))
    rope = make("position", spec.positions["rope"])
    runner, cache = context_for(dtype, [(block.mixer.cache_spec(), None)], None)
    T = 21
    x = torch.randn(T, tiny["hidden_size"])
    cos, sin = plain.rope_cos_sin(torch.arange(T), tiny["head_dim"], tiny["rope_theta"])
    want = plain.decoder_layer(x, weights, 1, tiny, cos, sin)
    ctx = runner._prepare([StepEntry("r", [1] * T, [])])
    ctx.position_tables = {"rope": rope.tables(ctx)}
    stream = ResidualStream(x.to(DEV))
    block.forward(stream, ctx, LayerCache(cache.pages_tensor(0), 0, None, True))
    got = stream.residual + stream.pending.float()
    assert torch.allclose(got.cpu(), want, atol=tol(dtype))


# ------------------------------------------------------------------------------------------
# A toy mixer with state of its own: a decayed running sum of its inputs per request.
#   s_t = decay * s_{t-1} + x_t ;  out_t = s_t * gain
# The state is one vector per request, kept in the request's slot between steps.
# ------------------------------------------------------------------------------------------

def _register_toy():
    from llm_pipeline_b200.cache import StateSpec
    from llm_pipeline_b200.config import (LayerSpec, ModelConfig, ModelSpec, PartSpec, ScheduleEntry,
                                          register_architecture)
    from llm_pipeline_b200.parts import Mixer, register_mixer
    from llm_pipeline_b200.weights import ParamSpec

    @register_mixer("toy_decayed_sum")
    class DecayedSum(Mixer):
        def __init__(self, prefix, hidden_size, decay):
            self.prefix, self.hidden_size, self.decay = prefix, hidden_size, decay
            self.gain = None

        def state_spec(self):
            return StateSpec((self.hidden_size,), torch.float32)

        def param_specs(self):
            return {f"{self.prefix}.gain": ParamSpec((self.hidden_size,), role="vector", init="norm")}

        def load(self, get):
            self.gain = get(f"{self.prefix}.gain", "vector").float()

        def forward(self, x, ctx, cache):
            out = torch.empty_like(x)
            row = 0
            for r, n in enumerate(ctx.q_lens):
                slot = int(ctx.slots[r])
                s = cache.state[slot]
                for i in range(n):
                    s = self.decay * s + x[row + i].float()
                    out[row + i] = (s * self.gain).to(x.dtype)
                cache.state[slot] = s
                row += n
            return out, None

    class ToyConfig(ModelConfig):
        architecture = "ToyHybridForCausalLM"

        def __init__(self, data):
            self.data = data

        @classmethod
        def from_json(cls, data):
            return cls(dict(data))

        def to_json(self):
            return dict(self.data)

        def model_spec(self):
            d = self.data
            H, V = d["hidden_size"], d["vocab_size"]
            norm = {"size": H, "eps": d["eps"]}
            ff = lambda i: PartSpec("swiglu", {"hidden_size": H, "intermediate_size": d["intermediate_size"]}, f"layers.{i}.ff")  # noqa: E731
            attn = PartSpec("attention", {"hidden_size": H, "num_heads": d["heads"], "num_kv_heads": d["kv_heads"],
                                          "head_dim": d["head_dim"], "scale": d["head_dim"] ** -0.5, "qk_norm": False,
                                          "window": d["window"], "position": "rope"}, "layers.1.attn")
            layers = (
                LayerSpec("pre_norm_residual", PartSpec("toy_decayed_sum", {"hidden_size": H, "decay": d["decay"]}, "layers.0.mix"),
                          ff(0), PartSpec("rms_norm", norm, "layers.0.n1"), PartSpec("rms_norm", norm, "layers.0.n2")),
                LayerSpec("pre_norm_residual", attn, ff(1), PartSpec("rms_norm", norm, "layers.1.n1"),
                          PartSpec("rms_norm", norm, "layers.1.n2")),
            )
            # layer 0 runs twice (two caches, so two states), the windowed attention layer once
            return ModelSpec("ToyHybridForCausalLM", V, H, PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H}, "embed"),
                             {"rope": PartSpec("rotary", {"rotary_dim": d["head_dim"], "theta": 10000.0})}, layers,
                             (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2)),
                             PartSpec("rms_norm", norm, "final"), PartSpec("linear_head", {"vocab_size": V, "hidden_size": H,
                                                                                           "tied_to": "embed"}, "head"), 512)

    register_architecture("ToyHybridForCausalLM", ToyConfig)


TOY = {"architectures": ["ToyHybridForCausalLM"], "hidden_size": 48, "vocab_size": 97, "intermediate_size": 80, "heads": 3,
       "kv_heads": 3, "head_dim": 16, "eps": 1e-5, "decay": 0.9, "window": 11}


def toy_reference(weights, ids):
    """The toy model on one whole sequence in plain PyTorch."""
    d = TOY
    H, T = d["hidden_size"], len(ids)
    x = weights["embed.weight"][torch.tensor(ids)]

    def ff(h, i):
        g, u = h @ weights[f"layers.{i}.ff.gate_proj.weight"].t(), h @ weights[f"layers.{i}.ff.up_proj.weight"].t()
        return (torch.nn.functional.silu(g) * u) @ weights[f"layers.{i}.ff.down_proj.weight"].t()

    def toy_layer(x):
        h = plain.rms_norm(x, weights["layers.0.n1.weight"], d["eps"])
        s, outs = torch.zeros(H), []
        for t in range(T):
            s = d["decay"] * s + h[t]
            outs.append(s * weights["layers.0.mix.gain"])
        x = x + torch.stack(outs)
        return x + ff(plain.rms_norm(x, weights["layers.0.n2.weight"], d["eps"]), 0)

    def attn_layer(x):
        h = plain.rms_norm(x, weights["layers.1.n1.weight"], d["eps"])
        nh, hd = d["heads"], d["head_dim"]
        cos, sin = plain.rope_cos_sin(torch.arange(T), hd, 10000.0)
        q = (h @ weights["layers.1.attn.q_proj.weight"].t()).view(T, nh, hd).transpose(0, 1)
        k = (h @ weights["layers.1.attn.k_proj.weight"].t()).view(T, nh, hd).transpose(0, 1)
        v = (h @ weights["layers.1.attn.v_proj.weight"].t()).view(T, nh, hd).transpose(0, 1)
        q, k = plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin)
        scores = (q @ k.transpose(1, 2)) * hd ** -0.5
        pos = torch.arange(T)
        masked = (pos[None, :] > pos[:, None]) | (pos[None, :] < pos[:, None] - d["window"] + 1)
        probs = torch.softmax(scores.masked_fill(masked[None], float("-inf")), dim=-1)
        a = (probs @ v).transpose(0, 1).reshape(T, nh * hd) @ weights["layers.1.attn.o_proj.weight"].t()
        x = x + a
        return x + ff(plain.rms_norm(x, weights["layers.1.n2.weight"], d["eps"]), 1)

    x = toy_layer(attn_layer(toy_layer(x)))
    return plain.rms_norm(x, weights["final.weight"], d["eps"]) @ weights["embed.weight"].t()


def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    """Different mixers in different layers, a layer named twice in the schedule, a windowed
    attention group that gives pages back, and per-request state carried across steps."""
    _register_toy()
    from llm_pipeline_b200.config import resolve_config
    from llm_pipeline_b200.weights import write_random_model
    from safetensors.torch import load_file
    folder = write_random_model(TOY, seed=11, out_dir=str(tmp_path), dtype=torch.float32, std=0.15)
    weights = load_file(f"{folder}/model.safetensors")
    assert "layers.0.mix.gain" in weights and "layers.1.attn.q_norm.weight" not in weights
    runner = H.make_runner(folder, torch.float32, page_size=4, num_pages=32, max_request_tokens=256)
    assert [kv is not None for kv, _ in runner.model.cache_specs()] == [False, True, False]
    assert [st is not None for _, st in runner.model.cache_specs()] == [True, False, True]
    requests = {f"t{i}": H.random_tokens(TOY["vocab_size"], n, 70 + i) for i, n in enumerate((40, 9, 23, 31, 17))}
    want = {rid: toy_reference(weights, ids) for rid, ids in requests.items()}
    H.assert_close(H.replay(runner, H.cut_whole(requests)), want, 1e-4, "toy whole")
    H.assert_close(H.replay(runner, H.cut_portions(requests, (5, 2, 9, 1))), want, 1e-4, "toy portions")
    H.assert_close(H.replay(runner, H.cut_mixed(requests, (5, 2, 9, 3), max_live=3)), want, 1e-4, "toy mixed")
    # Steps of single tokens: the attention layer between the two runs of the stateful layer is replayed from a CUDA
    # graph, as are the embedding before and the head after them; the stateful layer runs eagerly every step.
    assert runner.use_graphs and runner.model.pieces() == [(0, 1, False), (1, 2, True), (2, 3, False)]
    before = runner.graph_replays
    H.assert_close(H.replay(runner, H.cut_tail_one_by_one(requests, tail=12)), want, 1e-4, "toy tail, token by token")
    assert runner.graph_replays >= before + 5 * 10
    two = {rid: requests[rid] for rid in ("t0", "t3")}                    # two requests decoding side by side
    steps = [([(rid, toks[:len(toks) - 9], [len(toks) - 10]) for rid, toks in two.items()], [])]
    steps += [([(rid, [toks[len(toks) - 9 + i]], [0]) for rid, toks in two.items()], []) for i in range(9)]
    steps[-1] = (steps[-1][0], list(two))
    got = H.replay(runner, steps)
    for rid, toks in two.items():
        assert float((got[rid] - want[rid][len(toks) - 10:]).abs().max()) < 1e-4, rid
    # the windowed group never held more pages per request than the window needs
    assert runner.cache.groups[0].pool.high_water < 32 and runner.cache.pages_reused > 0


# ------------------------------------------------------------------------------------------
# Two more toy parts defined here, not in the framework: a feed-forward with routing (top-1 of a few
# small SwiGLU experts, router logits in float32) and another position encoding (positions divided by a
# factor, rotation of only the first half of every head).
# ------------------------------------------------------------------------------------------

def _register_toy_routing_and_positions():
    from llm_pipeline_b200.config import (LayerSpec, ModelConfig, ModelSpec, PartSpec, ScheduleEntry,
                                          register_architecture)
    from llm_pipeline_b200.parts import FeedForward, PositionEncoding, register_feed_forward, register_position
    from llm_pipeline_b200.weights import ParamSpec

    @register_feed_forward("toy_top1_experts")
    class Top1Experts(FeedForward):
        def __init__(self, prefix, hidden_size, intermediate_size, num_experts):
            self.prefix, self.H, self.I, self.E = prefix, hidden_size, intermediate_size, num_experts

        def param_specs(self):
            specs = {f"{self.prefix}.router.weight": ParamSpec((self.E, self.H))}
            for e in range(self.E):
                specs[f"{self.prefix}.experts.{e}.gate_up.weight"] = ParamSpec((2 * self.I, self.H))
                specs[f"{self.prefix}.experts.{e}.down.weight"] = ParamSpec((self.H, self.I))
            return specs

        def load(self, get):
            self.router = get(f"{self.prefix}.router.weight", "matrix").float()
            self.gate_up = [get(f"{self.prefix}.experts.{e}.gate_up.weight", "matrix") for e in range(self.E)]
            self.down = [get(f"{self.prefix}.experts.{e}.down.weight", "matrix") for e in range(self.E)]

        def forward(self, x, ctx):
            from llm_pipeline_b200.ops import kernels
            from llm_pipeline_b200.ops.linear import linear
            choice = (x.float() @ self.router.t()).argmax(dim=-1)          # router logits in float32
            out = torch.zeros_like(x)
            for e in range(self.E):
                rows = (choice == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                gu = linear(x[rows].contiguous(), self.gate_up[e])          # the framework's own kernels per expert
                act = torch.empty((rows.numel(), self.I), dtype=x.dtype, device=x.device)
                kernels.swiglu(gu, act)
                out[rows] = linear(act, self.down[e])
            return out, None

    @register_position("toy_scaled_half_rotary")
    class ScaledHalfRotary(PositionEncoding):
        def __init__(self, prefix, rotary_dim, theta, factor):
            self.rotary_dim, self.theta, self.factor = rotary_dim, theta, factor

        def tables(self, ctx):
            j = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32, device=ctx.device)
            inv_freq = 1.0 / (self.theta ** (j / self.rotary_dim))
            angles = (ctx.positions.float() / self.factor)[:, None] * inv_freq[None, :]
            return angles.cos().contiguous(), angles.sin().contiguous()

    class ToyRoutedConfig(ModelConfig):
        architecture = "ToyRoutedForCausalLM"

        def __init__(self, data):
            self.data = data

        @classmethod
        def from_json(cls, data):
            return cls(dict(data))

        def to_json(self):
            return dict(self.data)

        def model_spec(self):
            d = self.data
            H, V, hd = d["hidden_size"], d["vocab_size"], d["head_dim"]
            norm = {"size": H, "eps": d["eps"]}
            layers = []
            for i in range(d["layers"]):
                attn = PartSpec("attention", {"hidden_size": H, "num_heads": d["heads"], "num_kv_heads": d["kv_heads"], "head_dim": hd,
                                              "scale": hd ** -0.5, "qk_norm": True, "qk_norm_eps": d["eps"], "position": "half",
                                              "rotary_dim": hd // 2}, f"blocks.{i}.attn")
                ff = PartSpec("toy_top1_experts", {"hidden_size": H, "intermediate_size": d["intermediate_size"],
                                                   "num_experts": d["experts"]}, f"blocks.{i}.moe")
                layers.append(LayerSpec("pre_norm_residual", attn, ff, PartSpec("rms_norm", norm, f"blocks.{i}.n1"),
                                        PartSpec("rms_norm", norm, f"blocks.{i}.n2")))
            return ModelSpec("ToyRoutedForCausalLM", V, H, PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H}, "embed"),
                             {"half": PartSpec("toy_scaled_half_rotary", {"rotary_dim": hd // 2, "theta": 5000.0, "factor": d["factor"]})},
                             tuple(layers), tuple(ScheduleEntry(i, i) for i in range(d["layers"])),
                             PartSpec("rms_norm", norm, "final"), PartSpec("linear_head", {"vocab_size": V, "hidden_size": H, "tied_to": None}, "head"), 512)

    register_architecture("ToyRoutedForCausalLM", ToyRoutedConfig)


TOY_ROUTED = {"architectures": ["ToyRoutedForCausalLM"], "hidden_size": 64, "vocab_size": 211, "intermediate_size": 48, "heads": 4,
              "kv_heads": 2, "head_dim": 32, "eps": 1e-5, "layers": 2, "experts": 3, "factor": 4.0}


def toy_routed_reference(w, ids):
    d = TOY_ROUTED
    T, nh, nkv, hd = len(ids), d["heads"], d["kv_heads"], d["head_dim"]
    x = w["embed.weight"][torch.tensor(ids)]
    rd = hd // 2
    j = torch.arange(0, rd, 2, dtype=torch.float32)
    angles = (torch.arange(T).float() / d["factor"])[:, None] * (1.0 / (5000.0 ** (j / rd)))[None, :]
    cos, sin = torch.cat((angles.cos(), angles.cos()), -1), torch.cat((angles.sin(), angles.sin()), -1)

    def rope(t):                                   # t [heads, T, hd]: only the first rd entries rotate
        head = t[..., :rd]
        return torch.cat((head * cos[None] + plain.rotate_half(head) * sin[None], t[..., rd:]), dim=-1)

    for i in range(d["layers"]):
        p = f"blocks.{i}"
        h = plain.rms_norm(x, w[f"{p}.n1.weight"], d["eps"])
        q = (h @ w[f"{p}.attn.q_proj.weight"].t()).view(T, nh, hd).transpose(0, 1)
        k = (h @ w[f"{p}.attn.k_proj.weight"].t()).view(T, nkv, hd).transpose(0, 1)
        v = (h @ w[f"{p}.attn.v_proj.weight"].t()).view(T, nkv, hd).transpose(0, 1)
        q = rope(plain.rms_norm(q, w[f"{p}.attn.q_norm.weight"], d["eps"]))
        k = rope(plain.rms_norm(k, w[f"{p}.attn.k_norm.weight"], d["eps"]))
        k, v = k.repeat_interleave(nh // nkv, 0), v.repeat_interleave(nh // nkv, 0)
        pos = torch.arange(T)
        scores = ((q @ k.transpose(1, 2)) * hd ** -0.5).masked_fill((pos[None, :] > pos[:, None])[None], float("-inf"))
        a = (torch.softmax(scores, -1) @ v).transpose(0, 1).reshape(T, nh * hd) @ w[f"{p}.attn.o_proj.weight"].t()
        x = x + a
        h = plain.rms_norm(x, w[f"{p}.n2.weight"], d["eps"])
        choice = (h @ w[f"{p}.moe.router.weight"].t()).argmax(-1)
        out = torch.zeros_like(h)
        for e in range(d["experts"]):
            rows = choice == e
            gu = h[rows] @ w[f"{p}.moe.experts.{e}.gate_up.weight"].t()
            I = d["intermediate_size"]
            out[rows] = (torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]) @ w[f"{p}.moe.experts.{e}.down.weight"].t()
        x = x + out
    return plain.rms_norm(x, w["final.weight"], d["eps"]) @ w["head.weight"].t()


def test_toy_routed_feed_forward_and_other_position_encoding(tmp_path):
    """A feed-forward that routes each token to one expert and a position encoding with its own angle
    formula and partial rotation, both registered from this file, through the unchanged step function:
    logits do not depend on how tokens are cut or batched (each token's expert depends on the token alone)."""
    _register_toy_routing_and_positions()
    from llm_pipeline_b200.weights import write_random_model
    from safetensors.torch import load_file
    folder = write_random_model(TOY_ROUTED, seed=21, out_dir=str(tmp_path), dtype=torch.float32, std=0.2)
    weights = load_file(f"{folder}/model.safetensors")
    assert "blocks.1.moe.experts.2.down.weight" in weights
    runner = H.make_runner(folder, torch.float32, page_size=8, num_pages=24, max_request_tokens=256)
    requests = {f"m{i}": H.random_tokens(TOY_ROUTED["vocab_size"], n, 40 + i) for i, n in enumerate((35, 8, 20, 27))}
    want = {rid: toy_routed_reference(weights, ids) for rid, ids in requests.items()}
    H.assert_close(H.replay(runner, H.cut_whole(requests)), want, 2e-4, "routed whole")
    H.assert_close(H.replay(runner, H.cut_tail_one_by_one(requests, tail=6)), want, 2e-4, "routed tail")
    H.assert_close(H.replay(runner, H.cut_mixed(requests, (5, 2, 9, 3), max_live=3)), want, 2e-4, "routed mixed")
    assert not runner.use_graphs and runner.graph_replays == 0   # the routed feed-forward does not declare graph_safe


# ------------------------------------------------------------------------------------------
# A toy mixer whose cache holds one latent vector per token (a width that is neither the hidden size nor a head
# size), and a toy block with four norms (one before and one after each of mixer and feed-forward). Both are
# registered from this file. The mixer attends over its own latents:
#   c_t = x_t Wc ;  p_tj = softmax_j<=t((x_t Wq) . c_j / sqrt(L)) ;  out_t = (sum_j p_tj c_j) Wo
# ------------------------------------------------------------------------------------------

def _register_toy_latent_and_sandwich():
    from llm_pipeline_b200.cache import TokenPagesSpec
    from llm_pipeline_b200.config import (LayerSpec, ModelConfig, ModelSpec, PartSpec, ScheduleEntry,
                                          register_architecture)
    from llm_pipeline_b200.parts import Block, Mixer, ResidualStream, register_block, register_mixer
    from llm_pipeline_b200.weights import ParamSpec

    @register_mixer("toy_latent_lookback")
    class LatentLookback(Mixer):
        def __init__(self, prefix, hidden_size, latent_size):
            self.prefix, self.H, self.L = prefix, hidden_size, latent_size

        def cache_spec(self):
            return TokenPagesSpec((self.L,), dtype=torch.float32)       # one vector per token, float32 whatever the model computes in

        def param_specs(self):
            p = self.prefix
            return {f"{p}.wc": ParamSpec((self.L, self.H)), f"{p}.wq": ParamSpec((self.L, self.H)), f"{p}.wo": ParamSpec((self.H, self.L))}

        def load(self, get):
            self.wc, self.wq, self.wo = (get(f"{self.prefix}.{n}", "matrix").float() for n in ("wc", "wq", "wo"))

        def forward(self, x, ctx, cache):
            page_size = cache.pages.shape[1]
            latents = cache.pages.view(-1, self.L)                        # [pages * page_size, L]
            c = x.float() @ self.wc.t()
            latents[ctx.slot_mapping[cache.group].long()] = c             # this step's tokens into their page slots
            q = x.float() @ self.wq.t()
            out = torch.empty((x.shape[0], self.H), dtype=x.dtype, device=x.device)
            row = 0
            for r, (start, n) in enumerate(zip(ctx.starts, ctx.q_lens)):
                pages = ctx.block_tables[cache.group][r, :-(-(start + n) // page_size)].long()
                mine = cache.pages[pages].reshape(-1, self.L)[:start + n]      # every latent of the request, through its block table
                scores = (q[row:row + n] @ mine.t()) * self.L ** -0.5
                keys = torch.arange(start + n, device=x.device)
                scores = scores.masked_fill(keys[None, :] > (start + torch.arange(n, device=x.device))[:, None], float("-inf"))
                out[row:row + n] = ((torch.softmax(scores, -1) @ mine) @ self.wo.t()).to(x.dtype)
                row += n
            return out, None

    @register_block("toy_sandwich")
    class Sandwich(Block):
        NORMS = ("mixer", "post_mixer", "feed_forward", "post_feed_forward")

        def forward(self, stream, ctx, cache):
            out, _ = self.mixer.forward(self.norms["mixer"].add_norm(stream, ctx), ctx, cache)
            stream.add(self._normed(self.norms["post_mixer"], out, ctx))
            out, _ = self.feed_forward.forward(self.norms["feed_forward"].add_norm(stream, ctx), ctx)
            stream.add(self._normed(self.norms["post_feed_forward"], out, ctx))

        @staticmethod
        def _normed(norm, out, ctx):
            return norm.add_norm(ResidualStream(out.float().contiguous()), ctx)      # the norm of a tensor that is no residual

    class ToyLatentConfig(ModelConfig):
        architecture = "ToyLatentForCausalLM"

        def __init__(self, data):
            self.data = data

        @classmethod
        def from_json(cls, data):
            return cls(dict(data))

        def to_json(self):
            return dict(self.data)

        def model_spec(self):
            d = self.data
            H, V = d["hidden_size"], d["vocab_size"]
            norm = lambda name: PartSpec("rms_norm", {"size": H, "eps": d["eps"]}, name)  # noqa: E731
            ff = lambda i: PartSpec("swiglu", {"hidden_size": H, "intermediate_size": d["intermediate_size"]}, f"layers.{i}.ff")  # noqa: E731
            attn = PartSpec("attention", {"hidden_size": H, "num_heads": d["heads"], "num_kv_heads": d["kv_heads"],
                                          "head_dim": d["head_dim"], "scale": d["head_dim"] ** -0.5, "qk_norm": False,
                                          "position": "rope"}, "layers.1.attn")
            layers = (
                LayerSpec("toy_sandwich", PartSpec("toy_latent_lookback", {"hidden_size": H, "latent_size": d["latent_size"]}, "layers.0.mix"),
                          ff(0), norm("layers.0.pre_mix"), norm("layers.0.pre_ff"),
                          norms={"post_mixer": norm("layers.0.post_mix"), "post_feed_forward": norm("layers.0.post_ff")}),
                LayerSpec("pre_norm_residual", attn, ff(1), norm("layers.1.n1"), norm("layers.1.n2")),
            )
            return ModelSpec("ToyLatentForCausalLM", V, H, PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H}, "embed"),
                             {"rope": PartSpec("rotary", {"rotary_dim": d["head_dim"], "theta": 10000.0})}, layers,
                             (ScheduleEntry(0, 0), ScheduleEntry(1, 1)), norm("final"),
                             PartSpec("linear_head", {"vocab_size": V, "hidden_size": H, "tied_to": "embed"}, "head"), 512)

    register_architecture("ToyLatentForCausalLM", ToyLatentConfig)


TOY_LATENT = {"architectures": ["ToyLatentForCausalLM"], "hidden_size": 40, "vocab_size": 89, "intermediate_size": 56, "heads": 2,
              "kv_heads": 1, "head_dim": 16, "eps": 1e-5, "latent_size": 24}


def toy_latent_reference(w, ids):
    d = TOY_LATENT
    T, L = len(ids), d["latent_size"]
    x = w["embed.weight"][torch.tensor(ids)]
    pos = torch.arange(T)
    causal = pos[None, :] > pos[:, None]
    norm = lambda t, name: plain.rms_norm(t, w[f"{name}.weight"], d["eps"])  # noqa: E731

    def ff(h, i):
        g, u = h @ w[f"layers.{i}.ff.gate_proj.weight"].t(), h @ w[f"layers.{i}.ff.up_proj.weight"].t()
        return (torch.nn.functional.silu(g) * u) @ w[f"layers.{i}.ff.down_proj.weight"].t()

    h = norm(x, "layers.0.pre_mix")
    c, q = h @ w["layers.0.mix.wc"].t(), h @ w["layers.0.mix.wq"].t()
    probs = torch.softmax(((q @ c.t()) * L ** -0.5).masked_fill(causal, float("-inf")), -1)
    x = x + norm((probs @ c) @ w["layers.0.mix.wo"].t(), "layers.0.post_mix")
    x = x + norm(ff(norm(x, "layers.0.pre_ff"), 0), "layers.0.post_ff")
    h = norm(x, "layers.1.n1")
    nh, nkv, hd = d["heads"], d["kv_heads"], d["head_dim"]
    cos, sin = plain.rope_cos_sin(pos, hd, 10000.0)
    qh = plain.apply_rope((h @ w["layers.1.attn.q_proj.weight"].t()).view(T, nh, hd).transpose(0, 1), cos, sin)
    kh = plain.apply_rope((h @ w["layers.1.attn.k_proj.weight"].t()).view(T, nkv, hd).transpose(0, 1), cos, sin)
    vh = (h @ w["layers.1.attn.v_proj.weight"].t()).view(T, nkv, hd).transpose(0, 1)
    kh, vh = kh.repeat_interleave(nh // nkv, 0), vh.repeat_interleave(nh // nkv, 0)
    probs = torch.softmax(((qh @ kh.transpose(1, 2)) * hd ** -0.5).masked_fill(causal[None], float("-inf")), -1)
    x = x + (probs @ vh).transpose(0, 1).reshape(T, nh * hd) @ w["layers.1.attn.o_proj.weight"].t()
    x = x + ff(norm(x, "layers.1.n2"), 1)
    return norm(x, "final") @ w["embed.weight"].t()


def test_toy_latent_cache_and_four_norm_block(tmp_path):
    """A cache whose payload per token is a single vector of a width of its own, beside an attention layer's keys and
    values (two groups of pages of different shapes and element types under one manager), and a block kind with four named
    norms: registered here, built from a model folder and stepped through the unchanged step function."""
    _register_toy_latent_and_sandwich()
    from llm_pipeline_b200.cache import CacheManager, KVPagesSpec, TokenPagesSpec
    from llm_pipeline_b200.weights import write_random_model
    from safetensors.torch import load_file
    folder = write_random_model(TOY_LATENT, seed=31, out_dir=str(tmp_path), dtype=torch.float32, std=0.2)
    weights = load_file(f"{folder}/model.safetensors")
    assert {"layers.0.post_mix.weight", "layers.0.post_ff.weight", "layers.0.mix.wc"} <= set(weights)
    runner = H.make_runner(folder, torch.float32, page_size=4, num_pages=40, max_request_tokens=256)
    specs = runner.model.cache_specs()
    assert isinstance(specs[0][0], TokenPagesSpec) and isinstance(specs[1][0], KVPagesSpec)
    cache = runner.cache
    assert len(cache.groups) == 2
    assert tuple(cache.pages_tensor(0).shape) == (40, 4, 24) and cache.pages_tensor(0).dtype == torch.float32
    assert tuple(cache.pages_tensor(1).shape) == (40, 2, 1, 4, 16)
    # a page id costs what its group's payloads say: 24 float32 per token here, keys and values of one head of 16 there
    assert CacheManager.bytes_per_page(specs, 4, torch.bfloat16) == [4 * 24 * 4, 4 * 2 * 16 * 2]
    requests = {f"l{i}": H.random_tokens(TOY_LATENT["vocab_size"], n, 90 + i) for i, n in enumerate((37, 6, 22, 29, 14))}
    want = {rid: toy_latent_reference(weights, ids) for rid, ids in requests.items()}
    H.assert_close(H.replay(runner, H.cut_whole(requests)), want, 1e-4, "latent whole")
    H.assert_close(H.replay(runner, H.cut_tail_one_by_one(requests, tail=8)), want, 1e-4, "latent tail")
    H.assert_close(H.replay(runner, H.cut_mixed(requests, (5, 2, 9, 3), max_live=3)), want, 1e-4, "latent mixed")
    assert cache.pages_reused > 0 and cache.num_live == 0
    # a block kind that is given too few norms says which are missing
    from llm_pipeline_b200.parts import lookup
    with pytest.raises(ValueError, match="post_mixer"):
        lookup("block", "toy_sandwich")(None, None, object(), object())


# ------------------------------------------------------------------------------------------
# A toy position encoding that reads two streams of positions, registered from this file: a token has a row and a
# column; the lower half of the rotation frequencies turns with the row, the upper half with the column. Requests
# bring their position ids with their tokens; the cache goes on counting places as always.
# ------------------------------------------------------------------------------------------

def _register_toy_grid_positions():
    from llm_pipeline_b200.config import (LayerSpec, ModelConfig, ModelSpec, PartSpec, ScheduleEntry,
                                          register_architecture)
    from llm_pipeline_b200.parts import PositionEncoding, register_position

    @register_position("toy_row_column_rotary")
    class RowColumnRotary(PositionEncoding):
        streams = 2
        graph_safe = True                  # torch operations on the step's static arrays only

        def __init__(self, prefix, rotary_dim, theta):
            self.rotary_dim, self.theta = rotary_dim, theta

        def tables(self, ctx):
            half = self.rotary_dim // 2
            j = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32, device=ctx.device)
            inv_freq = 1.0 / (self.theta ** (j / self.rotary_dim))
            ids = ctx.position_ids.float()                                   # [2, N]
            which = (torch.arange(half, device=ctx.device) >= half // 2).long()       # frequency j reads stream which[j]
            angles = ids[which].t() * inv_freq[None, :]                      # [N, half]
            return angles.cos().contiguous(), angles.sin().contiguous()

    class ToyGridConfig(ModelConfig):
        architecture = "ToyGridForCausalLM"

        def __init__(self, data):
            self.data = data

        @classmethod
        def from_json(cls, data):
            return cls(dict(data))

        def to_json(self):
            return dict(self.data)

        def model_spec(self):
            d = self.data
            H, V, hd = d["hidden_size"], d["vocab_size"], d["head_dim"]
            norm = {"size": H, "eps": d["eps"]}
            layers = []
            for i in range(d["layers"]):
                attn = PartSpec("attention", {"hidden_size": H, "num_heads": d["heads"], "num_kv_heads": d["kv_heads"], "head_dim": hd,
                                              "scale": hd ** -0.5, "qk_norm": True, "qk_norm_eps": d["eps"], "position": "grid"},
                                f"blocks.{i}.attn")
                ff = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": d["intermediate_size"]}, f"blocks.{i}.mlp")
                layers.append(LayerSpec("pre_norm_residual", attn, ff, PartSpec("rms_norm", norm, f"blocks.{i}.n1"),
                                        PartSpec("rms_norm", norm, f"blocks.{i}.n2")))
            return ModelSpec("ToyGridForCausalLM", V, H, PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H}, "embed"),
                             {"grid": PartSpec("toy_row_column_rotary", {"rotary_dim": hd, "theta": 300.0})},
                             tuple(layers), tuple(ScheduleEntry(i, i) for i in range(d["layers"])),
                             PartSpec("rms_norm", norm, "final"), PartSpec("linear_head", {"vocab_size": V, "hidden_size": H, "tied_to": None}, "head"), 512)

    register_architecture("ToyGridForCausalLM", ToyGridConfig)


TOY_GRID = {"architectures": ["ToyGridForCausalLM"], "hidden_size": 64, "vocab_size": 173, "intermediate_size": 80, "heads": 4,
            "kv_heads": 2, "head_dim": 32, "eps": 1e-5, "layers": 2}


def toy_grid_reference(w, ids, rows, cols):
    d = TOY_GRID
    T, nh, nkv, hd = len(ids), d["heads"], d["kv_heads"], d["head_dim"]
    x = w["embed.weight"][torch.tensor(ids)]
    half = hd // 2
    inv_freq = 1.0 / (300.0 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
    place = torch.stack([torch.tensor(rows).float()] * (half // 2) + [torch.tensor(cols).float()] * (half - half // 2), dim=1)
    angles = place * inv_freq[None, :]
    cos, sin = torch.cat((angles.cos(), angles.cos()), -1), torch.cat((angles.sin(), angles.sin()), -1)

    def rope(t):                                   # t [heads, T, hd]
        return t * cos[None] + plain.rotate_half(t) * sin[None]

    for i in range(d["layers"]):
        p = f"blocks.{i}"
        h = plain.rms_norm(x, w[f"{p}.n1.weight"], d["eps"])
        q = (h @ w[f"{p}.attn.q_proj.weight"].t()).view(T, nh, hd).transpose(0, 1)
        k = (h @ w[f"{p}.attn.k_proj.weight"].t()).view(T, nkv, hd).transpose(0, 1)
        v = (h @ w[f"{p}.attn.v_proj.weight"].t()).view(T, nkv, hd).transpose(0, 1)
        q = rope(plain.rms_norm(q, w[f"{p}.attn.q_norm.weight"], d["eps"]))
        k = rope(plain.rms_norm(k, w[f"{p}.attn.k_norm.weight"], d["eps"]))
        k, v = k.repeat_interleave(nh // nkv, 0), v.repeat_interleave(nh // nkv, 0)
        pos = torch.arange(T)
        scores = ((q @ k.transpose(1, 2)) * hd ** -0.5).masked_fill((pos[None, :] > pos[:, None])[None], float("-inf"))
        x = x + (torch.softmax(scores, -1) @ v).transpose(0, 1).reshape(T, nh * hd) @ w[f"{p}.attn.o_proj.weight"].t()
        h = plain.rms_norm(x, w[f"{p}.n2.weight"], d["eps"])
        I = d["intermediate_size"]
        x = x + (torch.nn.functional.silu(h @ w[f"{p}.mlp.gate_proj.weight"].t()) * (h @ w[f"{p}.mlp.up_proj.weight"].t())) \
            @ w[f"{p}.mlp.down_proj.weight"].t()
        assert w[f"{p}.mlp.gate_proj.weight"].shape[0] == I
    return plain.rms_norm(x, w["final.weight"], d["eps"]) @ w["head.weight"].t()


def test_toy_position_encoding_with_two_streams_of_positions(tmp_path):
    """A position encoding that reads a row and a column for every token, registered from this file: requests bring
    both with their tokens through the unchanged step function (whole, in portions, mixed, the tail token by token
    through replayed graphs), and through the generation engine, where generated tokens go on from the largest id of
    the prompt. Without position ids every stream holds the tokens' places."""
    _register_toy_grid_positions()
    from llm_pipeline_b200.engine import StepEntry
    from llm_pipeline_b200.engine.generate import GenerationEngine
    from llm_pipeline_b200.models import load_model
    from llm_pipeline_b200.sampling import SamplingConfig
    from llm_pipeline_b200.weights import write_random_model
    from safetensors.torch import load_file
    folder = write_random_model(TOY_GRID, seed=33, out_dir=str(tmp_path), dtype=torch.float32, std=0.2)
    weights = load_file(f"{folder}/model.safetensors")
    runner = H.make_runner(folder, torch.float32, page_size=8, num_pages=40, max_request_tokens=256)
    assert runner.position_streams == 2 and runner.use_graphs
    requests = {f"g{i}": H.random_tokens(TOY_GRID["vocab_size"], n, 60 + i) for i, n in enumerate((45, 8, 52, 27))}
    # a grid of 7 columns, row by row, the second request starting in the middle of the grid
    place = {rid: ([(t + 3 * i) // 7 for t in range(len(toks))], [(t + 3 * i) % 7 for t in range(len(toks))])
             for i, (rid, toks) in enumerate(requests.items())}
    want = {rid: toy_grid_reference(weights, toks, *place[rid]) for rid, toks in requests.items()}

    def replay(steps):
        rows, done = {}, {rid: 0 for rid in requests}
        for entries, end in steps:
            batch = []
            for rid, toks, wanted in entries:
                a, b = done[rid], done[rid] + len(toks)
                batch.append(StepEntry(rid, toks, wanted, [place[rid][0][a:b], place[rid][1][a:b]]))
                done[rid] = b
            logits = runner.step(batch)
            cursor = 0
            for rid, _toks, wanted in entries:
                rows.setdefault(rid, []).append(logits[cursor:cursor + len(wanted)].float().cpu())
                cursor += len(wanted)
            for rid in end:
                runner.release(rid)
            runner.cache.check()
        return {rid: torch.cat(parts) for rid, parts in rows.items()}

    H.assert_close(replay(H.cut_whole(requests)), want, 2e-4, "grid whole")
    H.assert_close(replay(H.cut_portions(requests, (5, 2, 9, 1))), want, 2e-4, "grid portions")
    H.assert_close(replay(H.cut_mixed(requests, (5, 2, 9, 3), max_live=3)), want, 2e-4, "grid mixed")
    before = runner.graph_replays
    H.assert_close(replay(H.cut_tail_one_by_one(requests, tail=20)), want, 2e-4, "grid tail")
    assert runner.graph_replays > before + 40
    # without position ids: the place in the request in both streams
    toks = requests["g1"]
    got = runner.step([StepEntry("plain", toks, list(range(len(toks))))]).float().cpu()
    runner.release("plain")
    assert float((got - toy_grid_reference(weights, toks, list(range(len(toks))), list(range(len(toks))))).abs().max()) < 2e-4
    with pytest.raises(ValueError, match="position ids of another shape"):
        runner.step([StepEntry("bad", toks, [0], [list(range(len(toks)))])])
    # through the generation engine: greedy tokens against the plain formulas, generated tokens at max id + 1, + 2, ...
    config, model = load_model(folder, "cuda:0", torch.float32)
    engine = GenerationEngine(model, config, page_size=8, num_pages=40, max_num_seqs=4, max_num_batched_tokens=16, max_model_len=256)
    greedy = SamplingConfig(temperature=0.0)
    ids = {}
    for rid in ("g0", "g3"):
        ids[rid] = engine.add_request(requests[rid], max_tokens=6, sampling=greedy, ignore_eos=True, position_ids=place[rid])
    outputs = {}
    while engine.has_unfinished():
        for request in engine.step():
            outputs[request.req_id] = list(request.output)
    for rid in ("g0", "g3"):
        toks, rows, cols = list(requests[rid]), list(place[rid][0]), list(place[rid][1])
        after = 1 + max(max(rows), max(cols))
        for step in range(6):
            logits = toy_grid_reference(weights, toks, rows, cols)[-1]
            top2 = logits.topk(2).values
            token = int(logits.argmax())
            if float(top2[0] - top2[1]) > 1e-3:                       # a near tie may fall either way
                assert outputs[ids[rid]][step] == token, (rid, step)
            toks.append(outputs[ids[rid]][step])
            rows.append(after + step)
            cols.append(after + step)
    with pytest.raises(ValueError, match="position ids must be"):
        engine.add_request(requests["g1"], position_ids=[place["g1"][0]])
