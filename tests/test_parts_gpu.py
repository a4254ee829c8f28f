"""Each part alone against the plain implementation, and parts that the framework does not
ship, defined here: a mixer with state of its own, a feed-forward with routing, another
position encoding, a schedule that runs a layer twice and lets a layer read another's pages.
None of them needs a change to the framework's files."""
from dataclasses import dataclass

import pytest
import torch

import helpers as H
import qwen3_plain as P

pytestmark = pytest.mark.gpu


def _env(dtype=torch.float32):
    from binfer_b200.engine import make_env
    return make_env(dtype)


def _ctx_for(runner, items):
    runner.reserve(items)
    return runner.build_context(items)


def _tiny_runner(which="A", dtype=torch.float32, tmp=None, **kw):
    from binfer_b200.engine import make_runner, model_from_dir
    env = _env(dtype)
    d = H.make_model_dir(tmp, which, dtype)
    model = model_from_dir(d, env)
    return model, make_runner(model, env, page_size=H.TINY[which]["page_size"], num_pages=64, **kw), d


# ------------------------------------------------------------------ parts alone
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1.2e-2)])
def test_norm_part_folds_the_pending_add(cuda_device, dtype, tol):
    from binfer_b200.config import NormSpec
    from binfer_b200.parts import ResidualStream, build_norm
    from binfer_b200.weights import ParamSpec
    env = _env(dtype)
    norm = build_norm(NormSpec(eps=3e-5), 100, "n.weight", env)
    assert [(s.name, s.shape, s.role) for s in norm.param_specs()] == [("n.weight", (100,), "vector")]
    w = 1 + 0.1 * torch.randn(100)
    norm.load(lambda spec: w.to(env.device))
    x = torch.randn(6, 100, device=env.device)
    delta = torch.randn(6, 100, device=env.device).to(dtype)
    stream = ResidualStream(x.clone())
    stream.add(delta)
    y = norm.forward(stream)
    want_x = x.double() + delta.double()
    assert stream.pending is None
    assert H.rel_err(stream.x.cpu(), want_x.cpu()) < 2e-6
    assert H.rel_err(y.cpu(), P.rms_norm(want_x.cpu(), w.double(), 3e-5)) < tol


def test_feed_forward_part(cuda_device, tmp_path):
    model, runner, d = _tiny_runner("B", tmp=tmp_path)
    raw, w = H.read_model_dir(d)
    ffn = model.blocks[1].ffn
    assert [s.shape for s in ffn.param_specs()] == [(160, 96), (160, 96), (96, 160)]
    x = torch.randn(13, 96, device=cuda_device)
    got = ffn.forward(x, None)
    want = P.swiglu_mlp(x.double().cpu(), {k: v.double() for k, v in w.items()},
                        "model.layers.1.mlp.")
    assert H.rel_err(got.cpu(), want) < 5e-6


def test_position_encoding_part(cuda_device):
    from binfer_b200.config import RopeSpec
    from binfer_b200.parts import build_position
    rope = build_position(RopeSpec(theta=1e6, rotary_dim=32, factor=4.0), 32, _env())
    i = torch.arange(16, dtype=torch.float64)
    assert torch.equal(rope.inv_freq.cpu(), ((1e6 ** (-2 * i / 32)) / 4.0).float())
    with pytest.raises(ValueError):
        build_position(RopeSpec(rotary_dim=48), 32, _env())


@pytest.mark.parametrize("which", ["A", "B", "W"])
def test_attention_part_alone(cuda_device, tmp_path, which):
    """The mixer on normed activations of a whole request, then again as two portions."""
    from binfer_b200.engine.runner import StepItem
    model, runner, d = _tiny_runner(which, tmp=tmp_path)
    raw, w = H.read_model_dir(d)
    c = P.read_config(raw)
    layer = 1
    mixer = model.blocks[layer].mixer
    view = runner.views[layer]
    n = 45
    x = torch.randn(n, c["hidden"], device=cuda_device)
    want = P.attention_block(x.double().cpu(), {k: v.double() for k, v in w.items()},
                             f"model.layers.{layer}.self_attn.", c, torch.arange(n),
                             c["windows"][layer])
    runner.add_request("r")
    ctx = _ctx_for(runner, [StepItem("r", list(range(n)), [])])
    got = mixer.forward(x, ctx, view)
    assert H.rel_err(got.cpu(), want) < 5e-6
    runner.free_request("r")
    runner.add_request("s")                         # the same in two portions, cut at 17
    ctx = _ctx_for(runner, [StepItem("s", list(range(17)), [])])
    a = mixer.forward(x[:17], ctx, view)
    runner.cache.commit("s", 17)
    ctx = _ctx_for(runner, [StepItem("s", list(range(17, n)), [])])
    b = mixer.forward(x[17:], ctx, view)
    assert torch.equal(torch.cat([a, b]), got)


def test_block_part_alone(cuda_device, tmp_path):
    from binfer_b200.engine.runner import StepItem
    from binfer_b200.parts import ResidualStream
    model, runner, d = _tiny_runner("B", tmp=tmp_path)
    raw, w = H.read_model_dir(d)
    c = P.read_config(raw)
    n = 21
    x = torch.randn(n, 96, device=cuda_device)
    want = P.decoder_layer(x.double().cpu(), {k: v.double() for k, v in w.items()}, 2, c,
                           torch.arange(n))
    runner.add_request("r")
    ctx = _ctx_for(runner, [StepItem("r", list(range(n)), [])])
    stream = ResidualStream(x.clone())
    model.blocks[2].forward(stream, ctx, runner.views[2])
    stream.flush()
    assert H.rel_err(stream.x.cpu(), want) < 5e-6


# --------------------------------------------- parts and models defined by the test
@dataclass(frozen=True)
class DecaySpec:
    kind: str = "test_decay_mixer"
    decay: float = 0.9


def _register_toy_parts():
    """A mixer with fixed-size state per request (an exponentially decaying sum of the
    projected inputs) and a feed-forward with top-1 routing over two experts; plain tensor
    code, float32.  (The position encodings: ``_register_toy_positions``.)"""
    from binfer_b200.cache import StateNeed
    from binfer_b200.parts import FeedForward, Mixer, register_ffn, register_mixer
    from binfer_b200.weights import ParamSpec

    class DecayMixer(Mixer):
        def __init__(self, spec, hidden, prefix, env):
            self.spec, self.hidden, self.prefix, self.env = spec, hidden, prefix, env

        def param_specs(self):
            return [ParamSpec(self.prefix + "in.weight", (self.hidden, self.hidden))]

        def load(self, get):
            self.w = get(self.param_specs()[0])

        def state_need(self):
            return StateNeed((self.hidden,), "float32")

        def forward(self, x, ctx, view):
            u = x.float() @ self.w.float().T
            out = torch.empty_like(u)
            starts = ctx.q_start.tolist()
            slots = ctx.state_slots.tolist()
            for b in range(ctx.B):
                s = view.state[slots[b]]
                for t in range(starts[b], starts[b + 1]):
                    s.mul_(self.spec.decay).add_(u[t])
                    out[t] = s
            return out.to(x.dtype)

    @dataclass(frozen=True)
    class RoutedSpec:
        kind: str = "test_routed_ffn"
        experts: int = 2

    class RoutedFFN(FeedForward):
        def __init__(self, spec, hidden, prefix, env):
            self.spec, self.hidden, self.prefix = spec, hidden, prefix

        def param_specs(self):
            e = self.spec.experts
            return [ParamSpec(self.prefix + "router.weight", (e, self.hidden)),
                    ParamSpec(self.prefix + "experts.weight", (e * self.hidden, self.hidden))]

        def load(self, get):
            r, e = self.param_specs()
            self.router, self.experts = get(r), get(e).view(self.spec.experts, self.hidden, -1)

        def forward(self, x, ctx):
            choice = (x.float() @ self.router.float().T).argmax(-1)      # router logits in float
            return torch.einsum("th,thk->tk", x.float(),
                                self.experts.float()[choice].transpose(1, 2)).to(x.dtype)

    register_mixer("test_decay_mixer", DecayMixer)
    register_ffn("test_routed_ffn", RoutedFFN)
    return DecaySpec, RoutedSpec


def _toy_spec(layers, schedule, vocab=50, hidden=32):
    from binfer_b200.config import ModelSpec, NameLayout, NormSpec
    return ModelSpec(architecture="ToyForCausalLM", hidden_size=hidden, vocab_size=vocab,
                     layers=tuple(layers), schedule=tuple(schedule), final_norm=NormSpec(eps=1e-5),
                     tie_word_embeddings=True, names=NameLayout())


def test_toy_mixer_with_state_and_routed_ffn(cuda_device):
    """Registered, built from specs, loaded by name, and stepped whole and in portions: the
    carried state makes the portions agree with the whole."""
    from binfer_b200.config import (AttentionSpec, GatedMLPSpec, LayerSpec, NormSpec, RopeSpec,
                                    ScheduleEntry, register_architecture, parse_config)
    from binfer_b200.engine import make_runner
    from binfer_b200.engine.runner import StepItem
    from binfer_b200.parts import build_model, param_specs_for
    from binfer_b200.weights import TensorSource, random_tensors
    DecaySpecT, RoutedSpecT = _register_toy_parts()
    norm = NormSpec(eps=1e-5)
    attn = AttentionSpec(num_heads=2, num_kv_heads=1, head_dim=16, position=RopeSpec(theta=100.0))
    layers = [LayerSpec(mixer=DecaySpecT(decay=0.8), ffn=RoutedSpecT(), norm=norm),
              LayerSpec(mixer=attn, ffn=GatedMLPSpec(intermediate_size=48), norm=norm),
              LayerSpec(mixer=DecaySpecT(decay=0.5), ffn=GatedMLPSpec(intermediate_size=40), norm=norm)]
    spec = _toy_spec(layers, [ScheduleEntry(i) for i in range(3)])
    # a whole architecture, chosen by config.json's name like any other
    register_architecture("ToyForCausalLM", lambda raw: type("C", (), {"to_spec": lambda self: spec})())
    assert parse_config({"architectures": ["ToyForCausalLM"]}).to_spec() is spec
    names = [s.name for s in param_specs_for(spec)]
    assert "model.layers.0.self_attn.in.weight" in names
    assert "model.layers.0.mlp.router.weight" in names
    env = _env()
    model = build_model(spec, env, TensorSource.from_dict(
        random_tensors(param_specs_for(spec), seed=1, std=0.2, norm_std=0.05)))
    assert [n is not None for n in model.kv_needs()] == [False, True, False]
    assert [n is not None for n in model.state_needs()] == [True, False, True]
    toks = H.random_tokens(23, 50, 3)

    def run(cuts):
        runner = make_runner(model, env, page_size=4, num_pages=16, max_requests=2)
        runner.add_request("other")               # another request's state must not leak in
        runner.step([StepItem("other", toks[::-1][:5], [])])
        runner.add_request("r")
        rows, a = [], 0
        for n in cuts:
            rows.append(runner.step([StepItem("r", toks[a:a + n], list(range(n)))]).clone())
            a += n
        return torch.cat(rows)

    whole = run([23])
    assert torch.isfinite(whole).all() and float(whole.abs().max()) > 0
    parts = run([7, 1, 2, 13])
    assert H.rel_err(parts, whole) < 1e-5
    # a slot that is handed out again starts from zero state
    runner = make_runner(model, env, page_size=4, num_pages=16, max_requests=1)
    runner.add_request("a")
    first = runner.step([StepItem("a", toks, [22])]).clone()
    runner.free_request("a")
    runner.add_request("b")
    assert torch.equal(runner.step([StepItem("b", toks, [22])]), first)


@dataclass(frozen=True)
class StretchedRotarySpec:
    """Rotations with frequencies base * (i + 1) over the first ``rotary_dim`` features."""
    kind: str = "test_stretched_rotary"
    base: float = 0.03
    rotary_dim: int = 8


@dataclass(frozen=True)
class BucketShiftSpec:
    """A learned vector per bucket of ``width`` positions, added to every q and k head."""
    kind: str = "test_bucket_shift"
    buckets: int = 6
    width: int = 3


def _register_toy_positions():
    from binfer_b200.parts import PositionEncoding, register_position
    from binfer_b200.weights import ParamSpec

    class StretchedRotary(PositionEncoding):
        def __init__(self, spec, head_dim, env):
            i = torch.arange(spec.rotary_dim // 2, dtype=torch.float32)
            self.inv_freq = (spec.base * (i + 1)).to(env.device)

    class BucketShift(PositionEncoding):
        def __init__(self, spec, head_dim, env):
            self.spec, self.head_dim = spec, head_dim

        def param_specs(self, prefix):
            self.table_spec = ParamSpec(prefix + "position_table.weight",
                                        (self.spec.buckets, self.head_dim))
            return [self.table_spec]

        def load(self, get):
            self.table = get(self.table_spec)

        def apply(self, q, k, positions):
            b = (positions.long() // self.spec.width).clamp(max=self.spec.buckets - 1)
            shift = self.table[b].to(q.dtype)[:, None, :]
            q.add_(shift)
            k.add_(shift)

    register_position("test_stretched_rotary", StretchedRotary)
    register_position("test_bucket_shift", BucketShift)


# (the bounds of the replay tests: largest difference and root mean square, over the logits')
@pytest.mark.parametrize("dtype,tol,tol_rms", [(torch.float32, 2e-5, 5e-6),
                                               (torch.bfloat16, 3e-2, 1e-2)])
def test_toy_position_encodings(cuda_device, dtype, tol, tol_rms):
    """Two position encodings that the framework does not ship, registered here: a rotation
    with another table of frequencies (it runs inside the fused kernel) and an additive one
    with a tensor of its own (it runs between the head norms and the store).  A third layer
    execution reads the second one's pages, so that the encoding meets a mixer that stores
    nothing.  Whole and in portions, against a plain restatement."""
    from binfer_b200.config import (AttentionSpec, GatedMLPSpec, LayerSpec, NormSpec,
                                    ScheduleEntry)
    from binfer_b200.engine import make_runner
    from binfer_b200.engine.runner import StepItem
    from binfer_b200.parts import build_model, param_specs_for
    from binfer_b200.weights import TensorSource, random_tensors
    _register_toy_positions()
    norm = NormSpec(eps=1e-6)
    stretched, shift = StretchedRotarySpec(), BucketShiftSpec()
    layers = [LayerSpec(mixer=AttentionSpec(num_heads=4, num_kv_heads=2, head_dim=16,
                                            position=stretched),
                        ffn=GatedMLPSpec(intermediate_size=24), norm=norm),
              LayerSpec(mixer=AttentionSpec(num_heads=4, num_kv_heads=1, head_dim=16, qk_norm=True,
                                            position=shift),
                        ffn=GatedMLPSpec(intermediate_size=40), norm=norm)]
    sched = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1, cache_from=1)]
    spec = _toy_spec(layers, sched, vocab=40, hidden=32)
    names = [s.name for s in param_specs_for(spec)]
    assert "model.layers.1.self_attn.position_table.weight" in names
    assert "model.layers.0.self_attn.position_table.weight" not in names
    env = _env(dtype)
    # (weights small enough that the scores stay of order one: with a sharp softmax the
    # bfloat16 rounding of this 32-wide model alone exceeds the bounds)
    weights = random_tensors(param_specs_for(spec), seed=9, std=0.1, norm_std=0.05)
    model = build_model(spec, env, TensorSource.from_dict(weights))
    n = 19
    toks = H.random_tokens(n, 40, 5)

    w = {k: v.double() for k, v in weights.items()}
    if dtype == torch.bfloat16:
        w = {k: v.to(torch.bfloat16).double() for k, v in w.items()}
    pos = torch.arange(n)
    x = P.embedding(torch.tensor(toks), w["model.embed_tokens.weight"])
    kept = {}
    for e, entry in enumerate(sched):
        p = f"model.layers.{entry.layer}."
        a, m = p + "self_attn.", layers[entry.layer].mixer
        h = P.rms_norm(x, w[p + "input_layernorm.weight"], 1e-6)
        q = (h @ w[a + "q_proj.weight"].T).view(n, m.num_heads, 16)
        k = (h @ w[a + "k_proj.weight"].T).view(n, m.num_kv_heads, 16)
        v = (h @ w[a + "v_proj.weight"].T).view(n, m.num_kv_heads, 16)
        if m.qk_norm:
            q = P.rms_norm(q, w[a + "q_norm.weight"], 1e-6)
            k = P.rms_norm(k, w[a + "k_norm.weight"], 1e-6)
        if entry.layer == 0:
            i = torch.arange(stretched.rotary_dim // 2, dtype=torch.float32)
            ang = pos.float()[:, None] * (stretched.base * (i + 1))[None, :]
            q, k = P.apply_rope(q, ang), P.apply_rope(k, ang)
        else:
            b = (pos // shift.width).clamp(max=shift.buckets - 1)
            add = w[a + "position_table.weight"][b][:, None, :]
            q, k = q + add, k + add
        kept[e] = (k, v)
        if entry.cache_from is not None:
            k, v = kept[entry.cache_from]
        att = P.causal_attention(q, k, v, 16 ** -0.5).reshape(n, -1) @ w[a + "o_proj.weight"].T
        x = x + att
        h = P.rms_norm(x, w[p + "post_attention_layernorm.weight"], 1e-6)
        x = x + P.swiglu_mlp(h, w, p + "mlp.")
    want = P.rms_norm(x, w["model.norm.weight"], 1e-5) @ w["model.embed_tokens.weight"].T

    for cuts in ([n], [6, 1, 2, 10]):
        runner = make_runner(model, env, page_size=4, num_pages=8, max_requests=2)
        runner.add_request("r")
        rows, at = [], 0
        for c in cuts:
            rows.append(runner.step([StepItem("r", toks[at:at + c], list(range(c)))]).clone())
            at += c
        got = torch.cat(rows).float().cpu()
        assert H.rel_err(got, want) < tol and H.rel_rms(got, want) < tol_rms, cuts


def _register_sandwich_block():
    """An arrangement of a layer's parts that the framework does not ship: every sublayer has a
    norm before it and one after it (``x += norm_b(mixer(norm_a(x)))``), four norms a layer,
    whose names come from the family's :class:`NameLayout`."""
    from binfer_b200.parts import build_ffn, build_mixer, build_norm, register_block
    from binfer_b200.parts.base import ResidualStream

    class SandwichBlock:
        def __init__(self, spec, hidden, names, index, env):
            p = names.layer_prefix.format(i=index)
            self.norms = {role: build_norm(spec.norm, hidden, f"{p}{names.norm(role)}.weight", env)
                          for role in ("input", "post_mixer", "pre_ffn", "post_ffn")}
            self.mixer = build_mixer(spec.mixer, hidden, f"{p}{names.mixer}.", env)
            self.ffn = build_ffn(spec.ffn, hidden, f"{p}{names.ffn}.", env)

        def parts(self):
            return [*self.norms.values(), self.mixer, self.ffn]

        def param_specs(self):
            return [s for part in self.parts() for s in part.param_specs()]

        def load(self, get):
            for part in self.parts():
                part.load(get)

        def _normed(self, role, h):
            """The norm ``role`` of a sublayer's output (a tensor, not the stream)."""
            return self.norms[role].forward(ResidualStream(h.float().contiguous()))

        def forward(self, stream, ctx, view):
            h = self.mixer.forward(self.norms["input"].forward(stream), ctx, view)
            stream.add(self._normed("post_mixer", h))
            h = self.ffn.forward(self.norms["pre_ffn"].forward(stream), ctx)
            stream.add(self._normed("post_ffn", h))

    register_block("test_sandwich", SandwichBlock)


@pytest.mark.parametrize("dtype,tol,tol_rms", [(torch.float32, 2e-5, 5e-6),
                                               (torch.bfloat16, 3e-2, 1e-2)])
def test_toy_block_arrangement(cuda_device, dtype, tol, tol_rms):
    """Another arrangement of a layer's parts, registered here, beside the shipped one in one
    model: its four norms get their names from the family's layout, the weights load by those
    names, and whole and cut prompts agree with a plain restatement."""
    from binfer_b200.config import (AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, NameLayout,
                                    NormSpec, RopeSpec, ScheduleEntry)
    from binfer_b200.engine import make_runner
    from binfer_b200.engine.runner import StepItem
    from binfer_b200.parts import build_model, param_specs_for
    from binfer_b200.weights import TensorSource, random_tensors
    _register_sandwich_block()
    norm = NormSpec(eps=1e-6)
    rope = RopeSpec(theta=50.0)
    attn = AttentionSpec(num_heads=4, num_kv_heads=2, head_dim=16, position=rope)
    layers = [LayerSpec(mixer=attn, ffn=GatedMLPSpec(intermediate_size=24), norm=norm,
                        block="test_sandwich"),
              LayerSpec(mixer=attn, ffn=GatedMLPSpec(intermediate_size=40), norm=norm)]
    names = NameLayout(more_norms=(("pre_ffn", "pre_feedforward_layernorm"),
                                   ("post_ffn", "post_feedforward_layernorm")))
    spec = ModelSpec(architecture="ToySandwichForCausalLM", hidden_size=32, vocab_size=40,
                     layers=tuple(layers), schedule=(ScheduleEntry(0), ScheduleEntry(1)),
                     final_norm=NormSpec(eps=1e-5), tie_word_embeddings=True, names=names)
    wanted = [s.name for s in param_specs_for(spec)]
    assert "model.layers.0.pre_feedforward_layernorm.weight" in wanted
    assert "model.layers.0.post_feedforward_layernorm.weight" in wanted
    assert "model.layers.1.pre_feedforward_layernorm.weight" not in wanted
    with pytest.raises(KeyError, match="known"):
        NameLayout().norm("pre_ffn")
    env = _env(dtype)
    weights = random_tensors(param_specs_for(spec), seed=4, std=0.1, norm_std=0.05)
    model = build_model(spec, env, TensorSource.from_dict(weights))
    n = 17
    toks = H.random_tokens(n, 40, 8)

    w = {k: v.double() for k, v in weights.items()}
    if dtype == torch.bfloat16:
        w = {k: v.to(torch.bfloat16).double() for k, v in w.items()}
    pos = torch.arange(n)
    ang = P.rope_angles(pos, 16, 50.0)
    x = P.embedding(torch.tensor(toks), w["model.embed_tokens.weight"])

    def attention(h, a):
        q = (h @ w[a + "q_proj.weight"].T).view(n, 4, 16)
        k = (h @ w[a + "k_proj.weight"].T).view(n, 2, 16)
        v = (h @ w[a + "v_proj.weight"].T).view(n, 2, 16)
        q, k = P.apply_rope(q, ang), P.apply_rope(k, ang)
        return P.causal_attention(q, k, v, 16 ** -0.5).reshape(n, -1) @ w[a + "o_proj.weight"].T

    p0, p1 = "model.layers.0.", "model.layers.1."
    h = attention(P.rms_norm(x, w[p0 + "input_layernorm.weight"], 1e-6), p0 + "self_attn.")
    x = x + P.rms_norm(h, w[p0 + "post_attention_layernorm.weight"], 1e-6)
    h = P.swiglu_mlp(P.rms_norm(x, w[p0 + "pre_feedforward_layernorm.weight"], 1e-6), w, p0 + "mlp.")
    x = x + P.rms_norm(h, w[p0 + "post_feedforward_layernorm.weight"], 1e-6)
    x = x + attention(P.rms_norm(x, w[p1 + "input_layernorm.weight"], 1e-6), p1 + "self_attn.")
    x = x + P.swiglu_mlp(P.rms_norm(x, w[p1 + "post_attention_layernorm.weight"], 1e-6), w, p1 + "mlp.")
    want = P.rms_norm(x, w["model.norm.weight"], 1e-5) @ w["model.embed_tokens.weight"].T

    for cuts in ([n], [5, 2, 1, 9]):
        runner = make_runner(model, env, page_size=4, num_pages=10, max_requests=1)
        runner.add_request("r")
        rows, at = [], 0
        for c in cuts:
            rows.append(runner.step([StepItem("r", toks[at:at + c], list(range(c)))]).clone())
            at += c
        got = torch.cat(rows).float().cpu()
        assert H.rel_err(got, want) < tol and H.rel_rms(got, want) < tol_rms, cuts


def test_schedule_runs_a_layer_twice_and_shares_pages(cuda_device):
    """The order of execution is data: layer 0 runs twice (two caches of its own), and the
    last entry reads the pages that the first one wrote."""
    from binfer_b200.config import (AttentionSpec, GatedMLPSpec, LayerSpec, NormSpec, RopeSpec,
                                    ScheduleEntry)
    from binfer_b200.engine import make_runner
    from binfer_b200.engine.runner import StepItem
    from binfer_b200.parts import build_model, param_specs_for
    from binfer_b200.weights import TensorSource, random_tensors
    norm = NormSpec(eps=1e-6)
    attn = AttentionSpec(num_heads=4, num_kv_heads=2, head_dim=8, qk_norm=True,
                         position=RopeSpec(theta=1000.0))
    layer = LayerSpec(mixer=attn, ffn=GatedMLPSpec(intermediate_size=24), norm=norm)
    sched = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_from=0)]
    spec = _toy_spec([layer, layer], sched, vocab=40, hidden=32)
    env = _env()
    weights = random_tensors(param_specs_for(spec), seed=4, std=0.3, norm_std=0.05)
    model = build_model(spec, env, TensorSource.from_dict(weights))
    assert [n is not None for n in model.kv_needs()] == [True, True, True, False]
    toks = H.random_tokens(19, 40, 8)

    # plain restatement of this schedule from the plain parts
    w = {k: v.double() for k, v in weights.items()}
    c = dict(heads=4, kv_heads=2, head_dim=8, eps=1e-6, theta=1000.0, factor=1.0)
    pos = torch.arange(19)
    x = P.embedding(torch.tensor(toks), w["model.embed_tokens.weight"])
    k0 = v0 = None
    for e, entry in enumerate(sched):
        p = f"model.layers.{entry.layer}."
        n = P.rms_norm(x, w[p + "input_layernorm.weight"], 1e-6)
        a = p + "self_attn."
        q = P.rms_norm((n @ w[a + "q_proj.weight"].T).view(19, 4, 8), w[a + "q_norm.weight"], 1e-6)
        k = P.rms_norm((n @ w[a + "k_proj.weight"].T).view(19, 2, 8), w[a + "k_norm.weight"], 1e-6)
        v = (n @ w[a + "v_proj.weight"].T).view(19, 2, 8)
        ang = P.rope_angles(pos, 8, 1000.0)
        q, k = P.apply_rope(q, ang), P.apply_rope(k, ang)
        if e == 0:
            k0, v0 = k, v
        if entry.cache_from is not None:
            k, v = k0, v0
        att = P.causal_attention(q, k, v, 8 ** -0.5).reshape(19, 32) @ w[a + "o_proj.weight"].T
        x = x + att
        n = P.rms_norm(x, w[p + "post_attention_layernorm.weight"], 1e-6)
        x = x + P.swiglu_mlp(n, w, p + "mlp.")
    want = P.rms_norm(x, w["model.norm.weight"], 1e-5) @ w["model.embed_tokens.weight"].T

    for cuts in ([19], [5, 1, 1, 12]):
        runner = make_runner(model, env, page_size=4, num_pages=8, max_requests=2)
        runner.add_request("r")
        rows, a = [], 0
        for n in cuts:
            rows.append(runner.step([StepItem("r", toks[a:a + n], list(range(n)))]).clone())
            a += n
        assert H.rel_err(torch.cat(rows).cpu(), want) < 2e-5, cuts


def _plain_scored_attention(q, k, v, scale, softcap, slopes, sinks):
    """softmax over keys j <= p of cap(q.k * scale) + slope_h (j - p), with a sink logit per
    head in the denominator; plain and whole, for the test below."""
    T, heads, d = q.shape
    group = heads // k.shape[1]
    pos = torch.arange(T)
    out = torch.empty_like(q)
    for h in range(heads):
        s = (q[:, h] @ k[:, h // group].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        if slopes is not None:
            s = s + slopes[h] * (pos[None, :] - pos[:, None])
        s = s.masked_fill(pos[None, :] > pos[:, None], float("-inf"))
        if sinks is not None:
            s = torch.cat([s, sinks[h].expand(T, 1)], dim=1)
        p = torch.softmax(s, dim=-1)[:, :T]
        out[:, h] = p @ v[:, h // group]
    return out


@pytest.mark.parametrize("dtype,tol,tol_rms", [(torch.float32, 2e-5, 5e-6),
                                               (torch.bfloat16, 3e-2, 1e-2)])
def test_attention_whose_scores_are_changed(cuda_device, dtype, tol, tol_rms):
    """Attention that this architecture does not have, named by the spec alone: a soft cap on
    the scores, a bias per distance, a sink logit per head (a tensor of the mixer).  One layer
    with all three, one with the cap only, one plain; whole, in portions and token by token,
    against a plain restatement.  The cap is low enough and the slopes steep enough that
    leaving either out shows."""
    from binfer_b200.config import (AttentionSpec, GatedMLPSpec, LayerSpec, NormSpec, RopeSpec,
                                    ScheduleEntry, ScoreSpec)
    from binfer_b200.engine import make_runner
    from binfer_b200.engine.runner import StepItem
    from binfer_b200.parts import build_model, param_specs_for
    from binfer_b200.weights import TensorSource, random_tensors
    norm, rope = NormSpec(eps=1e-6), RopeSpec(theta=1e4, rotary_dim=16)
    slopes = (0.5, 0.25, 0.125, 0.0625)
    scores = [ScoreSpec(softcap=0.6, slopes=slopes, sinks=True), ScoreSpec(softcap=0.3), None]
    layers = [LayerSpec(mixer=AttentionSpec(num_heads=4, num_kv_heads=2, head_dim=16,
                                            position=rope, score=sc),
                        ffn=GatedMLPSpec(intermediate_size=24), norm=norm) for sc in scores]
    spec = _toy_spec(layers, [ScheduleEntry(i) for i in range(3)], vocab=40, hidden=32)
    names = [s.name for s in param_specs_for(spec)]
    assert "model.layers.0.self_attn.sinks" in names and "model.layers.1.self_attn.sinks" not in names
    env = _env(dtype)
    # (weights small enough that the scores stay of order one: with a sharp softmax the
    # bfloat16 rounding of this 32-wide model alone exceeds the bounds)
    weights = random_tensors(param_specs_for(spec), seed=4, std=0.12, norm_std=0.1)
    model = build_model(spec, env, TensorSource.from_dict(weights))
    n = 41
    toks = H.random_tokens(n, 40, 8)

    w = {k: v.double() for k, v in weights.items()}
    if dtype == torch.bfloat16:
        w = {k: (v.to(torch.bfloat16).double() if v.dim() > 1 else v) for k, v in w.items()}
    pos = torch.arange(n)
    ang = P.rope_angles(pos, 16, 1e4)

    def plain(with_scores=True):
        x = P.embedding(torch.tensor(toks), w["model.embed_tokens.weight"])
        for i, sc in enumerate(scores):
            p = f"model.layers.{i}."
            a = p + "self_attn."
            h = P.rms_norm(x, w[p + "input_layernorm.weight"], 1e-6)
            q = P.apply_rope((h @ w[a + "q_proj.weight"].T).view(n, 4, 16), ang)
            k = P.apply_rope((h @ w[a + "k_proj.weight"].T).view(n, 2, 16), ang)
            v = (h @ w[a + "v_proj.weight"].T).view(n, 2, 16)
            if sc is None or not with_scores:
                att = P.causal_attention(q, k, v, 16 ** -0.5)
            else:
                att = _plain_scored_attention(
                    q, k, v, 16 ** -0.5, sc.softcap,
                    torch.tensor(sc.slopes, dtype=torch.float64) if sc.slopes else None,
                    w[a + "sinks"] if sc.sinks else None)
            x = x + att.reshape(n, -1) @ w[a + "o_proj.weight"].T
            h = P.rms_norm(x, w[p + "post_attention_layernorm.weight"], 1e-6)
            x = x + P.swiglu_mlp(h, w, p + "mlp.")
        return P.rms_norm(x, w["model.norm.weight"], 1e-5) @ w["model.embed_tokens.weight"].T

    want = plain()
    assert H.rel_err(plain(with_scores=False), want) > 0.2, "the changes would not show"
    for cuts in ([n], [6, 1, 2, 17, 15], [20] + [1] * 21):
        runner = make_runner(model, env, page_size=4, num_pages=12, max_requests=2)
        runner.add_request("r")
        rows, at = [], 0
        for c in cuts:
            rows.append(runner.step([StepItem("r", toks[at:at + c], list(range(c)))]).clone())
            at += c
        runner.check_errors()
        got = torch.cat(rows).float().cpu()
        assert H.rel_err(got, want) < tol and H.rel_rms(got, want) < tol_rms, (
            cuts, H.rel_err(got, want), H.rel_rms(got, want))
