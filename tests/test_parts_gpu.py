"""Each part alone against the plain implementation; schedules; and a toy architecture with a mixer
that keeps state of its own, registered from here without touching the framework's files."""
import dataclasses
import math
import os
from dataclasses import dataclass

import pytest
import torch

import helpers
from helpers import plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _env(dtype):
    from return_b200.parts import BuildEnv
    return BuildEnv(dtype, torch.device(DEV))


def _tol(dtype):
    return dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=4e-2, rtol=4e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from return_b200.parts import NORMS, NormSpec
    norm = NORMS.build(NormSpec(size=72, eps=1e-5), _env(dtype))
    assert list(norm.params()) == ["weight"] and norm.params()["weight"].shape == (72,)
    w = 1 + 0.1 * torch.randn(72, device=DEV)
    norm.bind({"weight": w})
    x = torch.randn(11, 72, device=DEV).to(dtype)
    out = torch.empty_like(x)
    norm.forward(x, out)
    assert torch.allclose(out.float(), plain.rms_norm(x.float(), w, 1e-5), **_tol(dtype))


def test_rope_part_tables():
    from return_b200.parts import POSITION_ENCODINGS, RopeSpec
    rope = POSITION_ENCODINGS.build(RopeSpec(rotary_dim=48, theta=50000.0, max_positions=300), _env(torch.float32))
    cos, sin, rot = rope.rotary_tables()
    c, s = plain.rope_tables(torch.arange(300), 48, 50000.0)
    assert rot == 48 and torch.equal(cos.cpu(), c) and torch.equal(sin.cpu(), s)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    from return_b200.parts import FEED_FORWARDS, SwiGLUSpec
    g, u, d = (0.2 * torch.randn(104, 40), 0.2 * torch.randn(104, 40), 0.2 * torch.randn(40, 104))
    rd = lambda t: t.to(dtype).float()
    w = {"mlp.gate_proj.weight": rd(g), "mlp.up_proj.weight": rd(u), "mlp.down_proj.weight": rd(d)}
    for interleave in (0, 8):
        ff = FEED_FORWARDS.build(SwiGLUSpec(hidden_size=40, intermediate_size=104, interleave=interleave), _env(dtype))
        assert {k: v.shape for k, v in ff.params().items()} == {"gate_up": (208, 40), "down": (40, 104)}
        gate_up = torch.cat([g, u]) if interleave == 0 else \
            torch.stack([g.view(-1, 8, 40), u.view(-1, 8, 40)], dim=1).reshape(208, 40)
        ff.bind({"gate_up": gate_up.to(dtype).to(DEV), "down": d.to(dtype).to(DEV)})
        for rows in (9, 40):                 # few rows and many rows take different kernels on the bfloat16 path
            x = torch.randn(rows, 40).to(dtype)
            y = ff.forward(x.to(DEV), None)
            assert torch.allclose(y.float().cpu(), plain.swiglu_mlp(w, "", x.float()), **_tol(dtype))


def _runner_for(spec, params, dtype, page_size=8, max_token=512, max_reside=4):
    from return_b200.engine.config import EngineConfig
    from return_b200.engine.runner import ModelRunner
    from return_b200.models.decoder import DecoderModel
    model = DecoderModel(spec, _env(dtype))
    model.bind(params)
    cfg = EngineConfig(max_token=max_token, max_reside=max_reside, page_size=page_size,
                       dtype="float32" if dtype == torch.float32 else "bfloat16", use_cuda_graph=False, device=DEV)
    r = ModelRunner(model, cfg, max_positions=max_token)
    r.storage.poison()
    return r


def _params_from_dir(model_dir, spec, dtype):
    from return_b200.config import registry
    from return_b200.models.decoder import DecoderModel
    from return_b200.weights import loader
    arch, cfg = registry.read_config(model_dir)
    model = DecoderModel(spec, _env(dtype))
    expected = {n: s for n, (s, _) in loader.checkpoint_shapes(arch, cfg).items()}
    # a spec with fewer or reordered layers still takes its parameters by name
    params = loader.load_parameters(DecoderModel(arch.decoder_spec(cfg, 512), _env(dtype)).params(),
                                    arch.weight_sources(cfg), expected, model_dir, dtype, DEV)
    return {k: v for k, v in params.items() if k in model.params()}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", ["A", "C"])
def test_attention_part_and_block_alone(tmp_path, case, dtype):
    """One block of the model, stepped in two portions, against plain.decoder_layer on the whole."""
    from return_b200.config import registry
    from return_b200.parts import LayerContext
    d = helpers.make_model_dir(tmp_path, case)
    arch, cfg = registry.read_config(d)
    full = arch.decoder_spec(cfg, 512)
    spec = dataclasses.replace(full, layers=full.layers[:1], schedule=full.schedule[:1])
    runner = _runner_for(spec, _params_from_dir(d, spec, dtype), dtype, page_size=helpers.CASES[case][2])
    c, w = plain.read_config(d), plain.read_weights(d)
    T, H = 45, cfg.hidden_size
    x = torch.randn(T, H)
    want, _ = plain.decoder_layer(c, w, 0, x, torch.arange(T), plain.layer_windows(c)[0])
    # the attention part alone: plain projections + attention + output projection of the normed input
    a = plain.rms_norm(x, w["model.layers.0.input_layernorm.weight"], c["rms_norm_eps"])
    q, k, v = plain.attention_project_qkv(c, w, "model.layers.0.", a, torch.arange(T))
    o = plain.attention_scores_softmax_pv(q, k, v, torch.arange(T), torch.arange(T), c["head_dim"] ** -0.5,
                                          plain.layer_windows(c)[0])
    want_mixer = plain.linear(o.reshape(T, -1), w["model.layers.0.self_attn.o_proj.weight"])

    from return_b200.engine.batch import StepBatch, build_host_batch
    runner.add_request("r")
    block = runner.model.blocks[0]
    got, got_mixer = [], []
    for lo, hi in ((0, 29), (29, T)):
        entry = runner.reserve("r", [0] * (hi - lo))
        batch = StepBatch(build_host_batch([entry], runner.manager, tilings=runner.tilings), torch.device(DEV), runner.staging)
        ctx = runner.storage.layer_context(0, batch, write=True)
        got_mixer.append(block.mixer.forward(a[lo:hi].to(dtype).to(DEV), ctx).float().cpu())
        stream = x[lo:hi].clone().to(DEV)
        delta = block.forward(stream, None, ctx)
        got.append((stream + delta.float()).cpu())
    assert torch.allclose(torch.cat(got_mixer), want_mixer, **_tol(dtype))
    assert torch.allclose(torch.cat(got), want, **_tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_schedule_names_a_layer_twice_and_shares_a_cache(tmp_path, dtype):
    from return_b200.config import registry
    from return_b200.parts import ScheduleEntry
    d = helpers.make_model_dir(tmp_path, "A")
    arch, cfg = registry.read_config(d)
    base = arch.decoder_spec(cfg, 512)
    ids = helpers.random_ids(256, 41, 9)
    for sched, plain_sched in (
            ((ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0)), [(0, None), (1, None), (0, None)]),
            ((ScheduleEntry(0), ScheduleEntry(1, cache_of=0)), [(0, None), (1, 0)]),
            ((ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_of=0), ScheduleEntry(0, cache_of=1)),
             [(1, None), (0, None), (1, 0), (0, 1)])):
        spec = dataclasses.replace(base, schedule=sched)
        runner = _runner_for(spec, _params_from_dir(d, spec, dtype), dtype, page_size=16)
        owners = sum(1 for e in sched if e.cache_of is None)
        assert runner.storage.pools[0].shape[0] == owners          # one cache layer per owning run
        runner.add_request("r")
        rows = []
        for lo, hi in ((0, 17), (17, 18), (18, 41)):
            e = runner.reserve("r", ids[lo:hi], list(range(hi - lo)))
            rows.append(runner.step([e]).cpu())
        want = helpers.plain_logits(d, ids, schedule=plain_sched)
        tol = 1e-4 if dtype == torch.float32 else 6e-2
        assert (torch.cat(rows) - want).abs().max() < tol


# ------------------------------------------------------------------------------- a toy architecture

@dataclass(frozen=True)
class RunningMeanSpec:
    hidden_size: int
    kind: str = "running_mean"


@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    rms_norm_eps: float
    architectures: tuple = ("ToyRunningMeanLM",)

    @classmethod
    def from_dict(cls, raw):
        return cls(raw["vocab_size"], raw["hidden_size"], raw["intermediate_size"], raw["num_hidden_layers"],
                   raw["rms_norm_eps"])

    def to_dict(self):
        d = dataclasses.asdict(self)
        d["architectures"] = list(self.architectures)
        d["model_type"] = "toy_running_mean"
        return d


def _register_toy():
    """A mixer whose state is the running sum of its inputs and their count: y_t = W mean(x_0..x_t)."""
    from return_b200.config import registry
    from return_b200.parts import MIXERS, BlockSpec, DecoderSpec, Mixer, NormSpec, ParamSpec, StateNeed, SwiGLUSpec
    from return_b200.weights.loader import Source

    class RunningMean(Mixer):
        graph_safe = False          # forward walks the segments on the host

        def params(self):
            return {"w": ParamSpec((self.spec.hidden_size, self.spec.hidden_size))}

        def cache_need(self):
            return StateNeed((self.spec.hidden_size + 1,), torch.float32)

        def forward(self, x, ctx):
            host = ctx.batch.host
            out = torch.empty_like(x)
            H = self.spec.hidden_size
            for i in range(host.num_segments):
                a, b, slot = int(host.cu_q[i]), int(host.cu_q[i + 1]), int(host.seg_slot[i])
                st = ctx.state[slot]
                sums = x[a:b].float().cumsum(0) + st[:H]
                counts = torch.arange(1, b - a + 1, device=x.device, dtype=torch.float32) + st[H]
                out[a:b] = ((sums / counts[:, None]) @ self.p_w.float().T).to(x.dtype)
                st[:H] = sums[-1]
                st[H] = counts[-1]
            return out

    MIXERS.register("running_mean", RunningMean)

    def decoder_spec(cfg, max_positions=None):
        norm = NormSpec(cfg.hidden_size, cfg.rms_norm_eps)
        block = BlockSpec(RunningMeanSpec(cfg.hidden_size), SwiGLUSpec(cfg.hidden_size, cfg.intermediate_size), norm, norm)
        return DecoderSpec(cfg.vocab_size, cfg.hidden_size, (block,) * cfg.num_hidden_layers,
                           DecoderSpec.in_order(cfg.num_hidden_layers), norm, tie_embeddings=True)

    def weight_sources(cfg):
        m = {"embed": Source(("tok.weight",)), "final_norm.weight": Source(("out_norm.weight",))}
        for i in range(cfg.num_hidden_layers):
            m[f"layers.{i}.mixer.w"] = Source((f"blocks.{i}.mean.w",))
            m[f"layers.{i}.feed_forward.gate_up"] = Source((f"blocks.{i}.ff.gate", f"blocks.{i}.ff.up"))
            m[f"layers.{i}.feed_forward.down"] = Source((f"blocks.{i}.ff.down",))
            m[f"layers.{i}.mixer_norm.weight"] = Source((f"blocks.{i}.n1",))
            m[f"layers.{i}.feed_forward_norm.weight"] = Source((f"blocks.{i}.n2",))
        return m

    registry.register_architecture(registry.Architecture(
        name="ToyRunningMeanLM", model_type="toy_running_mean", config_cls=ToyConfig,
        decoder_spec=decoder_spec, weight_sources=weight_sources))


def _toy_reference(model_dir, cfg, ids):
    from safetensors.torch import load_file
    w = load_file(os.path.join(model_dir, "model.safetensors"))
    x = w["tok.weight"][torch.tensor(ids)]
    for i in range(cfg.num_hidden_layers):
        a = plain.rms_norm(x, w[f"blocks.{i}.n1"], cfg.rms_norm_eps)
        mean = a.cumsum(0) / torch.arange(1, len(ids) + 1)[:, None]
        x = x + mean @ w[f"blocks.{i}.mean.w"].T
        b = plain.rms_norm(x, w[f"blocks.{i}.n2"], cfg.rms_norm_eps)
        g, u = b @ w[f"blocks.{i}.ff.gate"].T, b @ w[f"blocks.{i}.ff.up"].T
        x = x + (g * torch.sigmoid(g) * u) @ w[f"blocks.{i}.ff.down"].T
    return plain.rms_norm(x, w["out_norm.weight"], cfg.rms_norm_eps) @ w["tok.weight"].T


def test_toy_mixer_with_state_of_its_own(tmp_path):
    from return_b200.config import registry
    from return_b200.engine.replay import TraceReplayer
    from return_b200.parts import MIXERS
    from return_b200.weights import loader
    _register_toy()
    try:
        cfg = ToyConfig(vocab_size=90, hidden_size=24, intermediate_size=40, num_hidden_layers=2, rms_norm_eps=1e-5)
        d = loader.write_random_model(os.path.join(str(tmp_path), "toy"), cfg, seed=11)
        arch, read = registry.read_config(d)
        assert arch.name == "ToyRunningMeanLM" and read == cfg
        reqs = {f"t{i}": helpers.random_ids(90, n, 100 + i) for i, n in enumerate((30, 7, 19, 12, 25))}
        steps = helpers.mixed(reqs, max_live=3, portion=6, decode_tail=3, seed=5)
        rp = TraceReplayer(d, "float32", helpers.pool_tokens(steps), page_size=16, max_reside=3)
        st = rp.runner.storage
        assert len(st.states) == 2 and all(t.shape == (3 + 1, 25) for t in st.states.values())   # + the slot of no request
        got = helpers.collect(steps, [None if (lg := rp.run_step(s)) is None else lg.cpu() for s in steps])
        for rid, ids in reqs.items():
            assert (got[rid] - _toy_reference(d, cfg, ids)).abs().max() < 1e-4, rid
        assert rp.runner.manager.free_slots == 3
    finally:
        registry.unregister_architecture("ToyRunningMeanLM")
        MIXERS.unregister("running_mean")


def test_toy_state_under_the_scheduler_with_reused_slots_and_a_preemption(tmp_path):
    """The same toy architecture through ``Engine.generate``: two slots for five requests, so slots are taken
    again, and a pool so small that one request is preempted and computed again.  Every admission must
    start from zero state, whoever admits: greedy tokens equal the toy reference's."""
    from return_b200.config import registry
    from return_b200.engine.config import EngineConfig
    from return_b200.engine.engine import Engine
    from return_b200.parts import MIXERS
    from return_b200.weights import loader
    _register_toy()
    try:
        cfg = ToyConfig(vocab_size=90, hidden_size=24, intermediate_size=40, num_hidden_layers=2, rms_norm_eps=1e-5)
        d = loader.write_random_model(os.path.join(str(tmp_path), "toy"), cfg, seed=11)
        prompts = [helpers.random_ids(90, n, 300 + i) for i, n in enumerate((30, 28, 9, 17, 22))]
        new = 26

        def greedy(ids):
            ids, out = list(ids), []
            for _ in range(new):
                out.append(int(_toy_reference(d, cfg, ids)[-1].argmax()))
                ids.append(out[-1])
            return out

        eng = Engine(d, EngineConfig(max_token=96, max_reside=2, page_size=16, prefill_chunk=16, dtype="float32",
                                     use_cuda_graph=True, max_model_len=80))
        got = eng.generate(prompts, max_new_tokens=new, temperature=0.0)
        assert [r.output_ids for r in got] == [greedy(p) for p in prompts]
        assert eng.stats()["preemptions"] > 0
        eng.runner.manager.check()
        assert eng.runner.manager.free_slots == 2
    finally:
        registry.unregister_architecture("ToyRunningMeanLM")
        MIXERS.unregister("running_mean")


# ------------------------------------------------------------------------------- a second toy architecture:
# the engine's attention with a position encoding of the test's own, and a feed-forward with routing

@dataclass(frozen=True)
class PairRotationSpec:
    """Neighbouring pairs (2i, 2i + 1) of a head rotated by position * base^(-i / (D/2))."""
    head_dim: int
    base: float
    kind: str = "pair_rotation"


@dataclass(frozen=True)
class RoutedSpec:
    """Top-1 of ``experts`` small SwiGLU experts, weighted by the router's softmax probability."""
    hidden_size: int
    intermediate_size: int
    experts: int
    kind: str = "toy_routed"


@dataclass(frozen=True)
class RoutedConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    experts: int
    heads: int
    kv_heads: int
    head_dim: int
    base: float
    eps: float
    architectures: tuple = ("ToyRoutedLM",)

    @classmethod
    def from_dict(cls, raw):
        return cls(*(raw[k] for k in ("vocab_size", "hidden_size", "intermediate_size", "experts", "heads", "kv_heads",
                                      "head_dim", "base", "eps")))

    def to_dict(self):
        d = dataclasses.asdict(self)
        d["architectures"] = list(self.architectures)
        d["model_type"] = "toy_routed"
        return d


def _pair_rotate(x, pos, base):
    """x [T, heads, D] float32, pos [T]: the toy encoding, shared by the part and the reference."""
    D = x.shape[-1]
    inv = base ** (-torch.arange(D // 2, dtype=torch.float32, device=x.device) / (D // 2))
    ang = pos.to(torch.float32)[:, None, None] * inv[None, None, :]
    c, s = ang.cos(), ang.sin()
    a, b = x[..., 0::2], x[..., 1::2]
    return torch.stack([a * c - b * s, a * s + b * c], dim=-1).reshape(x.shape)


def _register_routed():
    from return_b200.config import registry
    from return_b200.parts import (FEED_FORWARDS, POSITION_ENCODINGS, AttentionSpec, BlockSpec, DecoderSpec, FeedForward,
                                   NormSpec, ParamSpec, PositionEncoding, SwiGLUSpec)
    from return_b200.weights.loader import Source

    class PairRotation(PositionEncoding):
        def apply(self, qkv, batch, num_heads, num_kv_heads, head_dim):
            T = qkv.shape[0]
            n = (num_heads + num_kv_heads) * head_dim                 # q and k heads; v stays
            x = qkv[:, :n].float().reshape(T, num_heads + num_kv_heads, head_dim)
            qkv[:, :n] = _pair_rotate(x, batch.pos, self.spec.base).reshape(T, n).to(qkv.dtype)

    class Routed(FeedForward):
        def params(self):
            s = self.spec
            return {"router": ParamSpec((s.experts, s.hidden_size)),
                    "w1": ParamSpec((s.experts * 2 * s.intermediate_size, s.hidden_size)),
                    "w2": ParamSpec((s.experts * s.hidden_size, s.intermediate_size))}

        def forward(self, x, ctx):
            s = self.spec
            logits = x.float() @ self.p_router.float().T              # router logits in 32-bit
            prob, pick = torch.softmax(logits, dim=-1).max(dim=-1)
            w1 = self.p_w1.float().reshape(s.experts, 2 * s.intermediate_size, s.hidden_size)
            w2 = self.p_w2.float().reshape(s.experts, s.hidden_size, s.intermediate_size)
            y = torch.zeros_like(x, dtype=torch.float32)
            for e in range(s.experts):                                # every expert on every row, masked: no host sync
                gu = x.float() @ w1[e].T
                g, u = gu[:, :s.intermediate_size], gu[:, s.intermediate_size:]
                y += ((g * torch.sigmoid(g) * u) @ w2[e].T) * (prob * (pick == e))[:, None]
            return y.to(x.dtype)

    POSITION_ENCODINGS.register("pair_rotation", PairRotation)
    FEED_FORWARDS.register("toy_routed", Routed)

    def decoder_spec(cfg, max_positions=None):
        norm = NormSpec(cfg.hidden_size, cfg.eps)
        att = lambda position: AttentionSpec(cfg.hidden_size, cfg.heads, cfg.kv_heads, cfg.head_dim, cfg.head_dim ** -0.5,
                                             position=position)
        routed = BlockSpec(att(PairRotationSpec(cfg.head_dim, cfg.base)),
                           RoutedSpec(cfg.hidden_size, cfg.intermediate_size, cfg.experts), norm, norm)
        dense = BlockSpec(att(None), SwiGLUSpec(cfg.hidden_size, cfg.intermediate_size), norm, norm)
        return DecoderSpec(cfg.vocab_size, cfg.hidden_size, (routed, dense), DecoderSpec.in_order(2), norm,
                           tie_embeddings=False)

    def weight_sources(cfg):
        m = {"embed": Source(("emb",)), "lm_head": Source(("head",)), "final_norm.weight": Source(("nf",))}
        for i in range(2):
            m[f"layers.{i}.mixer.qkv"] = Source((f"l{i}.q", f"l{i}.k", f"l{i}.v"))
            m[f"layers.{i}.mixer.o"] = Source((f"l{i}.o",))
            m[f"layers.{i}.mixer_norm.weight"] = Source((f"l{i}.n1",))
            m[f"layers.{i}.feed_forward_norm.weight"] = Source((f"l{i}.n2",))
        m["layers.0.feed_forward.router"] = Source(("l0.router",))
        m["layers.0.feed_forward.w1"] = Source(("l0.w1",))
        m["layers.0.feed_forward.w2"] = Source(("l0.w2",))
        m["layers.1.feed_forward.gate_up"] = Source(("l1.gate", "l1.up"))
        m["layers.1.feed_forward.down"] = Source(("l1.down",))
        return m

    def split_rows(cfg, pname):
        if pname.endswith("mixer.qkv"):
            return [cfg.heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim]
        return None

    registry.register_architecture(registry.Architecture(
        name="ToyRoutedLM", model_type="toy_routed", config_cls=RoutedConfig,
        decoder_spec=decoder_spec, weight_sources=weight_sources, split_rows=split_rows))


def _routed_reference(model_dir, cfg, ids):
    from safetensors.torch import load_file
    w = {k: v.float() for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}
    T = len(ids)
    pos = torch.arange(T)
    x = w["emb"][torch.tensor(ids)]
    for i in range(2):
        a = plain.rms_norm(x, w[f"l{i}.n1"], cfg.eps)
        q = (a @ w[f"l{i}.q"].T).reshape(T, cfg.heads, cfg.head_dim)
        k = (a @ w[f"l{i}.k"].T).reshape(T, cfg.kv_heads, cfg.head_dim)
        v = (a @ w[f"l{i}.v"].T).reshape(T, cfg.kv_heads, cfg.head_dim)
        if i == 0:
            q, k = _pair_rotate(q, pos, cfg.base), _pair_rotate(k, pos, cfg.base)
        o = plain.attention_scores_softmax_pv(q, k, v, pos, pos, cfg.head_dim ** -0.5, None)
        x = x + o.reshape(T, -1) @ w[f"l{i}.o"].T
        b = plain.rms_norm(x, w[f"l{i}.n2"], cfg.eps)
        if i == 0:
            prob, pick = torch.softmax(b @ w["l0.router"].T, dim=-1).max(dim=-1)
            w1 = w["l0.w1"].reshape(cfg.experts, 2 * cfg.intermediate_size, cfg.hidden_size)
            w2 = w["l0.w2"].reshape(cfg.experts, cfg.hidden_size, cfg.intermediate_size)
            y = torch.zeros_like(b)
            for t in range(T):
                e = int(pick[t])
                gu = w1[e] @ b[t]
                g, u = gu[:cfg.intermediate_size], gu[cfg.intermediate_size:]
                y[t] = (w2[e] @ (g * torch.sigmoid(g) * u)) * prob[t]
            x = x + y
        else:
            g, u = b @ w["l1.gate"].T, b @ w["l1.up"].T
            x = x + (g * torch.sigmoid(g) * u) @ w["l1.down"].T
    return plain.rms_norm(x, w["nf"], cfg.eps) @ w["head"].T


def test_toy_position_encoding_and_routed_feed_forward(tmp_path):
    """An architecture registered from this file: the engine's paged attention with a position encoding
    defined here (layer 0) and with none (layer 1), a routed feed-forward defined here (layer 0) beside
    the engine's dense one (layer 1).  Replayed in portions and mixed batches against plain math."""
    from return_b200.config import registry
    from return_b200.engine.replay import TraceReplayer
    from return_b200.parts import FEED_FORWARDS, POSITION_ENCODINGS
    from return_b200.weights import loader
    _register_routed()
    try:
        cfg = RoutedConfig(vocab_size=70, hidden_size=32, intermediate_size=24, experts=3, heads=4, kv_heads=2,
                           head_dim=16, base=50.0, eps=1e-5)
        d = loader.write_random_model(os.path.join(str(tmp_path), "routed"), cfg, seed=3)
        arch, read = registry.read_config(d)
        assert arch.name == "ToyRoutedLM" and read == cfg
        reqs = {f"t{i}": helpers.random_ids(70, n, 200 + i) for i, n in enumerate((33, 9, 21, 14))}
        steps = helpers.mixed(reqs, max_live=3, portion=7, decode_tail=4, seed=9)
        rp = TraceReplayer(d, "float32", helpers.pool_tokens(steps), page_size=16, max_reside=3)
        got = helpers.collect(steps, [None if (lg := rp.run_step(s)) is None else lg.cpu() for s in steps])
        for rid, ids in reqs.items():
            assert (got[rid] - _routed_reference(d, cfg, ids)).abs().max() < 2e-4, rid
    finally:
        registry.unregister_architecture("ToyRoutedLM")
        POSITION_ENCODINGS.unregister("pair_rotation")
        FEED_FORWARDS.unregister("toy_routed")
