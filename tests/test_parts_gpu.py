"""Each part alone against its plain formula, and the claim that the engine is open to other parts: a toy
mixer with state of its own and a toy architecture (different mixers in different layers, a layer that
runs twice, a layer that reads another layer's cache, a windowed layer) are defined HERE, registered, built
and stepped without touching the framework's files."""
import json
import math
import os
from dataclasses import asdict, dataclass

import pytest
import torch

from helpers import TOL, max_rel_err, random_tokens
from plain import llama as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rt(dtype):
    from forge_b200.parts import Runtime
    return Runtime(torch.device(DEV), dtype)


def _rand(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


DT = [torch.float32, torch.bfloat16]
PART_TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2}


@pytest.mark.parametrize("dtype", DT)
def test_rmsnorm_part(dtype):
    from forge_b200.config import PartSpec
    from forge_b200.parts import build_part
    part = build_part("norm", PartSpec("rmsnorm", {"size": 88, "eps": 1e-4}), _rt(dtype))
    assert list(part.tensor_specs()) == ["weight"] and part.tensor_specs()["weight"].shape == (88,)
    w, x = _rand(88, seed=1) + 1.0, _rand(9, 88, scale=2.0)
    part.bind({"weight": w})
    got = part.forward(x.to(DEV)).float().cpu()
    want = P.rms_norm(x.double(), w.double(), 1e-4).float()
    assert got.dtype == torch.float32 and max_rel_err(got, want) <= PART_TOL[dtype]


@pytest.mark.parametrize("dtype", DT)
def test_swiglu_part(dtype):
    from forge_b200.config import PartSpec
    from forge_b200.parts import build_part
    H, I, T = 72, 200, 11
    part = build_part("feed_forward", PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I}), _rt(dtype))
    specs = part.tensor_specs()
    assert specs["mlp.gate_proj.weight"].shape == (I, H) and specs["mlp.down_proj.weight"].shape == (H, I)
    t = {n: _rand(*s.shape, seed=i, scale=0.2).to(torch.bfloat16) for i, (n, s) in enumerate(specs.items())}
    part.bind(t)
    x = _rand(T, H, seed=9).to(dtype)
    residual = _rand(T, H, seed=10)
    res_dev = residual.clone().to(DEV)
    part.forward(x.to(DEV), res_dev)
    want = residual.double() + P.swiglu(x.double(), t["mlp.gate_proj.weight"].double(), t["mlp.up_proj.weight"].double(),
                                        t["mlp.down_proj.weight"].double())
    assert max_rel_err(res_dev, want) <= PART_TOL[dtype]


@pytest.mark.parametrize("dtype", DT)
def test_embedding_and_tied_head(dtype):
    from forge_b200.config import PartSpec
    from forge_b200.parts import build_part
    V, H = 130, 40
    emb = build_part("embedding", PartSpec("embedding", {"vocab_size": V, "hidden_size": H}), _rt(dtype))
    head = build_part("lm_head", PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "tied": True}), _rt(dtype))
    table = _rand(V, H).to(torch.bfloat16)
    emb.bind({"weight": table})
    head.bind({}, shared_table=emb.table)
    assert head.tensor_specs()["weight"].required is False
    ids = torch.tensor([3, 129, 0], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(ids).cpu(), table.float()[ids.cpu().long()])
    x = _rand(4, H, seed=2).to(dtype)
    want = P.linear(x.double(), table.double())
    assert max_rel_err(head.forward(x.to(DEV)), want) <= PART_TOL[dtype]


def _attention_harness(dtype, window, page_size=8):
    """An attention mixer with a cache of its own, fed one request in two portions and a decode token."""
    from forge_b200.cache import CacheStorage
    from forge_b200.config import PartSpec
    from forge_b200.engine import StepEntry, build_step_batch
    from forge_b200.parts import build_part
    H, NH, NKV, HD, theta = 48, 6, 2, 16, 777.0
    spec = PartSpec("attention", {"hidden_size": H, "num_heads": NH, "num_kv_heads": NKV, "head_dim": HD,
                                  "qkv_bias": True, "window": window,
                                  "position": PartSpec("rope", {"head_dim": HD, "theta": theta})})
    mixer = build_part("mixer", spec, _rt(dtype))
    t = {n: _rand(*s.shape, seed=i, scale=0.3).to(torch.bfloat16) for i, (n, s) in enumerate(mixer.tensor_specs().items())}
    mixer.bind(t)
    storage = CacheStorage([mixer.cache_spec()], [None], page_size, 16, 2, dtype, torch.device(DEV))
    T = 29
    x = _rand(T, H, seed=50).to(dtype)
    got = torch.zeros(T, H)
    storage.manager.admit("r")
    for a, b in [(0, 13), (13, 28), (28, 29)]:
        batch = build_step_batch([StepEntry("r", [0] * (b - a), [])], storage.manager, torch.device(DEV), 8)
        res = torch.zeros(b - a, H, device=DEV)
        mixer.forward(x[a:b].to(DEV), batch, storage.layers[0], res)
        got[a:b] = res.cpu()
        storage.manager.release_out_of_window("r")
        storage.manager.check()
    # plain: whole sequence
    xd = x.double()
    w = {k: v.double() for k, v in t.items()}
    q = P.linear(xd, w["self_attn.q_proj.weight"], w["self_attn.q_proj.bias"]).view(T, NH, HD)
    k = P.linear(xd, w["self_attn.k_proj.weight"], w["self_attn.k_proj.bias"]).view(T, NKV, HD)
    v = P.linear(xd, w["self_attn.v_proj.weight"], w["self_attn.v_proj.bias"]).view(T, NKV, HD)
    pos = torch.arange(T)
    o = P.attention(P.rope(q, pos, theta), P.rope(k, pos, theta), v, window=window)
    want = P.linear(o.reshape(T, NH * HD), w["self_attn.o_proj.weight"])
    return got, want, storage


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("window", [None, 5])
def test_attention_part_with_its_position_encoding_and_cache(dtype, window):
    got, want, storage = _attention_harness(dtype, window)
    assert max_rel_err(got, want) <= PART_TOL[dtype]
    if window is not None:      # 29 tokens, window 5, pages of 8: positions 0..23 are behind every future query
        assert storage.manager.block_table("r", "kv2x16_win5")[:3] == [-1, -1, -1]


# ---------------------------------------------------------------------------------------------------
# A toy mixer with state of its own, and a toy architecture around it, defined in this test file only.

H_TOY = 40


def _toy_mixer_class():
    from forge_b200.parts import Part, StateSpec
    from forge_b200.weights import TensorSpec

    class RunningMeanMixer(Part):
        """y_t = W . mean(x_1..x_t): per request it keeps the running sum of its inputs and their count, a
        state of fixed size that must survive being cut into portions."""

        def __init__(self, rt, hidden_size):
            self.rt, self.h = rt, hidden_size
            self.w = None

        def tensor_specs(self):
            return {"mixer.proj.weight": TensorSpec((self.h, self.h))}

        def bind(self, tensors):
            self.w = tensors["mixer.proj.weight"].to(device=self.rt.device, dtype=torch.float32)

        def cache_spec(self):
            return StateSpec((self.h + 1,), torch.float32)

        def forward(self, x, batch, cache, residual):
            xs = x.float()
            for s in range(batch.num_requests):
                a, b = batch.host_q_start[s], batch.host_q_start[s + 1]
                st = cache.state[batch.host_slots[s]]
                csum = torch.cumsum(xs[a:b], 0) + st[:self.h]
                cnt = st[self.h] + torch.arange(1, b - a + 1, device=xs.device)
                residual[a:b] += (csum / cnt[:, None]) @ self.w.t()
                st[:self.h] = csum[-1]
                st[self.h] = cnt[-1]

    return RunningMeanMixer


@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int = 97
    hidden_size: int = H_TOY
    intermediate_size: int = 56
    num_heads: int = 5
    num_kv_heads: int = 5
    head_dim: int = 8
    eps: float = 1e-5
    theta: float = 100.0
    window: int = 7
    max_position_embeddings: int = 256

    @classmethod
    def from_dict(cls, d, architecture="ToyForCausalLM"):
        return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})

    def to_dict(self):
        return dict(asdict(self), architectures=["ToyForCausalLM"])

    def plan(self):
        from forge_b200.config import LayerSpec, ModelPlan, PartSpec
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.eps})
        ffn = PartSpec("swiglu", {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size})

        def attn(window):
            return PartSpec("attention", {"hidden_size": self.hidden_size, "num_heads": self.num_heads,
                                          "num_kv_heads": self.num_kv_heads, "head_dim": self.head_dim, "window": window,
                                          "position": PartSpec("rope", {"head_dim": self.head_dim, "theta": self.theta})})
        toy = PartSpec("toy_running_mean", {"hidden_size": self.hidden_size})
        norms = {"input": norm, "post_mixer": norm}
        layers = [
            LayerSpec("pre_norm", attn(None), ffn, norms, "model.layers.0."),
            LayerSpec("pre_norm", toy, ffn, norms, "model.layers.1."),
            LayerSpec("pre_norm", attn(None), ffn, norms, "model.layers.2.", cache_from=0),   # reads layer 0's keys
            LayerSpec("pre_norm", attn(self.window), ffn, norms, "model.layers.3."),           # a window of its own
        ]
        return ModelPlan(hidden_size=self.hidden_size, vocab_size=self.vocab_size, max_positions=self.max_position_embeddings,
                         embedding=PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}),
                         final_norm=norm,
                         lm_head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size, "tied": False}),
                         layers=layers, schedule=[0, 1, 0, 2, 3])                              # layer 0 runs twice


def plain_toy_logits(cfg, w, ids):
    """The toy model on one whole sequence, from the plain functions, float64."""
    T = len(ids)
    pos = torch.arange(T)
    h = P.embedding(torch.tensor(ids), w["model.embed_tokens.weight"])
    kv_of_run = {}

    def attn_layer(p, h, run, window, read_run=None):
        x = P.rms_norm(h, w[p + "input_layernorm.weight"], cfg.eps)
        q = P.rope(P.linear(x, w[p + "self_attn.q_proj.weight"]).view(T, cfg.num_heads, cfg.head_dim), pos, cfg.theta)
        if read_run is None:
            k = P.rope(P.linear(x, w[p + "self_attn.k_proj.weight"]).view(T, cfg.num_kv_heads, cfg.head_dim), pos, cfg.theta)
            v = P.linear(x, w[p + "self_attn.v_proj.weight"]).view(T, cfg.num_kv_heads, cfg.head_dim)
            kv_of_run[run] = (k, v)
        else:
            k, v = kv_of_run[read_run]
        a = P.attention(q, k, v, window=window)
        return h + P.linear(a.reshape(T, -1), w[p + "self_attn.o_proj.weight"])

    def ffn(p, h):
        x = P.rms_norm(h, w[p + "post_attention_layernorm.weight"], cfg.eps)
        return h + P.swiglu(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])

    for run, layer in enumerate([0, 1, 0, 2, 3]):
        p = f"model.layers.{layer}."
        if layer == 1:
            x = P.rms_norm(h, w[p + "input_layernorm.weight"], cfg.eps)
            mean = torch.cumsum(x, 0) / torch.arange(1, T + 1, dtype=x.dtype)[:, None]
            h = h + P.linear(mean, w[p + "mixer.proj.weight"])
        elif layer == 2:
            h = attn_layer(p, h, run, None, read_run=2)        # the latest earlier run of layer 0 is run 2
        else:
            h = attn_layer(p, h, run, cfg.window if layer == 3 else None)
        h = ffn(p, h)
    return P.linear(P.rms_norm(h, w["model.norm.weight"], cfg.eps), w["lm_head.weight"])


@pytest.fixture
def toy_registered():
    from forge_b200.config import register_architecture, unregister_architecture
    from forge_b200.parts import register_part, unregister_part
    register_part("mixer", "toy_running_mean", _toy_mixer_class())
    register_architecture("ToyForCausalLM", ToyConfig)
    yield
    unregister_part("mixer", "toy_running_mean")
    unregister_architecture("ToyForCausalLM")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_is_registered_built_and_stepped(toy_registered, dtype, tmp_path):
    import schedules
    from forge_b200.config import load_config
    from forge_b200.engine import ModelRunner, StepEntry
    from forge_b200.weights import write_random_model
    from plain.safetensors_reader import read_safetensors
    cfg = ToyConfig()
    d = write_random_model(cfg, str(tmp_path / "toy"), seed=4, std=0.12, embed_std=0.6, norm_std=0.15)
    assert isinstance(load_config(d), ToyConfig)
    assert json.load(open(os.path.join(d, "config.json")))["architectures"] == ["ToyForCausalLM"]
    w = {k: torch.from_numpy(v).double() for k, v in read_safetensors(os.path.join(d, "model.safetensors")).items()}
    assert "model.layers.1.mixer.proj.weight" in w and "model.layers.1.self_attn.q_proj.weight" not in w
    reqs = {f"t{i}": random_tokens(n, cfg.vocab_size, seed=30 + i) for i, n in enumerate([41, 64, 23, 90])}
    want = {rid: plain_toy_logits(cfg, w, toks).float() for rid, toks in reqs.items()}
    # the toy mixer plans its work from host lists and does not declare itself graph_safe: the runner finds
    # that out by itself and decodes through the ordinary step
    runner = ModelRunner(d, dtype=dtype, page_size=8, cache_tokens=240, max_requests=3)
    assert runner.graph_safe is False and runner.cuda_graphs is False
    groups = set(runner.manager.groups)
    assert groups == {"kv5x8_full", "kv5x8_win7"}, groups          # two needs, two pools; the toy layer has none
    for steps in (schedules.whole(reqs), schedules.changing_portions(reqs), schedules.mixed(reqs, max_live=3)):
        got = {rid: torch.zeros(len(t), cfg.vocab_size) for rid, t in reqs.items()}
        for entries, end in steps:
            for rid, p, n in entries:
                if not runner.is_live(rid):
                    runner.admit(rid)
            lg = runner.step([StepEntry(rid, reqs[rid][p:p + n], list(range(n))) for rid, p, n in entries]).cpu()
            o = 0
            for rid, p, n in entries:
                got[rid][p:p + n] = lg[o:o + n]
                o += n
            for rid in end:
                runner.release(rid)
            runner.manager.check()
        for rid in reqs:
            assert max_rel_err(got[rid], want[rid]) <= TOL[dtype], rid
        assert runner.manager.num_free_pages() == {g: runner.num_pages for g in groups}
    del runner
    # and through the Python entry point with its default settings: prompt, then tokens one by one
    import forge_b200 as forge
    from helpers import assert_greedy_follows_plain
    model = forge.Model(d, dtype=dtype, block_size=8, max_num_seqs=3, cache_tokens=240)
    prompt = reqs["t2"][:11]
    out = model.generate(prompt, max_new_tokens=14, do_sample=False)
    assert out["num_generated_tokens"] == 14
    assert_greedy_follows_plain(lambda ids: plain_toy_logits(cfg, w, ids), prompt, out["token_ids"], TOL[dtype], "toy")
    # decoding far beyond what the windowed group's pool could hold if its pages were not given back
    ctx = model.create_context()
    long = random_tokens(200, cfg.vocab_size, seed=77)
    got_long = torch.cat([torch.from_numpy(ctx.forward(long[:9], 0))] +
                         [torch.from_numpy(ctx.forward([t], 9 + i)) for i, t in enumerate(long[9:])])
    assert max_rel_err(got_long, plain_toy_logits(cfg, w, long).float()) <= TOL[dtype]


# ---------------------------------------------------------------------------------------------------
# Two more toy parts, again defined here only: a feed-forward with a router, and another position encoding.

def _interleaved_rope(x, positions, theta):
    """Rotary encoding on neighbouring pairs (2d, 2d+1) instead of the half-split pairs; x [T, heads, HD]."""
    T, _, hd = x.shape
    d = torch.arange(hd // 2, dtype=x.dtype, device=x.device)
    ang = positions.to(x.dtype)[:, None] * torch.exp(d * (-2.0 * math.log(float(theta)) / hd))    # 1 / theta^(2d/hd)
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x0, x1 = x[..., 0::2], x[..., 1::2]
    return torch.stack([x0 * cos - x1 * sin, x0 * sin + x1 * cos], dim=-1).reshape(x.shape)


def _toy_part_classes():
    from forge_b200.parts import Part
    from forge_b200.weights import TensorSpec

    from forge_b200.parts.position import RotaryEmbedding

    class HalfSpeedRope(RotaryEmbedding):
        """A subclass of the stock rotary part with other arithmetic (positions advance at half speed).  It
        inherits ``theta`` and ``rotary``, but not the offer to the one-launch decode kernel, which would
        rotate by the stock angles."""

        def encode_and_store(self, qkv, positions, *args, **kwargs):
            return super().encode_and_store(qkv, positions // 2, *args, **kwargs)

    class InterleavedRope(Part):
        """A position encoding the framework does not have.  It meets the interface of the category: rotate q
        and k, put k and v into the pages at slot_mapping (cache layout [pages, 2, kv heads, page, head]),
        return q.  Everything it reads of the step is a device tensor, so it may be captured."""
        graph_safe = True

        def __init__(self, rt, head_dim, theta):
            self.rt, self.head_dim, self.theta = rt, head_dim, theta

        def encode_and_store(self, qkv, positions, slot_mapping, kv_cache, num_heads, num_kv_heads, page_size, batch=None):
            T, hd = qkv.shape[0], self.head_dim
            x = qkv.float().view(T, num_heads + 2 * num_kv_heads, hd)
            q = _interleaved_rope(x[:, :num_heads], positions, self.theta)
            if slot_mapping is not None and kv_cache is not None:
                k = _interleaved_rope(x[:, num_heads:num_heads + num_kv_heads], positions, self.theta)
                v = x[:, num_heads + num_kv_heads:]
                page, off = (slot_mapping // page_size).long(), (slot_mapping % page_size).long()
                kv_cache[page, 0, :, off, :] = k.to(kv_cache.dtype)
                kv_cache[page, 1, :, off, :] = v.to(kv_cache.dtype)
            return q.reshape(T, num_heads * hd).to(self.rt.dtype).contiguous()

    class RoutedFeedForward(Part):
        """residual += sum_e softmax(x . Wr^T)_e * W2_e . relu(W1_e . x): the router's logits and weights in
        32-bit, every expert weighted (no hard choice, so the result is continuous in x)."""
        graph_safe = True

        def __init__(self, rt, hidden_size, expert_size, num_experts):
            self.rt, self.h, self.f, self.e = rt, hidden_size, expert_size, num_experts

        def tensor_specs(self):
            specs = {"moe.router.weight": TensorSpec((self.e, self.h))}
            for i in range(self.e):
                specs[f"moe.experts.{i}.w1.weight"] = TensorSpec((self.f, self.h))
                specs[f"moe.experts.{i}.w2.weight"] = TensorSpec((self.h, self.f))
            return specs

        def bind(self, tensors):
            dev = self.rt.device
            self.router = tensors["moe.router.weight"].to(device=dev, dtype=torch.float32)
            self.w1 = [tensors[f"moe.experts.{i}.w1.weight"].to(device=dev, dtype=self.rt.dtype) for i in range(self.e)]
            self.w2 = [tensors[f"moe.experts.{i}.w2.weight"].to(device=dev, dtype=self.rt.dtype) for i in range(self.e)]

        def forward(self, x, residual):
            gate = torch.softmax(x.float() @ self.router.t(), dim=-1)
            for i in range(self.e):
                y = torch.relu(x @ self.w1[i].t()) @ self.w2[i].t()
                residual += gate[:, i:i + 1] * y.float()

    return InterleavedRope, RoutedFeedForward, HalfSpeedRope


@dataclass(frozen=True)
class Toy2Config:
    vocab_size: int = 61
    hidden_size: int = 48
    num_heads: int = 6
    num_kv_heads: int = 2
    head_dim: int = 16
    expert_size: int = 24
    num_experts: int = 3
    intermediate_size: int = 72
    eps: float = 1e-6
    theta: float = 50.0
    max_position_embeddings: int = 192
    second_position: str = "rope"

    @classmethod
    def from_dict(cls, d, architecture="Toy2ForCausalLM"):
        return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})

    def to_dict(self):
        return dict(asdict(self), architectures=["Toy2ForCausalLM"])

    def plan(self):
        from forge_b200.config import LayerSpec, ModelPlan, PartSpec
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.eps})

        def attn(position):
            return PartSpec("attention", {"hidden_size": self.hidden_size, "num_heads": self.num_heads,
                                          "num_kv_heads": self.num_kv_heads, "head_dim": self.head_dim, "position": position})
        norms = {"input": norm, "post_mixer": norm}
        layers = [
            LayerSpec("pre_norm", attn(PartSpec("toy_interleaved_rope", {"head_dim": self.head_dim, "theta": self.theta})),
                      PartSpec("toy_routed", {"hidden_size": self.hidden_size, "expert_size": self.expert_size,
                                              "num_experts": self.num_experts}), norms, "model.layers.0."),
            LayerSpec("pre_norm", attn(PartSpec(self.second_position, {"head_dim": self.head_dim, "theta": self.theta})),
                      PartSpec("swiglu", {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size}),
                      norms, "model.layers.1."),
        ]
        return ModelPlan(hidden_size=self.hidden_size, vocab_size=self.vocab_size, max_positions=self.max_position_embeddings,
                         embedding=PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}),
                         final_norm=norm,
                         lm_head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size, "tied": True}),
                         layers=layers, schedule=[0, 1])


def plain_toy2_logits(cfg, w, ids):
    T, pos = len(ids), torch.arange(len(ids))
    h = P.embedding(torch.tensor(ids), w["model.embed_tokens.weight"])
    second = P.rope if cfg.second_position == "rope" else (lambda x, pos, theta: P.rope(x, pos // 2, theta))
    for layer, enc in ((0, _interleaved_rope), (1, second)):
        p = f"model.layers.{layer}."
        x = P.rms_norm(h, w[p + "input_layernorm.weight"], cfg.eps)
        q = enc(P.linear(x, w[p + "self_attn.q_proj.weight"]).view(T, cfg.num_heads, cfg.head_dim), pos, cfg.theta)
        k = enc(P.linear(x, w[p + "self_attn.k_proj.weight"]).view(T, cfg.num_kv_heads, cfg.head_dim), pos, cfg.theta)
        v = P.linear(x, w[p + "self_attn.v_proj.weight"]).view(T, cfg.num_kv_heads, cfg.head_dim)
        h = h + P.linear(P.attention(q, k, v).reshape(T, -1), w[p + "self_attn.o_proj.weight"])
        x = P.rms_norm(h, w[p + "post_attention_layernorm.weight"], cfg.eps)
        if layer == 0:
            gate = torch.softmax(P.linear(x, w[p + "moe.router.weight"]), dim=-1)
            for e in range(cfg.num_experts):
                y = P.linear(torch.relu(P.linear(x, w[p + f"moe.experts.{e}.w1.weight"])), w[p + f"moe.experts.{e}.w2.weight"])
                h = h + gate[:, e:e + 1] * y
        else:
            h = h + P.swiglu(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return P.linear(P.rms_norm(h, w["model.norm.weight"], cfg.eps), w["model.embed_tokens.weight"])


@pytest.mark.parametrize("second_position", ["rope", "toy_half_speed_rope"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_feed_forward_with_a_router_and_toy_position_encoding(dtype, second_position, tmp_path):
    """A feed-forward with routing and a position encoding of another kind, registered from this file, in one
    layer beside a stock layer; embeddings tied.  Whole, in changing portions (whose single tokens replay the
    decode graph, the toy parts inside it) and mixed with page reuse.  With ``toy_half_speed_rope`` the second
    layer's position part is a SUBCLASS of the stock rotary part with other arithmetic: its decode steps must
    run its own arithmetic too, not the stock rotation of the one-launch decode kernel."""
    import schedules
    from forge_b200.config import register_architecture, unregister_architecture
    from forge_b200.engine import ModelRunner, StepEntry
    from forge_b200.parts import register_part, unregister_part
    from forge_b200.weights import write_random_model
    from plain.safetensors_reader import read_safetensors
    rope_cls, ffn_cls, half_cls = _toy_part_classes()
    register_part("position", "toy_interleaved_rope", rope_cls)
    register_part("position", "toy_half_speed_rope", half_cls)
    register_part("feed_forward", "toy_routed", ffn_cls)
    register_architecture("Toy2ForCausalLM", Toy2Config)
    try:
        cfg = Toy2Config(second_position=second_position)
        d = write_random_model(cfg, str(tmp_path / "toy2"), seed=7, std=0.12, embed_std=0.6, norm_std=0.15)
        w = {k: torch.from_numpy(v).double() for k, v in read_safetensors(os.path.join(d, "model.safetensors")).items()}
        assert "model.layers.0.moe.experts.2.w2.weight" in w and "lm_head.weight" not in w
        reqs = {f"t{i}": random_tokens(n, cfg.vocab_size, seed=50 + i) for i, n in enumerate([37, 70, 19, 52])}
        want = {rid: plain_toy2_logits(cfg, w, toks).float() for rid, toks in reqs.items()}
        runner = ModelRunner(d, dtype=dtype, page_size=8, cache_tokens=200, max_requests=3)
        assert runner.graph_safe and runner.cuda_graphs        # both toy parts read device tensors only
        for steps in (schedules.whole(reqs), schedules.changing_portions(reqs), schedules.last_one_by_one(reqs, tail=12),
                      schedules.mixed(reqs, max_live=3)):
            got = {rid: torch.zeros(len(t), cfg.vocab_size) for rid, t in reqs.items()}
            for entries, end in steps:
                for rid, p, n in entries:
                    if not runner.is_live(rid):
                        runner.admit(rid)
                lg = runner.step([StepEntry(rid, reqs[rid][p:p + n], list(range(n))) for rid, p, n in entries]).cpu()
                o = 0
                for rid, p, n in entries:
                    got[rid][p:p + n] = lg[o:o + n]
                    o += n
                for rid in end:
                    runner.release(rid)
                runner.manager.check()
            for rid in reqs:
                assert max_rel_err(got[rid], want[rid]) <= TOL[dtype], rid
    finally:
        unregister_part("position", "toy_interleaved_rope")
        unregister_part("position", "toy_half_speed_rope")
        unregister_part("feed_forward", "toy_routed")
        unregister_architecture("Toy2ForCausalLM")


# ---------------------------------------------------------------------------------------------------
# A model whose every layer keeps a window only: its requests may run far past what the pool holds.

@dataclass(frozen=True)
class ToyWindowConfig:
    vocab_size: int = 53
    hidden_size: int = 32
    num_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 16
    intermediate_size: int = 40
    eps: float = 1e-5
    theta: float = 200.0
    window: int = 11
    num_layers: int = 2
    max_position_embeddings: int = 512

    @classmethod
    def from_dict(cls, d, architecture="ToyWindowForCausalLM"):
        return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})

    def to_dict(self):
        return dict(asdict(self), architectures=["ToyWindowForCausalLM"])

    def plan(self):
        from forge_b200.config import LayerSpec, ModelPlan, PartSpec
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.eps})
        mixer = PartSpec("attention", {"hidden_size": self.hidden_size, "num_heads": self.num_heads,
                                       "num_kv_heads": self.num_kv_heads, "head_dim": self.head_dim, "window": self.window,
                                       "position": PartSpec("rope", {"head_dim": self.head_dim, "theta": self.theta})})
        ffn = PartSpec("swiglu", {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size})
        layers = [LayerSpec("pre_norm", mixer, ffn, {"input": norm, "post_mixer": norm}, f"model.layers.{i}.")
                  for i in range(self.num_layers)]
        return ModelPlan(hidden_size=self.hidden_size, vocab_size=self.vocab_size, max_positions=self.max_position_embeddings,
                         embedding=PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}),
                         final_norm=norm,
                         lm_head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size, "tied": True}),
                         layers=layers, schedule=list(range(self.num_layers)))


def plain_window_logits(cfg, w, ids):
    T, pos = len(ids), torch.arange(len(ids))
    h = P.embedding(torch.tensor(ids), w["model.embed_tokens.weight"])
    for layer in range(cfg.num_layers):
        p = f"model.layers.{layer}."
        x = P.rms_norm(h, w[p + "input_layernorm.weight"], cfg.eps)
        q = P.rope(P.linear(x, w[p + "self_attn.q_proj.weight"]).view(T, cfg.num_heads, cfg.head_dim), pos, cfg.theta)
        k = P.rope(P.linear(x, w[p + "self_attn.k_proj.weight"]).view(T, cfg.num_kv_heads, cfg.head_dim), pos, cfg.theta)
        v = P.linear(x, w[p + "self_attn.v_proj.weight"]).view(T, cfg.num_kv_heads, cfg.head_dim)
        h = h + P.linear(P.attention(q, k, v, window=cfg.window).reshape(T, -1), w[p + "self_attn.o_proj.weight"])
        x = P.rms_norm(h, w[p + "post_attention_layernorm.weight"], cfg.eps)
        h = h + P.swiglu(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return P.linear(P.rms_norm(h, w["model.norm.weight"], cfg.eps), w["model.embed_tokens.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windowed_model_decodes_past_the_pools_capacity(dtype, tmp_path):
    """Four pages of eight tokens; a request of 300 tokens.  Pages that the window has passed are given back
    and taken again, the block table keeps its logical length, and a step that the table cannot hold is
    refused before anything is appended."""
    import schedules
    from forge_b200.cache import OutOfPages
    from forge_b200.config import register_architecture, unregister_architecture
    from forge_b200.engine import ModelRunner, StepEntry
    from forge_b200.weights import write_random_model
    from plain.safetensors_reader import read_safetensors
    register_architecture("ToyWindowForCausalLM", ToyWindowConfig)
    try:
        cfg = ToyWindowConfig()
        d = write_random_model(cfg, str(tmp_path / "toywin"), seed=9, std=0.15, embed_std=0.6, norm_std=0.15)
        w = {k: torch.from_numpy(v).double() for k, v in read_safetensors(os.path.join(d, "model.safetensors")).items()}
        toks = random_tokens(300, cfg.vocab_size, seed=3)
        want = plain_window_logits(cfg, w, toks).float()
        runner = ModelRunner(d, dtype=dtype, page_size=8, cache_tokens=32, max_requests=2)
        assert runner.num_pages == 4 and runner.max_pages_per_request == 64
        runner.admit("x")
        got = [runner.step([StepEntry("x", toks[:5], list(range(5)))]).cpu()]
        p = 5
        for n in (3, 1, 1, 7, 2, 1, 1, 1, 6):                      # portions beside single tokens, then decode only
            got.append(runner.step([StepEntry("x", toks[p:p + n], list(range(n)))]).cpu())
            p += n
        while p < 300:
            got.append(runner.step([StepEntry("x", [toks[p]], [0])]).cpu())
            p += 1
            runner.manager.check()
        assert max_rel_err(torch.cat(got), want) <= TOL[dtype]
        assert runner.manager.num_tokens("x") == 300 and sum(t >= 0 for t in runner.manager.block_table("x", "kv2x16_win11")) <= 3
        # a portion that needs more pages than are free is refused, and nothing of it stays behind
        with pytest.raises(OutOfPages):
            runner.step([StepEntry("x", toks[:40], [])])
        assert runner.manager.num_tokens("x") == 300
        runner.release("x")
        runner.manager.check()
        assert runner.manager.num_free_pages() == {"kv2x16_win11": 4}
    finally:
        unregister_architecture("ToyWindowForCausalLM")
