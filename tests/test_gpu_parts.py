"""Each part alone against the plain implementation, at sizes other than the tiny models';
and a toy architecture defined here (a mixer with state of its own beside attention, a layer
run twice, a layer reading another layer's cache) that is registered, given random weights,
built and stepped without any change to the framework's files."""
import math
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_llama as plain
import replay_util as ru

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 1e-4, "bfloat16": 2e-2}


def runtime(dtype, max_tokens=128, max_requests=4, page=16):
    from hfee_b200.parts import Runtime
    return Runtime(DT[dtype], DEV, max_tokens, max_requests, page)


def make_step(lengths_before, new_counts, rt, tokens=None, want=None):
    from hfee_b200.engine import Step, StepBuffers, StepEntry
    buf = StepBuffers(rt.max_tokens, rt.max_requests, DEV)
    entries = [StepEntry(i, (tokens[i] if tokens else [0] * n), (want[i] if want else ())) for i, n in enumerate(new_counts)]
    return Step(entries, lengths_before, buf)


def rnd(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(dtype):
    from hfee_b200 import PartSpec
    from hfee_b200.parts import build_part
    rt = runtime(dtype)
    w = 1 + rnd((200,), 1, 0.1)
    part = build_part("norm", PartSpec("rms_norm", width=200, eps=3e-6), {"weight": w.to(DEV)}, rt)
    x = rnd((9, 200), 2, 4.0).to(DEV)
    out = torch.empty(9, 200, dtype=DT[dtype], device=DEV)
    part.forward(x, out)
    ref = plain.rms_norm(x.double().cpu().numpy(), w.double().numpy(), 3e-6)
    assert ru.rel_err(out.float().cpu().numpy(), ref) < (1e-5 if dtype == "float32" else 6e-3)


def test_rotary_part_tables_and_scaling():
    from hfee_b200 import PartSpec
    from hfee_b200.config import RopeScaling
    from hfee_b200.parts import build_part
    rt = runtime("float32")
    sc = RopeScaling(8.0, 1.0, 4.0, 64)
    part = build_part("position", PartSpec("rotary", head_dim=48, rope_dim=32, theta=500000.0, scaling=sc,
                                           pairing="interleaved"), {}, rt)
    ref_inv = plain.rope_inv_freq(32, 500000.0, {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                 "high_freq_factor": 4.0, "original_max_position_embeddings": 64})
    assert np.allclose(part.inv_freq_host, ref_inv, rtol=1e-15)
    step = make_step([7, 0, 100], [3, 2, 1], rt)
    cs = part.table(step)
    assert part.table(step) is cs                                # one table per step, shared by layers
    pos = np.array([7, 8, 9, 0, 1, 100], dtype=np.float64)
    ang = pos[:, None] * ref_inv[None, :]
    assert np.abs(cs[..., 0].cpu().numpy() - np.cos(ang)).max() < 1e-7
    assert np.abs(cs[..., 1].cpu().numpy() - np.sin(ang)).max() < 1e-7


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv,hd,window,pairing", [(6, 2, 48, None, "half"), (5, 5, 16, 9, "interleaved"),
                                                         (8, 1, 64, None, "interleaved")])
def test_attention_part_in_two_portions(dtype, heads, kv, hd, window, pairing):
    """The attention part alone: a sequence fed as two portions equals the plain whole-sequence
    attention layer (projections, rotation, cache, attention, output projection, residual)."""
    from hfee_b200 import CacheManager, PartSpec
    from hfee_b200.parts import build_part
    width, n = 72, 41
    rt = runtime(dtype)
    pos_spec = PartSpec("rotary", head_dim=hd, rope_dim=hd, theta=10000.0, scaling=None, pairing=pairing)
    spec = PartSpec("attention", width=width, heads=heads, kv_heads=kv, head_dim=hd, position=pos_spec,
                    window=window, scale=None)
    w = {"q": rnd((heads * hd, width), 1, 0.1), "k": rnd((kv * hd, width), 2, 0.1),
         "v": rnd((kv * hd, width), 3, 0.1), "o": rnd((width, heads * hd), 4, 0.1)}
    wd = {k: v.to(DT[dtype]).to(DEV) for k, v in w.items()}
    part = build_part("mixer", spec, wd, rt)
    cache = CacheManager({0: part.cache_need()}, 16, 8, 4, 128, DT[dtype], DEV)
    x = rnd((n, width), 5)
    xq = x.to(DT[dtype])
    slot = cache.open()
    residual = torch.zeros(n, width, dtype=torch.float32, device=DEV)
    at = 0
    for count in (30, 11):
        cache.reserve(slot, at + count); cache.sync()
        step = make_step([at], [count], rt)
        part.forward(xq[at:at + count].to(DEV).contiguous(), residual[at:at + count], step, cache.view(0), True)
        cache.commit(slot, at + count)
        at += count
    f = lambda t: t.to(DT[dtype]).double().numpy()
    xn = f(x)
    inv = plain.rope_inv_freq(hd, 10000.0)
    q = plain.rope(plain.linear(xn, f(w["q"])), heads, hd, range(n), inv, pairing)
    k = plain.rope(plain.linear(xn, f(w["k"])), kv, hd, range(n), inv, pairing)
    att = plain.attention(q, k, plain.linear(xn, f(w["v"])), heads, kv, hd, window)
    ref = plain.linear(att, f(w["o"]))
    assert ru.rel_err(residual.cpu().numpy(), ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,width,inner", [(5, 40, 100), (70, 64, 172), (3, 96, 90)])
def test_feed_forward_part(dtype, n, width, inner):
    from hfee_b200 import PartSpec
    from hfee_b200.parts import build_part
    rt = runtime(dtype)
    w = {"gate": rnd((inner, width), 1, 0.2), "up": rnd((inner, width), 2, 0.2), "down": rnd((width, inner), 3, 0.2)}
    part = build_part("feed_forward", PartSpec("swiglu", width=width, inner=inner),
                      {k: v.to(DT[dtype]).to(DEV) for k, v in w.items()}, rt)
    x = rnd((n, width), 4)
    base = rnd((n, width), 5)
    residual = base.clone().to(DEV)
    part.forward(x.to(DT[dtype]).to(DEV), residual, make_step([0], [n], rt))
    f = lambda t: t.to(DT[dtype]).double().numpy()
    ref = base.double().numpy() + plain.feed_forward(f(x), f(w["gate"]), f(w["up"]), f(w["down"]))
    assert ru.rel_err(residual.cpu().numpy(), ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tied", [False, True])
def test_embedding_and_head_parts(dtype, tied):
    from hfee_b200 import PartSpec
    from hfee_b200.parts import part_class
    rt = runtime(dtype)
    vocab, width = 301, 56
    table = rnd((vocab, width), 1).to(DT[dtype]).to(DEV)
    emb = part_class("embedding", "token")(PartSpec("token", vocab=vocab, width=width), {"table": table}, rt)
    toks = [300, 0, 17, 17, 5]
    step = make_step([0], [5], rt, tokens=[toks])
    residual = torch.empty(5, width, dtype=torch.float32, device=DEV)
    emb.forward(step, residual)
    assert torch.equal(residual, table[torch.tensor(toks, device=DEV)].float())
    wh = rnd((vocab, width), 2).to(DT[dtype]).to(DEV)
    head = part_class("head", "linear")(PartSpec("linear", vocab=vocab, width=width, tied=tied),
                                        {} if tied else {"weight": wh}, rt, embedding=emb)
    xn = rnd((5, width), 3).to(DT[dtype]).to(DEV)
    logits = torch.empty(5, vocab, dtype=torch.float32, device=DEV)
    head.forward(xn, logits)
    ref = xn.double().cpu().numpy() @ (table if tied else wh).double().cpu().numpy().T
    assert ru.rel_err(logits.cpu().numpy(), ref) < 1e-5


# ---------------------------------------------------------------------------------------------
# A toy architecture, defined and registered here only.

def _register_toy():
    from hfee_b200 import (FixedState, LayerSpec, Mixer, ModelSpec, PartSpec, RunSpec, TensorNeed,
                           register_architecture, register_part)
    from hfee_b200.parts import part_class

    class RunningMeanMixer(Mixer):
        """y_t = W . mean(x_0..x_t): the state is the running sum of the inputs, one row per request."""

        @staticmethod
        def tensor_needs(spec):
            return {"w": TensorNeed((spec.width, spec.width))}

        def __init__(self, spec, tensors, rt):
            super().__init__(spec, tensors, rt)
            self.w = tensors["w"].float()

        def cache_need(self):
            return FixedState((int(self.spec.width),), "float32")

        def forward(self, xn, residual, step, cache, writes_cache):
            at = 0
            for slot, start, count in step.requests:
                x = xn[at:at + count].float()
                sums = cache.state[slot][None, :] + torch.cumsum(x, dim=0)
                denom = torch.arange(start + 1, start + count + 1, device=x.device, dtype=torch.float32)[:, None]
                residual[at:at + count] += (sums / denom) @ self.w.t()
                if writes_cache:
                    cache.state[slot] = sums[-1]
                at += count

    try:
        part_class("mixer", "running_mean")
    except ValueError:
        register_part("mixer", "running_mean", RunningMeanMixer)

    @dataclass(frozen=True)
    class ToyConfig:
        width: int
        heads: int
        head_dim: int
        inner: int
        vocab: int
        eps: float
        window: int

        @classmethod
        def from_dict(cls, d):
            return cls(d["width"], d["heads"], d["head_dim"], d["inner"], d["vocab_size"], d["eps"], d["window"])

    def toy_spec(c):
        pos = PartSpec("rotary", head_dim=c.head_dim, rope_dim=c.head_dim // 2, theta=1000.0, scaling=None, pairing="half")
        attn = PartSpec("attention", width=c.width, heads=c.heads, kv_heads=1, head_dim=c.head_dim, position=pos,
                        window=None, scale=None)
        mean = PartSpec("running_mean", width=c.width)
        ffn = PartSpec("swiglu", width=c.width, inner=c.inner)
        norm = PartSpec("rms_norm", width=c.width, eps=c.eps)
        block = PartSpec("pre_norm", width=c.width)

        def layer(i, mixer, mixer_names):
            p = f"toy.{i}."
            names = {"ffn.gate": p + "gate", "ffn.up": p + "up", "ffn.down": p + "down",
                     "mixer_norm.weight": p + "n1", "ffn_norm.weight": p + "n2"}
            names.update({f"mixer.{k}": p + k for k in mixer_names})
            return LayerSpec.pre_norm(block, mixer, ffn, norm, norm, names=names)

        local = attn.replace(window=c.window, position=PartSpec("none"))
        layers = (layer(0, attn, "qkvo"), layer(1, mean, "w"), layer(2, attn, "qkvo"), layer(3, local, "qkvo"))
        # layer 0 (attention), layer 1 (running mean), layer 1 again with a state of its own,
        # layer 2, which projects only queries and attends over the cache layer 0 wrote, and
        # layer 3: attention over a window of its own cache, without position encoding
        schedule = (RunSpec(0, cache=0), RunSpec(1, cache=1), RunSpec(1, cache=2), RunSpec(2, cache=0, writes_cache=False),
                    RunSpec(3, cache=3))
        return ModelSpec(width=c.width, vocab=c.vocab, embedding=PartSpec("token", vocab=c.vocab, width=c.width),
                         layers=layers, schedule=schedule, final_norm=norm,
                         head=PartSpec("linear", vocab=c.vocab, width=c.width, tied=True),
                         names={"embedding.table": "toy.embed", "final_norm.weight": "toy.norm"}, max_positions=512)

    register_architecture("ToyStateForCausalLM", ToyConfig.from_dict, toy_spec)


TOY = {"architectures": ["ToyStateForCausalLM"], "width": 80, "heads": 5, "head_dim": 32, "inner": 116,
       "vocab_size": 211, "eps": 1e-5, "window": 21}


def toy_plain_forward(w, tokens, bf16):
    f = (lambda a: plain.to_bf16_grid(a)) if bf16 else (lambda a: a)
    c = TOY
    n = len(tokens)
    inv = plain.rope_inv_freq(16, 1000.0)

    def rope_partial(x, heads):
        x = x.reshape(n, heads, 32).copy()
        rot = plain.rope(x[:, :, :16].reshape(n, heads * 16), heads, 16, range(n), inv, "half")
        x[:, :, :16] = rot.reshape(n, heads, 16)
        return x.reshape(n, heads * 32)

    def ffn(x, p):
        xb = plain.rms_norm(x, w[p + "n2"], c["eps"])
        return x + plain.feed_forward(xb, f(w[p + "gate"]), f(w[p + "up"]), f(w[p + "down"]))

    x = plain.embed(f(w["toy.embed"]), tokens)
    xb = plain.rms_norm(x, w["toy.0.n1"], c["eps"])
    k0 = rope_partial(plain.linear(xb, f(w["toy.0.k"])), 1)
    v0 = plain.linear(xb, f(w["toy.0.v"]))
    q0 = rope_partial(plain.linear(xb, f(w["toy.0.q"])), 5)
    x = ffn(x + plain.linear(plain.attention(q0, k0, v0, 5, 1, 32), f(w["toy.0.o"])), "toy.0.")
    for _ in range(2):                                                   # layer 1 twice
        xb = plain.rms_norm(x, w["toy.1.n1"], c["eps"])
        mean = np.cumsum(xb, axis=0) / np.arange(1, n + 1)[:, None]
        x = ffn(x + plain.linear(mean, f(w["toy.1.w"])), "toy.1.")
    xb = plain.rms_norm(x, w["toy.2.n1"], c["eps"])
    q2 = rope_partial(plain.linear(xb, f(w["toy.2.q"])), 5)
    x = ffn(x + plain.linear(plain.attention(q2, k0, v0, 5, 1, 32), f(w["toy.2.o"])), "toy.2.")
    xb = plain.rms_norm(x, w["toy.3.n1"], c["eps"])                      # windowed, no position encoding
    att = plain.attention(plain.linear(xb, f(w["toy.3.q"])), plain.linear(xb, f(w["toy.3.k"])),
                          plain.linear(xb, f(w["toy.3.v"])), 5, 1, 32, window=c["window"])
    x = ffn(x + plain.linear(att, f(w["toy.3.o"])), "toy.3.")
    return plain.linear(plain.rms_norm(x, w["toy.norm"], c["eps"]), f(w["toy.embed"]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_state_runs_through_the_engine(tmp_path, dtype):
    from hfee_b200 import EngineConfig, FixedState, ModelRunner, PagedKV, write_random_model
    _register_toy()
    d = str(tmp_path / "toy")
    write_random_model(d, TOY, seed=5, dtype="float32")
    w = plain.read_safetensors(d + "/model.safetensors")
    assert "toy.2.k" in w        # layer 2's own k/v are in the checkpoint but unused: it reads layer 0's cache
    rng = np.random.default_rng(9)
    seqs = [rng.integers(0, 211, size=n).tolist() for n in (50, 9, 33, 70)]
    refs = [toy_plain_forward(w, s, dtype == "bfloat16") for s in seqs]
    e = EngineConfig(dtype=dtype, page_size=16, max_requests=3, max_context=128, max_cache_tokens=10 * 16,
                     max_batch_tokens=96)                   # CUDA graphs stay at their default: on
    runner = ModelRunner(d, e)
    # the toy mixer walks the step's host-side list of requests, so it does not declare itself safe
    # to capture, and a model with such a part never replays a graph
    assert not runner.model.graph_safe
    needs = runner.model.cache_needs()
    assert needs[0] == PagedKV(1, 32, None) and needs[1] == needs[2] == FixedState((80,), "float32")
    assert needs[3] == PagedKV(1, 32, 21)
    assert len(runner.cache.paged) == 2 and len(runner.cache.states) == 1
    windowed = [g for g in runner.cache.paged if g.need.window][0]
    # the last scheme: decode-only steps of equal batch size while slots and positions change
    # (requests leave after 5 to 40 tokens, the fourth joins in a freed slot): a slot id or a
    # position frozen into a replayed graph would show here
    together = ru.batched_decode(seqs, tails=[40, 5, 30, 35], live=3)
    assert sum(all(len(t) == 1 for _, t, _ in st["entries"]) for st in together) >= 30
    for steps in (ru.whole(seqs), ru.portions(seqs, sizes=(7, 2, 16, 3, 2, 33)), ru.mixed(seqs, live=3, seed=1), together):
        got = ru.run_in_process(runner, steps)
        for i in range(len(seqs)):
            assert ru.rel_err(got[i], refs[i]) < TOL[dtype], f"request {i}"
    assert runner.graph_replays == 0
    # the windowed group gave pages back while requests were still running: a request of 70 tokens
    # never held more than ceil((21 + longest portion) / 16) + 1 of them
    s = runner.open()
    for t in range(0, 70, 2):
        runner.step([__import__("hfee_b200").StepEntry(s, seqs[3][t:t + 2], [])])
        assert int((windowed.table[s] >= 0).sum()) <= 3
    runner.close(s)


# ---------------------------------------------------------------------------------------------
# A second toy architecture: a feed-forward with routing and another position encoding, both
# defined here, beside the framework's attention.

def _register_routed_toy():
    from hfee_b200 import (LayerSpec, ModelSpec, Part, PartSpec, TensorNeed, register_architecture, register_part)
    from hfee_b200.parts import part_class
    from hfee_b200.parts.rotary import Rotary

    class RoutedFeedForward(Part):
        """Top-1 routing over small gated experts: router logits in float32, each token runs
        through the expert with the largest logit, scaled by that logit's softmax weight."""
        category = "feed_forward"

        @staticmethod
        def tensor_needs(spec):
            e, w, i = spec.experts, spec.width, spec.inner
            return {"router": TensorNeed((e, w), role="vector"), "gate": TensorNeed((e * i, w)),
                    "up": TensorNeed((e * i, w)), "down": TensorNeed((e * w, i))}

        def __init__(self, spec, tensors, rt):
            super().__init__(spec, tensors, rt)
            e, w, i = spec.experts, spec.width, spec.inner
            self.router = tensors["router"].float()
            self.gate = tensors["gate"].float().reshape(e, i, w)
            self.up = tensors["up"].float().reshape(e, i, w)
            self.down = tensors["down"].float().reshape(e, w, i)

        def forward(self, xn, residual, step):
            x = xn.float()
            logits = x @ self.router.t()                       # float32 router
            weight, choice = torch.softmax(logits, dim=-1).max(dim=-1)
            for e in range(self.router.shape[0]):
                rows = (choice == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                xe = x[rows]
                g, u = xe @ self.gate[e].t(), xe @ self.up[e].t()
                residual[rows] += ((g / (1 + torch.exp(-g)) * u) @ self.down[e].t()) * weight[rows, None]

    class ScaledRotary(Rotary):
        """Rotary encoding with positions divided by ``factor`` (linear position interpolation)."""

        def __init__(self, spec, tensors, rt):
            super().__init__(spec, tensors, rt)
            self.inv_freq_host = [f / spec.factor for f in self.inv_freq_host]
            self.inv_freq = torch.tensor(self.inv_freq_host, dtype=torch.float64, device=rt.device)

    for cat, kind, cls in (("feed_forward", "toy_routed", RoutedFeedForward), ("position", "scaled_rotary", ScaledRotary)):
        try:
            part_class(cat, kind)
        except ValueError:
            register_part(cat, kind, cls)

    @dataclass(frozen=True)
    class RoutedConfig:
        d: dict

        @classmethod
        def from_dict(cls, d):
            return cls(dict(d))

    def spec_of(c):
        d = c.d
        w = d["width"]
        pos = PartSpec("scaled_rotary", head_dim=d["head_dim"], rope_dim=d["head_dim"], theta=777.0, scaling=None,
                       pairing="interleaved", factor=d["factor"])
        attn = PartSpec("attention", width=w, heads=d["heads"], kv_heads=d["kv_heads"], head_dim=d["head_dim"],
                        position=pos, window=None, scale=None)
        dense = PartSpec("swiglu", width=w, inner=d["inner"])
        routed = PartSpec("toy_routed", width=w, inner=d["expert_inner"], experts=d["experts"])
        norm = PartSpec("rms_norm", width=w, eps=d["eps"], add_unit=True)
        layers = []
        for i in range(d["layers"]):
            p = f"l{i}."
            ffn = routed if i % 2 == 1 else dense                # dense and routed layers alternate
            names = {"mixer.q": p + "q", "mixer.k": p + "k", "mixer.v": p + "v", "mixer.o": p + "o",
                     "mixer_norm.weight": p + "n1", "ffn_norm.weight": p + "n2"}
            names.update({"ffn." + k: p + "ffn_" + k for k in (("router", "gate", "up", "down") if i % 2 else ("gate", "up", "down"))})
            layers.append(LayerSpec.pre_norm(PartSpec("pre_norm", width=w), attn, ffn, norm, norm, names=names))
        return ModelSpec(width=w, vocab=d["vocab_size"], embedding=PartSpec("token", vocab=d["vocab_size"], width=w),
                         layers=tuple(layers), schedule=ModelSpec.sequential(len(layers)), final_norm=norm,
                         head=PartSpec("linear", vocab=d["vocab_size"], width=w, tied=False),
                         names={"embedding.table": "emb", "final_norm.weight": "norm", "head.weight": "head"}, max_positions=512)

    register_architecture("ToyRoutedForCausalLM", RoutedConfig.from_dict, spec_of)


ROUTED = {"architectures": ["ToyRoutedForCausalLM"], "width": 48, "heads": 6, "kv_heads": 3, "head_dim": 16,
          "inner": 100, "experts": 3, "expert_inner": 40, "layers": 4, "vocab_size": 97, "eps": 1e-6, "factor": 4.0}


def routed_plain_forward(w, tokens):
    c = ROUTED
    n = len(tokens)
    inv = plain.rope_inv_freq(c["head_dim"], 777.0) / c["factor"]
    norm = lambda x, name: plain.rms_norm(x, 1.0 + w[name], c["eps"])         # add_unit: scale by 1 + w
    x = plain.embed(w["emb"], tokens)
    for i in range(c["layers"]):
        p = f"l{i}."
        xb = norm(x, p + "n1")
        q = plain.rope(plain.linear(xb, w[p + "q"]), c["heads"], c["head_dim"], range(n), inv, "interleaved")
        k = plain.rope(plain.linear(xb, w[p + "k"]), c["kv_heads"], c["head_dim"], range(n), inv, "interleaved")
        att = plain.attention(q, k, plain.linear(xb, w[p + "v"]), c["heads"], c["kv_heads"], c["head_dim"])
        x = x + plain.linear(att, w[p + "o"])
        xb = norm(x, p + "n2")
        if i % 2 == 0:
            x = x + plain.feed_forward(xb, w[p + "ffn_gate"], w[p + "ffn_up"], w[p + "ffn_down"])
        else:
            e_n, ei = c["experts"], c["expert_inner"]
            logits = xb @ w[p + "ffn_router"].T
            probs = np.exp(logits - logits.max(1, keepdims=True))
            probs /= probs.sum(1, keepdims=True)
            out = np.zeros_like(x)
            for t in range(n):
                e = int(np.argmax(logits[t]))
                g = w[p + "ffn_gate"].reshape(e_n, ei, -1)[e] @ xb[t]
                u = w[p + "ffn_up"].reshape(e_n, ei, -1)[e] @ xb[t]
                out[t] = (w[p + "ffn_down"].reshape(e_n, -1, ei)[e] @ plain.swiglu(g, u)) * probs[t, e]
            x = x + out
    return plain.linear(norm(x, "norm"), w["head"])


def test_routed_feed_forward_and_another_position_encoding(tmp_path):
    """Float32 (the bfloat16 rounding of the router's input could flip a near-tied expert choice)."""
    from hfee_b200 import EngineConfig, ModelRunner, write_random_model
    _register_routed_toy()
    d = str(tmp_path / "routed")
    write_random_model(d, ROUTED, seed=6, dtype="float32", std=0.08)
    w = plain.read_safetensors(d + "/model.safetensors")
    rng = np.random.default_rng(4)
    seqs = [rng.integers(0, 97, size=n).tolist() for n in (45, 12, 30)]
    refs = [routed_plain_forward(w, s) for s in seqs]
    runner = ModelRunner(d, EngineConfig(dtype="float32", page_size=16, max_requests=3, max_context=64,
                                         max_cache_tokens=7 * 16, max_batch_tokens=64))
    assert not runner.model.graph_safe            # the routed feed-forward picks its rows on the host
    for steps in (ru.whole(seqs), ru.portions(seqs, sizes=(5, 2, 9, 2, 20)), ru.mixed(seqs, live=3, seed=2),
                  ru.batched_decode(seqs, tails=[33, 6, 20])):
        got = ru.run_in_process(runner, steps)
        for i in range(len(seqs)):
            assert ru.rel_err(got[i], refs[i]) < 1e-4, f"request {i}"


# ---------------------------------------------------------------------------------------------
# A third toy architecture: other arrangements of the same parts.  A block with a norm in front of
# and behind each of its two branches (four norms), and a block without a feed-forward; both are
# block parts defined and registered here, the layers name their parts as data.

def _register_sandwich_toy():
    from hfee_b200 import LayerSpec, ModelSpec, PartSpec, register_architecture, register_part
    from hfee_b200.parts import Block, part_class

    class SandwichBlock(Block):
        """``x += post1(mixer(pre1(x))); x += post2(ffn(pre2(x)))``.  Mixers and feed-forwards add
        into the float32 buffer they are given; here that is a zeroed scratch, whose norm then joins
        the stream."""
        needs = ("mixer", "ffn", "pre_mixer_norm", "post_mixer_norm", "pre_ffn_norm", "post_ffn_norm")
        graph_safe = True            # device-side work on buffers that live as long as the engine

        def __init__(self, spec, tensors, rt, parts):
            super().__init__(spec, tensors, rt, parts)
            self.width = int(spec.width)

        def _branch(self, pre, part, post, residual, step, *more):
            rt, n = self.rt, step.n
            xn = rt.scratch("sandwich_in", (rt.max_tokens, self.width))[:n]
            branch = rt.scratch("sandwich_branch", (rt.max_tokens, self.width), torch.float32)[:n]
            normed = rt.scratch("sandwich_out", (rt.max_tokens, self.width), torch.float32)[:n]
            pre.forward(residual, xn)
            branch.zero_()
            part.forward(xn, branch, step, *more)
            post.forward(branch, normed)
            residual += normed

        def forward(self, residual, step, cache, writes_cache):
            p = self.parts
            self._branch(p["pre_mixer_norm"], p["mixer"], p["post_mixer_norm"], residual, step, cache, writes_cache)
            self._branch(p["pre_ffn_norm"], p["ffn"], p["post_ffn_norm"], residual, step)

    class MixerOnlyBlock(Block):
        """``x += mixer(norm(x))``: a layer without a feed-forward."""
        needs = ("mixer", "norm")
        graph_safe = True

        def forward(self, residual, step, cache, writes_cache):
            xn = self.rt.scratch("mixer_only_in", (self.rt.max_tokens, int(self.spec.width)))[:step.n]
            self.parts["norm"].forward(residual, xn)
            self.parts["mixer"].forward(xn, residual, step, cache, writes_cache)

    for kind, cls in (("toy_sandwich", SandwichBlock), ("toy_mixer_only", MixerOnlyBlock)):
        try:
            part_class("block", kind)
        except ValueError:
            register_part("block", kind, cls)

    @dataclass(frozen=True)
    class SandwichConfig:
        d: dict

        @classmethod
        def from_dict(cls, d):
            return cls(dict(d))

    def spec_of(c):
        d = c.d
        w = d["width"]
        pos = PartSpec("rotary", head_dim=d["head_dim"], rope_dim=d["head_dim"], theta=5000.0, scaling=None, pairing="half")
        attn = PartSpec("attention", width=w, heads=d["heads"], kv_heads=d["kv_heads"], head_dim=d["head_dim"],
                        position=pos, window=None, scale=None)
        ffn = PartSpec("swiglu", width=w, inner=d["inner"])
        norm = PartSpec("rms_norm", width=w, eps=d["eps"])
        layers = []
        for i in range(d["layers"]):
            p = f"s{i}."
            names = {"mixer.q": p + "q", "mixer.k": p + "k", "mixer.v": p + "v", "mixer.o": p + "o"}
            if i % 2 == 0:
                parts = {"mixer": ("mixer", attn), "ffn": ("feed_forward", ffn)}
                parts.update({k: ("norm", norm) for k in ("pre_mixer_norm", "post_mixer_norm", "pre_ffn_norm", "post_ffn_norm")})
                names.update({"ffn.gate": p + "gate", "ffn.up": p + "up", "ffn.down": p + "down"})
                names.update({k + ".weight": p + k for k in ("pre_mixer_norm", "post_mixer_norm", "pre_ffn_norm", "post_ffn_norm")})
                layers.append(LayerSpec(PartSpec("toy_sandwich", width=w), parts, names))
            else:
                names["norm.weight"] = p + "norm"
                layers.append(LayerSpec(PartSpec("toy_mixer_only", width=w), {"mixer": ("mixer", attn), "norm": ("norm", norm)}, names))
        return ModelSpec(width=w, vocab=d["vocab_size"], embedding=PartSpec("token", vocab=d["vocab_size"], width=w),
                         layers=tuple(layers), schedule=ModelSpec.sequential(len(layers)), final_norm=norm,
                         head=PartSpec("linear", vocab=d["vocab_size"], width=w, tied=True),
                         names={"embedding.table": "emb", "final_norm.weight": "norm"}, max_positions=256)

    register_architecture("ToySandwichForCausalLM", SandwichConfig.from_dict, spec_of)


SANDWICH = {"architectures": ["ToySandwichForCausalLM"], "width": 72, "heads": 6, "kv_heads": 2, "head_dim": 16,
            "inner": 88, "layers": 3, "vocab_size": 131, "eps": 1e-5}


def sandwich_plain_forward(w, tokens, bf16):
    f = (lambda a: plain.to_bf16_grid(a)) if bf16 else (lambda a: a)
    c = SANDWICH
    n = len(tokens)
    inv = plain.rope_inv_freq(c["head_dim"], 5000.0)
    norm = lambda x, name: plain.rms_norm(x, w[name], c["eps"])

    def attend(xb, p):
        q = plain.rope(plain.linear(xb, f(w[p + "q"])), c["heads"], c["head_dim"], range(n), inv, "half")
        k = plain.rope(plain.linear(xb, f(w[p + "k"])), c["kv_heads"], c["head_dim"], range(n), inv, "half")
        att = plain.attention(q, k, plain.linear(xb, f(w[p + "v"])), c["heads"], c["kv_heads"], c["head_dim"])
        return plain.linear(att, f(w[p + "o"]))

    x = plain.embed(f(w["emb"]), tokens)
    for i in range(c["layers"]):
        p = f"s{i}."
        if i % 2 == 0:
            x = x + norm(attend(norm(x, p + "pre_mixer_norm"), p), p + "post_mixer_norm")
            h = plain.feed_forward(norm(x, p + "pre_ffn_norm"), f(w[p + "gate"]), f(w[p + "up"]), f(w[p + "down"]))
            x = x + norm(h, p + "post_ffn_norm")
        else:
            x = x + attend(norm(x, p + "norm"), p)
    return plain.linear(norm(x, "norm"), f(w["emb"]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_blocks_with_four_norms_and_without_a_feed_forward(tmp_path, dtype):
    from hfee_b200 import EngineConfig, ModelRunner, write_random_model
    _register_sandwich_toy()
    d = str(tmp_path / "sandwich")
    write_random_model(d, SANDWICH, seed=8, dtype="float32", std=0.08)
    w = plain.read_safetensors(d + "/model.safetensors")
    assert "s0.post_ffn_norm" in w and "s1.norm" in w and "s1.gate" not in w       # the layers' parts decide the tensors
    rng = np.random.default_rng(3)
    seqs = [rng.integers(0, 131, size=n).tolist() for n in (47, 11, 60, 35)]
    refs = [sandwich_plain_forward(w, s, dtype == "bfloat16") for s in seqs]
    runner = ModelRunner(d, EngineConfig(dtype=dtype, page_size=16, max_requests=3, max_context=64,
                                         max_cache_tokens=11 * 16, max_batch_tokens=64))
    assert runner.model.graph_safe
    for steps in (ru.whole(seqs), ru.portions(seqs, sizes=(5, 2, 9, 2, 20)), ru.mixed(seqs, live=3, seed=4),
                  ru.batched_decode(seqs, tails=[34, 6, 30, 25], live=3)):
        got = ru.run_in_process(runner, steps)
        for i in range(len(seqs)):
            assert ru.rel_err(got[i], refs[i]) < TOL[dtype], f"request {i}"
    assert runner.graph_replays > 10          # decode-only steps of these blocks replay from CUDA graphs
