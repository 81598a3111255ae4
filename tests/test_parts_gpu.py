"""Each part of a layer alone against the plain implementation, at sizes that are not the tiny models',
and a toy mixer with a state of its own, a toy feed-forward with routing, another position encoding, a scaled
embedding and a capped head, all defined HERE: they are registered, built into a model by a toy architecture and stepped through the
engine without any change to the library's files."""
import math
import os
import tempfile
from dataclasses import dataclass

import pytest
import torch

import helpers
import plain_apertus as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def rnd(x, dtype):
    return x if dtype == torch.float32 else x.to(dtype).float()


def tol(dtype, ref):
    return (2e-5 if dtype == torch.float32 else 6 * 2.0 ** -8) * max(float(ref.abs().max()), 1e-3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    from tileinfer_b200.config import NormSpec
    from tileinfer_b200.parts import Runtime, lookup
    torch.manual_seed(0)
    spec = NormSpec("rmsnorm", 200, 3e-6, "n.weight")
    w = rnd(1 + 0.2 * torch.randn(200), dtype)
    part = lookup("norm", "rmsnorm")(spec, {"n.weight": w.to(dtype)}, Runtime(dtype))
    assert [d.name for d in part.tensors(spec)] == ["n.weight"]
    x = rnd(torch.randn(9, 200) * 2, dtype)
    out = torch.empty(9, 200, dtype=dtype, device="cuda")
    part.forward(x.to(dtype).cuda(), out)
    ref = plain.rmsnorm(x, w, 3e-6, dtype)
    assert float((out.float().cpu() - ref).abs().max()) <= tol(dtype, ref)
    xs, d = x.to(dtype).cuda(), rnd(torch.randn(9, 200), dtype)
    part.add_forward(xs, d.to(dtype).cuda(), out)
    ref = plain.rmsnorm(rnd(x + d, dtype), w, 3e-6, dtype)
    assert float((out.float().cpu() - ref).abs().max()) <= tol(dtype, ref)


def test_rope_tables_follow_the_reference_recipe():
    """32-bit inverse frequencies and angles, 64-bit cos/sin of the 32-bit angle, llama3 scaling per
    frequency (src/model/rope.jl:15-48), beyond the original length where the scaling matters."""
    from tileinfer_b200.config import Llama3RopeScaling, PositionSpec
    from tileinfer_b200.parts import Runtime, lookup
    for scaling, sdict in ((None, None), (Llama3RopeScaling(8.0, 1.0, 4.0, 64), {"rope_type": "llama3", "factor": 8.0,
                           "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 64})):
        spec = PositionSpec("rope", 48, 12e6, scaling, 4096)
        part = lookup("position", "rope")(spec, Runtime(torch.float32), 300)
        cfg = plain.read_config({"vocab_size": 1, "hidden_size": 48, "intermediate_size": 1, "num_hidden_layers": 1,
                                 "num_attention_heads": 1, "head_dim": 48, "rms_norm_eps": 1e-5, "rope_theta": 12e6,
                                 "max_position_embeddings": 4096, "rope_scaling": sdict})
        cos, sin = plain.rope_tables(cfg, torch.arange(300), torch.float32)
        table = part.cos_sin.cpu()
        assert table.shape == (300, 24, 2)
        assert torch.equal(table[:, :, 0], cos[:, :24]) and torch.equal(table[:, :, 1], sin[:, :24])
        assert torch.equal(cos[:, :24], cos[:, 24:])            # both halves share the angles


class OneStep:
    """A minimal stand-in for the engine around a part: a cache for one layer and step contexts."""

    def __init__(self, mixer, dtype, max_tokens=512, max_seqs=4):
        from tileinfer_b200.cache import Cache
        from tileinfer_b200.engine.step import StepPlanner
        self.cache = Cache([mixer.cache_request()], dtype, "cuda", max_tokens=max_tokens, max_seqs=max_seqs)
        self.planner = StepPlanner(self.cache, 512, "cuda")
        self.planner.runtime = mixer.rt

    def run(self, mixer, entries, hidden):
        """entries: (slot, [n, H] activations). Returns the mixer's output rows in the same order."""
        self.cache.reserve([(s, h.shape[0]) for s, h in entries])
        ctx = self.planner.plan([(s, [0] * h.shape[0]) for s, h in entries], [[] for _ in entries])
        x = torch.cat([h for _, h in entries]).cuda()
        out = mixer.forward(x, ctx, self.cache.layer(0))
        if out.dim() == 3:
            out = out.sum(0)
        for s, h in entries:
            self.cache.advance(s, h.shape[0])
        return out.float().cpu().clone()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("qk_norm", [True, False])
def test_attention_part_whole_then_continued(dtype, qk_norm):
    """The attention mixer alone: sequences of unequal lengths in one step, then continued by chunks and
    single tokens, against the plain attention block on the whole sequences."""
    from tileinfer_b200.config import Llama3RopeScaling, MixerSpec, PositionSpec
    from tileinfer_b200.parts import Runtime, lookup
    torch.manual_seed(1)
    H, nq, nkv, D = 72, 6, 2, 32
    rt = Runtime(dtype)
    pos_spec = PositionSpec("rope", D, 50000.0, Llama3RopeScaling(4.0, 1.0, 2.0, 32), 4096)
    names = {"q": "q.w", "k": "k.w", "v": "v.w", "o": "o.w", "q_norm": "qn.w", "k_norm": "kn.w"}
    spec = MixerSpec("attention", "a.", H, nq, nkv, D, qk_norm, 1e-6, 1 / math.sqrt(D), None, None, pos_spec, names)
    cls = lookup("mixer", "attention")
    decls = cls.tensors(spec)
    assert len(decls) == (6 if qk_norm else 4)
    W = {d.name: rnd(torch.randn(d.shape) * (0.1 if len(d.shape) == 2 else 0.2) + (0 if len(d.shape) == 2 else 1), dtype) for d in decls}
    mixer = cls(spec, {k: v.to(dtype) for k, v in W.items()}, rt, lookup("position", "rope")(pos_spec, rt, 512))
    cfg = plain.read_config({"vocab_size": 1, "hidden_size": H, "intermediate_size": 1, "num_hidden_layers": 1,
                             "num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": D, "rms_norm_eps": 1e-6,
                             "rope_theta": 50000.0, "max_position_embeddings": 4096, "qk_norm": qk_norm,
                             "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0,
                                              "high_freq_factor": 2.0, "original_max_position_embeddings": 32}})
    pw = {"L.self_attn.q_proj.weight": W["a.q.w"], "L.self_attn.k_proj.weight": W["a.k.w"], "L.self_attn.v_proj.weight": W["a.v.w"],
          "L.self_attn.o_proj.weight": W["a.o.w"]}
    if qk_norm:
        pw["L.self_attn.q_norm.weight"], pw["L.self_attn.k_norm.weight"] = W["a.qn.w"], W["a.kn.w"]
    hs = [rnd(torch.randn(n, H), dtype) for n in (100, 37)]
    refs = [plain.attention_block(h, pw, "L.", cfg, torch.arange(h.shape[0]), dtype) for h in hs]
    env = OneStep(mixer, dtype)
    a, b = env.cache.alloc_slot(), env.cache.alloc_slot()
    cut = lambda h: h.to(dtype)
    got_a, got_b = [], []
    out = env.run(mixer, [(a, cut(hs[0][:70])), (b, cut(hs[1][:5]))], H)
    got_a.append(out[:70]); got_b.append(out[70:])
    out = env.run(mixer, [(b, cut(hs[1][5:36])), (a, cut(hs[0][70:71]))], H)      # a chunk and a single token, order swapped
    got_b.append(out[:31]); got_a.append(out[31:])
    for t in range(71, 100):
        entries = [(a, cut(hs[0][t:t + 1]))] + ([(b, cut(hs[1][36:37]))] if t == 71 else [])
        out = env.run(mixer, entries, H)
        got_a.append(out[:1])
        if t == 71:
            got_b.append(out[1:])
    for got, ref in ((torch.cat(got_a), refs[0]), (torch.cat(got_b), refs[1])):
        assert float((got - ref).abs().max()) <= tol(dtype, ref)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_part_with_another_rotation(dtype):
    """The attention mixer asks its position encoding for a rotation and knows nothing else about it: here
    the rope part with interleaved pairs over half of each head (options of its record), a prompt and
    then single tokens, against the plain functions with that rotation written out."""
    from tileinfer_b200.config import MixerSpec, PositionSpec
    from tileinfer_b200.parts import Runtime, lookup
    torch.manual_seed(6)
    H, nq, nkv, D, rotary = 72, 4, 2, 64, 32
    rt = Runtime(dtype)
    pos_spec = PositionSpec("rope", D, 50000.0, None, 4096, {"rotary_dim": rotary, "pairing": "interleaved"})
    names = {"q": "q.w", "k": "k.w", "v": "v.w", "o": "o.w", "q_norm": "qn.w", "k_norm": "kn.w"}
    spec = MixerSpec("attention", "a.", H, nq, nkv, D, True, 1e-6, 1 / math.sqrt(D), None, None, pos_spec, names)
    cls = lookup("mixer", "attention")
    W = {d.name: rnd(torch.randn(d.shape) * (0.1 if len(d.shape) == 2 else 0.2) + (0 if len(d.shape) == 2 else 1), dtype)
         for d in cls.tensors(spec)}
    position = lookup("position", "rope")(pos_spec, rt, 256)
    rotation = position.rotation()
    assert rotation.rotary_dim == rotary and rotation.interleaved and rotation.cos_sin.shape == (256, rotary // 2, 2)
    mixer = cls(spec, {k: v.to(dtype) for k, v in W.items()}, rt, position)
    cfg = plain.read_config({"vocab_size": 1, "hidden_size": H, "intermediate_size": 1, "num_hidden_layers": 1,
                             "num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": rotary, "rms_norm_eps": 1e-6,
                             "rope_theta": 50000.0, "max_position_embeddings": 4096})
    n = 90
    h = rnd(torch.randn(n, H), dtype)
    cos, sin = plain.rope_tables(cfg, torch.arange(n), dtype)             # frequencies over the rotated width

    def rotate(x):
        y = x.clone()
        for i in range(rotary // 2):
            a, b, c, s_ = 2 * i, 2 * i + 1, cos[:, i, None], sin[:, i, None]
            y[..., a] = rnd(rnd(x[..., a] * c, dtype) + rnd(-x[..., b] * s_, dtype), dtype)
            y[..., b] = rnd(rnd(x[..., b] * c, dtype) + rnd(x[..., a] * s_, dtype), dtype)
        return y

    q = plain.linear(h, W["a.q.w"], dtype).view(n, nq, D)
    k = plain.linear(h, W["a.k.w"], dtype).view(n, nkv, D)
    v = plain.linear(h, W["a.v.w"], dtype).view(n, nkv, D)
    q, k = rotate(plain.rmsnorm(q, W["a.qn.w"], 1e-6, dtype)), rotate(plain.rmsnorm(k, W["a.kn.w"], 1e-6, dtype))
    ref = plain.linear(plain.attention(q, k, v, 1 / math.sqrt(D), dtype).reshape(n, nq * D), W["a.o.w"], dtype)
    env = OneStep(mixer, dtype)
    a = env.cache.alloc_slot()
    got = [env.run(mixer, [(a, h[:70].to(dtype))], H)] + [env.run(mixer, [(a, h[t:t + 1].to(dtype))], H) for t in range(70, n)]
    assert float((torch.cat(got) - ref).abs().max()) <= tol(dtype, ref)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [1, 7, 150])
def test_feed_forward_part(dtype, n):
    from tileinfer_b200.config import FeedForwardSpec
    from tileinfer_b200.parts import Runtime, lookup
    torch.manual_seed(2)
    H, I = 72, 200
    names = {"up": "up.w", "down": "down.w", "alpha_p": "ap", "alpha_n": "an", "beta": "b", "eps": "e"}
    spec = FeedForwardSpec("xielu_mlp", "m.", H, I, names)
    cls = lookup("feed_forward", "xielu_mlp")
    W = {"m.up.w": rnd(torch.randn(I, H) * 0.2, dtype), "m.down.w": rnd(torch.randn(H, I) * 0.2, dtype),
         "m.ap": torch.tensor([18.125]), "m.an": torch.tensor([10.5]), "m.b": torch.tensor(0.5), "m.e": torch.tensor(-1e-6)}
    assert {d.name for d in cls.tensors(spec)} == set(W)
    part = cls(spec, {k: (v.to(dtype) if v.numel() > 1 else v) for k, v in W.items()}, Runtime(dtype))
    h = rnd(torch.randn(n, H), dtype)
    out = part.forward(h.to(dtype).cuda(), None)
    out = out.sum(0) if out.dim() == 3 else out
    pw = {"L.mlp.up_proj.weight": W["m.up.w"], "L.mlp.down_proj.weight": W["m.down.w"], "L.mlp.act_fn.alpha_p": W["m.ap"],
          "L.mlp.act_fn.alpha_n": W["m.an"], "L.mlp.act_fn.beta": W["m.b"], "L.mlp.act_fn.eps": W["m.e"]}
    ref = plain.feed_forward(h, pw, "L.", dtype)
    # alpha_p = 18 amplifies a one-step difference of the rounded up-projection (the reference notes the
    # same: test/ops/tile.jl:168-174); the bound is a few steps of the activation's scale, not of the output's.
    a = plain.xielu_scalars(W["m.ap"], W["m.an"], W["m.b"], W["m.e"], dtype)
    act = plain.xielu(plain.linear(h, W["m.up.w"], dtype), a, dtype)
    bound = (2e-5 if dtype == torch.float32 else 4 * 2.0 ** -8) * float(act.abs().max()) * float(W["m.down.w"].abs().sum(1).max()) / 8
    assert float((out.float().cpu() - ref).abs().max()) <= max(bound, tol(dtype, ref))


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_part(dtype):
    """The pre-norm arrangement alone, around a mixer and a feed-forward that exist only here (plain
    torch arithmetic on the device): the residual stream after each of the two adds and the normed
    input handed to the next block."""
    from tileinfer_b200.config import NormSpec
    from tileinfer_b200.parts import Runtime, lookup
    torch.manual_seed(4)
    H, n = 136, 11
    rt = Runtime(dtype)

    class Scale:
        def __init__(self, factor):
            self.factor = factor

        def forward(self, h, step, cache=None):
            return (h.float() * self.factor).to(h.dtype)

    ws = {f"n{i}.weight": rnd(1 + 0.2 * torch.randn(H), dtype) for i in range(3)}
    norms = [lookup("norm", "rmsnorm")(NormSpec("rmsnorm", H, 1e-6, f"n{i}.weight"), {k: v.to(dtype) for k, v in ws.items()}, rt)
             for i in range(3)]
    block = lookup("block", "pre_norm")(None, Scale(0.75), Scale(-0.5), norms[0], norms[1])
    assert block.input_norm is norms[0]
    x = rnd(torch.randn(n, H) * 2, dtype)
    xs = x.to(dtype).cuda()
    h = torch.empty(n, H, dtype=dtype, device="cuda")
    norms[0].forward(xs, h)
    h_out = torch.empty_like(h)
    assert block.forward(xs, h, None, None, norms[2], h_out) is h_out
    h0 = plain.rmsnorm(x, ws["n0.weight"], 1e-6, dtype)
    x1 = rnd(x + rnd(h0 * 0.75, dtype), dtype)
    h1 = plain.rmsnorm(x1, ws["n1.weight"], 1e-6, dtype)
    x2 = rnd(x1 + rnd(h1 * -0.5, dtype), dtype)
    ref = plain.rmsnorm(x2, ws["n2.weight"], 1e-6, dtype)
    assert float((xs.float().cpu() - x2).abs().max()) <= tol(dtype, x2)
    assert float((h_out.float().cpu() - ref).abs().max()) <= tol(dtype, ref)


# ------------------------------------------------------------------------------------------------
# Toy parts, defined in this test only.
def build_toy_architecture():
    from tileinfer_b200.config import (FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec,
                                       TensorDecl, register_architecture)
    from tileinfer_b200.parts import (CacheRequest, Embedding, FeedForward, Head, Mixer, PositionEncoding, register_embedding,
                                      register_feed_forward, register_head, register_mixer, register_position)

    @register_embedding("toy_scaled")
    class ScaledEmbedding(Embedding):
        """Rows of the table times a multiplier from the model's options: an end of the model that is not Apertus's."""

        def __init__(self, spec, tensors, rt):
            self.table = rt.param(tensors[spec.embed_name])
            self.scale = float(spec.options["embed_scale"])

        @classmethod
        def tensors(cls, spec):
            return [TensorDecl(spec.embed_name, (spec.vocab_size, spec.hidden_size), ("normal", 0.5))]

        def forward(self, token_ids, out, status):
            out.copy_((self.table[token_ids.long()].float() * self.scale).to(out.dtype))
            return out

    @register_head("toy_capped")
    class CappedHead(Head):
        """logits = cap * tanh(W h / cap), with a head matrix of its own."""

        def __init__(self, spec, tensors, rt, embedding):
            self.weight = tensors[spec.lm_head_name].to(rt.device).float()
            self.cap = float(spec.options["logit_cap"])

        @classmethod
        def tensors(cls, spec):
            return [TensorDecl(spec.lm_head_name, (spec.vocab_size, spec.hidden_size), ("normal", 0.3))]

        def forward(self, h, logits):
            logits.copy_(self.cap * torch.tanh(h.float() @ self.weight.t() / self.cap))
            return logits

    @register_position("toy_learned")
    class LearnedOffsets(PositionEncoding):
        """Adds sin(position · rate) to the mixer input: a position encoding that is not a rotation."""

        def __init__(self, spec, rt, max_positions):
            self.rate = float(spec.options["rate"])

        def apply(self, h, positions):
            return h + torch.sin(positions.float()[:, None] * self.rate).to(h.dtype)

    @register_mixer("toy_decay")
    class DecayMixer(Mixer):
        """s <- decay · s + W_in x per sequence, y = W_out s: a running state of fixed size per sequence,
        kept in the cache's state slot between steps."""

        def __init__(self, spec, tensors, rt, position):
            self.spec, self.rt, self.position = spec, rt, position
            self.w_in = tensors[spec.prefix + "w_in"].to(rt.device).float()
            self.w_out = tensors[spec.prefix + "w_out"].to(rt.device).float()
            self.decay = float(spec.options["decay"])

        @classmethod
        def tensors(cls, spec):
            S = spec.options["state"]
            return [TensorDecl(spec.prefix + "w_in", (S, spec.hidden_size), ("normal", 0.3)),
                    TensorDecl(spec.prefix + "w_out", (spec.hidden_size, S), ("normal", 0.3))]

        def cache_request(self):
            return CacheRequest("state", shape=(self.spec.options["state"],), dtype=torch.float32)

        def forward(self, h, step, cache):
            h = self.position.apply(h, step.positions).float()
            out = torch.empty_like(h)
            row = 0
            for slot, n in zip(step.host_slots, step.host_q_lens):          # tokens of a sequence run in order
                s = cache.state[slot]
                for t in range(row, row + n):
                    s = self.decay * s + self.w_in @ h[t]
                    out[t] = self.w_out @ s
                cache.state[slot] = s
                row += n
            return out.to(self.rt.dtype)

    @register_feed_forward("toy_routed")
    class RoutedFeedForward(FeedForward):
        """Two experts, each token goes to the one with the larger router logit (32-bit router)."""

        def __init__(self, spec, tensors, rt):
            self.rt = rt
            self.router = tensors[spec.prefix + "router"].to(rt.device).float()
            self.experts = tensors[spec.prefix + "experts"].to(rt.device).float()

        @classmethod
        def tensors(cls, spec):
            return [TensorDecl(spec.prefix + "router", (2, spec.hidden_size), ("normal", 0.5)),
                    TensorDecl(spec.prefix + "experts", (2, spec.hidden_size, spec.hidden_size), ("normal", 0.2))]

        def forward(self, h, step):
            x = h.float()
            choice = (x @ self.router.t()).argmax(-1)
            return torch.einsum("nij,nj->ni", self.experts[choice], x).to(self.rt.dtype)

    @dataclass(frozen=True)
    class ToyConfig:
        vocab_size: int
        hidden_size: int
        state: int
        max_position_embeddings: int = 512

        @classmethod
        def from_dict(cls, c):
            return cls(c["vocab_size"], c["hidden_size"], c["state_size"])

        def to_dict(self):
            return {"architectures": ["ToyForCausalLM"], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                    "state_size": self.state}

        def model_spec(self):
            H = self.hidden_size
            norm = lambda name: NormSpec("rmsnorm", H, 1e-5, name)
            toy = LayerSpec("pre_norm",
                            MixerSpec("toy_decay", "l0.mix.", H, position=PositionSpec("toy_learned", options={"rate": 0.37}),
                                      options={"state": self.state, "decay": 0.8}),
                            norm("l0.n1"), FeedForwardSpec("toy_routed", "l0.ffn.", H), norm("l0.n2"))
            attn = LayerSpec("pre_norm",
                             MixerSpec("attention", "l1.attn.", H, 2, 1, 16, False, 1e-5, 0.25, None, None,
                                       PositionSpec("rope", 16, 10000.0, None, 512),
                                       {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "qn", "k_norm": "kn"}),
                             norm("l1.n1"),
                             FeedForwardSpec("xielu_mlp", "l1.mlp.", H, 40, {"up": "up", "down": "down", "alpha_p": "ap",
                                                                           "alpha_n": "an", "beta": "b", "eps": "e"}),
                             norm("l1.n2"))
            # The order names the toy layer twice: its second run has a state of its own.
            return ModelSpec("ToyForCausalLM", self.vocab_size, H, (toy, attn), (0, 1, 0), norm("final"),
                             "embed", "head", self.max_position_embeddings, embedding_kind="toy_scaled", head_kind="toy_capped",
                             options={"embed_scale": 3.0, "logit_cap": 2.5})

    register_architecture("ToyForCausalLM", ToyConfig)
    return ToyConfig


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_parts_are_registered_built_and_stepped(dtype):
    """A mixer with a state of its own, a routed feed-forward and another position encoding run through the
    library's engine next to its attention layer; cutting the work differently changes nothing."""
    from tileinfer_b200.engine import Engine
    from tileinfer_b200.weights import write_model_folder
    ToyConfig = build_toy_architecture()
    cfg = ToyConfig(50, 24, 6)
    with tempfile.TemporaryDirectory() as d:
        folder = write_model_folder(cfg, 3, os.path.join(d, "toy"))
        eng = Engine.load(folder, dtype=dtype, max_context=128, max_seqs=3, max_tokens=512, graphs=False)
        kinds = sorted(g.kind for g in eng.cache.groups)
        assert kinds == ["paged_kv", "state"] and eng.cache.state_groups[0].state.shape[:2] == (2, 3)
        prompts = helpers.random_prompts(50, [20, 7, 33], 4)
        a, b, c = (eng.new_sequence() for _ in range(3))
        whole = eng.step([(a, prompts[0]), (b, prompts[1]), (c, prompts[2])], [list(range(len(p))) for p in prompts]).cpu()
        for s in (a, b, c):
            eng.free_sequence(s)
        # Again, cut differently, in reused slots (whose state must have been zeroed): prefixes, then one token each.
        c, a, b = (eng.new_sequence() for _ in range(3))
        slot = {0: a, 1: b, 2: c}
        rows = {i: [] for i in range(3)}
        head = {0: 15, 1: 1, 2: 30}
        out = eng.step([(slot[i], prompts[i][:head[i]]) for i in range(3)], [list(range(head[i])) for i in range(3)]).cpu()
        r = 0
        for i in range(3):
            rows[i].append(out[r:r + head[i]]); r += head[i]
        t = 0
        while any(head[i] + t < len(prompts[i]) for i in range(3)):
            live = [i for i in range(3) if head[i] + t < len(prompts[i])]
            out = eng.step([(slot[i], [prompts[i][head[i] + t]]) for i in live]).cpu()
            for k, i in enumerate(live):
                rows[i].append(out[k:k + 1])
            t += 1
        again = torch.cat([torch.cat(rows[i]) for i in range(3)])
        assert again.shape == whole.shape and bool(torch.isfinite(whole).all())
        limit = 1e-4 if dtype == "float32" else 4 * 2.0 ** -8 * float(whole.abs().max())
        assert float((again - whole).abs().max()) <= limit
        assert 1.0 < float(whole.abs().max()) <= 2.5                     # the toy head's cap is in effect
        assert type(eng.model.embedding).__name__ == "ScaledEmbedding" and type(eng.model.head).__name__ == "CappedHead"
