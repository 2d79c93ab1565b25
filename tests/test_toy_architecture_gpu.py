"""The framework is open: a mixer with state of its own, a feed-forward with routing, a position
encoding, an embedding, an output head and a whole architecture are defined HERE, registered, built,
loaded from a random model folder and stepped without touching the library's files.  The architecture
mixes what the Qwen3 plan never does: a scaled embedding with learned absolute positions added, a
stateful mixer, a windowed attention layer beside full ones (two cache groups plus a state group), a
layer that runs twice, a layer execution that reads the cache of an earlier one, a layer whose
attention rotates by half positions and whose feed-forward sends each token to one of three experts,
and a head whose logits are soft-capped.  It is a toy for this test only."""

import json
import math
from dataclasses import dataclass

import pytest
import torch

import plain_qwen3 as plain
from helpers import assert_logits_close
from ondeviceinfer_b200 import (StateNeed, load_resident_model, register_architecture, register_part,
                                write_random_model)
from ondeviceinfer_b200.config import (AttentionSpec, EmbeddingSpec, GatedMLPSpec, HeadSpec, ModelPlan, OrderEntry,
                                       PreNormBlockSpec, RMSNormSpec, RotarySpec, names)
from ondeviceinfer_b200.weights import SafetensorsSource
from ondeviceinfer_b200.weights.tensors import TensorDecl

pytestmark = pytest.mark.gpu
WINDOW = 40


# ----------------------------------------------------------------------------- a toy mixer


@dataclass(frozen=True)
class DecaySpec:
    hidden_size: int
    decay: float
    weight_name: str


class DecayMixer:
    """s_t = decay * s_{t-1} + x_t (per sequence, fp32, kept in the cache's state region);
    y_t = s_t W^T."""

    def __init__(self, spec):
        self.spec = spec

    def tensor_decls(self):
        return [TensorDecl(self.spec.weight_name, (self.spec.hidden_size, self.spec.hidden_size))]

    def load(self, fetch, runtime):
        self.weight = fetch.matrix(self.spec.weight_name).float()

    def cache_needs(self):
        return (StateNeed((self.spec.hidden_size,)),)

    def forward(self, x, ctx, view, residual):
        x = x.float()
        offset = 0
        for slot, n in zip(ctx.slot_list, ctx.q_lens):
            state = view.state[slot]
            rows = []
            for t in range(n):
                state = self.spec.decay * state + x[offset + t]
                rows.append(state)
            view.state[slot] = state
            residual[offset:offset + n] += torch.stack(rows) @ self.weight.t()
            offset += n


# ----------------------------------------------------------------------------- a toy position encoding


@dataclass(frozen=True)
class HalfStepRotarySpec:
    rot_dim: int
    theta: float


class HalfStepRotary:
    """Rotary embedding whose angle advances by half a step per position (position interpolation)."""

    def __init__(self, spec):
        self.spec = spec
        self.rot_dim = spec.rot_dim

    def tensor_decls(self):
        return []

    def load(self, fetch, runtime):
        d = self.spec.rot_dim
        self.inv_freq = (1.0 / (self.spec.theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(runtime.device)

    def rotary_tables(self, ctx):
        def make():
            angles = (ctx.tok_pos.float() * 0.5)[:, None] * self.inv_freq[None, :]
            return torch.cos(angles).contiguous(), torch.sin(angles).contiguous()
        return ctx.memo(("half-step rotary", self.spec), make)


# ----------------------------------------------------------------------------- a toy feed-forward with routing


@dataclass(frozen=True)
class RoutedSpec:
    hidden_size: int
    intermediate_size: int
    experts: int
    prefix: str


class RoutedFeedForward:
    """Each token goes to the expert with the largest router logit (fp32), whose gated MLP output is
    scaled by that expert's softmax probability and added to the residual."""

    def __init__(self, spec):
        self.spec = spec

    def tensor_decls(self):
        s = self.spec
        decls = [TensorDecl(s.prefix + "router", (s.experts, s.hidden_size))]
        for e in range(s.experts):
            decls += [TensorDecl(f"{s.prefix}{e}.g", (s.intermediate_size, s.hidden_size)),
                      TensorDecl(f"{s.prefix}{e}.u", (s.intermediate_size, s.hidden_size)),
                      TensorDecl(f"{s.prefix}{e}.d", (s.hidden_size, s.intermediate_size))]
        return decls

    def load(self, fetch, runtime):
        s = self.spec
        self.router = fetch.matrix(s.prefix + "router").float()
        self.experts = [tuple(fetch.matrix(f"{s.prefix}{e}.{n}").float() for n in "gud") for e in range(s.experts)]

    def forward(self, x, ctx, residual):
        x = x.float()
        prob = torch.softmax(x @ self.router.t(), -1)
        weight, choice = prob.max(-1)
        for e, (g, u, d) in enumerate(self.experts):
            rows = torch.nonzero(choice == e).flatten()
            if rows.numel():
                y = (torch.nn.functional.silu(x[rows] @ g.t()) * (x[rows] @ u.t())) @ d.t()
                residual[rows] += weight[rows, None] * y


# ----------------------------------------------------------------------------- toy ends: embedding and head


@dataclass(frozen=True)
class ScaledEmbeddingSpec:
    vocab_size: int
    hidden_size: int
    weight_name: str
    positions_name: str
    max_positions: int
    scale: float


class ScaledEmbedding:
    """hidden[t] = scale * table[token[t]] + learned[position[t]]."""

    def __init__(self, spec):
        self.spec = spec

    def tensor_decls(self):
        s = self.spec
        return [TensorDecl(s.weight_name, (s.vocab_size, s.hidden_size)),
                TensorDecl(s.positions_name, (s.max_positions, s.hidden_size))]

    def load(self, fetch, runtime):
        self.table = fetch.matrix(self.spec.weight_name)
        self.learned = fetch.matrix(self.spec.positions_name)

    def forward(self, ctx):
        return self.spec.scale * self.table[ctx.token_ids.long()].float() + self.learned[ctx.tok_pos.long()].float()


@dataclass(frozen=True)
class SoftCapHeadSpec:
    vocab_size: int
    hidden_size: int
    weight_name: str
    cap: float
    tied: bool = True          # binds the embedding's table, declares nothing


class SoftCapHead:
    """logits = cap * tanh((rows W^T) / cap)."""

    def __init__(self, spec):
        self.spec = spec

    def tensor_decls(self):
        return []

    def load(self, fetch, runtime):
        self.weight = fetch.matrix(self.spec.weight_name)

    def forward(self, rows, ctx):
        return self.spec.cap * torch.tanh(rows.float() @ self.weight.float().t() / self.spec.cap)


# ----------------------------------------------------------------------------- a toy architecture


@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int
    hidden_size: int
    eps: float

    @classmethod
    def from_dict(cls, raw):
        return cls(raw["vocab_size"], raw["hidden_size"], raw["eps"])

    def to_dict(self):
        return {"architectures": ["ToyForCausalLM"], "vocab_size": self.vocab_size,
                "hidden_size": self.hidden_size, "eps": self.eps}

    def to_plan(self):
        H = self.hidden_size

        def attention(i, window, nq, nkv, d):
            return AttentionSpec(H, nq, nkv, d, RotarySpec(d, 3000.0), f"l{i}.attn.",
                                 names(q="q", k="k", v="v", o="o", q_norm="qn", k_norm="kn"),
                                 qk_norm_eps=self.eps, window=window)

        def block(i, mixer):
            return PreNormBlockSpec(RMSNormSpec(H, self.eps, f"l{i}.n1"), mixer, RMSNormSpec(H, self.eps, f"l{i}.n2"),
                                    GatedMLPSpec(H, 2 * H, "silu", f"l{i}.ff.", names(gate="g", up="u", down="d")))

        routed = PreNormBlockSpec(
            RMSNormSpec(H, self.eps, "l3.n1"),
            AttentionSpec(H, 3, 3, 16, HalfStepRotarySpec(16, 500.0), "l3.attn.",
                          names(q="q", k="k", v="v", o="o", q_norm="qn", k_norm="kn"), qk_norm_eps=self.eps),
            RMSNormSpec(H, self.eps, "l3.n2"), RoutedSpec(H, 40, 3, "l3.moe."))
        layers = (block(0, attention(0, None, 4, 2, 16)), block(1, DecaySpec(H, 0.9, "l1.mix")),
                  block(2, attention(2, WINDOW, 2, 1, 32)), routed)
        order = (OrderEntry(0), OrderEntry(1), OrderEntry(2), OrderEntry(0), OrderEntry(2, cache_from=2), OrderEntry(3))
        return ModelPlan(ScaledEmbeddingSpec(self.vocab_size, H, "emb", "pos", MAX_POSITIONS, EMB_SCALE), layers, order,
                         RMSNormSpec(H, self.eps, "nf"), SoftCapHeadSpec(self.vocab_size, H, "emb", LOGIT_CAP))


MAX_POSITIONS, EMB_SCALE, LOGIT_CAP = 640, 3.0, 0.25
TOY = {"architectures": ["ToyForCausalLM"], "vocab_size": 211, "hidden_size": 48, "eps": 1e-5}


def toy_plain_logits(w, ids):
    """Whole sequence, no cache, from the plain functions plus the toy's own rules."""
    H, eps = TOY["hidden_size"], TOY["eps"]
    T = len(ids)
    pos = torch.arange(T)
    h = EMB_SCALE * w["emb"][torch.tensor(ids)] + w["pos"][pos]

    def qkv(i, x, nq, nkv, d, theta=3000.0, step=1.0):
        p = f"l{i}.attn."
        q = plain.rms_norm(plain.linear(x, w[p + "q"]).view(T, nq, d), w[p + "qn"], eps).transpose(0, 1)
        k = plain.rms_norm(plain.linear(x, w[p + "k"]).view(T, nkv, d), w[p + "kn"], eps).transpose(0, 1)
        v = plain.linear(x, w[p + "v"]).view(T, nkv, d).transpose(0, 1)
        cos, sin = plain.rope_tables(pos.float() * step, d, theta, torch.float32)
        return plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v

    def attend(i, q, k, v, window):
        g = q.shape[0] // k.shape[0]
        scores = q @ k.repeat_interleave(g, 0).transpose(-1, -2) / math.sqrt(q.shape[-1])
        visible = pos[None, :] <= pos[:, None]
        if window:
            visible = visible & (pos[None, :] > pos[:, None] - window)
        o = torch.softmax(scores.masked_fill(~visible, float("-inf")), -1) @ v.repeat_interleave(g, 0)
        return plain.linear(o.transpose(0, 1).reshape(T, -1), w[f"l{i}.attn.o"])

    def ffn(i, h):
        m = plain.rms_norm(h, w[f"l{i}.n2"], eps)
        return h + plain.linear(torch.nn.functional.silu(plain.linear(m, w[f"l{i}.ff.g"])) * plain.linear(m, w[f"l{i}.ff.u"]),
                                w[f"l{i}.ff.d"])

    def attention_layer(i, h, nq, nkv, d, window, shared=None):
        q, k, v = qkv(i, plain.rms_norm(h, w[f"l{i}.n1"], eps), nq, nkv, d)
        if shared is not None:
            k, v = shared
        return ffn(i, h + attend(i, q, k, v, window)), (k, v)

    def decay_layer(h):
        x = plain.rms_norm(h, w["l1.n1"], eps)
        state, rows = torch.zeros(H), []
        for t in range(T):
            state = 0.9 * state + x[t]
            rows.append(state)
        return ffn(1, h + torch.stack(rows) @ w["l1.mix"].t())

    h, _ = attention_layer(0, h, 4, 2, 16, None)
    h = decay_layer(h)
    h, kv2 = attention_layer(2, h, 2, 1, 32, WINDOW)
    h, _ = attention_layer(0, h, 4, 2, 16, None)               # the same layer again, on its own cache
    h, _ = attention_layer(2, h, 2, 1, 32, WINDOW, shared=kv2)  # reads the third execution's keys and values
    # half-step rotation, then a routed feed-forward
    q, k, v = qkv(3, plain.rms_norm(h, w["l3.n1"], eps), 3, 3, 16, theta=500.0, step=0.5)
    h = h + attend(3, q, k, v, None)
    m = plain.rms_norm(h, w["l3.n2"], eps)
    prob = torch.softmax(m @ w["l3.moe.router"].t(), -1)
    weight, choice = prob.max(-1)
    routed = torch.zeros_like(h)
    for t in range(T):
        e = int(choice[t])
        y = plain.linear(torch.nn.functional.silu(plain.linear(m[t:t + 1], w[f"l3.moe.{e}.g"])) *
                         plain.linear(m[t:t + 1], w[f"l3.moe.{e}.u"]), w[f"l3.moe.{e}.d"])
        routed[t] = weight[t] * y[0]
    h = h + routed
    return LOGIT_CAP * torch.tanh(plain.linear(plain.rms_norm(h, w["nf"], eps), w["emb"]) / LOGIT_CAP)


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    register_part(DecaySpec, DecayMixer)
    register_part(HalfStepRotarySpec, HalfStepRotary)
    register_part(RoutedSpec, RoutedFeedForward)
    register_part(ScaledEmbeddingSpec, ScaledEmbedding)
    register_part(SoftCapHeadSpec, SoftCapHead)
    register_architecture("ToyForCausalLM", ToyConfig)
    folder = write_random_model(tmp_path_factory.mktemp("toy"), TOY, seed=5)
    source = SafetensorsSource(folder)
    weights = {n: source.fetch(n).float() for n in source.stored()}
    return folder, weights


def test_registered_toy_is_built_with_its_cache_groups(toy):
    folder, weights = toy
    assert json.loads((folder / "config.json").read_text())["architectures"] == ["ToyForCausalLM"]
    assert "l1.mix" in weights and "l2.attn.kn" in weights and "l3.moe.router" in weights and "l3.moe.2.d" in weights
    assert weights["pos"].shape == (MAX_POSITIONS, TOY["hidden_size"]) and "head" not in weights
    model = load_resident_model(folder, dtype="float32")
    cache = model.make_cache(max_tokens=1024, max_seqs=2)
    assert len(cache.kv_groups) == 3 and len(cache.state_groups) == 1
    windowed = next(g for g in cache.kv_groups if g.need.window == WINDOW)
    full = next(g for g in cache.kv_groups if g.need.window is None and g.need.num_kv_heads == 2)
    routed = next(g for g in cache.kv_groups if g.need.num_kv_heads == 3)
    assert full.owners == [0, 3] and windowed.owners == [2] and routed.owners == [5] and cache.state_groups[0].owners == [1]
    assert cache.max_step_tokens == 256 and windowed.ring_pages > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_model_steps_like_its_plain_form_however_it_is_cut(toy, dtype):
    folder, weights = toy
    model = load_resident_model(folder, dtype=dtype)
    gen = torch.Generator().manual_seed(9)
    lengths = [600, 45, 130, 41, 90, 300]      # 600 > the ring of the windowed group and > one step's limit
    requests = [torch.randint(0, TOY["vocab_size"], (n,), generator=gen).tolist() for n in lengths]
    expected = [toy_plain_logits(weights, r) for r in requests]
    cache = model.make_cache(max_tokens=2048, max_seqs=3)

    # each alone and whole (the 600-token request is cut into sub-steps by the step function)
    for r in (0, 1):
        slot = cache.alloc()
        assert_logits_close(model.step(cache, [slot], [requests[r]], "all"), expected[r], dtype, f"toy whole {r}")
        cache.free(slot)

    # around the window's edge one token at a time: positions WINDOW-2 .. WINDOW+2 and on
    slot = cache.alloc()
    rows = [model.step(cache, [slot], [requests[2][:WINDOW - 2]], "all")]
    rows += [model.step(cache, [slot], [[t]], "last") for t in requests[2][WINDOW - 2:]]
    assert_logits_close(torch.cat(rows), expected[2], dtype, "toy token by token over the window's edge")
    cache.free(slot)

    # batches of three on three slots, unequal prompts, shorter requests end earlier, slots reused:
    # the state of a reused slot must start from zero
    got = {r: [] for r in range(6)}
    for batch in ([0, 1, 2], [3, 4, 5]):
        slots = {r: cache.alloc() for r in batch}
        cut = {r: max(1, len(requests[r]) - 5 - 3 * (r % 3)) for r in batch}
        logits = model.step(cache, [slots[r] for r in batch], [requests[r][:cut[r]] for r in batch], "all")
        offset = 0
        for r in batch:
            got[r].append(logits[offset:offset + cut[r]])
            offset += cut[r]
        live = list(batch)
        while live:
            for r in [r for r in live if cut[r] == len(requests[r])]:
                cache.free(slots.pop(r))
                live.remove(r)
            if not live:
                break
            logits = model.step(cache, [slots[r] for r in live], [[requests[r][cut[r]]] for r in live], "last")
            for i, r in enumerate(live):
                got[r].append(logits[i:i + 1])
                cut[r] += 1
        cache.check()
    for r in range(6):
        assert_logits_close(torch.cat(got[r]), expected[r], dtype, f"toy batched {r}")
