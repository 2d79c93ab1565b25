"""Each part alone, built from its spec through the registry and loaded from a plain
dictionary of tensors, against the plain functions; sizes and options differ from the
tiny models' (no Q/K norm, partial rotary, a given scale, a width of 72)."""

import math

import pytest
import torch

import plain_qwen3 as plain
from helpers import assert_logits_close
from ondeviceinfer_b200.cache import SequenceCache
from ondeviceinfer_b200.config import (AttentionSpec, GatedMLPSpec, NoPositionSpec, PreNormBlockSpec, RMSNormSpec,
                                       RotarySpec, names)
from ondeviceinfer_b200.engine.step import StepContext
from ondeviceinfer_b200.parts import Runtime, build_part
from ondeviceinfer_b200.parts.linear import flush_residual_add
from ondeviceinfer_b200.weights import Fetcher, StoredTensor, check

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


class DictSource:
    def __init__(self, tensors):
        self.tensors = tensors

    def stored(self):
        return {n: StoredTensor(tuple(t.shape), t.dtype) for n, t in self.tensors.items()}

    def fetch(self, name):
        return self.tensors[name]


def load(part, tensors, dtype):
    check(part.tensor_decls(), DictSource(tensors).stored())
    part.load(Fetcher(DictSource(tensors), DT[dtype], DEV), Runtime(DT[dtype], DEV))
    return part


def random_tensors(part, seed):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for decl in part.tensor_decls():
        t = torch.randn(decl.shape, generator=g)
        out[decl.name] = (1 + 0.1 * t if decl.init == "one_plus_normal" else t / math.sqrt(decl.shape[-1])).to(torch.bfloat16)
    return out


def context_for(part_needs, lengths, past, dtype, tokens_dummy=True):
    """A cache with one layer execution and a step context for sequences that already hold
    `past` positions (filled by earlier steps of the caller)."""
    cache = SequenceCache([part_needs], [None], dtype=DT[dtype], device=DEV, max_tokens=2048, max_seqs=len(lengths))
    return cache


@pytest.mark.parametrize("dtype", DT)
def test_rmsnorm_part(dtype):
    part = build_part(RMSNormSpec(200, 1e-4, "n.weight"))
    tensors = random_tensors(part, 0)
    load(part, tensors, dtype)
    x = torch.randn(5, 200) * 2
    out = part(x.to(DEV))
    assert out.dtype == DT[dtype]
    expected = plain.rms_norm(x.to(DT[dtype]), tensors["n.weight"].to(DT[dtype]), 1e-4)
    assert_logits_close(out, expected, dtype)
    rows = torch.tensor([4, 1], dtype=torch.int32, device=DEV)
    assert torch.equal(part(x.to(DEV), rows), out[[4, 1]])


def test_rotary_part_tables_are_shared_within_a_step():
    part = build_part(RotarySpec(head_dim=48, theta=5000.0, rotary_dim=32))
    load(part, {}, "float32")
    cache = SequenceCache([()], [None], dtype=torch.float32, device=DEV, max_tokens=64, max_seqs=2)
    a, b = cache.alloc(), cache.alloc()
    cache.advance([b], [9])
    ctx = StepContext(cache, [a, b], [[1, 2, 3], [4]], [], DEV)
    cos, sin = part.rotary_tables(ctx)
    assert part.rotary_tables(ctx)[0] is cos
    ec, es = plain.rope_tables(torch.tensor([0, 1, 2, 9]), 32, 5000.0, torch.float32)
    assert torch.allclose(cos.cpu(), ec[:, :16], atol=2e-7) and torch.allclose(sin.cpu(), es[:, :16], atol=2e-7)
    assert build_part(NoPositionSpec()).rotary_tables(ctx) is None


def plain_attention_part(x, w, spec, dtype):
    """Whole-sequence attention with the part's options, from the plain functions."""
    T = x.shape[0]
    nq, nkv, d = spec.num_heads, spec.num_kv_heads, spec.head_dim
    q = plain.linear(x, w[spec.name("q")]).view(T, nq, d).transpose(0, 1)
    k = plain.linear(x, w[spec.name("k")]).view(T, nkv, d).transpose(0, 1)
    v = plain.linear(x, w[spec.name("v")]).view(T, nkv, d).transpose(0, 1)
    if spec.qk_norm_eps is not None:
        q = plain.rms_norm(q, w[spec.name("q_norm")], spec.qk_norm_eps)
        k = plain.rms_norm(k, w[spec.name("k_norm")], spec.qk_norm_eps)
    if isinstance(spec.position, RotarySpec):
        rot = spec.position.dim
        cos, sin = plain.rope_tables(torch.arange(T), rot, spec.position.theta, x.dtype)
        q = torch.cat((plain.apply_rope(q[..., :rot], cos, sin), q[..., rot:]), -1)
        k = torch.cat((plain.apply_rope(k[..., :rot], cos, sin), k[..., rot:]), -1)
    scale = spec.scale if spec.scale is not None else 1 / math.sqrt(d)
    g = nq // nkv
    scores = q.float() @ k.float().repeat_interleave(g, 0).transpose(-1, -2) * scale
    pos = torch.arange(T)
    visible = pos[None, :] <= pos[:, None]
    if spec.window:
        visible &= pos[None, :] > pos[:, None] - spec.window
    scores = scores.masked_fill(~visible, float("-inf"))
    o = (torch.softmax(scores, -1) @ v.float().repeat_interleave(g, 0)).to(x.dtype)
    return plain.linear(o.transpose(0, 1).reshape(T, nq * d), w[spec.name("o")])


ATTENTION_SPECS = {
    "no_norm_partial_rotary_scaled": dict(qk_norm_eps=None, position=RotarySpec(48, 5000.0, 32), scale=0.2, window=None),
    "norm_no_position": dict(qk_norm_eps=1e-4, position=NoPositionSpec(), scale=None, window=None),
    "window": dict(qk_norm_eps=1e-5, position=RotarySpec(48, 1e4), scale=None, window=24),
}


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("variant", ATTENTION_SPECS)
def test_attention_part_alone(variant, dtype):
    spec = AttentionSpec(hidden_size=72, num_heads=6, num_kv_heads=2, head_dim=48, prefix="attn.",
                         names=names(q="wq", k="wk", v="wv", o="wo", q_norm="qn", k_norm="kn"),
                         **ATTENTION_SPECS[variant])
    part = build_part(spec)
    tensors = random_tensors(part, 1)
    load(part, tensors, dtype)
    torch.manual_seed(2)
    lengths = [90, 7]
    xs = [torch.randn(n, 72).to(DT[dtype]) for n in lengths]
    w = {n: t.to(DT[dtype]) for n, t in tensors.items()}
    expected = [plain_attention_part(x, w, spec, dtype).float() for x in xs]
    cache = SequenceCache([part.cache_needs()], [None], dtype=DT[dtype], device=DEV, max_tokens=512, max_seqs=2,
                          max_step_tokens=64)
    slots = [cache.alloc(), cache.alloc()]
    got = [[], []]
    # three steps: a chunk of each, then the rest of the long one token by token with the short one's rest
    cuts = [[0, 50, 88, 89, 90], [0, 3, 5, 6, 7]]
    for step in range(4):
        runs = [xs[i][cuts[i][step]:cuts[i][step + 1]] for i in range(2)]
        q_lens = [len(r) for r in runs]
        cache.reserve(slots, q_lens)
        ctx = StepContext(cache, slots, [[0] * n for n in q_lens], [], DEV)
        residual = torch.zeros(sum(q_lens), 72, device=DEV)
        part.forward(torch.cat(runs).to(DEV), ctx, cache.view(0), residual)
        cache.advance(slots, q_lens)
        got[0].append(residual[:q_lens[0]])
        got[1].append(residual[q_lens[0]:])
    for i in range(2):
        assert_logits_close(torch.cat(got[i]), expected[i], dtype, f"{variant} sequence {i}")


@pytest.mark.parametrize("dtype", DT)
def test_gated_mlp_part_adds_into_the_residual(dtype):
    spec = GatedMLPSpec(72, 200, "silu", "ff.", names(gate="g", up="u", down="d"))
    part = build_part(spec)
    tensors = random_tensors(part, 3)
    load(part, tensors, dtype)
    x = torch.randn(9, 72).to(DT[dtype])
    residual = torch.randn(9, 72)
    r = residual.clone().to(DEV)
    part.forward(x.to(DEV), None, r)
    w = {k.replace("ff.", "") + "_proj.weight": v.to(DT[dtype]) for k, v in
         {"ff.gate": tensors["ff.g"], "ff.up": tensors["ff.u"], "ff.down": tensors["ff.d"]}.items()}
    expected = residual + plain.swiglu(x, w, "").float()
    assert_logits_close(r, expected, dtype)
    with pytest.raises(ValueError):
        build_part(GatedMLPSpec(8, 16, "gelu", "", names(gate="g", up="u", down="d")))


@pytest.mark.parametrize("dtype", DT)
def test_prenorm_block_alone(dtype):
    cfg = {"num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 16, "hidden_size": 112,
           "rms_norm_eps": 2e-5, "intermediate_size": 48}
    p = "model.layers.0."
    spec = PreNormBlockSpec(
        mixer_norm=RMSNormSpec(112, 2e-5, p + "input_layernorm.weight"),
        mixer=AttentionSpec(112, 5, 5, 16, RotarySpec(16, 777.0), p + "self_attn.",
                            names(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", o="o_proj.weight",
                                  q_norm="q_norm.weight", k_norm="k_norm.weight"), qk_norm_eps=2e-5),
        ffn_norm=RMSNormSpec(112, 2e-5, p + "post_attention_layernorm.weight"),
        ffn=GatedMLPSpec(112, 48, "silu", p + "mlp.", names(gate="gate_proj.weight", up="up_proj.weight",
                                                           down="down_proj.weight")))
    block = build_part(spec)
    tensors = random_tensors(block, 4)
    load(block, tensors, dtype)
    hidden = torch.randn(70, 112)
    cos, sin = plain.rope_tables(torch.arange(70), 16, 777.0, DT[dtype])
    expected = plain.decoder_layer(hidden.to(DT[dtype]), {k: v.to(DT[dtype]) for k, v in tensors.items()}, 0, cfg, cos, sin)
    cache = SequenceCache([block.cache_needs()], [None], dtype=DT[dtype], device=DEV, max_tokens=128, max_seqs=1)
    slot = cache.alloc()
    cache.reserve([slot], [70])
    ctx = StepContext(cache, [slot], [[0] * 70], [], DEV)
    h = hidden.clone().to(DEV)
    block.forward(h, ctx, cache.view(0))
    flush_residual_add(ctx)          # the block may leave its last product's add to the norm that follows
    assert h.dtype == torch.float32
    assert_logits_close(h, expected.float(), dtype)


def test_two_blocks_decode_through_the_fused_products(monkeypatch):
    """Two blocks with heads of 128 at decode width: the second norm of a block and the first of the next
    are left to the following product (`NormedRows`), the heads are prepared in the q/k/v product's epilogue.
    Against the plain layers over the whole sequence, and against the same blocks with the fusions refused."""
    from ondeviceinfer_b200.parts import Attention, GatedMLP
    import importlib
    linear_module = importlib.import_module("ondeviceinfer_b200.parts.linear")
    cfg = {"num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 128, "hidden_size": 192,
           "rms_norm_eps": 1e-5, "intermediate_size": 320}
    blocks, tensors = [], {}
    for i in range(2):
        p = f"model.layers.{i}."
        spec = PreNormBlockSpec(
            mixer_norm=RMSNormSpec(192, 1e-5, p + "input_layernorm.weight"),
            mixer=AttentionSpec(192, 2, 1, 128, RotarySpec(128, 5000.0), p + "self_attn.",
                                names(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", o="o_proj.weight",
                                      q_norm="q_norm.weight", k_norm="k_norm.weight"), qk_norm_eps=1e-5),
            ffn_norm=RMSNormSpec(192, 1e-5, p + "post_attention_layernorm.weight"),
            ffn=GatedMLPSpec(192, 320, "silu", p + "mlp.", names(gate="gate_proj.weight", up="up_proj.weight",
                                                                down="down_proj.weight")))
        block = build_part(spec)
        mine = random_tensors(block, 40 + i)
        load(block, mine, "bfloat16")
        blocks.append(block)
        tensors.update(mine)
    n, tail = 75, 5
    hidden = torch.randn(n, 192)
    cos, sin = plain.rope_tables(torch.arange(n), 128, 5000.0, torch.bfloat16)
    w = {k: v.to(torch.bfloat16) for k, v in tensors.items()}
    expected = plain.decoder_layer(plain.decoder_layer(hidden.bfloat16(), w, 0, cfg, cos, sin), w, 1, cfg, cos, sin).float()

    def run(count_fused):
        cache = SequenceCache([b.cache_needs() for b in blocks], [None, None], dtype=torch.bfloat16, device=DEV,
                              max_tokens=128, max_seqs=1)
        slot = cache.alloc()
        rows, seen = [], {"lazy": 0, "heads": 0}
        real_operand, real_heads = linear_module._operand, linear_module.project_heads

        def counting_operand(x, *args):
            seen["lazy"] += isinstance(x, linear_module.NormedRows)
            return real_operand(x, *args)

        def counting_heads(*args, **kwargs):
            seen["heads"] += 1
            return real_heads(*args, **kwargs)

        monkeypatch.setattr(linear_module, "_operand", counting_operand)
        monkeypatch.setattr("ondeviceinfer_b200.parts.attention.project_heads", counting_heads)
        for start, stop in [(0, n - tail)] + [(t, t + 1) for t in range(n - tail, n)]:
            cache.reserve([slot], [stop - start])
            ctx = StepContext(cache, [slot], [[0] * (stop - start)], [], DEV)
            ctx.residual_sumsq = None
            h = hidden[start:stop].clone().to(DEV)
            for i, block in enumerate(blocks):
                block.forward(h, ctx, cache.view(i))
            flush_residual_add(ctx)
            cache.advance([slot], [stop - start])
            rows.append(h.cpu())
        assert (seen["lazy"] > 0) == count_fused and (seen["heads"] > 0) == count_fused, seen
        return torch.cat(rows)

    fused = run(True)
    assert_logits_close(fused, expected, "bfloat16")
    monkeypatch.setattr(Attention, "takes_lazy_norm", False)
    monkeypatch.setattr(GatedMLP, "takes_lazy_norm", False)
    monkeypatch.setattr("ondeviceinfer_b200.parts.attention.heads_in_epilogue", lambda *a, **k: False)
    plain_way = run(False)
    assert_logits_close(plain_way, expected, "bfloat16")
    assert float((fused - plain_way).abs().max()) <= 0.02 * float(expected.abs().max())


def test_unknown_spec_and_bad_sizes_are_refused():
    class Unknown:
        pass

    with pytest.raises(KeyError):
        build_part(Unknown())
    base = dict(hidden_size=64, num_kv_heads=2, position=NoPositionSpec(), prefix="", names=names(q="q", k="k", v="v", o="o"))
    with pytest.raises(ValueError):
        build_part(AttentionSpec(num_heads=3, head_dim=16, **base))        # heads not divisible by groups
    with pytest.raises(ValueError):
        build_part(AttentionSpec(num_heads=4, head_dim=24, **base))        # head size not a multiple of 16
    with pytest.raises(ValueError):
        build_part(RotarySpec(head_dim=16, theta=1e4, rotary_dim=18))
