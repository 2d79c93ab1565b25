"""The decode path that generation really runs, compared at the level of logits.

``generate()`` does not decode through the generic step function: its one-token steps replay CUDA graphs
on fixed buffers (``engine/decode.py``): rows of a fixed width with padding rows on a slot outside the
cache, page tables of fixed stride, key splits bounded by the graph, counters advanced by the sampling
kernel.  Here given tokens are fed through exactly that path (each step's inputs copied from the host, as
``generate()`` does) and the logits that each replay leaves are compared, per request and position, with
the plain implementation: a wrong page-table row, a padding row that leaks, a dropped key split or a
stale position in one sequence fails these tests, where a comparison of sampled tokens might not.
"""

import pytest
import torch

import ondeviceinfer_b200 as odi
import plain_qwen3 as plain
from helpers import CASES, assert_logits_close, engine_model, plain_logits

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="session")
def tmp_root(tmp_path_factory):
    return tmp_path_factory.mktemp("models")


def replay_batches(model, cache, requests, batches, tails, *, drop=False):
    """Feed ``requests`` (token lists) batch by batch: all but the last ``tails[r]`` tokens of each request in
    one prompt step, then one token per live request per graph replay; a request that has been fed whole
    leaves and gives its slot back.  Returns, per request, the logits at positions ``cut - 1 .. len - 1``."""
    got = {}
    runner = odi.api.decode_runner(model, cache)
    for batch in batches:
        slots = {r: cache.alloc() for r in batch}
        fed = {r: len(requests[r]) - tails[r] for r in batch}
        assert all(n >= 1 for n in fed.values())
        logits = model.step(cache, [slots[r] for r in batch], [requests[r][:fed[r]] for r in batch], "last")
        for i, r in enumerate(batch):
            got[r] = [logits[i:i + 1].clone()]
        live = [r for r in batch]
        begun = False          # whether the runner's live set is this batch's
        changed = True
        while True:
            done = [i for i, r in enumerate(live) if fed[r] == len(requests[r])]
            if done:
                for i in done:
                    cache.free(slots.pop(live[i]))
                stay = [r for i, r in enumerate(live) if i not in done]
                if stay and drop and begun:
                    runner.drop(done, stay, [fed[r] for r in stay])      # the runner narrows its own live set
                else:
                    changed = True
                live = stay
            if not live:
                break
            feed = [requests[r][fed[r]] for r in live]
            if changed:
                runner.begin([slots[r] for r in live], feed, live, [fed[r] for r in live])
                changed, begun = False, True
            runner.step(feed)
            rows = runner.last_logits()
            assert rows.shape == (len(live), model.vocab_size) and rows.dtype == torch.float32
            for i, r in enumerate(live):
                got[r].append(rows[i:i + 1].clone())
                fed[r] += 1
        cache.check()
    return {r: torch.cat(rows) for r, rows in got.items()}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["A", "B", "C", "Cb", "D"])
def test_graph_replay_logits_of_unequal_batches_that_shrink_and_reuse_slots(case, dtype, tmp_root):
    """Seven requests in batches of three on a cache of three slots; in each batch the tails are unequal, so the
    batch narrows (widths 4, 2, 1 with padding rows) while it runs; the second and third batch run in the
    slots and pages the first gave back."""
    model, _, cfg = engine_model(case, dtype, tmp_root)
    lengths = [70, 9, 33, 130, 64, 65, 20]
    requests = plain.random_prompts(cfg, lengths, CASES[case][1] + 200)
    tails = {r: min(len(requests[r]) - 1, [3, 8, 5][r % 3]) for r in range(len(requests))}
    cache = model.make_cache(max_tokens=3 * 192, max_seqs=3)
    for drop in (False, True):
        got = replay_batches(model, cache, requests, [[0, 1, 2], [3, 4, 5], [6]], tails, drop=drop)
        assert cache.slots.held_count == 0
        for r, tokens in enumerate(requests):
            expected = plain_logits(case, tokens)[len(tokens) - tails[r] - 1:]
            assert_logits_close(got[r], expected, dtype, f"{case} request {r} through graph replay (drop={drop})")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case,count", [("B", 40), ("C", 64), ("Cb", 37)])
def test_graph_replay_logits_at_wide_batches(case, count, dtype, tmp_root):
    """37, 40 and 64 live sequences: the captured widths 48 and 64 (multiples of 16, with 11 and 8 padding rows
    or none), whose products go other ways than those of narrow batches; unequal lengths and tails, so the
    batch also passes through narrower widths while it empties."""
    model, _, cfg = engine_model(case, dtype, tmp_root)
    lengths = [2 + (7 * i) % 45 for i in range(count)]
    requests = plain.random_prompts(cfg, lengths, CASES[case][1] + 300)
    tails = {r: min(len(requests[r]) - 1, 1 + r % 4) for r in range(count)}
    cache = model.make_cache(max_tokens=count * 64, max_seqs=count)
    got = replay_batches(model, cache, requests, [list(range(count))], tails)
    runner = odi.api.decode_runner(model, cache)
    assert {key[0] for key in runner._graphs} >= {DecodeRunner_width(count)}
    for r, tokens in enumerate(requests):
        expected = plain_logits(case, tokens)[len(tokens) - tails[r] - 1:]
        assert_logits_close(got[r], expected, dtype, f"{case} request {r} of {count} through graph replay")


def DecodeRunner_width(n):
    from ondeviceinfer_b200.engine.decode import DecodeRunner
    return DecodeRunner._width_for(n)


@pytest.mark.parametrize("dtype", DTYPES)
def test_graph_replay_matches_the_step_path_row_by_row(dtype, tmp_root):
    """The same steps through the generic step function and through graph replay: 32-bit logits are the
    same bits (the same kernels on the same values; only the launch differs), bfloat16 logits as close as
    two runs of different kernel forms may be (the replayed width pads the batch, which may choose another
    token tile)."""
    model, _, cfg = engine_model("C", dtype, tmp_root)
    requests = plain.random_prompts(cfg, [100, 7, 64, 190, 31], 401)
    tails = {r: 6 for r in range(5)}
    cache = model.make_cache(max_tokens=5 * 256, max_seqs=5)
    replayed = replay_batches(model, cache, requests, [[0, 1, 2, 3, 4]], tails)
    slots = [cache.alloc() for _ in requests]
    stepped = [model.step(cache, slots, [r[:-6] for r in requests], "last")]
    for t in range(6):
        stepped.append(model.step(cache, slots, [[r[len(r) - 6 + t]] for r in requests], "last"))
    for slot in slots:
        cache.free(slot)
    for r in range(5):
        mine = torch.stack([rows[r] for rows in stepped])
        if dtype == "float32":
            assert torch.equal(mine, replayed[r]), r
        else:
            assert_logits_close(replayed[r], mine, dtype, f"request {r}: replay against stepping")


@pytest.mark.parametrize("V,K", [(389, 96), (1000, 4096), (40000, 256), (523, 84)])
def test_logits_keep_fp32_at_every_number_of_rows(V, K):
    """The head product returns fp32 from fp32 accumulators whether 1, 64, 65 or 300 rows are wanted (the kernel
    form changes with the count, the precision does not): a row's logits in a wide batch equal its logits in
    a narrow one far below bf16's spacing, and they are not bf16 numbers.  K = 84 is a width that the
    tensor-core kernels refuse."""
    import math

    from ondeviceinfer_b200.parts.linear import linear

    torch.manual_seed(3)
    x = torch.randn(300, K).bfloat16().cuda()
    w = (torch.randn(V, K) / math.sqrt(K)).bfloat16().cuda()
    exact = x.double().cpu() @ w.double().cpu().t()
    outs = {n: linear(x[:n], w, out_dtype=torch.float32) for n in (1, 64, 65, 255, 300)}
    for n, out in outs.items():
        assert out.dtype == torch.float32 and out.shape == (n, V)
        assert float((out.double().cpu() - exact[:n]).abs().max()) < 2e-5 * math.sqrt(K), n
        assert not torch.equal(out.bfloat16().float(), out), f"{n} rows: the logits were rounded to bf16 on the way"
    assert float((outs[65][:64] - outs[64]).abs().max()) < 1e-4
    assert float((outs[300][:64] - outs[64]).abs().max()) < 1e-4


# ----------------------------------------------------------------------------- a windowed model under graph replay
#
# Graph replay is only exercised by the Qwen3 plan's full attention otherwise.  This plan, defined here and made of
# the library's graph-safe parts only, has a windowed attention layer beside a full one: under replay its
# CUDA-core decode kernel runs with ring page tables, splits fixed from the graph's length bucket, padding rows
# on the pad slot, and captures in the middle of a batch.

WINDOW = 40
WINDOWED = {"architectures": ["WindowedForCausalLM"], "vocab_size": 173, "hidden_size": 64, "eps": 1e-5}


class WindowedConfig:
    def __init__(self, raw):
        self.raw = dict(raw)

    @classmethod
    def from_dict(cls, raw):
        return cls(raw)

    def to_dict(self):
        return dict(self.raw)

    def to_plan(self):
        from ondeviceinfer_b200.config import (AttentionSpec, EmbeddingSpec, GatedMLPSpec, HeadSpec, ModelPlan, OrderEntry,
                                               PreNormBlockSpec, RMSNormSpec, RotarySpec, names)
        H, V, eps = self.raw["hidden_size"], self.raw["vocab_size"], self.raw["eps"]

        def block(i, window, nq, nkv, d):
            attention = AttentionSpec(H, nq, nkv, d, RotarySpec(d, 3000.0), f"l{i}.attn.",
                                      names(q="q", k="k", v="v", o="o", q_norm="qn", k_norm="kn"),
                                      qk_norm_eps=eps, window=window)
            return PreNormBlockSpec(RMSNormSpec(H, eps, f"l{i}.n1"), attention, RMSNormSpec(H, eps, f"l{i}.n2"),
                                    GatedMLPSpec(H, 2 * H, "silu", f"l{i}.ff.", names(gate="g", up="u", down="d")))

        layers = (block(0, None, 4, 2, 16), block(1, WINDOW, 2, 1, 32))
        return ModelPlan(EmbeddingSpec(V, H, "emb"), layers, (OrderEntry(0), OrderEntry(1)), RMSNormSpec(H, eps, "nf"),
                         HeadSpec(V, H, None))


def windowed_plain_logits(w, ids):
    import math
    H, eps, T = WINDOWED["hidden_size"], WINDOWED["eps"], len(ids)
    h = w["emb"][torch.tensor(ids)]
    pos = torch.arange(T)
    for i, (window, nq, nkv, d) in enumerate(((None, 4, 2, 16), (WINDOW, 2, 1, 32))):
        p = f"l{i}.attn."
        x = plain.rms_norm(h, w[f"l{i}.n1"], eps)
        q = plain.rms_norm(plain.linear(x, w[p + "q"]).view(T, nq, d), w[p + "qn"], eps).transpose(0, 1)
        k = plain.rms_norm(plain.linear(x, w[p + "k"]).view(T, nkv, d), w[p + "kn"], eps).transpose(0, 1)
        v = plain.linear(x, w[p + "v"]).view(T, nkv, d).transpose(0, 1)
        cos, sin = plain.rope_tables(pos, d, 3000.0, torch.float32)
        q, k = plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin)
        g = nq // nkv
        scores = q @ k.repeat_interleave(g, 0).transpose(-1, -2) / math.sqrt(d)
        visible = pos[None, :] <= pos[:, None]
        if window:
            visible = visible & (pos[None, :] > pos[:, None] - window)
        o = torch.softmax(scores.masked_fill(~visible, float("-inf")), -1) @ v.repeat_interleave(g, 0)
        h = h + plain.linear(o.transpose(0, 1).reshape(T, -1), w[p + "o"])
        m = plain.rms_norm(h, w[f"l{i}.n2"], eps)
        h = h + plain.linear(torch.nn.functional.silu(plain.linear(m, w[f"l{i}.ff.g"])) * plain.linear(m, w[f"l{i}.ff.u"]),
                             w[f"l{i}.ff.d"])
    return plain.linear(plain.rms_norm(h, w["nf"], eps), w["emb"])


@pytest.mark.parametrize("dtype", DTYPES)
def test_graph_replay_of_a_windowed_layer_past_the_rings_wrap_and_across_a_bucket(dtype, tmp_path):
    from ondeviceinfer_b200 import load_resident_model, register_architecture, write_random_model
    from ondeviceinfer_b200.weights import SafetensorsSource

    register_architecture("WindowedForCausalLM", WindowedConfig)
    folder = write_random_model(tmp_path / "windowed", WINDOWED, seed=6)
    source = SafetensorsSource(folder)
    weights = {n: source.fetch(n).float() for n in source.stored()}
    model = load_resident_model(folder, dtype=dtype)
    assert model.decoder.graph_safe
    gen = torch.Generator().manual_seed(10)
    # request 1 decodes 240 .. 269 alone and first (the sequence passes 256 in the middle of the batch: another
    # graph is captured there), request 0 decodes positions 380 .. 419 (its ring of 6 pages wraps at 384),
    # request 2 is short and leaves the second batch early
    lengths, tails = [420, 270, 100], {0: 40, 1: 30, 2: 10}
    requests = [torch.randint(0, WINDOWED["vocab_size"], (n,), generator=gen).tolist() for n in lengths]
    cache = model.make_cache(max_tokens=2 * 448, max_seqs=2)
    windowed = next(g for g in cache.kv_groups if g.need.window == WINDOW)
    assert windowed.ring_pages == 6
    got = replay_batches(model, cache, requests, [[1], [0, 2]], tails)
    runner = odi.api.decode_runner(model, cache)
    assert {key[1] for key in runner._graphs} >= {256, 512}, "the batch of request 1 should have crossed a length bucket"
    for r, tokens in enumerate(requests):
        expected = windowed_plain_logits(weights, tokens)[len(tokens) - tails[r] - 1:]
        assert_logits_close(got[r], expected, dtype, f"windowed request {r} through graph replay")
    # and the same tokens from generate() with and without graphs
    prompts = [r[:-8] for r in requests[:2]]
    with_graphs = odi.generate(model, prompts, max_new_tokens=12, use_graphs=True)
    without = odi.generate(model, prompts, max_new_tokens=12, use_graphs=False)
    if dtype == "float32":
        assert with_graphs.generated_ids == without.generated_ids


@pytest.mark.parametrize("case", ["C", "Cb"])
def test_a_thousand_replayed_steps_are_the_step_paths_bit_for_bit(case, tmp_root):
    """Three sequences of 40, 300 and 1,000 tokens decode 1,200 given tokens each: the longest passes 1,024 and 2,048
    keys (other graphs take over), every sequence enters a new tile of keys every 64 steps (the host's list of key
    blocks is renewed) and the cut of the keys changes as they grow.  bf16 with heads of 128 (the TMA-fed decode
    attention).  The logits of every replayed step equal those of the generic step function bit for bit."""
    model, _, cfg = engine_model(case, "bfloat16", tmp_root)
    lengths, steps = [40, 300, 1000], 1200
    streams = plain.random_prompts(cfg, [n + steps for n in lengths], 77)
    room = -(-(max(lengths) + steps + 8) // 64) * 64

    def run(graphs):
        cache = model.make_cache(max_tokens=3 * room, max_seqs=3)
        slots = [cache.alloc() for _ in lengths]
        rows = [model.step(cache, slots, [s[:n] for s, n in zip(streams, lengths)], "last").clone()]
        runner = None
        if graphs:
            runner = odi.api.decode_runner(model, cache)
            runner.begin(slots, [s[n] for s, n in zip(streams, lengths)], [0, 1, 2], [1, 1, 1])
        for t in range(steps):
            feed = [s[n + t] for s, n in zip(streams, lengths)]
            if graphs:
                runner.step(feed)
                rows.append(runner.last_logits().clone())
            else:
                rows.append(model.step(cache, slots, [[f] for f in feed], "last").clone())
        cache.check()
        assert [cache.length(slot) for slot in slots] == [n + steps for n in lengths]
        return torch.stack(rows), (len(runner._graphs) if graphs else 0)

    replayed, graphs = run(True)
    stepped, _ = run(False)
    assert graphs >= 3                                   # up to 2,048 keys, up to 4,096, and the splits' bounds
    assert torch.isfinite(replayed).all()
    differing = (replayed != stepped).flatten(1).any(1).nonzero().flatten().tolist()
    assert not differing, f"steps whose logits differ: {differing[:10]}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_shorter_batch_after_a_longer_one_captures_its_graph_on_the_same_buffers(dtype, tmp_root):
    """Two sequences of about 1,500 keys, then, in the same slots and the same width, two of about 300: the second
    batch needs a graph for shorter sequences (several key blocks each, but fewer than the first batch's), which
    is captured while the buffers still hold the first batch's lengths.  The capture's own run must go by the
    lengths its list of key blocks was planned for (a kernel that finds longer sequences than its list covers
    reports it), and the logits must be those of the plain implementation."""
    model, _, cfg = engine_model("C", dtype, tmp_root)
    lengths = [1500, 1400, 300, 280]
    requests = plain.random_prompts(cfg, lengths, 321)
    tails = {r: 6 for r in range(4)}
    cache = model.make_cache(max_tokens=2 * 1536, max_seqs=2)
    got = replay_batches(model, cache, requests, [[0, 1], [2, 3]], tails)
    runner = odi.api.decode_runner(model, cache)
    assert {key[1] for key in runner._graphs} >= {512, 2048}
    for r, tokens in enumerate(requests):
        assert_logits_close(got[r], plain_logits("C", tokens)[len(tokens) - tails[r] - 1:], dtype, f"request {r}")
