"""The engine against the plain implementation, in 32-bit and in bfloat16, under every
way of cutting and batching the same requests."""

import pytest
import torch

import plain_qwen3 as plain
from helpers import CASES, assert_logits_close, engine_model, plain_logits

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
# request lengths: one token, a page minus / exactly / plus one, several pages, odd sizes
LENGTHS = {"A": [5, 11, 17, 64, 33, 100], "B": [1, 7, 30, 64, 65, 130, 63, 2], "C": [3, 200, 77, 129, 64, 31]}
LENGTHS.update({"Ab": LENGTHS["A"], "Bb": LENGTHS["B"], "Cb": LENGTHS["C"]})      # the same with projection biases
LENGTHS["D"] = [2, 40, 65, 9, 128, 33]
ALL_CASES = ["A", "B", "C", "Ab", "Bb", "Cb", "D"]


@pytest.fixture(scope="session")
def tmp_root(tmp_path_factory):
    return tmp_path_factory.mktemp("models")


def requests_of(case):
    cfg, seed = CASES[case]
    return plain.random_prompts(cfg, LENGTHS[case], seed + 100)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ALL_CASES)
def test_each_request_alone_and_whole(case, dtype, tmp_root):
    model, _, _ = engine_model(case, dtype, tmp_root)
    cache = model.make_cache(max_tokens=256, max_seqs=1)
    for r, tokens in enumerate(requests_of(case)):
        slot = cache.alloc()
        logits = model.step(cache, [slot], [tokens], "all")
        assert logits.dtype == torch.float32 and logits.shape == (len(tokens), model.vocab_size)
        assert_logits_close(logits, plain_logits(case, tokens), dtype, f"{case} request {r} whole")
        assert cache.length(slot) == len(tokens)
        cache.free(slot)
    cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ALL_CASES)
def test_last_32_tokens_one_by_one(case, dtype, tmp_root):
    model, _, _ = engine_model(case, dtype, tmp_root)
    cache = model.make_cache(max_tokens=256, max_seqs=1)
    for r, tokens in enumerate(requests_of(case)):
        expected = plain_logits(case, tokens)
        cut = max(1, len(tokens) - 32)
        slot = cache.alloc()
        rows = [model.step(cache, [slot], [tokens[:cut]], "all")]
        for t in range(cut, len(tokens)):
            rows.append(model.step(cache, [slot], [[tokens[t]]], "last"))
        assert_logits_close(torch.cat(rows), expected, dtype, f"{case} request {r} tail one by one")
        cache.free(slot)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ALL_CASES)
def test_batches_of_unequal_lengths_reuse_slots(case, dtype, tmp_root):
    """Batches of three requests on a cache with three slots, one batch after another: the
    prompts (all but the last d_i tokens, d_i unequal) in one step, then one token per live
    request per step; shorter requests end earlier and give their slot back at once."""
    model, _, _ = engine_model(case, dtype, tmp_root)
    requests = requests_of(case)
    cache = model.make_cache(max_tokens=3 * 256, max_seqs=3)
    got = {r: [] for r in range(len(requests))}
    seen_slots = []
    for first in range(0, len(requests), 3):
        batch = list(range(first, min(first + 3, len(requests))))
        tails = {r: min(len(requests[r]) - 1, 3 + 7 * (r % 3)) for r in batch}
        slots = {r: cache.alloc() for r in batch}
        seen_slots.append(sorted(slots.values()))
        prompts = [requests[r][:len(requests[r]) - tails[r]] for r in batch]
        logits = model.step(cache, [slots[r] for r in batch], prompts, "all")
        offset = 0
        for r, p in zip(batch, prompts):
            got[r].append(logits[offset:offset + len(p)])
            offset += len(p)
        fed = {r: len(p) for r, p in zip(batch, prompts)}
        live = list(batch)
        while True:
            for r in [r for r in live if fed[r] == len(requests[r])]:
                cache.free(slots.pop(r))
                live.remove(r)
            if not live:
                break
            logits = model.step(cache, [slots[r] for r in live], [[requests[r][fed[r]]] for r in live], "last")
            for i, r in enumerate(live):
                got[r].append(logits[i:i + 1])
                fed[r] += 1
        cache.check()
    assert seen_slots[0] == seen_slots[1], "the second batch must run in the slots of the first"
    for r, tokens in enumerate(requests):
        assert_logits_close(torch.cat(got[r]), plain_logits(case, tokens), dtype, f"{case} request {r} batched")


@pytest.mark.parametrize("dtype", DTYPES)
def test_what_else_is_in_the_batch_changes_nothing(dtype, tmp_root):
    """The same request alone, first of a batch, last of a batch, and in another slot:
    bit-equal in 32-bit (each row's arithmetic does not depend on the batch)."""
    model, _, _ = engine_model("B", dtype, tmp_root)
    requests = requests_of("B")
    target = requests[5]
    cache = model.make_cache(max_tokens=1024, max_seqs=4)

    def run(batch, which):
        slots = [cache.alloc() for _ in batch]
        logits = model.step(cache, slots, batch, "all")
        start = sum(len(b) for b in batch[:which])
        out = logits[start:start + len(batch[which])].clone()
        for s in slots:
            cache.free(s)
        return out

    alone = run([target], 0)
    first = run([target, requests[3], requests[0]], 0)
    last = run([requests[4], requests[6], requests[1], target], 3)
    if dtype == "float32":
        assert torch.equal(alone, first) and torch.equal(alone, last)
    else:
        expected = plain_logits("B", target)
        assert_logits_close(first, expected, dtype, "first of a batch")
        assert_logits_close(last, expected, dtype, "last of a batch")
        assert_logits_close(first, alone, dtype, "batch against alone")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_across_pages(dtype, tmp_root):
    """A 40-token prompt, then 300 tokens one by one: positions cross pages 64, 128, 192,
    256, 320 and the decode kernels split their key range."""
    model, _, cfg = engine_model("C", dtype, tmp_root)
    tokens = plain.random_prompts(cfg, [340], 77)[0]
    expected = plain_logits("C", tokens)
    cache = model.make_cache(max_tokens=384, max_seqs=1)
    slot = cache.alloc()
    rows = [model.step(cache, [slot], [tokens[:40]], "all")]
    for t in range(40, len(tokens)):
        rows.append(model.step(cache, [slot], [[tokens[t]]], "last"))
    assert_logits_close(torch.cat(rows), expected, dtype, "long decoding")
    assert cache.length(slot) == 340 and cache.tokens_held == 384
    cache.free(slot)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["A", "B"])
def test_first_tokens_of_a_sequence(case, dtype, tmp_root):
    """A sequence fed one token at a time from its very first token: positions 0, 1, 2, ..."""
    model, _, cfg = engine_model(case, dtype, tmp_root)
    tokens = plain.random_prompts(cfg, [6], 5)[0]
    expected = plain_logits(case, tokens)
    cache = model.make_cache(max_tokens=64, max_seqs=1)
    slot = cache.alloc()
    rows = [model.step(cache, [slot], [[t]], "last") for t in tokens]
    assert_logits_close(torch.cat(rows), expected, dtype, "first tokens")
    cache.free(slot)


@pytest.mark.parametrize("dtype", DTYPES)
def test_chunks_of_a_few_tokens_and_chosen_places(dtype, tmp_root):
    """Steps of several tokens on top of a cache (neither prompt nor single token), with
    logits wanted at chosen places only, in a batch whose members bring unequal chunks."""
    model, _, _ = engine_model("B", dtype, tmp_root)
    requests = requests_of("B")
    a, b = requests[5], requests[2]          # 130 and 30 tokens
    cache = model.make_cache(max_tokens=512, max_seqs=2)
    sa, sb = cache.alloc(), cache.alloc()
    none = model.step(cache, [sa, sb], [a[:50], b[:10]], "none")
    assert none.shape == (0, model.vocab_size)
    logits = model.step(cache, [sa, sb], [a[50:90], b[10:13]], [[0, 39], [1]])
    ea, eb = plain_logits("B", a), plain_logits("B", b)
    assert_logits_close(logits, torch.stack([ea[50], ea[89], eb[11]]), dtype, "chunk on a cache")
    logits = model.step(cache, [sb, sa], [b[13:], a[90:]], "last")
    assert_logits_close(logits, torch.stack([eb[-1], ea[-1]]), dtype, "swapped order")
    cache.free(sa)
    cache.free(sb)


def test_a_tied_head_shares_the_embedding_table(tmp_root):
    """Model A ties its head to the embedding: the two parts bind the same tensor (the loader hands out one tensor per
    name), so the table is on the device once; model B has a head of its own."""
    tied, _, _ = engine_model("A", "bfloat16", tmp_root)
    assert tied.decoder.head.weight.data_ptr() == tied.decoder.embedding.table.data_ptr()
    assert tied.decoder.head.tensor_decls() == []
    own, _, _ = engine_model("B", "bfloat16", tmp_root)
    assert own.decoder.head.weight.data_ptr() != own.decoder.embedding.table.data_ptr()
    assert [d.name for d in own.decoder.head.tensor_decls()] == ["lm_head.weight"]


def test_capacity_and_misuse_are_host_errors(tmp_root):
    from ondeviceinfer_b200 import CacheCapacityError

    model, _, _ = engine_model("A", "float32", tmp_root)
    cache = model.make_cache(max_tokens=128, max_seqs=2)
    slot = cache.alloc()
    with pytest.raises(CacheCapacityError):
        model.step(cache, [slot], [[1] * 129], "last")
    assert cache.length(slot) == 0
    with pytest.raises(ValueError):
        model.step(cache, [slot], [[256]], "last")           # token id outside the vocabulary
    with pytest.raises(ValueError):
        model.step(cache, [slot + 1], [[1]], "last")         # slot not held
    model.step(cache, [slot], [[1] * 128], "none")
    with pytest.raises(CacheCapacityError):
        model.step(cache, [slot], [[1]], "last")
    cache.free(slot)
    cache.check()


LARGE = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 1, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 40960, "hidden_act": "silu",
}


# two layers with the sizes of Qwen3-14B (width 5120, 40 query heads): seven K splits, a fused norm at the
# start of a layer as well as in its middle, a tied head over a small vocabulary
LARGE_TWO = dict(LARGE, num_hidden_layers=2, hidden_size=5120, num_attention_heads=40, intermediate_size=17408,
                 vocab_size=30000, tie_word_embeddings=True)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", ["8B", "14B"])
def test_qwen3_8b_layer_sizes(sizes, dtype, tmp_path):
    """One layer with the sizes of Qwen3-8B (width 4096, 32 query and 8 key/value heads of 128,
    feed-forward 12288, vocabulary 151936), and two with those of Qwen3-14B: whole, the last tokens one
    by one, and an unequal batch, against the plain implementation.  Logits of wide sums are compared
    at the wanted places."""
    import ondeviceinfer_b200 as odi
    from helpers import write_model_folder

    LARGE = {"8B": globals()["LARGE"], "14B": LARGE_TWO}[sizes]
    weights = plain.random_weights(LARGE, 3)
    model = odi.load_resident_model(write_model_folder(tmp_path / "large", LARGE, weights), dtype=dtype)
    requests = plain.random_prompts(LARGE, [70, 9, 33], 3)
    expected = [plain.forward_logits(weights, LARGE, r) for r in requests]
    cache = model.make_cache(max_tokens=3 * 128, max_seqs=3)
    # whole, alone
    slot = cache.alloc()
    assert_logits_close(model.step(cache, [slot], [requests[0]], "all"), expected[0], dtype, "8B sizes whole", longest_sum=LARGE["intermediate_size"])
    cache.free(slot)
    # unequal batch: prompts without their last 4 tokens, then one token each
    slots = [cache.alloc() for _ in requests]
    cut = [len(r) - 4 for r in requests]
    logits = model.step(cache, slots, [r[:c] for r, c in zip(requests, cut)], "last")
    assert_logits_close(logits, torch.stack([e[c - 1] for e, c in zip(expected, cut)]), dtype, "8B sizes batch prompt", longest_sum=LARGE["intermediate_size"])
    for t in range(4):
        logits = model.step(cache, slots, [[r[c + t]] for r, c in zip(requests, cut)], "last")
        assert_logits_close(logits, torch.stack([e[c + t] for e, c in zip(expected, cut)]), dtype, f"8B sizes decode {t}", longest_sum=LARGE["intermediate_size"])
    for slot in slots:
        cache.free(slot)
    cache.check()
    if sizes == "8B":
        # 40 sequences of one or two tokens: the logits of 40 rows over the whole vocabulary in one product
        many = plain.random_prompts(LARGE, [1 + i % 2 for i in range(40)], 4)
        wide = model.make_cache(max_tokens=40 * 64, max_seqs=40)
        slots = [wide.alloc() for _ in many]
        logits = model.step(wide, slots, many, "last")
        follow = plain.random_prompts(LARGE, [1] * 40, 5)              # one more token each, fed through graph replay
        whole = [plain.forward_logits(weights, LARGE, r + f) for r, f in zip(many, follow)]
        expected = torch.stack([w[len(r) - 1] for w, r in zip(whole, many)])
        assert_logits_close(logits, expected, dtype, "8B sizes, 40 sequences", longest_sum=LARGE["intermediate_size"])
        # the same 40 rows one step on through the decode path of generate(): a captured graph of width 48
        runner = odi.api.decode_runner(model, wide)
        feed = [f[0] for f in follow]
        runner.begin(slots, feed, list(range(40)), [1] * 40)
        runner.step(feed)
        assert runner.ctx.width == 48
        assert_logits_close(runner.last_logits(), torch.stack([w[-1] for w in whole]), dtype,
                            "8B sizes, 40 sequences, graph replay", longest_sum=LARGE["intermediate_size"])
        for slot in slots:
            wide.free(slot)
        wide.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_context(dtype, tmp_root):
    """1,100 tokens (18 pages): whole in one step, then in two chunks with 40 single tokens at the
    end; prefill tiles, page rings and decode splits all wrap several times."""
    model, _, cfg = engine_model("C", dtype, tmp_root)
    tokens = plain.random_prompts(cfg, [1100], 91)[0]
    expected = plain_logits("C", tokens)
    cache = model.make_cache(max_tokens=1152, max_seqs=1)
    slot = cache.alloc()
    whole = model.step(cache, [slot], [tokens], "all")
    assert_logits_close(whole, expected, dtype, "long context whole")
    cache.free(slot)
    slot = cache.alloc()
    rows = [model.step(cache, [slot], [tokens[:700]], [[0, 350, 699]]),
            model.step(cache, [slot], [tokens[700:1060]], [[0, 359]])]
    picks = [0, 350, 699, 700, 1059]
    for t in range(1060, 1100):
        rows.append(model.step(cache, [slot], [[tokens[t]]], "last"))
        picks.append(t)
    assert_logits_close(torch.cat(rows), expected[picks], dtype, "long context in chunks")
    cache.free(slot)


# heads of 128 at a small width: a prompt of 2,100 tokens goes through the many-token kernels (every
# projection, with the head preparation, the SiLU gate and the residual adds in their epilogues)
WIDE_HEADS = dict(LARGE, num_hidden_layers=2, hidden_size=1024, num_attention_heads=8, num_key_value_heads=2,
                  intermediate_size=2048, vocab_size=1000, tie_word_embeddings=True)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_prompt_through_the_many_token_kernels(dtype, tmp_path):
    import ondeviceinfer_b200 as odi
    from helpers import write_model_folder

    weights = plain.random_weights(WIDE_HEADS, 5)
    model = odi.load_resident_model(write_model_folder(tmp_path / "wide", WIDE_HEADS, weights), dtype=dtype)
    tokens = plain.random_prompts(WIDE_HEADS, [2100], 6)[0]
    expected = plain.forward_logits(weights, WIDE_HEADS, tokens)
    cache = model.make_cache(max_tokens=2176, max_seqs=1)
    slot = cache.alloc()
    picks = [0, 127, 128, 1023, 1024, 2047, 2048, 2089]
    whole = model.step(cache, [slot], [tokens[:2090]], [picks])
    rows = [whole] + [model.step(cache, [slot], [[t]], "last") for t in tokens[2090:]]
    assert_logits_close(torch.cat(rows), expected[picks + list(range(2090, 2100))], dtype, "long prompt", longest_sum=2048)
    cache.free(slot)
    cache.check()


# One layer with the sizes of Qwen3-8B (a small vocabulary keeps the plain implementation affordable) and a
# prompt of 2,100 tokens: every projection goes through the many-token tensor-core kernel at the shapes the
# prefill benchmark stands on (q/k/v 6,144 x 4,096 with the head preparation, output projection, gate/up
# 2 x 12,288 x 4,096 with the SiLU gate, down 4,096 x 12,288 with the reduce-add), attention through the
# tcgen05 kernel at 32 query and 8 key/value heads.
LARGE_PREFILL = dict(LARGE, vocab_size=1000)
_LARGE_PREFILL_EXPECTED = {}


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_prompt_at_qwen3_8b_layer_sizes(dtype, tmp_path):
    import ondeviceinfer_b200 as odi
    from helpers import write_model_folder
    from ondeviceinfer_b200.kernels import ops

    weights = plain.random_weights(LARGE_PREFILL, 8)
    tokens = plain.random_prompts(LARGE_PREFILL, [2100], 9)[0]
    if "logits" not in _LARGE_PREFILL_EXPECTED:
        _LARGE_PREFILL_EXPECTED["logits"] = plain.forward_logits(weights, LARGE_PREFILL, tokens)
    expected = _LARGE_PREFILL_EXPECTED["logits"]
    model = odi.load_resident_model(write_model_folder(tmp_path / "large_prefill", LARGE_PREFILL, weights), dtype=dtype)
    cache = model.make_cache(max_tokens=2112, max_seqs=1)
    slot = cache.alloc()
    picks = [0, 63, 64, 255, 256, 1000, 2047, 2048, 2095]
    before = dict(ops.LAUNCHES)
    whole = model.step(cache, [slot], [tokens[:2096]], [picks])
    if dtype == "bfloat16":
        assert ops.LAUNCHES["library"] == before["library"], "a projection of the long prompt went to the vendor library"
    rows = [whole] + [model.step(cache, [slot], [[t]], "last") for t in tokens[2096:]]
    torch.cuda.synchronize()
    ops.raise_on_kernel_fault()
    assert_logits_close(torch.cat(rows), expected[picks + list(range(2096, 2100))], dtype, "2,100 tokens at 8B layer sizes",
                        longest_sum=LARGE_PREFILL["intermediate_size"])
    cache.free(slot)
    cache.check()
    # An unequal batch at these sizes: five sequences that are the same tokens cut at different places (so one plain
    # pass gives every expected row), decoded for four steps through graph replay and through the step function:
    # 8 key/value heads with 33, 24, 11, 2 and 1 tiles of keys, cut into blocks by the host's list.
    cuts = [2090, 1500, 700, 65, 3]
    wide = model.make_cache(max_tokens=len(cuts) * 2112, max_seqs=len(cuts))

    def decode(graphs):
        slots = [wide.alloc() for _ in cuts]
        rows = [model.step(wide, slots, [tokens[:c] for c in cuts], "last")]
        runner = odi.api.decode_runner(model, wide) if graphs else None
        if graphs:
            runner.begin(slots, [tokens[c] for c in cuts], list(range(len(cuts))), [1] * len(cuts))
        for t in range(4):
            feed = [tokens[c + t] for c in cuts]
            if graphs:
                runner.step(feed)
                rows.append(runner.last_logits().clone())
            else:
                rows.append(model.step(wide, slots, [[f] for f in feed], "last"))
        for slot in slots:
            wide.free(slot)
        wide.check()
        return torch.cat(rows)

    replayed, stepped = decode(True), decode(False)
    places = [c - 1 + t for t in range(5) for c in cuts]
    assert_logits_close(replayed, expected[places], dtype, "unequal batch at 8B layer sizes, graph replay",
                        longest_sum=LARGE_PREFILL["intermediate_size"])
    assert_logits_close(stepped, expected[places], dtype, "unequal batch at 8B layer sizes, step function",
                        longest_sum=LARGE_PREFILL["intermediate_size"])
    # (the two need not agree bit for bit: the replayed graph is eight rows wide, and its three padding rows
    # change how the host cuts the keys into blocks, so the splits' partial sums are grouped differently)
    assert_logits_close(replayed, stepped, dtype, "graph replay against the step function at 8B layer sizes",
                        longest_sum=LARGE_PREFILL["intermediate_size"])


def test_decode_with_the_splits_merged_in_the_output_projection(monkeypatch, tmp_root):
    """The optional form in which a decode attention leaves its key splits unmerged and the output projection
    merges them in its prologue: the same logits, bit for bit, as with the combine kernel, on sequences long
    enough for several splits (and one short one that uses a single split of the bound)."""
    import importlib
    linear_module = importlib.import_module("ondeviceinfer_b200.parts.linear")
    from ondeviceinfer_b200.kernels import ops
    model, weights, cfg = engine_model("Cb", "bfloat16", tmp_root)
    prompts = plain.random_prompts(cfg, [700, 300, 70], 21)

    def run(merge_in_product):
        monkeypatch.setattr(linear_module, "MERGE_IN_PRODUCT", merge_in_product)
        merged_calls = []
        real = ops.gemm_bf16

        def counting(*args, **kwargs):
            merged_calls.append(kwargs.get("merge") is not None)
            return real(*args, **kwargs)

        monkeypatch.setattr(ops, "gemm_bf16", counting)
        cache = model.make_cache(max_tokens=3 * 768, max_seqs=3)
        slots = [cache.alloc() for _ in prompts]
        rows = [model.step(cache, slots, prompts, "last")]
        for t in range(3):
            rows.append(model.step(cache, slots, [[5 + t], [9 + t], [11 + t]], "last"))
        monkeypatch.setattr(ops, "gemm_bf16", real)
        for slot in slots:
            cache.free(slot)
        return torch.cat(rows), sum(merged_calls)

    plain_way, none = run(False)
    fused_way, some = run(True)
    assert none == 0 and some == 3 * cfg["num_hidden_layers"]
    assert torch.equal(fused_way, plain_way)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_step_longer_than_the_token_limit_runs_in_passes(dtype, monkeypatch, tmp_root):
    """With the limit at 128 tokens a pass, prompts of 300, 70 and 129 tokens run as five passes of up to 64
    tokens per sequence over the same cache: the logits at every place are those of the plain implementation,
    and those of the step in one pass within rounding; decoding goes on from the cache they left."""
    import importlib
    step_module = importlib.import_module("ondeviceinfer_b200.engine.step")
    model, weights, cfg = engine_model("B", dtype, tmp_root)
    prompts = plain.random_prompts(cfg, [300, 70, 129], 33)
    passes = []
    real = step_module._run_chunk

    def counting(model_, cache_, slots_, tokens_, places_):
        passes.append([len(t) for t in tokens_])
        return real(model_, cache_, slots_, tokens_, places_)

    monkeypatch.setattr(step_module, "_run_chunk", counting)

    def run(limit):
        monkeypatch.setattr(step_module, "STEP_TOKEN_LIMIT", limit)
        del passes[:]
        cache = model.make_cache(max_tokens=3 * 384, max_seqs=3)
        slots = [cache.alloc() for _ in prompts]
        logits = model.step(cache, slots, prompts, "all")
        shape = list(passes)
        more = model.step(cache, slots, [[7], [8], [9]], "last")
        return logits, more, shape

    whole, whole_next, one = run(32768)
    cut, cut_next, five = run(128)
    assert one == [[300, 70, 129]]
    assert five == [[64, 64, 64], [64, 6, 64], [64, 1], [64], [44]]
    offset = 0
    for r, prompt in enumerate(prompts):
        expected = plain_logits("B", prompt, dtype)
        assert_logits_close(cut[offset:offset + len(prompt)], expected, dtype, f"request {r} in passes")
        offset += len(prompt)
    if dtype == "float32":
        assert float((cut - whole).abs().max()) < 2e-4 and float((cut_next - whole_next).abs().max()) < 2e-4
    for r, (prompt, token) in enumerate(zip(prompts, (7, 8, 9))):
        assert_logits_close(cut_next[r:r + 1], plain_logits("B", prompt + [token], dtype)[-1:], dtype, f"request {r} next")


def _drawn_config(rng):
    nkv, group = rng.choice([1, 2, 3, 5]), rng.choice([1, 2, 3, 4, 7])
    return {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
            "num_hidden_layers": rng.choice([1, 2, 3]), "hidden_size": rng.choice([36, 50, 72, 100, 104, 136, 250]),
            "num_attention_heads": nkv * group, "num_key_value_heads": nkv,
            "head_dim": rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 144, 192, 256]),
            "intermediate_size": rng.choice([33, 64, 135, 136, 200, 264]), "vocab_size": rng.choice([50, 301, 1000, 2049]),
            "rope_theta": rng.choice([10000.0, 1000000.0, 50000.0]), "rms_norm_eps": rng.choice([1e-6, 1e-5, 3e-6]),
            "tie_word_embeddings": rng.random() < 0.5, "max_position_embeddings": 4096, "hidden_act": "silu",
            "attention_bias": rng.random() < 0.4}


@pytest.mark.parametrize("draw", [3, 12, 27, 41])
def test_drawn_configurations(draw, tmp_path):
    """Configurations drawn at random from sizes that are no powers of two (widths and feed-forward sizes that are
    no multiples of 8, odd vocabularies, 1 to 35 query heads in groups of 1 to 7, head sizes from 16 to 256), with and
    without biases and a tied head: a whole prompt, an unequal batch of four, and its tails one token at a time
    through the step function and through graph replay, in both precisions, against the plain implementation."""
    import random

    import ondeviceinfer_b200 as odi
    from helpers import write_model_folder
    from ondeviceinfer_b200.kernels import ops

    rng = random.Random(draw)
    cfg = _drawn_config(rng)
    weights = plain.random_weights(cfg, draw)
    folder = write_model_folder(tmp_path / "drawn", cfg, weights)
    lengths = [rng.choice([1, 5, 33, 64, 65, 100, 130, 257, 700]) for _ in range(4)]
    requests = plain.random_prompts(cfg, lengths, draw + 1)
    expected = [plain.forward_logits(weights, cfg, r) for r in requests]
    room = -(-max(lengths) // 64) * 64 + 64
    for dtype in DTYPES:
        model = odi.load_resident_model(folder, device="cuda:0", dtype=dtype)
        cache = model.make_cache(max_tokens=4 * room, max_seqs=4)
        slot = cache.alloc()
        assert_logits_close(model.step(cache, [slot], [requests[3]], "all"), expected[3], dtype, f"{cfg} whole")
        cache.free(slot)
        for graphs in (False, True):
            slots = [cache.alloc() for _ in requests]
            cut = [max(1, len(r) - 1 - 3 * (i % 3)) for i, r in enumerate(requests)]
            logits = model.step(cache, slots, [r[:c] for r, c in zip(requests, cut)], "last")
            assert_logits_close(logits, torch.stack([e[c - 1] for e, c in zip(expected, cut)]), dtype, f"{cfg} prompts")
            live, fed, changed = list(range(4)), list(cut), True
            runner = odi.api.decode_runner(model, cache) if graphs else None
            while True:
                done = [i for i in live if fed[i] == len(requests[i])]
                for i in done:
                    cache.free(slots[i])
                changed = changed or bool(done)
                live = [i for i in live if i not in done]
                if not live:
                    break
                feed = [requests[i][fed[i]] for i in live]
                if graphs:
                    if changed:
                        runner.begin([slots[i] for i in live], feed, live, [fed[i] for i in live])
                        changed = False
                    runner.step(feed)
                    rows = runner.last_logits()
                else:
                    rows = model.step(cache, [slots[i] for i in live], [[f] for f in feed], "last")
                assert_logits_close(rows, torch.stack([expected[i][fed[i]] for i in live]), dtype,
                                    f"{cfg} one token each, graphs={graphs}")
                for i in live:
                    fed[i] += 1
            cache.check()
        torch.cuda.synchronize()
        ops.raise_on_kernel_fault()
