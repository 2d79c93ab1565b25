"""The decode runner's bookkeeping without a GPU: which graph it replays, what it saves around a capture in
the middle of a batch, page tables, padding rows, dropped rows.

CUDA graphs, streams and the sampling kernel are replaced by stand-ins on the CPU: a "graph" replays by
running the captured step again, as a CUDA graph would, and remembers the bound on the key splits that it
was captured with.  The model is a toy whose next token is a known function of the token and the position,
and which checks the page table it is given against the cache."""

import math

import pytest
import torch

from ondeviceinfer_b200.cache import KVNeed, SequenceCache
from ondeviceinfer_b200.engine import decode as decode_module
from ondeviceinfer_b200.engine.decode import DecodeRunner

VOCAB, BLOCK_ROWS = 97, 8


class FakeGraph:
    def __init__(self):
        self.run, self.bound = None, None

    def replay(self):
        self.run()


class FakeCapture:
    current = None

    def __init__(self, graph):
        self.graph = graph

    def __enter__(self):
        FakeCapture.current = self.graph

    def __exit__(self, *exc):
        FakeCapture.current = None
        return False


class FakeStream:
    def __init__(self, device=None):
        pass

    def wait_stream(self, other):
        pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


class ToyModel:
    """logits whose argmax is (token + position) mod VOCAB; asks for the key-split plan as an attention part does
    and checks that the graph being replayed was captured with room for it."""

    graph_safe = True

    def __init__(self, cache):
        self.device = torch.device("cpu")
        self.cache = cache
        self.seen = []

    def forward(self, ctx, cache):
        per_tensor, bound = ctx.key_splits(BLOCK_ROWS)
        graph = FakeCapture.current
        if graph is not None:            # being captured: the bound becomes a constant of this graph
            graph.bound = bound
        for row in range(ctx.width):
            if int(ctx.active[row]) == 0:
                continue
            slot, pos = int(ctx.slots[row]), int(ctx.tok_pos[row])
            if slot == cache.pad_slot:   # the runs of a capture: every row on the pad slot, results dropped
                continue
            assert pos == int(ctx.past[row]) == cache.lengths[slot] + self.offset, (row, pos)
            # the list of key blocks is the one for this step: the row's blocks cover its keys, the last one marked
            per, count = int(per_tensor[0]), int(per_tensor[1])
            mine = sorted(e & 255 for e in per_tensor[2:2 + count].tolist() if e >> 8 == row)
            needed = -(-(pos // 64 + 1) // per)
            assert mine == list(range(needed - 1)) + [128 | (needed - 1)] and needed <= bound, (row, pos, mine)
            for g, group in enumerate(cache.kv_groups):
                start, ids = ctx.page_table(g)
                pages = ids[int(start[row]):int(start[row]) + pos // 64 + 1].tolist()
                assert pages == group.slot_pages[slot][:pos // 64 + 1], "the page table lags behind the cache"
        wanted = (ctx.token_ids.long() + ctx.tok_pos.long()) % VOCAB
        logits = torch.zeros(ctx.width, VOCAB)
        logits[torch.arange(ctx.width), wanted] = 1.0
        return logits

    offset = 0          # steps replayed since the cache's lengths were last advanced


def fake_sample(logits, out, temperature, seed, streams, steps, *, advance_pos, advance_past, active):
    out[:logits.shape[0]] = logits.argmax(-1).to(torch.int32)
    advance_pos += active
    advance_past += active
    steps += active


@pytest.fixture
def cpu_graphs(monkeypatch):
    monkeypatch.setattr(torch.cuda, "CUDAGraph", FakeGraph)
    monkeypatch.setattr(torch.cuda, "graph", FakeCapture)
    monkeypatch.setattr(torch.cuda, "Stream", FakeStream)
    monkeypatch.setattr(torch.cuda, "stream", lambda s: s)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda device=None: FakeStream())
    monkeypatch.setattr(torch.cuda, "synchronize", lambda device=None: None)
    monkeypatch.setattr(decode_module.ops, "sample", fake_sample)
    original = DecodeRunner._capture

    def capture(self, ctx, bucket):
        graph, launches, logits = original(self, ctx, bucket)

        def run():
            logits.copy_(self._run_once(ctx))      # a replay leaves the step's logits where the capture saw them

        graph.run = run
        return graph, launches, logits

    monkeypatch.setattr(DecodeRunner, "_capture", capture)


def prefilled(cache, lengths):
    slots = [cache.alloc() for _ in lengths]
    cache.reserve(slots, lengths)
    cache.advance(slots, lengths)
    return slots


def test_runner_follows_the_sequences_through_graphs_captures_and_dropped_rows(cpu_graphs):
    cache = SequenceCache([(KVNeed(2, 16),)] * 2, [None, None], dtype=torch.float32, device="cpu",
                          max_tokens=4 * 640, max_seqs=4)
    model = ToyModel(cache)
    lengths = [250, 17, 100]
    slots = prefilled(cache, lengths)
    runner = DecodeRunner(model, cache)
    tokens = [5, 6, 7]
    runner.begin(slots, tokens, [0, 1, 2], [1, 1, 1])
    assert runner.ctx.width == 4 and int(runner.ctx.active.sum()) == 3
    first_keys = set(runner._graphs)
    assert first_keys == {(4, 256, (decode_module._power_of_two(2),))}        # 4 tiles of the longest, 2 a block

    def expect(tokens, lengths):
        return [(t + n) % VOCAB for t, n in zip(tokens, lengths)]

    for step in range(12):                  # the longest sequence passes 256 keys at the seventh step
        runner.step_device(1)
        tokens, lengths = expect(tokens, lengths), [n + 1 for n in lengths]
        assert runner.ctx.token_ids[:3].tolist() == tokens, step
        assert [cache.lengths[s] for s in slots] == lengths
        # the logits of the replayed step stay readable: the token each live row chose is their argmax
        assert runner.last_logits().shape == (3, VOCAB) and runner.last_logits().argmax(-1).tolist() == tokens
        graph, _, _ = runner._graph_for(4, [n + 1 for n in lengths])
        per = runner.ctx._key_splits[BLOCK_ROWS][1][0]
        assert math.ceil(max(-(-(n + 1) // 64) for n in lengths) / per) <= graph.bound
    assert any(key[1] == 512 for key in runner._graphs) and first_keys < set(runner._graphs)
    assert int(runner.ctx.active.sum()) == 3 and runner.ctx.slot_list[3] == cache.pad_slot   # restored after the capture

    # several steps in one call: the host plans each of them ahead of the cache's lengths
    steps_before = [int(v) for v in runner.ctx.steps[:3]]
    original_forward = model.forward

    def forward(ctx, cache_):
        model.offset = forward.calls
        forward.calls += 1
        return original_forward(ctx, cache_)

    forward.calls = 0
    model.forward = forward
    runner.step_device(5)
    for _ in range(5):
        tokens, lengths = expect(tokens, lengths), [n + 1 for n in lengths]
    assert runner.ctx.token_ids[:3].tolist() == tokens
    assert [int(v) for v in runner.ctx.steps[:3]] == [s + 5 for s in steps_before]
    model.forward, model.offset = original_forward, 0

    # the middle sequence ends: the others go on in a narrower batch with their tokens, positions and pages
    cache.free(slots[1])
    runner.drop([1], [0, 2], [int(runner.ctx.steps[0]), int(runner.ctx.steps[2])])
    slots, tokens, lengths = [slots[0], slots[2]], [tokens[0], tokens[2]], [lengths[0], lengths[2]]
    assert runner.ctx.width == 2 and runner.live_slots == slots
    for step in range(4):
        runner.step_device(1)
        tokens, lengths = expect(tokens, lengths), [n + 1 for n in lengths]
        assert runner.ctx.token_ids[:2].tolist() == tokens
    cache.check()

    # a graph made for twice the splits serves; no capture when a shorter batch follows on the same cache
    for slot in slots:
        cache.free(slot)
    graphs_before = len(runner._graphs)
    slots = prefilled(cache, [300, 280])
    runner.begin(slots, [1, 2], [0, 1], [1, 1])
    assert len(runner._graphs) == graphs_before
    runner.step_device(1)
    assert runner.ctx.token_ids[:2].tolist() == [(1 + 300) % VOCAB, (2 + 280) % VOCAB]
