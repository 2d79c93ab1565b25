"""The generation loop's decisions, driven by a scripted model (no GPU)."""

import pytest

from ondeviceinfer_b200.engine.generate import generate_requests, plan_batches


class Script:
    """A stand-in for model and cache.  The "logits" of a run are its request's script
    position; sampling reads the scripted token.  Records every call."""

    def __init__(self, scripts, n_slots=8):
        self.scripts = scripts          # request -> tokens it will produce
        self.free_slots = list(range(n_slots))
        self.held = {}
        self.steps = []                 # (slots, runs)
        self.freed = []

    def alloc(self):
        slot = self.free_slots.pop(0)
        self.held[slot] = 0
        return slot

    def free(self, slot):
        assert slot in self.held, "slot freed twice or never allocated"
        del self.held[slot]
        self.free_slots.append(slot)
        self.freed.append(slot)

    def step(self, slots, runs):
        assert all(s in self.held for s in slots)
        for s, run in zip(slots, runs):
            self.held[s] += len(run)
        self.steps.append((list(slots), [list(r) for r in runs]))
        return len(self.steps) - 1

    def sample(self, logits, requests, steps):
        return [self.scripts[r][t] for r, t in zip(requests, steps)]


def run(scripts, prompts, batches, n_slots=8, **kw):
    script = Script(scripts, n_slots)
    result = generate_requests(prompts, alloc=script.alloc, free=script.free, step=script.step,
                               sample=script.sample, batches=batches, **kw)
    assert not script.held, "slots still held at the end"
    return script, result


def test_unequal_prompts_shrinking_batch_and_stop_token_kept():
    prompts = [[1, 2, 3], [4], [5, 6]]
    scripts = {0: [10, 11, 12, 13], 1: [20, 99, 21, 22], 2: [30, 31, 32, 33]}
    script, result = run(scripts, prompts, [[0, 1, 2]], max_new_tokens=4, stop_token_ids=[99])
    assert result.generated_ids == [[10, 11, 12, 13], [20, 99], [30, 31, 32, 33]]
    assert result.finish_reasons == ["length", "stop", "length"]
    assert result.token_ids[1] == [4, 20, 99]
    # step 0: all prompts together; then one token each; request 1 leaves after its stop token
    assert script.steps[0][1] == prompts
    assert script.steps[1][1] == [[10], [20], [30]]
    assert script.steps[2][1] == [[11], [30 + 1]] and len(script.steps[2][0]) == 2
    assert len(script.steps) == 4 and result.decode_steps == 3
    assert len(result.step_seconds) == 3 and all(t >= 0 for t in result.step_seconds)
    assert result.decode_tokens == 3 + 1 + 3


def test_max_new_tokens_counts_the_prompts_token():
    script, result = run({0: [7, 8, 9]}, [[1, 2]], [[0]], max_new_tokens=1)
    assert result.generated_ids == [[7]] and len(script.steps) == 1
    with pytest.raises(ValueError):
        run({0: [7]}, [[1]], [[0]], max_new_tokens=0)


def test_stop_token_from_the_prompt_step_ends_the_sequence_at_once():
    script, result = run({0: [99, 1], 1: [5, 6]}, [[1], [2]], [[0, 1]], max_new_tokens=2, stop_token_ids=(99,))
    assert result.generated_ids == [[99], [5, 6]]
    assert script.steps[1][1] == [[5]]


def test_batches_run_one_after_another_and_reuse_slots():
    prompts = [[1]] * 5
    scripts = {r: [r, r, r] for r in range(5)}
    script, result = run(scripts, prompts, [[0, 1], [2, 3], [4]], n_slots=2, max_new_tokens=3)
    assert result.generated_ids == [[r] * 3 for r in range(5)]
    first_slots, second_slots = script.steps[0][0], script.steps[3][0]
    assert sorted(first_slots) == sorted(second_slots)            # the second batch got the first one's slots
    assert len(script.freed) == 5 and result.batches == [[0, 1], [2, 3], [4]]


def test_slots_are_freed_when_a_step_raises():
    script = Script({0: [1, 2, 3]})

    def failing_step(slots, runs):
        raise RuntimeError("boom")

    with pytest.raises(RuntimeError):
        generate_requests([[1]], max_new_tokens=2, alloc=script.alloc, free=script.free, step=failing_step,
                          sample=script.sample, batches=[[0]])
    assert not script.held


def test_step_numbers_given_to_the_sampler_are_tokens_generated_so_far():
    seen = []
    script = Script({0: [1, 2, 3], 1: [4, 5, 6]})

    def sample(logits, requests, steps):
        seen.append((list(requests), list(steps)))
        return script.sample(logits, requests, steps)

    generate_requests([[1], [2]], max_new_tokens=3, alloc=script.alloc, free=script.free, step=script.step,
                      sample=sample, batches=[[0, 1]])
    assert seen == [([0, 1], [0, 0]), ([0, 1], [1, 1]), ([0, 1], [2, 2])]


def test_plan_batches_respects_slots_and_tokens():
    # 64-token pages: footprints are 64, 128, 64, 192
    lengths = [10, 100, 60, 150]
    assert plan_batches(lengths, 5, max_seqs=8, max_tokens=10_000, page_size=64) == [[0, 1, 2, 3]]
    assert plan_batches(lengths, 5, max_seqs=2, max_tokens=10_000, page_size=64) == [[0, 1], [2, 3]]
    assert plan_batches(lengths, 5, max_seqs=8, max_tokens=256, page_size=64) == [[0, 1, 2], [3]]
    with pytest.raises(ValueError):
        plan_batches(lengths, 5, max_seqs=8, max_tokens=128, page_size=64)
    with pytest.raises(ValueError):
        plan_batches([0], 5, max_seqs=8, max_tokens=128, page_size=64)
    # prompt + max_new_tokens - 1 positions are cached: 64 + 1 - 1 fits one page, 64 + 2 - 1 does not
    assert plan_batches([64, 64], 1, max_seqs=8, max_tokens=128, page_size=64) == [[0, 1]]
    assert plan_batches([64, 64], 2, max_seqs=8, max_tokens=128, page_size=64) == [[0], [1]]


def test_fused_decoder_is_told_when_the_live_set_changes():
    """With a decoder, one-token steps go through begin/step instead of step/sample; begin is
    called again only when a sequence has left the batch."""
    scripts = {0: [10, 11, 12, 13], 1: [20, 99, 21, 22], 2: [30, 31, 32, 33]}
    script = Script(scripts)

    class Decoder:
        begins, live, position = [], [], {}

        def begin(self, slots, tokens, requests, steps):
            self.begins.append((list(slots), list(tokens), list(requests), list(steps)))
            self.live = list(requests)
            self.position = dict(zip(requests, steps))

        def step(self, last_tokens):
            # the loop feeds each live sequence's last token from its own record
            assert last_tokens == [scripts[r][self.position[r] - 1] for r in self.live]
            out = [scripts[r][self.position[r]] for r in self.live]
            for r in self.live:
                self.position[r] += 1
            return out

    decoder = Decoder()
    result = generate_requests([[1, 2, 3], [4], [5, 6]], max_new_tokens=4, alloc=script.alloc, free=script.free,
                               step=script.step, sample=script.sample, batches=[[0, 1, 2]], stop_token_ids=[99],
                               decoder=decoder)
    assert result.generated_ids == [[10, 11, 12, 13], [20, 99], [30, 31, 32, 33]]
    assert len(script.steps) == 1                      # only the prompts went through step()
    assert [b[2] for b in decoder.begins] == [[0, 1, 2], [0, 2]]
    assert decoder.begins[0][1] == [10, 20, 30] and decoder.begins[0][3] == [1, 1, 1]
    assert decoder.begins[1][1] == [11, 31] and decoder.begins[1][3] == [2, 2]
    assert result.decode_steps == 3 and not script.held


def test_decode_widths_pad_little_above_32():
    """Captured decode widths: powers of two up to 32, multiples of 16 beyond (33 must not run as 64)."""
    from ondeviceinfer_b200.engine.decode import DecodeRunner
    widths = {n: DecodeRunner._width_for(n) for n in (1, 2, 3, 8, 9, 17, 32, 33, 48, 49, 64, 65, 100)}
    assert widths == {1: 1, 2: 2, 3: 4, 8: 8, 9: 16, 17: 32, 32: 32, 33: 48, 48: 48, 49: 64, 64: 64, 65: 80, 100: 112}


def test_a_dropped_cache_takes_its_decode_runner_along_at_once():
    """The cache keeps its decode runners and a runner only a weak reference to the cache: when the last
    reference to the cache goes, both go at that moment, not when the cycle collector next runs (which may be
    in the middle of somebody else's graph capture, where destroying a graph is not allowed)."""
    import gc
    import weakref

    import torch

    from ondeviceinfer_b200.api import decode_runner
    from ondeviceinfer_b200.cache import KVNeed, SequenceCache

    class Model:            # what decode_runner touches before the first step
        decoder = object()

    gc.collect()
    gc.disable()
    try:
        cache = SequenceCache([(KVNeed(2, 16),)], [None], dtype=torch.float32, device="cpu", max_tokens=256, max_seqs=2)
        runner = decode_runner(Model, cache)
        assert decode_runner(Model, cache) is runner and runner.cache is cache
        gone = weakref.ref(runner)
        del runner, cache
        assert gone() is None
    finally:
        gc.enable()


def test_which_captured_graph_serves_a_step():
    """The decode runner replays the graph made for the step's width, length bucket and split bounds, or one
    made for up to twice the length and twice the splits; anything else needs a capture."""
    from ondeviceinfer_b200.engine.decode import DecodeRunner, serving_graph_key

    keys = {(8, 4096, (4,)): "a", (8, 8192, (8,)): "b", (16, 4096, (4,)): "c", (8, 4096, ()): "d"}
    assert serving_graph_key(keys, 8, 4096, (4,)) == (8, 4096, (4,))
    assert serving_graph_key(keys, 8, 4096, (2,)) == (8, 4096, (4,))        # twice the splits: serves
    assert serving_graph_key(keys, 8, 4096, (1,)) is None                    # four times: a graph of its own
    assert serving_graph_key(keys, 8, 4096, (8,)) == (8, 8192, (8,))        # twice the length: serves
    assert serving_graph_key(keys, 8, 2048, (4,)) == (8, 4096, (4,))
    assert serving_graph_key(keys, 8, 1024, (4,)) is None
    assert serving_graph_key(keys, 8, 8192, (4,)) == (8, 8192, (8,))
    assert serving_graph_key(keys, 8, 16384, (8,)) is None                   # longer than any graph was made for
    assert serving_graph_key(keys, 8, 4096, (16,)) is None                   # more splits than any graph has
    assert serving_graph_key(keys, 4, 4096, (4,)) is None                    # another width
    assert serving_graph_key(keys, 8, 4096, ()) == (8, 4096, ())             # a model whose parts cut no keys
    assert serving_graph_key(keys, 8, 4096, (4, 4)) is None
    assert [DecodeRunner._bucket_for(n) for n in (1, 256, 257, 4096, 4097)] == [256, 256, 512, 4096, 8192]
