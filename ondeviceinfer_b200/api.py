"""The Python entry point, in the manner of UESlubei/ondeviceinfer's own.

Reference                                              Here
``load_resident_model(path, device=, dtype=)``          same name and arguments
  (ondeviceinfer/weights.py:60-81)                      (the model class is chosen by config.json)
``model.make_resident_cache(batch_size=, max_seq_len=)`` same; room for batch_size sequences of
  (ondeviceinfer/model.py:165-181)                      max_seq_len tokens, in pages
``model(input_ids, cache=, logits_to_keep=)``           ``model.step(cache, slots, tokens, want=)``
  (ondeviceinfer/model.py:146-163)                      (unequal lengths, a slot per sequence)
``greedy_generate(model, input_ids, max_new_tokens=,    same name; any batch size; plus
  cache=, eos_token_id=)``                              ``generate(...)`` with temperature, seed and
  (ondeviceinfer/generation.py:28-70)                   requests of unequal length
"""

from __future__ import annotations

from pathlib import Path
from typing import List, Optional, Sequence, Union

import torch

from . import models  # noqa: F401  (registers the architectures)
from .cache import PAGE_SIZE, SequenceCache, pages_for
from .engine.decode import DecodeRunner
from .engine.generate import GenerationResult, generate_requests, plan_batches
from .engine.model import DecoderModel
from .engine.step import run_step
from .kernels import ops
from .registry import config_from_dict, config_from_folder
from .sampling import Sampler
from .weights import RandomSource, SafetensorsSource

DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _dtype(dtype) -> torch.dtype:
    if isinstance(dtype, str):
        if dtype not in DTYPES:
            raise ValueError(f"dtype must be one of {sorted(DTYPES)}, not {dtype!r}")
        return DTYPES[dtype]
    return dtype


class ResidentModel:
    """A loaded model: typed configuration, the decoder built from its plan, weights on the device."""

    def __init__(self, config, decoder: DecoderModel) -> None:
        self.config, self.decoder = config, decoder

    @property
    def device(self) -> torch.device:
        return self.decoder.device

    @property
    def dtype(self) -> torch.dtype:
        return self.decoder.dtype

    @property
    def vocab_size(self) -> int:
        return self.decoder.vocab_size

    def make_cache(self, *, max_tokens: int, max_seqs: Optional[int] = None) -> SequenceCache:
        """A cache for at most ``max_tokens`` tokens held by live sequences (each sequence
        rounded up to pages of 64) and at most ``max_seqs`` sequences at a time."""
        if max_seqs is None:
            max_seqs = max(1, pages_for(max_tokens))
        return self.decoder.make_cache(max_tokens=max_tokens, max_seqs=max_seqs)

    def make_resident_cache(self, *, batch_size: int, max_seq_len: int) -> SequenceCache:
        if max_seq_len <= 0:
            raise ValueError("max_seq_len must be positive")
        return self.make_cache(max_tokens=batch_size * pages_for(max_seq_len) * PAGE_SIZE, max_seqs=batch_size)

    def step(self, cache: SequenceCache, slots: Sequence[int], tokens: Sequence[Sequence[int]],
             want="last") -> torch.Tensor:
        """One step of the batch; fp32 logits [wanted, vocab].  See ``engine.step``."""
        return run_step(self.decoder, cache, slots, tokens, want)

    def generate(self, prompts, **kwargs) -> GenerationResult:
        return generate(self, prompts, **kwargs)


def load_resident_model(model_path, *, device="cuda:0", dtype=torch.bfloat16) -> ResidentModel:
    """Load a model folder (``config.json`` + safetensors) onto ``device``."""
    model_path = Path(model_path)
    config = config_from_folder(model_path)
    source = SafetensorsSource(model_path)
    try:
        decoder = DecoderModel(config.to_plan()).load(source, dtype=_dtype(dtype), device=device)
    finally:
        source.close()
    return ResidentModel(config, decoder)


def random_resident_model(config, seed: int, *, device="cuda:0", dtype=torch.bfloat16) -> ResidentModel:
    """A model with seeded random weights drawn on the device (nothing is written to disk).
    ``config`` is a typed configuration or a ``config.json`` dictionary."""
    if isinstance(config, dict):
        config = config_from_dict(config)
    decoder = DecoderModel(config.to_plan())
    source = RandomSource(decoder.tensor_decls(), seed, dtype=torch.bfloat16, device=device)
    decoder.load(source, dtype=_dtype(dtype), device=device)
    return ResidentModel(config, decoder)


def _as_prompts(prompts) -> List[List[int]]:
    if isinstance(prompts, torch.Tensor):
        if prompts.ndim != 2:
            raise ValueError("input_ids must have shape [batch, sequence]")
        return prompts.tolist()
    return [list(map(int, p)) for p in prompts]


def generate(model: ResidentModel, prompts, *, max_new_tokens: int, cache: Optional[SequenceCache] = None,
             temperature: float = 0.0, seed: int = 0,
             eos_token_id: Union[int, Sequence[int], None] = None, use_graphs: bool = True) -> GenerationResult:
    """Generate for every prompt (lists of token ids of any lengths, or a ``[batch, T]``
    tensor).  ``eos_token_id`` None disables stopping, as in the reference; a stop token
    is kept in the output.  Without ``cache`` one is made that fits all requests at once.
    Decode steps replay CUDA graphs (``use_graphs``) when every part of the model allows it;
    the kernels and the results are the same either way."""
    prompts = _as_prompts(prompts)
    if cache is None:
        need = sum(pages_for(len(p) + max_new_tokens) * PAGE_SIZE for p in prompts)
        cache = model.make_cache(max_tokens=need, max_seqs=len(prompts))
    if eos_token_id is None:
        stop = ()
    elif isinstance(eos_token_id, int):
        stop = (eos_token_id,)
    else:
        stop = tuple(eos_token_id)
    batches = plan_batches([len(p) for p in prompts], max_new_tokens, max_seqs=cache.max_seqs,
                           max_tokens=cache.max_tokens, page_size=PAGE_SIZE)
    sampler = Sampler(temperature, seed)

    def synchronize() -> None:
        # where the loop waits for the device anyway, it also learns whether a kernel gave up on a barrier
        torch.cuda.synchronize(model.device)
        ops.raise_on_kernel_fault()

    decoder = None
    if use_graphs and model.decoder.graph_safe:
        decoder = decode_runner(model, cache, temperature=temperature, seed=seed)
    return generate_requests(
        prompts, max_new_tokens=max_new_tokens, alloc=cache.alloc, free=cache.free,
        step=lambda slots, runs: model.step(cache, slots, runs, "last"),
        sample=sampler, batches=batches, stop_token_ids=stop,
        synchronize=synchronize, decoder=decoder)


def decode_runner(model: ResidentModel, cache: SequenceCache, *, temperature: float = 0.0, seed: int = 0) -> DecodeRunner:
    """The graph-replaying decoder of ``cache`` for these sampling settings (made once, kept on the cache)."""
    runners = cache.__dict__.setdefault("_decode_runners", {})
    key = (id(model.decoder), float(temperature), int(seed))
    if key not in runners:
        runners[key] = DecodeRunner(model.decoder, cache, temperature=temperature, seed=seed)
    return runners[key]


def greedy_generate(model: ResidentModel, input_ids, *, max_new_tokens: int,
                    cache: Optional[SequenceCache] = None, eos_token_id=None) -> GenerationResult:
    """The reference's entry point (ondeviceinfer/generation.py:28-36), for any batch."""
    return generate(model, input_ids, max_new_tokens=max_new_tokens, cache=cache, temperature=0.0,
                    eos_token_id=eos_token_id)
