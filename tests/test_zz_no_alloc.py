"""The allocation-free entry point (csrc/attention_noalloc.h), called through its exported C symbol.

Some callers of split-key decode attention cannot ask for device memory at the moment they
need the result: a host loop whose memory plan is frozen after start-up, a plugin inside an
engine that owns the allocator, code that runs while an allocator lock is held.  For them
the library keeps the scratch for the split partials in a fixed 8 MiB array of its own.
This test checks that the entry point gives what the ordinary entry point gives (which
takes a scratch buffer from the caller), twice in a row on different inputs so that the
second call runs on whatever the first one left in the array, and that a call that would
not fit is refused with a clear message instead of being launched.

It is collected last (file name) so that a run which stops at the first failure has already
run every other test; it passes alone in a fresh process as well as after the others.
"""

import ctypes
import math

import pytest
import torch

from ondeviceinfer_b200.kernels import ops
from ondeviceinfer_b200.kernels.build import load_library
from test_kernels_gpu import paged_setup, plain_attention

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
D = 128
ERR_SCRATCH_LIMIT = 10003


def call_noalloc(lib, q, setup, out, *, n_seqs, nq, nkv, splits, scale):
    args = ops._MmaAttnArgs(q.data_ptr(), setup["k_pool"].data_ptr(), setup["v_pool"].data_ptr(), out.data_ptr(),
                            0, setup["cu_q"].data_ptr(), setup["past"].data_ptr(), setup["page_start"].data_ptr(),
                            setup["page_ids"].data_ptr(), n_seqs, nq, nkv, splits, 0, scale)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.odi_attention_decode_noalloc(ctypes.byref(args), ctypes.c_int(n_seqs), stream)


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    lib = load_library("attention_mma", {"ODI_HEAD_DIM": D})
    lib.odi_attention_decode_noalloc_error.restype = ctypes.c_char_p
    lib.odi_attention_decode_noalloc_capacity.restype = ctypes.c_long
    lib.odi_attention_decode_noalloc_need.restype = ctypes.c_long
    assert lib.odi_attention_decode_noalloc_capacity() == 2 * 1024 * 1024
    scale = 1.0 / math.sqrt(D)
    torch.cuda.set_device(0)
    calls = [
        dict(nq=32, nkv=8, past=[300, 64, 63, 1000, 5], splits=6, seed=41),
        dict(nq=8, nkv=2, past=[700, 129], splits=3, seed=42),        # smaller: reads slots the first call wrote
        dict(nq=32, nkv=8, past=[300, 64, 63, 1000, 5], splits=1, seed=41),
    ]
    for call in calls:
        n = len(call["past"])
        setup = paged_setup([1] * n, call["past"], call["nkv"], D, "bfloat16", seed=call["seed"])
        torch.manual_seed(call["seed"])
        q = torch.randn(n, call["nq"], D).bfloat16().to(DEV)
        # every input and output exists before the call; the call itself must not allocate
        mine = torch.empty(n, call["nq"] * D, dtype=torch.bfloat16, device=DEV)
        theirs = torch.empty_like(mine)
        partial = torch.empty(n * call["nq"] * call["splits"] * (D + 2), dtype=torch.float32, device=DEV)
        torch.cuda.synchronize()
        allocated = torch.cuda.memory_allocated()
        rc = call_noalloc(lib, q, setup, mine, n_seqs=n, nq=call["nq"], nkv=call["nkv"], splits=call["splits"], scale=scale)
        assert rc == 0, (rc, lib.odi_attention_decode_noalloc_error())
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == allocated
        ops.attention_mma(q, setup["k_pool"], setup["v_pool"], theirs, setup["cu_q"], setup["past"],
                          setup["page_start"], setup["page_ids"], n_seqs=n, max_q_len=1, nq=call["nq"],
                          nkv=call["nkv"], d=D, page_size=64, scale=scale, splits=call["splits"],
                          partial=partial if call["splits"] > 1 else None, cluster=False)   # the caller-buffer form
        torch.cuda.synchronize()
        expected = plain_attention(q.float().cpu(), setup["dense"], [1] * n, call["past"], call["nq"], call["nkv"], D, 0,
                                   scale, "bfloat16")
        # the tolerance of the kernel tests: 2e-2 * max(1, max |expected|) for bf16 outputs
        limit = 2e-2 * max(1.0, float(expected.abs().max()))
        assert float((mine.float().cpu() - theirs.float().cpu()).abs().max()) <= limit
        assert float((mine.float().cpu() - expected).abs().max()) <= limit
        assert torch.equal(mine, theirs), "the same kernels on the same inputs: the results should be identical"


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    lib = load_library("attention_mma", {"ODI_HEAD_DIM": D})
    lib.odi_attention_decode_noalloc_error.restype = ctypes.c_char_p
    lib.odi_attention_decode_noalloc_need.restype = ctypes.c_long
    n, nq, nkv, splits = 64, 64, 8, 8
    assert lib.odi_attention_decode_noalloc_need(n, nq, splits) == n * nq * splits * (D + 2) > 2 * 1024 * 1024
    setup = paged_setup([1] * 2, [10, 20], nkv, D, "bfloat16", seed=43)
    q = torch.zeros(n, nq, D, dtype=torch.bfloat16, device=DEV)
    out = torch.full((n, nq * D), 7.0, dtype=torch.bfloat16, device=DEV)
    rc = call_noalloc(lib, q, setup, out, n_seqs=n, nq=nq, nkv=nkv, splits=splits, scale=1.0)
    assert rc == ERR_SCRATCH_LIMIT
    message = lib.odi_attention_decode_noalloc_error().decode()
    assert "2097152" in message and str(n * nq * splits * (D + 2)) in message
    torch.cuda.synchronize()
    assert float(out.float().min()) == 7.0, "a refused call must not launch anything"


def test_no_alloc_entry_point_refuses_null_pointers():
    lib = load_library("attention_mma", {"ODI_HEAD_DIM": D})
    lib.odi_attention_decode_noalloc_error.restype = ctypes.c_char_p
    setup = paged_setup([1] * 2, [10, 20], 2, D, "bfloat16", seed=44)
    out = torch.full((2, 4 * D), 7.0, dtype=torch.bfloat16, device=DEV)
    args = ops._MmaAttnArgs(0, setup["k_pool"].data_ptr(), setup["v_pool"].data_ptr(), out.data_ptr(),
                            0, setup["cu_q"].data_ptr(), setup["past"].data_ptr(), setup["page_start"].data_ptr(),
                            setup["page_ids"].data_ptr(), 2, 4, 2, 2, 0, 1.0)       # q is null
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.odi_attention_decode_noalloc(ctypes.byref(args), ctypes.c_int(2), stream) == ops.ODI_ERR_ARGUMENT
    assert "null" in lib.odi_attention_decode_noalloc_error().decode()
    assert lib.odi_attention_decode_noalloc(None, ctypes.c_int(2), stream) == ops.ODI_ERR_ARGUMENT
    torch.cuda.synchronize()
    assert float(out.float().min()) == 7.0
