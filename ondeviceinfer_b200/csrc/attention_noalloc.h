// Declaration of the one allocation-free entry point of this library.
//
// It has no counterpart in UESlubei/ondeviceinfer: the reference is PyTorch code and lets
// the framework allocate whatever an operation needs.
//
// Who needs it: code that has to run split-key decode attention from a place where device
// memory cannot be requested -- a real-time or safety-certified host loop whose memory plan
// is frozen after start-up, a plugin inside another engine that owns the allocator and hands
// out no workspace, a callback that runs while an allocator lock is held.  For those callers
// cudaMalloc (or any caching allocator built on it) is either forbidden or may block or
// fail at a moment when failing is not an option.
//
// What it does: the same computation as odi_attention_mma in its decode form (one query
// token per sequence, bf16, paged cache, keys cut into `splits` ranges whose partial results
// are merged), but the scratch for the partial results lives in a fixed array inside the
// library instead of in a buffer the caller passes.
//
// The limit: ODI_NOALLOC_SCRATCH_FLOATS floats (8 MiB).  Every GPU that loads the library
// holds that array until the process exits.  A call needs
//     n_tokens * nq * splits * (head_dim + 2)  floats
// and is refused with ODI_ERR_SCRATCH_LIMIT (and a message from
// odi_attention_decode_noalloc_error) when that is more; nothing is launched then.
//
// Rules of use:
//  * Inputs and outputs are still the caller's: args->q, k_pool, v_pool, out and the index
//    arrays must be device memory the caller owns.  args->partial is ignored.
//  * The first call on a device looks up the device address of the array (the array's name
//    in host code is only a handle, not an address a kernel could use) and sets a function
//    attribute.  Make that first call, once per device and with that device current,
//    during start-up and before any stream capture begins.
//  * All calls share the one array and it keeps what the previous call left in it.  Nothing
//    in it has to start at zero: every (token, head, split) slot that a call reads is written
//    by that same call first, so stale contents are never seen.  Two calls whose kernels may
//    overlap on the GPU (different streams without an ordering between them) race on the
//    array; order them, or use odi_attention_mma with separate buffers.
//  * Threads: the entry point may be called from several host threads.  The per-device set-up is published
//    atomically, so first calls that run side by side are safe (each may do the look-up; they agree), and
//    the refusal text is kept per thread.  What threads cannot share without ordering is the array itself:
//    the rule above on overlapping kernels holds whichever threads launched them.
//  * A null args, or a null q, k_pool, v_pool, out, cu_q, past, page_start or page_ids, is refused with
//    ODI_ERR_ARGUMENT and a message; nothing is launched.
//  * The entry point calls no cudaMalloc, cudaFree or any other allocating routine.
#pragma once

#include <cuda_runtime.h>

#define ODI_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define ODI_ERR_SCRATCH_LIMIT 10003

struct MmaAttnArgs;

extern "C" int odi_attention_decode_noalloc(const MmaAttnArgs* args, int n_tokens, cudaStream_t stream);

// Scratch floats a call with these sizes needs, and the fixed capacity.
extern "C" long odi_attention_decode_noalloc_need(int n_tokens, int nq, int splits);
extern "C" long odi_attention_decode_noalloc_capacity();

// Text of the last refusal on this thread ("" if the last call was accepted).
extern "C" const char* odi_attention_decode_noalloc_error();
