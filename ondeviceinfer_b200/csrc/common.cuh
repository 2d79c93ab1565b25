// Shared device helpers for the sm_100a kernels of this library.
//
// Conventions used by every kernel file:
//  * launchers are extern "C", take raw device pointers plus a cudaStream_t, allocate
//    nothing and return a cudaError_t value as int (0 = launched);
//  * the residual stream and all statistics (norms, softmax, rotation angles) are fp32;
//    `T` is the activation / weight / cache element type (float or __nv_bfloat16);
//  * sizes are runtime arguments unless a file says otherwise; a launcher that cannot
//    handle a size returns ODI_ERR_UNSUPPORTED instead of computing something else.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define ODI_ERR_UNSUPPORTED 10001  // size or alignment the kernel refuses
#define ODI_ERR_ARGUMENT 10002     // inconsistent arguments

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

// Round a float to the precision of T and back: marks the places where an activation
// is materialised in the model dtype.
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f<T>(from_f<T>(v)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` is
// 33 floats of shared memory.  The order of additions is fixed by the thread layout.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Result of the launches since the last call: the first launch error, else cudaGetLastError().
static thread_local int odi_rc = 0;
static inline int launch_status() {
  const int rc = odi_rc != 0 ? odi_rc : (int)cudaGetLastError();
  odi_rc = 0;
  return rc;
}

// Programmatic dependent launch.  Every kernel of this library starts with pdl_wait() before it
// touches memory that an earlier kernel of the stream may write or read, and tells the runtime
// with pdl_launch_dependents() that the next kernel may be scheduled; launched through
// launch_pdl() the next kernel's launch latency and set-up then overlap this kernel's run.
// Both instructions do nothing in a kernel that was launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <stdlib.h>
static inline int pdl_enabled() {
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("ODI_PDL");
    enabled = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return enabled;
}

template <typename... KArgs, typename... Args>
static inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled();
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args...);
  return odi_rc != 0 ? odi_rc : (int)e;      // keep the first error of a launcher
}

// Arguments of the fused head preparation (elementwise.cu; also the epilogue of the tensor-core
// product that makes the projections).
struct HeadPrepArgs {
  const void* qkv;
  void* q_out;
  void* k_pool;
  void* v_pool;
  const float* q_norm_w;  // null: no norm
  const float* k_norm_w;
  const float* cos_t;     // null: no rotation; [n_tokens, rot_dim / 2]
  const float* sin_t;
  const int* tok_seq;
  const int* tok_pos;
  const int* page_start;
  const int* page_ids;
  int n_tokens, nq, nkv, d, rot_dim, page_size, ring_pages, write_kv;
  float eps;
};

// The output of a decode attention whose key splits have not been merged yet (attention_mma.cu leaves it when
// asked to skip its combine kernel; the output projection's product can take it as its operand).
struct MergeArgs {
  const float* partial;   // [tokens, nq, splits, d + 2]: per split the weighted values, their maximum (natural-log
                          // domain, -inf for a split without keys) and their sum
  const int* past;        // [tokens]: the position of each token's query (one token per sequence)
  const int* plan;        // null: every token uses all `splits`; else plan[0] = tiles of 64 keys per split
  int splits, nq, d;
};

// How many of its `splits` partials a token at position `pos` has: all of them without a plan, else what its
// tiles need at plan[0] tiles a split (never fewer tiles a split than `splits` blocks need to cover the sequence).
__device__ __forceinline__ int merge_used_splits(const int* plan, int splits, int pos) {
  if (plan == nullptr) return splits;
  const int n_tiles = pos / 64 + 1;
  const int even = (n_tiles + splits - 1) / splits;
  const int per = max(plan[0], even);
  return (n_tiles + per - 1) / per;
}

// Position of key `pos` inside a sequence's page list.  A group that keeps every key
// has ring_pages == 0; a windowed group keeps a ring of ring_pages pages per sequence.
__device__ __forceinline__ int page_slot_of(int pos, int page_size, int ring_pages) {
  int p = pos / page_size;
  return ring_pages > 0 ? p % ring_pages : p;
}
