// bf16 causal grouped-query attention for prefill on the 5th-generation tensor cores.
//
// One CTA owns 128 consecutive query tokens of one sequence for one query head (optionally two
// heads that share a key/value head) and walks that sequence's key/value pages (64 positions
// each) up to the diagonal.  Per head:
//
//   S_j = Q K_j^T        tcgen05.mma, M = 128 query rows, N = 64 keys, K = head size; Q and K_j
//                        in shared memory (TMA, 128-byte swizzle), S_j in tensor memory
//   P_j = softmax part   by 8 warps: a query row is handled by two threads (32 keys each); fp32
//                        running maximum and sum; P_j rounded to bf16 and written, in the swizzled
//                        K-major layout the MMA reads, over the shared memory of K_j (which S_j
//                        has consumed by then)
//   O  += P_j V_j        tcgen05.mma, M = 128, N = head size, K = 64 keys; V_j is read as it lies
//                        in its page (MN-major operand); O accumulates in tensor memory
//
// The accumulator in tensor memory cannot be scaled by the MMA, so the running maximum that P is
// taken against is only raised when a row's new maximum exceeds it by more than 2^8: then that
// row of O is read, scaled and written back (tcgen05.ld / st) before the row's next product is
// issued.  P stays below 2^8, which bf16 and the fp32 accumulator hold without loss, and the
// result is the same as with a maximum that is raised every time.
//
// Per head S is double buffered in tensor memory (2 x 64 columns) and O takes head-size columns:
// 256 columns a head.  K/V pages sit in two shared-memory stages, so the scores of page j + 1 are
// computed while page j is in the softmax.  With one head per CTA (the default) a CTA takes 97 KB
// of shared memory, 256 columns and 80 registers a thread, so two CTAs share an SM and one's MMAs
// run under the other's softmax: measured 381 / 562 / 620 TFLOP/s at 1 x 2048, 8 x 2048 and
// 1 x 8192 tokens.  Two heads of a key/value group per CTA (K/V pages loaded once for both, the
// second head's P in buffers of its own) measured no faster (284-462 TFLOP/s with two stages,
// 323-551 with three) and stays an option.  Warps: 0 = TMA producer, 1 = MMA issuer (one thread)
// and tensor-memory owner, 2..9 = softmax of the first head, 10..17 = of the second.
//
// Works for any q_len >= 1 on top of any cached length (query t of the step sits at position
// past + t).  No window.  Compile with -DODI_HEAD_DIM=64 or 128.
//
// Every wait on an mbarrier is bounded (about two seconds of SM clock): a role that gives up
// records a code in `status`, raises the CTA's abort flag, and all roles fall through to the
// common exit, where tensor memory is freed.
#include <cuda.h>

#include "common.cuh"

#ifndef ODI_HEAD_DIM
#error "compile with -DODI_HEAD_DIM=<head size>"
#endif
#define D ODI_HEAD_DIM
#if D != 64 && D != 128
#error "the tcgen05 attention takes head sizes 64 and 128"
#endif

#define BM 128                 // query rows per CTA
#define BNK 64                 // keys per page / tile
#define KB (D / 64)            // 64-wide blocks of the head size
#ifndef NST
#define NST 2                  // key/value stages
#endif
#define Q_BYTES (KB * BM * 128)
#define KV_BYTES (KB * BNK * 128)     // one of K or V for a page
#define P_BYTES (BM * 128)            // 128 rows x 64 keys bf16
#define KP_BYTES (KV_BYTES > P_BYTES ? KV_BYTES : P_BYTES)   // K_j, later overwritten by P_j
#define STAGE_BYTES (KP_BYTES + KV_BYTES)
#define HEAD_COLS 256                  // tensor-memory columns per head: S0, S1, O
#define S_COL(t, b) ((t) * HEAD_COLS + (b) * BNK)
#define O_COL(t) ((t) * HEAD_COLS + 2 * BNK)
#define RESCALE_THRESHOLD 8.0f        // log2 units
#define WAIT_CYCLES 4000000000ll
#define LOG2E 1.4426950408889634f

#ifndef ODI_ATT_DEFAULT_HEADS_PER_CTA
#define ODI_ATT_DEFAULT_HEADS_PER_CTA 1
#endif
#define ATT_ERR_PRODUCER 11
#define ATT_ERR_MMA 12
#define ATT_ERR_SOFTMAX 13

struct TcAttnArgs {
  bf16* out;              // [n_tokens, nq * D]
  const int* cu_q;
  const int* past;
  const int* page_start;
  const int* page_ids;
  int* status;
  int n_seqs, nq, nkv;
  float scale;
};

// ------------------------------------------------------------------------------ PTX wrappers

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  const long long start = clock64();
  for (uint32_t i = 0;; ++i) {
    if (mbar_test(bar, parity)) return true;
    // try_wait suspends the thread for a bounded, implementation-defined time instead of spinning
    if ((i & 0xf) == 0xf) {
      if (*abort_flag) return false;
      if (clock64() - start > WAIT_CYCLES) break;
    }
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// 32 consecutive columns of this thread's lane: two loads in flight, one wait.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 2^x for x <= 8 (the scores minus the maximum in use); large negative x gives 0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// K-major operand tile written by TMA with the 128-byte swizzle (rows of 128 bytes, 8-row groups
// 1024 bytes apart): Q, K and P.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3ffff) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// MN-major operand (V as the B operand of P V: rows are keys = the MMA's K, the 128-byte row holds
// 64 consecutive head elements = the MMA's N): 8-key groups 1024 bytes apart (stride byte offset),
// 64-element column blocks KV_BYTES / KB apart (leading byte offset).
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3ffff) >> 4);
  d |= (uint64_t)((BNK * 128) >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// kind::f16, fp32 accumulator, bf16 operands; b_mn selects an MN-major B operand.
__host__ __device__ constexpr uint32_t idesc_bf16(int m, int n, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}

// ------------------------------------------------------------------------------ the kernel

template <int TILES>
__global__ void __launch_bounds__(64 + 256 * TILES, TILES == 1 ? 2 : 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const TcAttnArgs a) {
  constexpr int TMEM_COLS = TILES * HEAD_COLS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  // barriers: q_full, kv_full[NST], kv_empty[NST], s_full[2], s_empty[2], p_full[TILES][2], pv_done[TILES]
  __shared__ __align__(8) uint64_t bars[1 + 2 * NST + 4 + 3 * TILES];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ float row_max[TILES][2][BM];   // the two halves of a row exchange their maxima (and sums) here

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Heads along x, sequences along y, query tiles along z from the last (which sees the most keys) to the
  // first: blocks are handed out x-fastest, so the long tiles of all heads and sequences start first and
  // the short ones fill the tail.
  const int seq = blockIdx.y, head0 = blockIdx.x * TILES, hk = head0 / (a.nq / a.nkv);
  const int q_begin = a.cu_q[seq], q_len = a.cu_q[seq + 1] - q_begin;
  const int t0 = (gridDim.z - 1 - blockIdx.z) * BM;
  if (t0 >= q_len) return;                       // whole CTA: nothing allocated yet
  const int past = a.past[seq];
  const int nt = min(BM, q_len - t0);
  const int n_tiles = (past + t0 + nt + BNK - 1) / BNK;
  const int* pages = a.page_ids + a.page_start[seq];

  const uint32_t bar0 = smem_u32(&bars[0]);
  const uint32_t q_full = bar0, kv_full = bar0 + 8, kv_empty = kv_full + 8 * NST, s_full = kv_empty + 8 * NST,
                 s_empty = s_full + 16, p_full = s_empty + 16, pv_done = p_full + 16 * TILES;
  uint8_t* q_smem = smem;                                    // head t at t * Q_BYTES
  uint8_t* kv_smem = smem + TILES * Q_BYTES;                 // stage s: K (later the first head's P), then V
  uint8_t* p1_smem = kv_smem + NST * STAGE_BYTES;            // the second head's P, two buffers

  if (threadIdx.x == 0) {
    for (int i = 0; i < 1 + 2 * NST + 4 + 3 * TILES; ++i) mbar_init(bar0 + 8 * i, 1);
    for (int b = 0; b < 2; ++b) {      // signalled by the pairs of softmax warps: four pairs a head
      mbar_init(s_empty + 8 * b, 4 * TILES);
      for (int t = 0; t < TILES; ++t) mbar_init(p_full + 16 * t + 8 * b, 4);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abort_ptr = &abort_flag;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      pdl_wait();      // queries and this step's keys/values come from the kernel before
      mbar_expect_tx(q_full, TILES * Q_BYTES);
      for (int t = 0; t < TILES; ++t)
        for (int kb = 0; kb < KB; ++kb)
          tma_load_2d(smem_u32(q_smem + t * Q_BYTES + kb * BM * 128), &map_q, (head0 + t) * D + kb * 64, q_begin + t0, q_full);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % NST;
        if (!mbar_wait(kv_empty + 8 * s, ((uint32_t)(j / NST) & 1u) ^ 1u, abort_ptr)) { atomicCAS(a.status, 0, ATT_ERR_PRODUCER); break; }
        const int row = (pages[j] * a.nkv + hk) * BNK;
        uint8_t* st = kv_smem + (size_t)s * STAGE_BYTES;
        mbar_expect_tx(kv_full + 8 * s, 2 * KV_BYTES);
        for (int kb = 0; kb < KB; ++kb) {
          tma_load_2d(smem_u32(st + kb * BNK * 128), &map_k, kb * 64, row, kv_full + 8 * s);
          tma_load_2d(smem_u32(st + KP_BYTES + kb * BNK * 128), &map_v, kb * 64, row, kv_full + 8 * s);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc_bf16(BM, BNK, false);
      constexpr uint32_t idesc_o = idesc_bf16(BM, D, true);
      bool ok = mbar_wait(q_full, 0, abort_ptr);
      auto issue_s = [&](int j) -> bool {
        const int s = j % NST, b = j & 1;
        if (!mbar_wait(kv_full + 8 * s, (uint32_t)(j / NST) & 1u, abort_ptr)) return false;
        if (!mbar_wait(s_empty + 8 * b, ((uint32_t)(j >> 1) & 1u) ^ 1u, abort_ptr)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(kv_smem + (size_t)s * STAGE_BYTES);
#pragma unroll
        for (int t = 0; t < TILES; ++t) {
#pragma unroll
          for (int kb = 0; kb < KB; ++kb) {
            const uint64_t dq = desc_k_major(smem_u32(q_smem + t * Q_BYTES + kb * BM * 128));
            const uint64_t dk = desc_k_major(k_addr + kb * BNK * 128);
#pragma unroll
            for (int i = 0; i < 4; ++i) umma(tmem_base + S_COL(t, b), dq + 2 * i, dk + 2 * i, idesc_s, (kb | i) ? 1u : 0u);
          }
        }
        umma_commit(s_full + 8 * b);       // both heads' scores done: K_j is free for the first head's P
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_s(j + 1);      // the next page's scores run under this page's softmax
        if (!ok) break;
        const int s = j % NST, b = j & 1;
        const uint32_t stage = smem_u32(kv_smem + (size_t)s * STAGE_BYTES);
        const uint64_t dv = desc_mn_major(stage + KP_BYTES);
#pragma unroll
        for (int t = 0; t < TILES; ++t) {
          if (!mbar_wait(p_full + 16 * t + 8 * b, (uint32_t)(j >> 1) & 1u, abort_ptr)) { ok = false; break; }
          tc_fence_after();
          const uint64_t dp = desc_k_major(t == 0 ? stage : smem_u32(p1_smem + b * P_BYTES));
#pragma unroll
          for (int i = 0; i < 4; ++i)      // 16 keys per MMA: 32 bytes along P's rows, 16 rows (2048 bytes) down V
            umma(tmem_base + O_COL(t), dp + 2 * i, dv + (uint64_t)(i * 2048 >> 4), idesc_o, (j | i) ? 1u : 0u);
          umma_commit(pv_done + 8 * t);
        }
        umma_commit(kv_empty + 8 * s);
      }
      if (!ok) atomicCAS(a.status, 0, ATT_ERR_MMA);
    }
  } else {
    // ---------------------------------------------------------------- softmax and output (8 warps a head)
    const int tile = (warp - 2) >> 3;                // which of the CTA's heads
    const int head = head0 + tile;
    const int lane_group = warp & 3;                 // the tensor-memory lanes this warp may read
    const int half = ((warp - 2) >> 2) & 1;          // keys 0..31 or 32..63 of a page
    const int row = lane_group * 32 + lane;          // query row inside the tile
    const int pos = past + t0 + row;
    const uint32_t lane_addr = (uint32_t)(lane_group * 32) << 16;
    const float sl2 = a.scale * LOG2E;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    // The two warps that share a lane group (the two halves of 32 rows of a head) synchronise among
    // themselves on a named barrier of their own; the mbarriers they signal expect one arrival per pair.
    const bool pair_leader = half == 0 && lane == 0;
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(2 + tile * 4 + lane_group) : "memory"); };
    const uint32_t my_p_full = p_full + 16 * tile, my_pv_done = pv_done + 8 * tile;

    for (int j = 0; j < n_tiles && ok; ++j) {
      const int b = j & 1, st = j % NST;
      if (!mbar_wait(s_full + 8 * b, (uint32_t)(j >> 1) & 1u, abort_ptr)) { ok = false; break; }
      tc_fence_after();
      // Two passes over this thread's 32 scores, 16 at a time, to keep few registers live: the
      // maximum first, then (after the exchange with the other half of the row) the exponentials.
      const uint32_t s_addr = tmem_base + lane_addr + S_COL(tile, b) + half * 32;
      const int kbase = j * BNK + half * 32;
      const bool all_visible = kbase + 31 <= pos;
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 32; c += 16) {
        float s[16];
        tmem_ld16(s_addr + c, s);
#pragma unroll
        for (int i = 0; i < 16; ++i) mx = fmaxf(mx, (all_visible || kbase + c + i <= pos) ? s[i] : -INFINITY);
      }
      row_max[tile][half][row] = mx * sl2;   // sl2 > 0: the maximum of the scaled scores
      pair_sync();                            // maxima exchanged
      const float m_tile = fmaxf(row_max[tile][0][row], row_max[tile][1][row]);    // finite: key 0 is visible to every row
      // Raise the maximum this row's P is taken against only when it is exceeded by a wide margin;
      // what O holds for the row was taken against the old one and is scaled down first.  The
      // tensor-memory accesses are warp-wide, so the warp goes through them together whenever
      // one of its rows needs it (the others scale by 1); the partner warp sees the same rows.
      const bool need = m_tile > m_used + RESCALE_THRESHOLD;
      const float alpha = need ? exp2f(m_used - m_tile) : 1.f;
      if (j > 0 && __any_sync(0xffffffffu, need)) {
        if (!mbar_wait(my_pv_done, (uint32_t)(j - 1) & 1u, abort_ptr)) { ok = false; break; }
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < D / 2; c += 16) {
          float v[16];
          tmem_ld16(tmem_base + lane_addr + O_COL(tile) + half * (D / 2) + c, v);
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] *= alpha;
          tmem_st16(tmem_base + lane_addr + O_COL(tile) + half * (D / 2) + c, v);
        }
      }
      if (need) { l *= alpha; m_used = m_tile; }
      // P_j: row `row`, keys half*32 .. +31 = 16-byte chunks half*4 .. +3 of the 128-byte row, swizzled.
      // The first head writes over K_j (both heads' S_j have consumed it), the second into its own buffer.
      uint8_t* prow = (tile == 0 ? kv_smem + (size_t)st * STAGE_BYTES : p1_smem + b * P_BYTES) + row * 128;
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 32; c += 16) {
        float s[16];
        tmem_ld16(s_addr + c, s);
        uint32_t packed[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const bool v0 = all_visible || kbase + c + 2 * i <= pos, v1 = all_visible || kbase + c + 2 * i + 1 <= pos;
          const float p0 = v0 ? fast_exp2(fmaf(s[2 * i], sl2, -m_used)) : 0.f;
          const float p1 = v1 ? fast_exp2(fmaf(s[2 * i + 1], sl2, -m_used)) : 0.f;
          sum += p0 + p1;
          __nv_bfloat162 pr = __floats2bfloat162_rn(p0, p1);
          packed[i] = *(uint32_t*)&pr;
        }
        const int chunk0 = (half * 4 + c / 8) ^ (row & 7), chunk1 = (half * 4 + c / 8 + 1) ^ (row & 7);
        *(uint4*)(prow + chunk0 * 16) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        *(uint4*)(prow + chunk1 * 16) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
      }
      l += sum;
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // P visible to the tensor core's reads
      // A parity wait tells two phases apart, no more.  Page j-1's product cannot have been followed by
      // page j's yet (that one needs this pair's P_j), so here its phase is the current or the last
      // one; seen complete here, it keeps every later wait on this barrier (the next page's rescale,
      // the output's) within one phase of the barrier's state, however far the pairs drift apart.
      if (j > 0 && !mbar_wait(my_pv_done, (uint32_t)(j - 1) & 1u, abort_ptr)) { ok = false; break; }
      tc_fence_before();
      pair_sync();                            // both halves have read S_j for the last time and written P_j
      if (pair_leader) { mbar_arrive(s_empty + 8 * b); mbar_arrive(my_p_full + 8 * b); }
    }
    if (ok && !mbar_wait(my_pv_done, (uint32_t)(n_tiles - 1) & 1u, abort_ptr)) ok = false;
    tc_fence_after();
    if (!ok && lane == 0) atomicCAS(a.status, 0, ATT_ERR_SOFTMAX);
    // total row sum = the two halves' sums (both taken against the same maxima)
    row_max[tile][half][row] = l;
    pair_sync();
    const float total = row_max[tile][0][row] + row_max[tile][1][row];
    if (ok) {
      const float inv = total > 0.f ? 1.f / total : 0.f;
      bf16* dst = a.out + ((size_t)(q_begin + t0 + row) * a.nq + head) * D + half * (D / 2);
#pragma unroll 1
      for (int c = 0; c < D / 2; c += 16) {
        float v[16];
        tmem_ld16(tmem_base + lane_addr + O_COL(tile) + half * (D / 2) + c, v);     // every thread of the warp loads
        if (row < nt) {
#pragma unroll
          for (int i = 0; i < 16; i += 8) {
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              __nv_bfloat162 pr = __floats2bfloat162_rn(v[i + 2 * k] * inv, v[i + 2 * k + 1] * inv);
              w[k] = *(uint32_t*)&pr;
            }
            *(uint4*)(dst + c + i) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
  }
}

// ------------------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// A [rows, cols] row-major bf16 matrix cut into boxes of box_rows x 64 with the 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, long rows, long cols, int box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (fn == nullptr) return ODI_ERR_UNSUPPORTED;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : ODI_ERR_ARGUMENT;
}

extern "C" int odi_attention_tcgen05_head_dim() { return D; }

// q [n_tokens, nq * D] bf16; k_pool, v_pool [pool_pages, nkv, 64, D] bf16; out [n_tokens, nq * D].
// heads_per_cta: 2 = two heads of a key/value group per CTA (needs an even group size), 1 = one, 0 = choose.
extern "C" int odi_attention_tcgen05(const void* q, const void* k_pool, const void* v_pool, const TcAttnArgs* args,
                                     int n_tokens, int max_q_len, long pool_pages, int heads_per_cta,
                                     cudaStream_t stream) {
  TcAttnArgs a = *args;
  if (a.n_seqs <= 0 || n_tokens <= 0) return 0;
  if (a.nq % a.nkv != 0 || a.n_seqs > 65535 || a.nq > 65535 || a.status == nullptr) return ODI_ERR_UNSUPPORTED;
  if (((uintptr_t)q & 15) || ((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15) || ((uintptr_t)a.out & 15))
    return ODI_ERR_UNSUPPORTED;
  if (pool_pages * a.nkv * BNK > 0x7fffffffL) return ODI_ERR_UNSUPPORTED;    // row coordinates are 32-bit
  CUtensorMap mq, mk, mv;
  int rc = make_map(&mq, q, n_tokens, (long)a.nq * D, BM);
  if (rc == 0) rc = make_map(&mk, k_pool, pool_pages * a.nkv * BNK, D, BNK);
  if (rc == 0) rc = make_map(&mv, v_pool, pool_pages * a.nkv * BNK, D, BNK);
  if (rc != 0) return rc;
  static bool configured = false;
  const int smem1 = Q_BYTES + NST * STAGE_BYTES + 1024;
  const int smem2 = 2 * Q_BYTES + NST * STAGE_BYTES + 2 * P_BYTES + 1024;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem1);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_tcgen05_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  if (heads_per_cta == 2 && (a.nq / a.nkv) % 2 != 0) return ODI_ERR_ARGUMENT;
  if ((max_q_len + BM - 1) / BM > 65535) return ODI_ERR_UNSUPPORTED;
  if (heads_per_cta == 0) heads_per_cta = ODI_ATT_DEFAULT_HEADS_PER_CTA;
  if (heads_per_cta == 2 && (a.nq / a.nkv) % 2 == 0) {
    dim3 grid(a.nq / 2, a.n_seqs, (max_q_len + BM - 1) / BM);
    odi_rc = launch_pdl((attention_tcgen05_kernel<2>), dim3(grid), dim3(64 + 512), smem2, stream, mq, mk, mv, a);
  } else {
    dim3 grid(a.nq, a.n_seqs, (max_q_len + BM - 1) / BM);
    odi_rc = launch_pdl((attention_tcgen05_kernel<1>), dim3(grid), dim3(64 + 256), smem1, stream, mq, mk, mv, a);
  }
  return launch_status();
}
