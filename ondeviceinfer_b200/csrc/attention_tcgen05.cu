// bf16 causal grouped-query attention for prefill on the 5th-generation tensor cores.
//
// One CTA owns 128 consecutive query tokens of one sequence for one query head (optionally two
// heads that share a key/value head) and walks that sequence's key/value pages (64 positions
// each) up to the diagonal.  Per head:
//
//   S_j = Q K_j^T        tcgen05.mma, M = 128 query rows, N = 64 keys, K = head size; Q and K_j
//                        in shared memory (TMA, 128-byte swizzle), S_j in tensor memory
//   P_j = softmax part   by 4 warps, a thread per query row: it reads its row's 64 scores into
//                        registers, keeps an fp32 running maximum and sum, and writes P_j (pairs of
//                        bf16, 32 columns) over the first half of those scores' columns
//   O  += P_j V_j        tcgen05.mma with the A operand (P_j) read from tensor memory; V_j is read as
//                        it lies in its page (MN-major operand); O accumulates in tensor memory
//
// The accumulator in tensor memory cannot be scaled by the MMA, so the running maximum that P is
// taken against is only raised when a row's new maximum exceeds it by more than 2^8: then that
// row of O is read, scaled and written back (tcgen05.ld / st) before the row's next product is
// issued.  P stays below 2^8, which bf16 and the fp32 accumulator hold without loss, and the
// result is the same as with a maximum that is raised every time.
//
// Per head S is double buffered in tensor memory (2 x 64 columns) and O takes head-size columns:
// 256 columns a head.  Shared memory holds Q and two rings of two K and two V pages with lives of
// their own: a K slot is free once its scores are computed, so the keys of page j + 2 are on their
// way while page j is still in the softmax; a V slot once its product has run.  The tensor pipe
// executes one thread's MMAs in order, so the scores of page j + 2, issued after the product of
// page j, cannot overwrite P_j before it has been read.  With one head per CTA (the default) a CTA
// takes 97 KB of shared memory, 256 columns and 127 registers a thread, so two CTAs share an SM and
// one's MMAs run under the other's softmax.  Query tiles are handed out longest first.  Measured
// on B200: 882 TFLOP/s at 8 sequences of 2,048 tokens, 1,128 at one of 8,192, 1,047 at one of 32,768
// (32 query / 8 key-value heads of 128).  The form this replaced kept P in shared memory (written
// swizzled over the consumed K tile, two threads per row): 578 / 719 TFLOP/s; its K slot stayed
// busy until the product, and the MMA thread spent 40 % of a page's time waiting for the next keys.
// Two heads of a key/value group per CTA (K/V pages loaded once for both) measured slower
// (676 / 823) and stays an option; so did a form with two heads per CTA and keys in blocks of two
// pages (scores as N = 128 products into a single buffer per head: 700 / 856 issued in a fixed
// order, 628 / 746 with the MMA thread issuing whichever head was ready): a trace showed its MMA
// thread blocked on issue for more than half of a block's time, the N = 128 products taking about
// 125 cycles each and the P V products about 190, twice what they take when two CTAs share the SM.  Warps: 0 = TMA producer, 1 = MMA issuer (one thread) and
// tensor-memory owner, 2..5 = softmax and output of the first head, 6..9 = of the second.
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
#define RING 2                 // K pages, and V pages, in flight
#define Q_BYTES (KB * BM * 128)
#define KV_BYTES (KB * BNK * 128)     // one of K or V for a page
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

// 64 consecutive columns of this thread's lane (a whole row of scores): two loads in flight, one wait.
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float* v) {
  uint32_t r[64];
#pragma unroll
  for (int h = 0; h < 2; ++h)
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[32 * h + 0]), "=r"(r[32 * h + 1]), "=r"(r[32 * h + 2]), "=r"(r[32 * h + 3]), "=r"(r[32 * h + 4]),
          "=r"(r[32 * h + 5]), "=r"(r[32 * h + 6]), "=r"(r[32 * h + 7]), "=r"(r[32 * h + 8]), "=r"(r[32 * h + 9]),
          "=r"(r[32 * h + 10]), "=r"(r[32 * h + 11]), "=r"(r[32 * h + 12]), "=r"(r[32 * h + 13]), "=r"(r[32 * h + 14]),
          "=r"(r[32 * h + 15]), "=r"(r[32 * h + 16]), "=r"(r[32 * h + 17]), "=r"(r[32 * h + 18]), "=r"(r[32 * h + 19]),
          "=r"(r[32 * h + 20]), "=r"(r[32 * h + 21]), "=r"(r[32 * h + 22]), "=r"(r[32 * h + 23]), "=r"(r[32 * h + 24]),
          "=r"(r[32 * h + 25]), "=r"(r[32 * h + 26]), "=r"(r[32 * h + 27]), "=r"(r[32 * h + 28]), "=r"(r[32 * h + 29]),
          "=r"(r[32 * h + 30]), "=r"(r[32 * h + 31])
        : "r"(taddr + 32 * h));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
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


// 32 columns of packed values (two bf16 each) into this thread's lane.
__device__ __forceinline__ void tmem_st32_packed(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
        "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
        "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// D += A B with A (M x 16, K-major, two bf16 per 32-bit column) read from tensor memory.
__device__ __forceinline__ void umma_a_tmem(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// One query row, 64 keys: the row's scores at s_addr (tensor memory, this thread's lane) become P (bf16
// pairs, 32 columns at p_addr) against the row's running maximum; n counts this head's PV products
// (the one that will read this P is product n), kbase is the first key's position.  Returns false if a
// wait gave up.  The caller signals P afterwards.
struct RowState { float m_used, l; };
__device__ __forceinline__ bool softmax_keys64(uint32_t s_addr, uint32_t p_addr, uint32_t o_addr, int kbase, int pos, float sl2,
                                               int n, uint32_t pv_done, RowState& st, volatile int* abort_ptr) {
  float s[BNK];
  tmem_ld64(s_addr, s);
  float mx = -INFINITY;
  if (kbase + BNK - 1 <= pos) {
#pragma unroll
    for (int i = 0; i < BNK; ++i) mx = fmaxf(mx, s[i]);
  } else {
#pragma unroll
    for (int i = 0; i < BNK; ++i) { if (kbase + i > pos) s[i] = -INFINITY; mx = fmaxf(mx, s[i]); }
  }
  // Raise the maximum this row's P is taken against only when it is exceeded by a wide margin;
  // what O holds for the row was taken against the old one and is scaled down first.  The
  // tensor-memory accesses are warp-wide, so the warp goes through them together whenever
  // one of its rows needs it (the others scale by 1).  A row that sees none of these keys
  // (mx = -inf) needs nothing and gets P = 0.
  const float m_tile = mx * sl2;                 // sl2 > 0
  const bool need = m_tile > st.m_used + RESCALE_THRESHOLD;
  const float alpha = need ? exp2f(st.m_used - m_tile) : 1.f;
  if (n > 0 && __any_sync(0xffffffffu, need)) {
    if (!mbar_wait(pv_done, (uint32_t)(n - 1) & 1u, abort_ptr)) return false;
    tc_fence_after();
#pragma unroll 1
    for (int c = 0; c < D; c += 32) {
      float v[32];
      tmem_ld32(o_addr + c, v);
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] *= alpha;
      tmem_st32(o_addr + c, v);
    }
  }
  if (need) { st.l *= alpha; st.m_used = m_tile; }
  uint32_t packed[BNK / 2];                      // masked scores are -inf: exp2 gives 0
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < BNK / 2; ++i) {
    const float p0 = fast_exp2(fmaf(s[2 * i], sl2, -st.m_used));
    const float p1 = fast_exp2(fmaf(s[2 * i + 1], sl2, -st.m_used));
    sum += p0 + p1;
    __nv_bfloat162 pr = __floats2bfloat162_rn(p0, p1);
    packed[i] = *(uint32_t*)&pr;
  }
  st.l += sum;
  tmem_st32_packed(p_addr, packed);
  // A parity wait tells two phases apart, no more.  Product n-1 cannot have been followed by product n
  // yet (that one needs this warp's P), so here its phase is the current or the last one; seen complete
  // here, it keeps every later wait on this barrier within one phase of its state.
  if (n > 0 && !mbar_wait(pv_done, (uint32_t)(n - 1) & 1u, abort_ptr)) return false;
  return true;
}

// The finished row of O, divided by the row's sum, as bf16 to dst (D elements).
__device__ __forceinline__ void write_row(uint32_t o_addr, bf16* dst, float l, bool valid) {
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll 1
  for (int c = 0; c < D; c += 32) {
    float v[32];
    tmem_ld32(o_addr + c, v);                    // every thread of the warp loads
    if (valid) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
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

template <int TILES>
__global__ void __launch_bounds__(64 + 128 * TILES, TILES == 1 ? 2 : 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const TcAttnArgs a) {
  constexpr int TMEM_COLS = TILES * HEAD_COLS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  // barriers: q_full, k_full[R], k_empty[R], v_full[R], v_empty[R], s_full[2], p_full[TILES][2], pv_done[TILES]
  __shared__ __align__(8) uint64_t bars[1 + 4 * RING + 2 + 3 * TILES];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heads along x, sequences along y, query tiles along z from the last (the most keys) to the first
  const int seq = blockIdx.y, head0 = blockIdx.x * TILES, hk = head0 / (a.nq / a.nkv);
  const int q_begin = a.cu_q[seq], q_len = a.cu_q[seq + 1] - q_begin;
  const int t0 = (gridDim.z - 1 - blockIdx.z) * BM;
  if (t0 >= q_len) return;                       // whole CTA: nothing allocated yet
  const int past = a.past[seq];
  const int nt = min(BM, q_len - t0);
  const int n_tiles = (past + t0 + nt + BNK - 1) / BNK;
  const int* pages = a.page_ids + a.page_start[seq];

  const uint32_t bar0 = smem_u32(&bars[0]);
  const uint32_t q_full = bar0, k_full = bar0 + 8, k_empty = k_full + 8 * RING, v_full = k_empty + 8 * RING,
                 v_empty = v_full + 8 * RING, s_full = v_empty + 8 * RING, p_full = s_full + 16,
                 pv_done = p_full + 16 * TILES;
  uint8_t* q_smem = smem;                                    // head t at t * Q_BYTES
  uint8_t* k_smem = smem + TILES * Q_BYTES;                  // ring of K pages
  uint8_t* v_smem = k_smem + RING * KV_BYTES;             // ring of V pages

  if (threadIdx.x == 0) {
    for (int i = 0; i < 1 + 4 * RING + 2 + 3 * TILES; ++i) mbar_init(bar0 + 8 * i, 1);
    for (int b = 0; b < 2; ++b)
      for (int t = 0; t < TILES; ++t) mbar_init(p_full + 16 * t + 8 * b, 4);     // one arrival per softmax warp
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
    // ---------------------------------------------------------------- TMA producer: K_0, K_1, V_0, then K_j, V_{j-1}
    if (lane == 0) {
      pdl_wait();      // queries and this step's keys/values come from the kernel before
      mbar_expect_tx(q_full, TILES * Q_BYTES);
      for (int t = 0; t < TILES; ++t)
        for (int kb = 0; kb < KB; ++kb)
          tma_load_2d(smem_u32(q_smem + t * Q_BYTES + kb * BM * 128), &map_q, (head0 + t) * D + kb * 64, q_begin + t0, q_full);
      bool ok = true;
      auto load_page = [&](int j, const CUtensorMap* map, uint8_t* ring, uint32_t full, uint32_t empty) {
        const int s = j % RING;
        if (!mbar_wait(empty + 8 * s, ((uint32_t)(j / RING) & 1u) ^ 1u, abort_ptr)) { ok = false; return; }
        const int row = (pages[j] * a.nkv + hk) * BNK;
        mbar_expect_tx(full + 8 * s, KV_BYTES);
        for (int kb = 0; kb < KB; ++kb)
          tma_load_2d(smem_u32(ring + (size_t)s * KV_BYTES + kb * BNK * 128), map, kb * 64, row, full + 8 * s);
      };
      // keys run one page ahead of values: a K slot is free as soon as its scores are computed
      load_page(0, &map_k, k_smem, k_full, k_empty);
      for (int j = 1; j <= n_tiles && ok; ++j) {
        if (j < n_tiles) load_page(j, &map_k, k_smem, k_full, k_empty);
        if (ok) load_page(j - 1, &map_v, v_smem, v_full, v_empty);
      }
      if (!ok) atomicCAS(a.status, 0, ATT_ERR_PRODUCER);
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc_bf16(BM, BNK, false);
      constexpr uint32_t idesc_o = idesc_bf16(BM, D, true);
      bool ok = mbar_wait(q_full, 0, abort_ptr);
      auto issue_s = [&](int j) -> bool {
        const int s = j % RING, b = j & 1;
        if (!mbar_wait(k_full + 8 * s, (uint32_t)(j / RING) & 1u, abort_ptr)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(k_smem + (size_t)s * KV_BYTES);
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
        umma_commit(s_full + 8 * b);       // the scores are done ...
        umma_commit(k_empty + 8 * s);      // ... and the K slot is free
        return true;
      };
      // S_{j+1} overwrites the buffer whose first columns held P_{j-1}: it is issued after the product of
      // page j - 1, and the softmax threads read S_{j-1} before they signalled P_{j-1}.
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_s(j + 1);      // the next page's scores run under this page's softmax
        if (!ok) break;
        const int s = j % RING, b = j & 1;
        if (!mbar_wait(v_full + 8 * s, (uint32_t)(j / RING) & 1u, abort_ptr)) { ok = false; break; }
        const uint64_t dv = desc_mn_major(smem_u32(v_smem + (size_t)s * KV_BYTES));
#pragma unroll
        for (int t = 0; t < TILES; ++t) {
          if (!mbar_wait(p_full + 16 * t + 8 * b, (uint32_t)(j >> 1) & 1u, abort_ptr)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int i = 0; i < 4; ++i)      // 16 keys per MMA: 8 columns of packed P, 16 rows (2048 bytes) down V
            umma_a_tmem(tmem_base + O_COL(t), tmem_base + S_COL(t, b) + 8 * i, dv + (uint64_t)(i * 2048 >> 4), idesc_o,
                        (j | i) ? 1u : 0u);
          umma_commit(pv_done + 8 * t);
        }
        umma_commit(v_empty + 8 * s);
      }
      if (!ok) atomicCAS(a.status, 0, ATT_ERR_MMA);
    }
  } else {
    // ---------------------------------------------------------------- softmax and output (4 warps a head, a thread a row)
    const int tile = (warp - 2) >> 2;                // which of the CTA's heads
    const int head = head0 + tile;
    const int lane_group = warp & 3;                 // the tensor-memory lanes this warp may read
    const int row = lane_group * 32 + lane;          // query row inside the tile
    const int pos = past + t0 + row;
    const uint32_t lane_addr = (uint32_t)(lane_group * 32) << 16;
    const float sl2 = a.scale * LOG2E;
    RowState st = {-INFINITY, 0.f};
    bool ok = true;
    const uint32_t my_p_full = p_full + 16 * tile, my_pv_done = pv_done + 8 * tile;
    const uint32_t o_addr = tmem_base + lane_addr + O_COL(tile);

    for (int j = 0; j < n_tiles && ok; ++j) {
      const int b = j & 1;
      if (!mbar_wait(s_full + 8 * b, (uint32_t)(j >> 1) & 1u, abort_ptr)) { ok = false; break; }
      tc_fence_after();
      const uint32_t s_addr = tmem_base + lane_addr + S_COL(tile, b);
      // P_j goes over the first 32 columns of this row's scores
      if (!softmax_keys64(s_addr, s_addr, o_addr, j * BNK, pos, sl2, j, my_pv_done, st, abort_ptr)) { ok = false; break; }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(my_p_full + 8 * b);
    }
    if (ok && !mbar_wait(my_pv_done, (uint32_t)(n_tiles - 1) & 1u, abort_ptr)) ok = false;
    tc_fence_after();
    if (!ok && lane == 0) atomicCAS(a.status, 0, ATT_ERR_SOFTMAX);
    if (ok) write_row(o_addr, a.out + ((size_t)(q_begin + t0 + row) * a.nq + head) * D, st.l, row < nt);
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
template <int TILES>
static int launch_attention(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const TcAttnArgs& a,
                            int max_q_len, cudaStream_t stream) {
  const int smem = TILES * Q_BYTES + 2 * RING * KV_BYTES + 1024;
  auto kernel = attention_tcgen05_kernel<TILES>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(a.nq / TILES, a.n_seqs, (max_q_len + BM - 1) / BM);
  odi_rc = launch_pdl((kernel), dim3(grid), dim3(64 + 128 * TILES), smem, stream, mq, mk, mv, a);
  return launch_status();
}

extern "C" int odi_attention_tcgen05(const void* q, const void* k_pool, const void* v_pool, const TcAttnArgs* args,
                                     int n_tokens, int max_q_len, long pool_pages, int heads_per_cta,
                                     cudaStream_t stream) {
  TcAttnArgs a = *args;
  if (a.n_seqs <= 0 || n_tokens <= 0) return 0;
  if (a.nq % a.nkv != 0 || a.n_seqs > 65535 || a.nq > 65535 || a.status == nullptr) return ODI_ERR_UNSUPPORTED;
  if (((uintptr_t)q & 15) || ((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15) || ((uintptr_t)a.out & 15))
    return ODI_ERR_UNSUPPORTED;
  if (pool_pages * a.nkv * BNK > 0x7fffffffL) return ODI_ERR_UNSUPPORTED;    // row coordinates are 32-bit
  if ((max_q_len + BM - 1) / BM > 65535) return ODI_ERR_UNSUPPORTED;
  if (heads_per_cta < 0 || heads_per_cta > 2) return ODI_ERR_ARGUMENT;
  if (heads_per_cta == 2 && (a.nq / a.nkv) % 2 != 0) return ODI_ERR_ARGUMENT;
  CUtensorMap mq, mk, mv;
  int rc = make_map(&mq, q, n_tokens, (long)a.nq * D, BM);
  if (rc == 0) rc = make_map(&mk, k_pool, pool_pages * a.nkv * BNK, D, BNK);
  if (rc == 0) rc = make_map(&mv, v_pool, pool_pages * a.nkv * BNK, D, BNK);
  if (rc != 0) return rc;
  if (heads_per_cta == 0) heads_per_cta = ODI_ATT_DEFAULT_HEADS_PER_CTA;
  return heads_per_cta == 2 ? launch_attention<2>(mq, mk, mv, a, max_q_len, stream)
                            : launch_attention<1>(mq, mk, mv, a, max_q_len, stream);
}
