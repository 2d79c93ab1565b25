// bf16 matrix product on the 5th-generation tensor cores of sm_100a:
//
//     out[token, n] = sum_k X[token, k] * W[n, k]        (X and W row-major, K contiguous)
//
// with fp32 accumulation in tensor memory, for few tokens (decode, short chunks): a tile is 128 output
// features on the lanes of the accumulator and BN = 16..256 tokens on its columns, so a step streams each
// weight once at HBM speed whatever the number of tokens.  (Many tokens: gemm_prefill_tcgen05.cu.)
//
// One CTA = one (feature tile, token tile, K split).  Six warps:
//   warp 0   TMA producer: cp.async.bulk.tensor loads of W and X tiles (64 k per stage,
//            128-byte swizzle) into a ring of shared-memory stages, completion on mbarriers;
//   warp 1   allocates tensor memory; one thread issues tcgen05.mma (M=128, N=BN, K=16, four
//            per stage) and tcgen05.commit, which releases stages and finally signals the epilogue;
//   warps 2-5 epilogue: tcgen05.ld the accumulators (one feature row per thread, 16 tokens
//            at a time) and write the result.
// DUAL mode runs two weight tiles (rows n and n + dual_offset: gate and up) against the
// same X tile into two accumulators and writes silu(gate) * up.
//
// K splits: when there are too few tiles to fill the GPU, grid.z CTAs share a tile.
//  * Up to 8 splits form a thread-block cluster: every CTA leaves its fp32 partial in its own
//    shared memory, the cluster synchronises, and CTA r adds, for the token columns it owns, the
//    partials of all CTAs in rank order through distributed shared memory and runs the epilogue.
//  * More splits: each CTA writes its partial to global scratch; the CTA that arrives last (an
//    atomic ticket, nobody waits) adds the partials in split order and runs the epilogue.
// Either way the sum is taken in a fixed order and does not depend on timing.
//
// Every wait on an mbarrier is bounded: after about two seconds the kernel records an
// error code in `status`, skips its work, still frees its tensor memory and returns.
#include <cuda.h>

#include "common.cuh"

#define EPI_STORE_BF16 0   // out_bf16[token, n] = acc
#define EPI_STORE_F32 1    // out_f32[token, n] = acc
#define EPI_RESIDUAL 2     // out_f32[token, n] += acc
#define EPI_SWIGLU 3       // out_bf16[token, n] = silu(acc_gate) * acc_up   (DUAL)
#define EPI_HEAD_PREP 4    // the rows are q, k and v heads of 128: per-head norm, rotation, cache write

#define BM 128             // features per tile (UMMA M)
#define BK 64              // k per stage: 64 bf16 = one 128-byte swizzle row
#define GEMM_THREADS 192
#ifndef ODI_WAIT_CYCLES
#define ODI_WAIT_CYCLES 4000000000ll   // about two seconds of SM clock; a self-test build makes it milliseconds
#endif
#define WAIT_CYCLES ((long long)ODI_WAIT_CYCLES)

#define GEMM_ERR_TIMEOUT_PRODUCER 1
#define GEMM_ERR_TIMEOUT_MMA 2
#define GEMM_ERR_TIMEOUT_EPILOGUE 3

struct GemmArgs {
  void* out;
  float* scratch;          // split partials
  int* tickets;            // one counter per tile, zero on entry, left zero
  int* status;             // error word, 0 = fine
  int tokens, N, K, ldo;
  int dual_offset;         // DUAL: row distance between the two weight tiles
  int splits;
  // NORM: the activation operand is rmsnorm(norm_x) * norm_w, made on the fly from the
  // fp32 rows norm_x [tokens, K]; a row's sum of squares is the sum of its norm_n_parts pieces in
  // norm_parts [norm_n_parts, tokens].
  const float* norm_x;
  const float* norm_w;
  const float* norm_parts;
  int norm_n_parts;
  float norm_eps;
  // EPI_RESIDUAL: when not null, the sums of squares of the rows it leaves, one piece
  // per tile of 128 features: sumsq_out [ceil(N / 128), tokens].
  float* sumsq_out;
  // When not null: bias [weight rows], added to the finished product (after the K splits are summed) before
  // anything else the epilogue does with it.
  const float* bias;
  // Self-test of the bounded waits: when set, the producer announces and requests nothing, so no copy is ever
  // in flight and the MMA role's first wait runs out; the kernel must record that, free its tensor memory and
  // return.  Never set on the product path.
  int no_loads;
  // EPI_HEAD_PREP: a tile of 128 features is one head (query heads, then key heads, then value heads);
  // what the stand-alone head preparation would do with the bf16 projections happens in the epilogue.
  HeadPrepArgs hp;
  // PRO_MERGE: the activation operand is the output of a decode attention whose key splits are still apart
  // (K = mg.nq * mg.d); merge_kb_cap = the most k-blocks that one CTA of this launch takes.
  MergeArgs mg;
  int merge_kb_cap;
};

#define PRO_NONE 0
#define PRO_NORM 1         // the operand is made from fp32 rows by RMSNorm
#define PRO_MERGE 2        // the operand is made from the split partials of a decode attention

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
// Bounded wait.  Returns false when it gave up or when another role already gave up.  The role whose own wait
// ran out records its code in `status` before it raises the abort flag, so the word names the role that
// waited in vain and not one that merely left after it.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  const long long start = clock64();
  for (uint32_t i = 0;; ++i) {
    if (mbar_test(bar, parity)) return true;
    // try_wait suspends the thread for a bounded, implementation-defined time instead of spinning
    if ((i & 0xf) == 0xf) {
      if (*abort_flag) return false;
      if (clock64() - start > WAIT_CYCLES) break;
    }
  }
  atomicCAS(status, 0, code);
  __threadfence_block();
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols));
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols));
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
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

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Read a float from the same shared-memory offset in the CTA of the given cluster rank.
__device__ __forceinline__ float ld_peer_f32(const float* local, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, written by TMA
// with the 128-byte swizzle: 8-row groups are 1024 bytes apart (stride byte offset), the
// leading byte offset is not used by swizzled K-major layouts, version 1, layout type 2.
__device__ __forceinline__ uint64_t smem_desc_k_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3ffff) >> 4);     // start address, bits [0, 14)
  d |= (uint64_t)1 << 16;                      // leading byte offset (ignored), bits [16, 30)
  d |= (uint64_t)(1024 >> 4) << 32;            // stride byte offset, bits [32, 46)
  d |= (uint64_t)1 << 46;                      // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                      // SWIZZLE_128B
  return d;
}

// Instruction descriptor of kind::f16: fp32 accumulator, bf16 A and B, both K-major.
__host__ __device__ constexpr uint32_t instr_desc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ float silu_f(float g) { return g / (1.f + __expf(-g)); }

// One warp finishes one head of one token: `vals` holds the head's 128 projections (already rounded
// to bf16), lane i takes elements 4i .. 4i+3, whose rotation partners sit in lane i ^ 16.  The
// arithmetic, its order and its roundings are those of head_prep_vec_kernel<4> (elementwise.cu).
// `pos` and `page` (the token's position and, for key and value heads, the cache page that holds it) come from
// head_prep_lookup, which the warp ran long before: the three dependent index loads do not sit behind the product.
__device__ __forceinline__ void head_prep_finish(const HeadPrepArgs& hp, int t, int h, const float* vals, int lane,
                                                 int pos, int page) {
  constexpr int d = 128, half = 64;
  const int kind = h < hp.nq ? 0 : (h < hp.nq + hp.nkv ? 1 : 2);     // 0 q, 1 k, 2 v
  bf16* dst;
  if (kind == 0) {
    dst = (bf16*)hp.q_out + ((size_t)t * hp.nq + h) * d;
  } else {
    const int hk = kind == 1 ? h - hp.nq : h - hp.nq - hp.nkv;
    bf16* pool = (bf16*)(kind == 1 ? hp.k_pool : hp.v_pool);
    dst = pool + (((size_t)page * hp.nkv + hk) * hp.page_size + (pos % hp.page_size)) * d;
  }
  const float4 in = *(const float4*)(vals + 4 * lane);
  float x[4] = {in.x, in.y, in.z, in.w};
  if (kind != 2) {
    const float* w = kind == 0 ? hp.q_norm_w : hp.k_norm_w;
    if (w != nullptr) {
      float ss = 0.f;
#pragma unroll
      for (int r = 0; r < 4; ++r) ss += x[r] * x[r];
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / (float)d + hp.eps);
#pragma unroll
      for (int r = 0; r < 4; ++r) x[r] = round_to<bf16>(w[4 * lane + r] * round_to<bf16>(x[r] * inv));
    }
    if (hp.cos_t != nullptr) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int i = 4 * lane + r, f = i < half ? i : i - half;
        const float cs = hp.cos_t[(size_t)t * half + f], sn = hp.sin_t[(size_t)t * half + f];
        const float partner = __shfl_xor_sync(0xffffffffu, x[r], 16);
        x[r] = x[r] * cs + (i < half ? -partner : partner) * sn;
      }
    }
  }
  __nv_bfloat162 lo = __floats2bfloat162_rn(x[0], x[1]), hi = __floats2bfloat162_rn(x[2], x[3]);
  *(uint2*)(dst + 4 * lane) = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
}

// Position and cache page of token t for head h (the page only for key and value heads).  The step's index arrays
// are written by the host, or by the sampling kernel of the step before: nothing of this step, so they may be
// read before the dependency wait.
__device__ __forceinline__ void head_prep_lookup(const HeadPrepArgs& hp, int t, int h, int& pos, int& page) {
  pos = hp.tok_pos[t];
  page = 0;
  if (h >= hp.nq) page = hp.page_ids[hp.page_start[hp.tok_seq[t]] + page_slot_of(pos, hp.page_size, hp.ring_pages)];
}

// ------------------------------------------------------------------------------ the kernel

// Features on the lanes: one value per call; the 32 lanes of a warp write 32
// consecutive features of one token.
// Returns what it left in `out` for EPI_RESIDUAL (0 outside the matrix), else 0.
template <int EPI>
__device__ __forceinline__ float emit(const GemmArgs& a, int token, int n, float v, float v2) {
  if (token >= a.tokens || n >= a.N) return 0.f;
  const size_t at = (size_t)token * a.ldo + n;
  if (EPI == EPI_STORE_BF16) ((bf16*)a.out)[at] = __float2bfloat16_rn(v);
  else if (EPI == EPI_STORE_F32) ((float*)a.out)[at] = v;
  else if (EPI == EPI_RESIDUAL) { const float r = ((float*)a.out)[at] + v; ((float*)a.out)[at] = r; return r; }
  else if (EPI == EPI_SWIGLU) ((bf16*)a.out)[at] = __float2bfloat16_rn(silu_f(v) * v2);
  return 0.f;
}


// The 128 lanes of the accumulator are features (weight rows), its BN columns are tokens.
// PRO_NORM: the four epilogue warps first serve as converters: for every k-block they
// read the fp32 rows, scale them by the row's 1/rms and the norm weight with the roundings of the
// stand-alone RMSNorm kernel, and write the bf16 operand tile in the swizzled layout that TMA would
// have produced; the MMA thread waits for them (`ready`) as well as for the weight tile (`full`).
// PRO_MERGE: the converters build the operand tiles of all the CTA's k-blocks at once, behind the ring of
// weight stages, from the split partials of the decode attention before (what its combine kernel would
// have rounded to bf16, bit for bit); the MMA thread waits for all of them before its first product.
template <int BN, bool DUAL, int EPI, int STAGES, bool CLUSTER, int PRO>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const GemmArgs a) {
  constexpr int L_BYTES = BM * BK * 2;                    // lanes operand tile, 16 KB
  constexpr int C_BYTES = BN * BK * 2;                    // columns operand tile
  constexpr int L_TILES = DUAL ? 2 : 1;                   // the gate and the up tile
  constexpr int C_TILES = 1;
  constexpr bool NORM = PRO == PRO_NORM, MERGE = PRO == PRO_MERGE;
  constexpr int STAGE_BYTES = L_BYTES * L_TILES + (MERGE ? 0 : C_BYTES * C_TILES);   // MERGE: the token tiles lie behind the ring
  constexpr int ACC_COLS = BN * (DUAL ? 2 : 1);
  constexpr int TMEM_COLS = ACC_COLS <= 32 ? 32 : (ACC_COLS <= 64 ? 64 : (ACC_COLS <= 128 ? 128 : (ACC_COLS <= 256 ? 256 : 512)));

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  static_assert(!NORM || (BN % 16 == 0 && BN <= 64), "the norm prologue takes token tiles of 16, 32 or 64");
  static_assert(!MERGE || (EPI == EPI_RESIDUAL && !DUAL && BN <= 32), "the merge prologue serves the output projection at decode widths");
  // EPI_HEAD_PREP stages the finished rows behind the split partials (which peers may still be reading)
  constexpr int HP_STAGE_OFFSET = BN * BM * 4;
  static_assert(EPI != EPI_HEAD_PREP || (!DUAL && BN <= 64 && 2 * BN * BM * 4 <= STAGES * STAGE_BYTES),
                "the head-preparation epilogue needs room behind the split partials");
  __shared__ __align__(8) uint64_t bars[3 * STAGES + 1];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int ticket_slot;
  __shared__ float sumsq_part[4][BN <= 64 ? BN : 1];    // per epilogue warp and token column

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tok0 = blockIdx.x * BN, n0 = blockIdx.y * BM, split = blockIdx.z;
  const int total_kb = (a.K + BK - 1) / BK;
  const int kb_begin = (int)((long)total_kb * split / a.splits);
  const int kb_count = (int)((long)total_kb * (split + 1) / a.splits) - kb_begin;
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]), acc_bar = smem_u32(&bars[2 * STAGES]);
  const uint32_t ready0 = smem_u32(&bars[2 * STAGES + 1]);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); mbar_init(ready0 + 8 * s, 4); }
    mbar_init(acc_bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) { tmem_alloc(smem_u32(&tmem_base_slot), TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abort_ptr = &abort_flag;
  pdl_launch_dependents();      // the next kernel may be scheduled; it waits for this grid before it reads
  int hp_pos = 0, hp_page = 0;  // EPI_HEAD_PREP, epilogue warps: what head_prep_lookup found for the lane's token column

  if (warp == 0) {
    if (lane == 0 && !a.no_loads) {
      const CUtensorMap* map_l = &map_w;       // the lanes' operand: weight rows
      const CUtensorMap* map_c = &map_x;       // the columns' operand: token rows
      const int l_row = n0, c_row = tok0;
      // Weights are never written by a kernel, so their first tiles are
      // requested before this grid waits for the kernels it depends on; only the activation
      // tiles (and everything the epilogue touches, which runs after them) come after the wait.
      constexpr uint32_t TX_BYTES = PRO != PRO_NONE ? L_BYTES * L_TILES : STAGE_BYTES;   // else the converters make the token tile
      const int pre = min(STAGES, kb_count);
      for (int i = 0; i < pre; ++i) {
        const uint32_t dst = smem_u32(smem + (size_t)i * STAGE_BYTES);
        const int k0 = (kb_begin + i) * BK;
        mbar_expect_tx(full0 + 8 * i, TX_BYTES);
        tma_load_2d(dst, map_l, k0, l_row, full0 + 8 * i);
        if (L_TILES == 2) tma_load_2d(dst + L_BYTES, map_l, k0, l_row + a.dual_offset, full0 + 8 * i);
      }
      // (Asking the rest of this CTA's weights into L2 here as well, with cp.async.bulk.prefetch.tensor, measured
      // no gain for two k-blocks beyond the ring (3.46 against 3.49 ms a step at batch 8) and a loss beyond that:
      // 3.55 with four, 3.67 with eight, 4.16 with all.)
      if (PRO == PRO_NONE) {
        pdl_wait();
        for (int i = 0; i < pre; ++i) {
          const uint32_t dst = smem_u32(smem + (size_t)i * STAGE_BYTES);
          tma_load_2d(dst + L_BYTES * L_TILES, map_c, (kb_begin + i) * BK, c_row, full0 + 8 * i);
        }
      }
      for (int i = pre; i < kb_count; ++i) {
        const int s = i % STAGES;
        const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
        if (!mbar_wait(empty0 + 8 * s, phase ^ 1u, abort_ptr, a.status, GEMM_ERR_TIMEOUT_PRODUCER)) break;
        const uint32_t dst = smem_u32(smem + (size_t)s * STAGE_BYTES);
        const int k0 = (kb_begin + i) * BK;
        mbar_expect_tx(full0 + 8 * s, TX_BYTES);
        tma_load_2d(dst, map_l, k0, l_row, full0 + 8 * s);
        if (L_TILES == 2) tma_load_2d(dst + L_BYTES, map_l, k0, l_row + a.dual_offset, full0 + 8 * s);
        if (PRO == PRO_NONE) tma_load_2d(dst + L_BYTES * L_TILES, map_c, k0, c_row, full0 + 8 * s);
        if (C_TILES == 2) tma_load_2d(dst + L_BYTES * L_TILES + C_BYTES, map_c, k0, c_row + a.dual_offset, full0 + 8 * s);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_bf16(BM, BN);
      // MERGE: every token tile of this CTA is ready at once (the first `ready` barrier)
      bool ok = !MERGE || mbar_wait(ready0, 0, abort_ptr, a.status, GEMM_ERR_TIMEOUT_MMA);
      for (int i = 0; i < kb_count && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
        if (!mbar_wait(full0 + 8 * s, phase, abort_ptr, a.status, GEMM_ERR_TIMEOUT_MMA) ||
            (NORM && !mbar_wait(ready0 + 8 * s, phase, abort_ptr, a.status, GEMM_ERR_TIMEOUT_MMA))) {
          ok = false; break;
        }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + (size_t)s * STAGE_BYTES);
        const uint64_t dl = smem_desc_k_sw128(sa);
        const uint64_t dl2 = smem_desc_k_sw128(sa + L_BYTES);
        const uint64_t dc = smem_desc_k_sw128(MERGE ? smem_u32(smem + (size_t)STAGES * STAGE_BYTES + (size_t)i * C_BYTES)
                                                    : sa + L_BYTES * L_TILES);
#pragma unroll
        for (int j = 0; j < BK / 16; ++j) {
          const uint32_t acc = (i > 0 || j > 0) ? 1u : 0u;
          // 16 k = 32 bytes further inside the swizzle row: +2 in the (address >> 4) field
          umma_bf16(tmem_base, dl + 2 * j, dc + 2 * j, idesc, acc);
          if (DUAL) umma_bf16(tmem_base + BN, dl2 + 2 * j, dc + 2 * j, idesc, acc);
        }
        umma_commit(empty0 + 8 * s);    // the stage is free once these MMAs have read it
      }
      if (ok) umma_commit(acc_bar);     // accumulators complete
    }
  } else {
    // epilogue warps 2..5 own tensor-memory lanes 32 * (warp % 4) .. + 31
    const int lane_group = warp & 3;
    const int row = lane_group * 32 + lane;              // lane of the accumulator
    const uint32_t taddr = tmem_base + ((uint32_t)(lane_group * 32) << 16);
    const int tile_id = blockIdx.y * gridDim.x + blockIdx.x;
    // EPI_HEAD_PREP: lane j looks up, now, the j-th token column that this warp will finish at the very end (one
    // split: columns lane_group, lane_group + 4, ...; a cluster: the columns this CTA owns, rank + splits * (lane_group + 4 j))
    if (EPI == EPI_HEAD_PREP) {
      const int nth = lane_group + 4 * lane;
      const int c = a.splits == 1 ? nth : (int)cluster_rank() + nth * a.splits;
      if (c < BN && tok0 + c < a.tokens) head_prep_lookup(a.hp, tok0 + c, blockIdx.y, hp_pos, hp_page);
    }
    if (NORM) {
      constexpr int ITEMS = BN / 16;                  // token rows per thread: trow, trow + 16, ...
      constexpr int WANT = ITEMS == 1 ? 4 : 2;        // k-blocks in flight per thread, as registers allow (three CTAs per SM)
      constexpr int DEPTH = STAGES < WANT ? STAGES : WANT;
      const int tid_c = threadIdx.x - 64, chunk = tid_c & 7, trow = tid_c >> 3;   // a 16-byte chunk of a 128-byte row
      struct Piece { float4 g[2]; float4 x[ITEMS][2]; };
      auto fetch_g = [&](Piece& pc, int i) {          // the norm weight: no kernel writes it
        const int k = (kb_begin + i) * BK + chunk * 8;
        const bool in = i < kb_count && k < a.K;      // K is a multiple of 8: a chunk is inside or outside
        pc.g[0] = in ? *(const float4*)(a.norm_w + k) : make_float4(0.f, 0.f, 0.f, 0.f);
        pc.g[1] = in ? *(const float4*)(a.norm_w + k + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
      };
      Piece ring[DEPTH];
#pragma unroll
      for (int j = 0; j < DEPTH; ++j) fetch_g(ring[j], j);
      pdl_wait();                                     // the rows and their sums of squares come from the kernel before
      auto fetch_x = [&](Piece& pc, int i) {
        const int k = (kb_begin + i) * BK + chunk * 8;
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
          const int token = tok0 + trow + 16 * it;
          const bool in = i < kb_count && k < a.K && token < a.tokens;
          const float* src = a.norm_x + (size_t)token * a.K + k;
          pc.x[it][0] = in ? *(const float4*)src : make_float4(0.f, 0.f, 0.f, 0.f);
          pc.x[it][1] = in ? *(const float4*)(src + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      };
#pragma unroll
      for (int j = 0; j < DEPTH; ++j) fetch_x(ring[j], j);     // in flight together with the sums below
      float rstd[ITEMS];
#pragma unroll
      for (int it = 0; it < ITEMS; ++it) {
        const int token = tok0 + trow + 16 * it;
        float ss = 0.f;
        if (token < a.tokens)
          for (int p = chunk; p < a.norm_n_parts; p += 8) ss += a.norm_parts[(size_t)p * a.tokens + token];
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);    // the eight threads of a row are neighbours in a warp
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        ss += __shfl_xor_sync(0xffffffffu, ss, 4);
        rstd[it] = rsqrtf(ss / (float)a.K + a.norm_eps);
      }
      auto norm2 = [](float x0, float x1, float g0, float g1, float r) -> uint32_t {
        // the stand-alone kernel's roundings: bf16(x / rms), then bf16(weight * that)
        const float y0 = __bfloat162float(__float2bfloat16_rn(x0 * r)), y1 = __bfloat162float(__float2bfloat16_rn(x1 * r));
        __nv_bfloat162 pr = __floats2bfloat162_rn(g0 * y0, g1 * y1);
        return *(uint32_t*)&pr;
      };
      bool conv_ok = true;
      for (int base = 0; base < kb_count && conv_ok; base += DEPTH) {
#pragma unroll
        for (int j = 0; j < DEPTH; ++j) {
          const int i = base + j;
          if (i >= kb_count) break;
          const int s = i % STAGES;
          if (i >= STAGES && !mbar_wait(empty0 + 8 * s, (((uint32_t)(i / STAGES) & 1u) ^ 1u), abort_ptr, a.status, GEMM_ERR_TIMEOUT_EPILOGUE)) { conv_ok = false; break; }
          const float4 g0 = ring[j].g[0], g1 = ring[j].g[1];
          uint8_t* tile = smem + (size_t)s * STAGE_BYTES + L_BYTES * L_TILES;
#pragma unroll
          for (int it = 0; it < ITEMS; ++it) {
            const int r = trow + 16 * it;
            const float4 x0 = ring[j].x[it][0], x1 = ring[j].x[it][1];
            const uint4 packed = make_uint4(norm2(x0.x, x0.y, g0.x, g0.y, rstd[it]), norm2(x0.z, x0.w, g0.z, g0.w, rstd[it]),
                                            norm2(x1.x, x1.y, g1.x, g1.y, rstd[it]), norm2(x1.z, x1.w, g1.z, g1.w, rstd[it]));
            *(uint4*)(tile + r * 128 + ((chunk ^ (r & 7)) << 4)) = packed;
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // visible to the tensor core's reads
          __syncwarp();
          if (lane == 0) mbar_arrive(ready0 + 8 * s);
          fetch_g(ring[j], i + DEPTH);                 // zeros past the end
          fetch_x(ring[j], i + DEPTH);
        }
      }
    }
    if (MERGE) {
      const MergeArgs& mg = a.mg;
      const int tid_c = threadIdx.x - 64;
      const int RS = mg.d + 2, WS = mg.splits + 2;
      const int k_begin = kb_begin * BK;                      // K is a multiple of 64 here: whole k-blocks
      const int n_chunks = kb_count * (BK / 8);               // 16-byte pieces of a token's row in this CTA's range
      const int head_begin = k_begin / mg.d;
      const int n_heads = (k_begin + kb_count * BK - 1) / mg.d - head_begin + 1;
      const int n_tok = min(BN, a.tokens - tok0);
      uint8_t* c_region = smem + (size_t)STAGES * STAGE_BYTES;
      float* wtab = (float*)(c_region + (size_t)a.merge_kb_cap * C_BYTES);   // per (token, head): weights, 1 / denominator, count
      pdl_wait();                                             // the partials come from the kernel before
      // a thread per (token, head): the weights of its splits, as the combine kernel makes them
      for (int pair = tid_c; pair < n_tok * n_heads; pair += 128) {
        const int token = tok0 + pair / n_heads, h = head_begin + pair % n_heads;
        const int used = merge_used_splits(mg.plan, mg.splits, mg.past[token]);
        const float* p = mg.partial + ((size_t)token * mg.nq + h) * mg.splits * RS + mg.d;
        float* wrow = wtab + (size_t)pair * WS;
        float M = -INFINITY;
#pragma unroll 4
        for (int s = 0; s < used; ++s) M = fmaxf(M, __ldcg(p + s * RS));
        float denom = 0.f;
#pragma unroll 4
        for (int s = 0; s < used; ++s) {
          const float ms = __ldcg(p + s * RS), ls = __ldcg(p + s * RS + 1);
          const float w = ms != -INFINITY ? expf(ms - M) : 0.f;       // an empty split (max -inf) adds nothing
          denom = __fadd_rn(denom, ms != -INFINITY ? __fmul_rn(w, ls) : 0.f);
          wrow[s] = w;
        }
        wrow[mg.splits] = denom > 0.f ? 1.f / denom : 0.f;
        wrow[mg.splits + 1] = __int_as_float(used);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");          // the four converter warps
      // a thread per (token row, 16-byte piece): the splits' values added in split order, rounded once
      for (int item = tid_c; item < BN * n_chunks; item += 128) {
        const int t = item / n_chunks, c = item % n_chunks;
        uint4 packed = make_uint4(0u, 0u, 0u, 0u);            // rows beyond the tokens are zeros
        if (t < n_tok) {
          const int k = k_begin + c * 8, h = k / mg.d, dd = k % mg.d;
          const float* wrow = wtab + (size_t)(t * n_heads + h - head_begin) * WS;
          const int used = __float_as_int(wrow[mg.splits + 1]);
          const float inv = wrow[mg.splits];
          const float* p = mg.partial + ((size_t)(tok0 + t) * mg.nq + h) * mg.splits * RS + dd;
          float v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = 0.f;
#pragma unroll 4
          for (int s = 0; s < used; ++s) {
            // rows of d + 2 floats are 8-byte aligned; whatever an empty split's slot holds is loaded but not added
            const float2* src = (const float2*)(p + (size_t)s * RS);
            const float2 x0 = __ldcg(src), x1 = __ldcg(src + 1), x2 = __ldcg(src + 2), x3 = __ldcg(src + 3);
            const float w = wrow[s];
            if (w > 0.f) {
              v[0] = __fmaf_rn(w, x0.x, v[0]); v[1] = __fmaf_rn(w, x0.y, v[1]);
              v[2] = __fmaf_rn(w, x1.x, v[2]); v[3] = __fmaf_rn(w, x1.y, v[3]);
              v[4] = __fmaf_rn(w, x2.x, v[4]); v[5] = __fmaf_rn(w, x2.y, v[5]);
              v[6] = __fmaf_rn(w, x3.x, v[6]); v[7] = __fmaf_rn(w, x3.y, v[7]);
            }
          }
          __nv_bfloat162 h0 = __floats2bfloat162_rn(__fmul_rn(v[0], inv), __fmul_rn(v[1], inv));
          __nv_bfloat162 h1 = __floats2bfloat162_rn(__fmul_rn(v[2], inv), __fmul_rn(v[3], inv));
          __nv_bfloat162 h2 = __floats2bfloat162_rn(__fmul_rn(v[4], inv), __fmul_rn(v[5], inv));
          __nv_bfloat162 h3 = __floats2bfloat162_rn(__fmul_rn(v[6], inv), __fmul_rn(v[7], inv));
          packed = make_uint4(*(uint32_t*)&h0, *(uint32_t*)&h1, *(uint32_t*)&h2, *(uint32_t*)&h3);
        }
        uint8_t* tile = c_region + (size_t)(c >> 3) * C_BYTES;
        *(uint4*)(tile + t * 128 + (((c & 7) ^ (t & 7)) << 4)) = packed;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) mbar_arrive(ready0);
    }
    bool ok = mbar_wait(acc_bar, 0, abort_ptr, a.status, GEMM_ERR_TIMEOUT_EPILOGUE);
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    tc_fence_after();
    if (ok && a.splits == 1) {
      const int n = n0 + row;
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        if (tok0 + c >= a.tokens) break;
        float v[16], u[16];
        tmem_ld16(taddr + c, v);
        if (DUAL) tmem_ld16(taddr + BN + c, u);
        if (a.bias != nullptr && n < a.N) {
          // this thread's feature row has one bias for every token (a weight: no kernel writes it)
          const float bias_v = a.bias[n], bias_u = DUAL ? a.bias[n + a.dual_offset] : 0.f;
#pragma unroll
          for (int i = 0; i < 16; ++i) { v[i] += bias_v; if (DUAL) u[i] += bias_u; }
        }
        if (EPI == EPI_RESIDUAL) {
          // read the 16 residual values first: the adds must not wait on one another
          float r[16];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            r[i] = (tok0 + c + i < a.tokens && n < a.N) ? ((const float*)a.out)[(size_t)(tok0 + c + i) * a.ldo + n] : 0.f;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const bool in = tok0 + c + i < a.tokens && n < a.N;
            const float left = in ? r[i] + v[i] : 0.f;
            if (in) ((float*)a.out)[(size_t)(tok0 + c + i) * a.ldo + n] = left;
            if (a.sumsq_out != nullptr && BN <= 64) {
              const float sq = warp_sum(left * left);
              if (lane == 0) sumsq_part[lane_group][BN <= 64 ? c + i : 0] = sq;
            }
          }
        } else if (EPI == EPI_HEAD_PREP) {
          float* stage = (float*)(smem + HP_STAGE_OFFSET);       // [token column][128]; every MMA has completed
#pragma unroll
          for (int i = 0; i < 16; ++i) stage[(c + i) * BM + row] = round_to<bf16>(v[i]);
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) emit<EPI>(a, tok0 + c + i, n, v[i], DUAL ? u[i] : 0.f);
        }
      }
    } else if (ok && CLUSTER) {
      // leave the partial in this CTA's shared memory (the stages are free: every MMA has completed)
      float* red = (float*)smem;
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        if (tok0 + c >= a.tokens) break;
        float v[16], u[16];
        tmem_ld16(taddr + c, v);
        if (DUAL) tmem_ld16(taddr + BN + c, u);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          red[(c + i) * BM + row] = v[i];
          if (DUAL) red[(BN + c + i) * BM + row] = u[i];
        }
      }
    } else if (ok) {
      const int n = n0 + row;
      constexpr int PER = (DUAL ? 2 : 1) * BN * BM;       // floats per partial
      float* mine = a.scratch + ((size_t)tile_id * a.splits + split) * PER;
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        if (tok0 + c >= a.tokens) break;
        float v[16], u[16];
        tmem_ld16(taddr + c, v);
        if (DUAL) tmem_ld16(taddr + BN + c, u);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          mine[(size_t)(c + i) * BM + row] = v[i];
          if (DUAL) mine[(size_t)(BN + c + i) * BM + row] = u[i];
        }
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");      // the four epilogue warps
      if (threadIdx.x == 64) ticket_slot = atomicAdd(&a.tickets[tile_id], 1);
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ticket_slot == a.splits - 1) {                   // every other split has published its partial
        __threadfence();
        const float* all = a.scratch + (size_t)tile_id * a.splits * PER;
#pragma unroll 1
        for (int c = 0; c < BN; c += 8) {
          if (tok0 + c >= a.tokens) break;
          float v[8], u[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) { v[i] = 0.f; u[i] = 0.f; }
          for (int s = 0; s < a.splits; ++s) {             // split order: the sum does not depend on timing
            float pv[8], pu[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              pv[i] = __ldcg(all + (size_t)s * PER + (size_t)(c + i) * BM + row);
              if (DUAL) pu[i] = __ldcg(all + (size_t)s * PER + (size_t)(BN + c + i) * BM + row);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) { v[i] += pv[i]; if (DUAL) u[i] += pu[i]; }
          }
          if (a.bias != nullptr && n < a.N) {
            const float bias_v = a.bias[n], bias_u = DUAL ? a.bias[n + a.dual_offset] : 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) { v[i] += bias_v; if (DUAL) u[i] += bias_u; }
          }
          if (EPI == EPI_RESIDUAL) {
            float r[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
              r[i] = (tok0 + c + i < a.tokens && n < a.N) ? ((const float*)a.out)[(size_t)(tok0 + c + i) * a.ldo + n] : 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (tok0 + c + i < a.tokens && n < a.N) ((float*)a.out)[(size_t)(tok0 + c + i) * a.ldo + n] = r[i] + v[i];
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) emit<EPI>(a, tok0 + c + i, n, v[i], u[i]);
          }
        }
        if (threadIdx.x == 64) a.tickets[tile_id] = 0;    // ready for the next launch
      }
    }
    if (EPI == EPI_HEAD_PREP && a.splits == 1) {
      // every epilogue warp comes here, whatever happened above; then a warp per token column
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const float* stage = (const float*)(smem + HP_STAGE_OFFSET);
      if (ok)
        for (int c = lane_group, j = 0; c < BN && tok0 + c < a.tokens; c += 4, ++j)
          head_prep_finish(a.hp, tok0 + c, blockIdx.y, stage + c * BM, lane, __shfl_sync(0xffffffffu, hp_pos, j),
                           __shfl_sync(0xffffffffu, hp_page, j));
    }
    if (EPI == EPI_RESIDUAL && BN <= 64 && a.sumsq_out != nullptr && a.splits == 1) {
      // every epilogue warp comes here, whatever happened above: the four warps' sums, in warp order
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const int c = threadIdx.x - 64;
      if (ok && c < BN && tok0 + c < a.tokens)
        a.sumsq_out[(size_t)blockIdx.y * a.tokens + tok0 + c] =
            sumsq_part[0][c] + sumsq_part[1][c] + sumsq_part[2][c] + sumsq_part[3][c];
    }
    tc_fence_before();
  }
  if (CLUSTER && a.splits > 1) {
    // Every thread of every CTA of the cluster takes part in both barriers, whatever happened before.
    __syncwarp();
    cluster_sync_all();
    if (warp >= 2) {
      const bool live = !abort_flag;            // nobody writes the flag any more: the same for all four warps
      const int row = (warp & 3) * 32 + lane, n = n0 + row;
      const float* red = (const float*)smem;
      const uint32_t rank = cluster_rank();
      const bool sums = EPI == EPI_RESIDUAL && BN <= 64 && a.sumsq_out != nullptr;
      int slot = 0;
      // The token columns this CTA owns, GROUP of them at a time: all peers' values of the whole group (and the
      // residual values they will be added to) are requested before the first is used, so a group costs one round
      // trip through the cluster's shared memory, not one per column; each column's values are then added in rank
      // order, a fixed sum.  (One column at a time, a tile of 32 tokens in 8 splits paid four round trips here.)
      constexpr int GROUP = (DUAL || BN <= 16) ? 2 : 4;
      if (live)
        for (int c0 = (int)rank; c0 < BN && tok0 + c0 < a.tokens; c0 += GROUP * a.splits) {
          float pv[GROUP][8], pu[DUAL ? GROUP : 1][8], res[GROUP];
#pragma unroll
          for (int g = 0; g < GROUP; ++g) {
            const int c = c0 + g * a.splits;
            const bool owned = c < BN && tok0 + c < a.tokens;
            const bool inside = owned && n < a.N;
            res[g] = (EPI == EPI_RESIDUAL && inside) ? ((const float*)a.out)[(size_t)(tok0 + c) * a.ldo + n] : 0.f;
#pragma unroll
            for (int p = 0; p < 8; ++p) {
              pv[g][p] = (owned && p < a.splits) ? ld_peer_f32(red + c * BM + row, (uint32_t)p) : 0.f;
              if (DUAL) pu[g][p] = (owned && p < a.splits) ? ld_peer_f32(red + (BN + c) * BM + row, (uint32_t)p) : 0.f;
            }
          }
#pragma unroll
          for (int g = 0; g < GROUP; ++g) {
            const int c = c0 + g * a.splits;
            if (c >= BN || tok0 + c >= a.tokens) break;       // the same for the whole warp
            const bool inside = n < a.N;
            float v = 0.f, u = 0.f;
#pragma unroll
            for (int p = 0; p < 8; ++p) {
              if (p < a.splits) { v += pv[g][p]; if (DUAL) u += pu[g][p]; }
            }
            if (a.bias != nullptr && n < a.N) { v += a.bias[n]; if (DUAL) u += a.bias[n + a.dual_offset]; }
            if (EPI == EPI_HEAD_PREP) ((float*)(smem + HP_STAGE_OFFSET))[slot * BM + row] = round_to<bf16>(v);
            float left = 0.f;
            if (EPI == EPI_RESIDUAL) {
              left = inside ? res[g] + v : 0.f;
              if (inside) ((float*)a.out)[(size_t)(tok0 + c) * a.ldo + n] = left;
            } else {
              emit<EPI>(a, tok0 + c, n, v, u);
            }
            if (sums) {
              const float sq = warp_sum(left * left);
              if (lane == 0) sumsq_part[warp & 3][BN <= 64 ? slot : 0] = sq;
            }
            ++slot;
          }
        }
      if (EPI == EPI_HEAD_PREP) {
        asm volatile("bar.sync 1, 128;" ::: "memory");      // the four epilogue warps: the owned columns are staged
        if (live)
          for (int sl = warp & 3, j = 0; sl < slot; sl += 4, ++j)       // a warp per owned token column
            head_prep_finish(a.hp, tok0 + (int)rank + sl * a.splits, blockIdx.y, (const float*)(smem + HP_STAGE_OFFSET) + sl * BM, lane,
                             __shfl_sync(0xffffffffu, hp_pos, j), __shfl_sync(0xffffffffu, hp_page, j));
      }
      if (sums) {
        asm volatile("bar.sync 1, 128;" ::: "memory");      // the four epilogue warps
        const int mine = threadIdx.x - 64, c = (int)rank + mine * a.splits;
        if (live && mine < slot && c < BN && tok0 + c < a.tokens)
          a.sumsq_out[(size_t)blockIdx.y * a.tokens + tok0 + c] =
              sumsq_part[0][mine] + sumsq_part[1][mine] + sumsq_part[2][mine] + sumsq_part[3][mine];
      }
    }
    __syncwarp();
    cluster_sync_all();     // nobody leaves while its shared memory may still be read
  }
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
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

// A [rows, K] row-major bf16 matrix cut into boxes of box_rows x 64 with the 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (fn == nullptr) return ODI_ERR_UNSUPPORTED;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {BK, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : ODI_ERR_ARGUMENT;
}

// Dynamic shared memory of the merge prologue's form beyond its ring of weight stages: the token tiles of
// `kb_cap` k-blocks and the table of the splits' weights for the heads those k-blocks can touch.
static inline int merge_extra_smem(int bn, int kb_cap, int splits, int d) {
  const int heads = (kb_cap * BK + d - 1) / d + 1;
  return kb_cap * bn * BK * 2 + bn * heads * (splits + 2) * 4;
}
#define MERGE_SMEM_LIMIT (96 * 1024)      // per CTA, so that two fit on an SM

template <int BN, bool DUAL, int EPI, bool CLUSTER, int PRO = PRO_NONE>
static int launch(const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& a, dim3 grid, cudaStream_t stream) {
  constexpr bool MERGE = PRO == PRO_MERGE;
  constexpr int STAGE_BYTES = BM * BK * 2 * (DUAL ? 2 : 1) + (MERGE ? 0 : BN * BK * 2);
  // A CTA takes about 72 KB (four stages of a 128 x 16 tile), so that three CTAs fit on an
  // SM: several short pipelines per SM hide each other's set-up, drain and split exchange, and the
  // CTAs of the next kernel of the stream find room to move in and request their first weight tiles
  // while this one drains.  Measured on whole captured decode steps (Qwen3-8B sizes, batch 1 / 8):
  // 72-84 KB 3.39 / 3.86 ms, 56-64 KB 3.46 / 4.13 ms, 100 KB 3.50 / 4.13 ms; one CTA of 144-200 KB
  // per SM is 1.5x slower per kernel.
#ifndef ODI_GEMM_DECODE_SMEM_KB
#define ODI_GEMM_DECODE_SMEM_KB 72
#endif
  // (Token tiles of 64 with a larger budget, tokens 64, us own at 72 / 108 / 160 KB against the library: down
  // projection 26.0 / 24.8 / 47.9 against 21.8, output projection 13.3 / 12.6 / 27.1 against 9.7, q/k/v 14.4 / 20.8 /
  // 34.2 against 11.3, gate/up with the SiLU gate 55 at every budget against 38.4 + 3.5: above 32 tokens the
  // projections go to the library, see parts/linear.py.)
  // (MERGE: three weight stages, so that with the token tiles behind them a CTA still takes about 72 KB.)
  constexpr int BUDGET = MERGE ? 48 * 1024 : ODI_GEMM_DECODE_SMEM_KB * 1024;
  constexpr int STAGES = BUDGET / STAGE_BYTES < 2 ? 2 : (BUDGET / STAGE_BYTES > 12 ? 12 : BUDGET / STAGE_BYTES);
  const int SMEM = STAGES * STAGE_BYTES + 1024 + (MERGE ? merge_extra_smem(BN, a.merge_kb_cap, a.mg.splits, a.mg.d) : 0);
  if (MERGE && SMEM > MERGE_SMEM_LIMIT) return ODI_ERR_UNSUPPORTED;
  static_assert(!CLUSTER || (DUAL ? 2 : 1) * BN * BM * 4 <= STAGES * STAGE_BYTES, "the split partial must fit the stage memory");
  auto kernel = gemm_tcgen05_kernel<BN, DUAL, EPI, STAGES, CLUSTER, PRO>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MERGE ? MERGE_SMEM_LIMIT : SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  if (CLUSTER) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled();
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 1;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = grid.z;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    odi_rc = (int)cudaLaunchKernelEx(&cfg, kernel, mw, mx, a);
    return launch_status();
  }
  odi_rc = launch_pdl((kernel), dim3(grid), dim3(GEMM_THREADS), SMEM, stream, mw, mx, a);
  return launch_status();
}

template <int BN, bool CLUSTER>
static int dispatch_epi(int epi, const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& a, dim3 grid,
                        cudaStream_t stream) {
  if (a.norm_x != nullptr) {
    // the norm prologue exists for the two products that follow a norm in a decoder layer, at decode widths
    if constexpr (BN <= 32) {
      if (epi == EPI_STORE_BF16) return launch<BN, false, EPI_STORE_BF16, CLUSTER, PRO_NORM>(mw, mx, a, grid, stream);
      if (epi == EPI_SWIGLU) return launch<BN, true, EPI_SWIGLU, CLUSTER, PRO_NORM>(mw, mx, a, grid, stream);
      if (epi == EPI_HEAD_PREP) return launch<BN, false, EPI_HEAD_PREP, CLUSTER, PRO_NORM>(mw, mx, a, grid, stream);
    }
    return ODI_ERR_UNSUPPORTED;
  }
  if (a.mg.partial != nullptr) {
    // the merge prologue exists for the product that follows a decode attention: the output projection
    if constexpr (BN <= 32) {
      if (epi == EPI_RESIDUAL) return launch<BN, false, EPI_RESIDUAL, CLUSTER, PRO_MERGE>(mw, mx, a, grid, stream);
    }
    return ODI_ERR_UNSUPPORTED;
  }
  if (epi == EPI_HEAD_PREP) {
    if constexpr (BN <= 32) return launch<BN, false, EPI_HEAD_PREP, CLUSTER>(mw, mx, a, grid, stream);
    else return ODI_ERR_UNSUPPORTED;
  }
  switch (epi) {
    case EPI_STORE_BF16: return launch<BN, false, EPI_STORE_BF16, CLUSTER>(mw, mx, a, grid, stream);
    case EPI_STORE_F32: return launch<BN, false, EPI_STORE_F32, CLUSTER>(mw, mx, a, grid, stream);
    case EPI_RESIDUAL: return launch<BN, false, EPI_RESIDUAL, CLUSTER>(mw, mx, a, grid, stream);
    case EPI_SWIGLU:
      if constexpr (BN <= 128 && !(CLUSTER && BN > 64)) return launch<BN, true, EPI_SWIGLU, CLUSTER>(mw, mx, a, grid, stream);
      else return ODI_ERR_UNSUPPORTED;
  }
  return ODI_ERR_ARGUMENT;
}

// Scratch floats a launch with these sizes needs (0 when splits == 1).
extern "C" long odi_gemm_bf16_scratch_floats(int tokens, int n_out, int bn, int splits, int dual) {
  if (splits <= 1) return 0;
  const long tiles = (long)((n_out + BM - 1) / BM) * ((tokens + bn - 1) / bn);
  return tiles * splits * (dual ? 2 : 1) * bn * BM;
}

// x [tokens, K] bf16, w [w_rows, K] bf16 (for EPI_SWIGLU w holds the gate rows followed by
// the up rows and n_out = w_rows / 2), out [tokens, ldo]; bias: null or fp32 [w_rows], added to the product.
// no_loads != 0: the self-test of the bounded waits (see GemmArgs); the result is invalid by design.
// Tiles of 128 features x bn tokens, bn in {16, 32, 64, 128, 256}, K splits allowed; cluster != 0 lets 2..8 splits
// (bn <= 64) exchange partials through distributed shared memory.  Many tokens are the business of
// gemm_prefill_tcgen05.cu; this kernel takes them too, tile by tile, but re-reads the weights for every token tile.
extern "C" int odi_gemm_bf16(const void* x, const void* w, void* out, int tokens, int n_out, int K, int w_rows,
                             int ldo, int epi, int bn, int splits, int cluster, float* scratch,
                             int* tickets, int* status, const float* norm_x, const float* norm_w,
                             const float* norm_parts, int norm_n_parts, float norm_eps, float* sumsq_out,
                             const HeadPrepArgs* head_prep, const float* bias, int no_loads, const MergeArgs* merge,
                             cudaStream_t stream) {
  if (tokens <= 0 || n_out <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return ODI_ERR_UNSUPPORTED;
  if ((x != nullptr) + (norm_x != nullptr) + (merge != nullptr) != 1) return ODI_ERR_ARGUMENT;
  const int total_kb = (K + BK - 1) / BK;
  if (splits < 1 || splits > total_kb) return ODI_ERR_ARGUMENT;
  const bool clustered = cluster && splits > 1 && splits <= 8 && bn <= 64;
  if (splits > 1 && !clustered && (scratch == nullptr || tickets == nullptr)) return ODI_ERR_ARGUMENT;
  if (status == nullptr) return ODI_ERR_ARGUMENT;
  const bool dual = epi == EPI_SWIGLU;
  if (dual && w_rows != 2 * n_out) return ODI_ERR_ARGUMENT;
  CUtensorMap mw, mx;
  int rc = make_map(&mw, w, w_rows, K, BM);
  if (rc != 0) return rc;
  rc = make_map(&mx, x == nullptr ? w : x, tokens, K, bn);    // with a prologue the map is not used
  if (rc != 0) return rc;
  GemmArgs a;
  a.out = out; a.scratch = scratch; a.tickets = tickets; a.status = status;
  a.tokens = tokens; a.N = n_out; a.K = K; a.ldo = ldo; a.dual_offset = dual ? n_out : 0; a.splits = splits;
  if (norm_x != nullptr) {
    if (bn > 32 || (epi != EPI_STORE_BF16 && epi != EPI_SWIGLU && epi != EPI_HEAD_PREP)) return ODI_ERR_UNSUPPORTED;
    if (norm_w == nullptr || norm_parts == nullptr || norm_n_parts < 1) return ODI_ERR_ARGUMENT;
    if (((uintptr_t)norm_x & 15) || ((uintptr_t)norm_w & 15)) return ODI_ERR_UNSUPPORTED;
  }
  if (sumsq_out != nullptr && (epi != EPI_RESIDUAL || bn > 64 || !(clustered || splits == 1))) return ODI_ERR_UNSUPPORTED;
  a.norm_x = norm_x; a.norm_w = norm_w; a.norm_parts = norm_parts; a.norm_n_parts = norm_n_parts; a.norm_eps = norm_eps;
  a.sumsq_out = sumsq_out;
  a.bias = bias;
  a.no_loads = no_loads;
  if (no_loads && (x == nullptr || splits != 1)) return ODI_ERR_ARGUMENT;     // the self-test is one plain tile
  a.mg = MergeArgs{};
  a.merge_kb_cap = 0;
  if (merge != nullptr) {
    // heads of a multiple of 64 (a k-block lies inside one head), K = all heads, one token per sequence, up to 32 splits
    a.mg = *merge;
    if (bn > 32 || epi != EPI_RESIDUAL || !(clustered || splits == 1)) return ODI_ERR_UNSUPPORTED;
    if (a.mg.partial == nullptr || a.mg.past == nullptr || a.mg.splits < 1 || a.mg.splits > 32 || a.mg.d <= 0 ||
        a.mg.d % BK != 0 || (long)a.mg.nq * a.mg.d != K || ((uintptr_t)a.mg.partial & 7))
      return ODI_ERR_UNSUPPORTED;
    a.merge_kb_cap = (total_kb + splits - 1) / splits;
  }
  if (epi == EPI_HEAD_PREP) {
    // heads of 128 (a tile is a head), whole-head rotation or none, keys and values written, tokens in columns
    if (head_prep == nullptr) return ODI_ERR_ARGUMENT;
    a.hp = *head_prep;
    const HeadPrepArgs& hp = a.hp;
    if (bn > 32 || !(clustered || splits == 1) || hp.d != BM || n_out != (hp.nq + 2 * hp.nkv) * BM ||
        !hp.write_kv || (hp.cos_t != nullptr && hp.rot_dim != hp.d) || hp.n_tokens != tokens)
      return ODI_ERR_UNSUPPORTED;
  } else {
    a.hp = HeadPrepArgs{};
  }
  dim3 grid((tokens + bn - 1) / bn, (n_out + BM - 1) / BM, splits);
  if (grid.y > 65535 || grid.z > 65535) return ODI_ERR_UNSUPPORTED;
  // 2..8 splits of a token tile of up to 64 exchange their partials inside a cluster
  if (cluster && splits > 1 && splits <= 8 && bn <= 64) {
    switch (bn) {
      case 16: return dispatch_epi<16, true>(epi, mw, mx, a, grid, stream);
      case 32: return dispatch_epi<32, true>(epi, mw, mx, a, grid, stream);
      case 64: return dispatch_epi<64, true>(epi, mw, mx, a, grid, stream);
    }
  }
  switch (bn) {
    case 16: return dispatch_epi<16, false>(epi, mw, mx, a, grid, stream);
    case 32: return dispatch_epi<32, false>(epi, mw, mx, a, grid, stream);
    case 64: return dispatch_epi<64, false>(epi, mw, mx, a, grid, stream);
    case 128: return dispatch_epi<128, false>(epi, mw, mx, a, grid, stream);
    case 256: return dispatch_epi<256, false>(epi, mw, mx, a, grid, stream);
  }
  return ODI_ERR_UNSUPPORTED;
}
