// bf16 matrix product for many tokens (prefill) on the 5th-generation tensor cores:
//   out[token, n] = epilogue( sum_k x[token, k] * w[n, k] ),  fp32 accumulation.
//
// A persistent kernel of clusters of two CTAs (two SMs), the two-CTA form of the MMA.  A cluster owns
// tiles of 256 tokens x 256 features and walks them (its own, then every n-th; token tiles vary fastest
// inside groups of 16, so that the clusters that run side by side share weight tiles and a bounded set of
// activation rows in L2).  CTA r of the pair holds token rows r * 128 .. + 127 of the activations and
// feature rows r * 128 .. + 127 of the weights: per k-block of 64 that is 16 KB + 16 KB by TMA (128-byte
// swizzle) into a ring of six stages.  One thread of the leader CTA issues tcgen05.mma.cta_group::2
// (M = 256, N = 256, K = 16), which reads both CTAs' shared memory and fills 128 lanes x 256 columns of
// tensor memory in each CTA.  A single CTA with a 128 x 256 tile moves 48 KB into shared memory and reads
// 48 KB back per 512 cycles of math, more than the 128 bytes per cycle shared memory delivers (measured:
// 1.3-1.4 PFLOP/s); the pair moves and reads 32 KB per CTA for the same math.
//
// Tensor memory holds two accumulators (2 x 256 columns): while the four epilogue warps of each CTA read
// one tile's result, convert it, stage it swizzled in shared memory (two buffers of 128 rows x 128 bytes)
// and hand it to a TMA store -- for the residual a TMA fp32 reduce-add, which never reads the residual --
// the MMA thread is already filling the other accumulator.
//
//   warp 0   TMA producer (one thread per CTA)
//   warp 1   allocates tensor memory; in the leader one thread issues the MMAs and commits
//   warps 2-5 epilogue: a thread per token row of the CTA's half tile
//
//   full[s]      (leader's) both producers announce their bytes and their TMA loads complete on it
//   empty[s]     (each CTA's) the leader's commit reaches both: the stage may be refilled
//   acc_full[b]  (each CTA's) the leader's commit reaches both: the tile's accumulator is complete
//   acc_empty[b] (leader's) the epilogue warps of both CTAs arrive: the accumulator may be overwritten
//
// Epilogues: store bf16, store fp32, add into an fp32 residual, SiLU gate, head preparation (the rows of w
// are query, key and value heads of 128: a tile's 256 columns are two heads, and a thread of the epilogue
// finishes its token's row of each: per-head norm, rotation, the write to the query buffer or the cache
// page; this one writes its rows itself, the others go through TMA).  For the gate the weight rows
// are the gate rows followed by the up rows; the leader holds 128 gate rows and the peer the same 128 up
// rows, a tile's 256 columns are gate | up, and silu(gate) * up gives 128 outputs.
//
// Measured on B200 against the library's product plus the elementwise kernel a fused epilogue saves
// (Qwen3-8B sizes, us): 2,048 tokens q/k/v 70 / 69, output projection + residual 49 / 46 + 11, gate/up +
// SiLU gate 273 / 274 + 24, down + residual 145 / 133 + 11; 8,192 tokens 267 / 270, 191 / 180 + 44,
// 1,040 / 1,031 + 96, 558 / 529 + 44.  Below about a thousand tokens there are too few tiles for 74 clusters.
//
// The output rows must start on 16-byte boundaries (the TMA store's rule); K a multiple of 8.
// Every wait on an mbarrier is bounded: after about two seconds of SM clock the role records an error code
// in `status`, all roles leave their loops, tensor memory is freed and the kernel returns.
#include <cuda.h>

#include "common.cuh"

#define EPI_STORE_BF16 0
#define EPI_STORE_F32 1
#define EPI_RESIDUAL 2
#define EPI_SWIGLU 3
#define EPI_HEAD_PREP 4    // the rows of w are q, k and v heads of 128: per-head norm, rotation, cache write

#define BM 128             // token rows per CTA (the lanes of its tensor memory); a tile has 2 * BM
#define BN 256             // accumulator columns per tile
#define BK 64              // k per stage: 64 bf16 = one 128-byte swizzle row
#define A_BYTES (BM * BK * 2)     // 128 rows of 64 k: a CTA's activation rows, and as much for its weight rows
#define THREADS 192
#define WAIT_CYCLES 4000000000ll

#define ERR_PRODUCER 21
#define ERR_MMA 22
#define ERR_EPILOGUE 23

struct PrefillGemmArgs {
  void* out;               // only its alignment matters here: the output goes through a tensor map
  int* status;
  int tokens, N, K, ldo;   // N: output features (for the gate: half of the weight rows)
  int up_offset;           // EPI_SWIGLU: row distance from a gate row to its up row
  int m_tiles, n_tiles;    // tiles of 256 tokens, tiles of 256 columns
  const float* bias;       // null, or fp32 [weight rows]: added to the product before the epilogue's own work
  // EPI_RESIDUAL: every tile's k-blocks in `parts` ranges that different pairs add into the residual one after the
  // other (see segment_of); flags: two counters per tile, zero on entry and left zero.
  int parts;
  int* flags;
  HeadPrepArgs hp;         // EPI_HEAD_PREP
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
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
// Bounded wait.  Returns false when it gave up or when another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  const long long start = clock64();
  for (uint32_t i = 0;; ++i) {
    if (mbar_test(bar, parity)) return true;
    if ((i & 0xf) == 0xf) {
      if (*abort_flag) return false;
      if (clock64() - start > WAIT_CYCLES) break;
    }
  }
  *abort_flag = 1;
  return false;
}
// A staged tile (128 rows of 128 bytes, 128-byte swizzle) to global memory: plain store, or fp32 add.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }   // the four epilogue warps

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
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

// K-major tile written by TMA with the 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_k_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3ffff) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// kind::f16: fp32 accumulator, bf16 A and B, both K-major.
__host__ __device__ constexpr uint32_t instr_desc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ float silu_f(float g) { return g / (1.f + __expf(-g)); }

// ------------------------------------------------------------------------------ the kernel

#define STAGES 6
#define STAGE_BYTES (2 * A_BYTES)

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The address, in the cluster's shared window, of the same variable in the CTA of the given rank.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  return remote;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t cluster_bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// A TMA load into this CTA's shared memory whose bytes are counted on a barrier of the pair's leader.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void umma_pair_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives, once the MMAs issued so far have completed, on the barrier at this offset in both CTAs.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(both) : "memory");
}

// One thread finishes one head of one token from the head's 128 projections in tensor memory (columns
// taddr .. + 127 of the thread's lane): rounded to bf16 as the stored projections would be, then the
// arithmetic of the stand-alone head preparation (per-head RMSNorm, half-split rotation), and the row goes to
// the query buffer or to the token's place in the key / value cache.
__device__ __forceinline__ void head_prep_row(const HeadPrepArgs& hp, int t, int h, uint32_t taddr, const float* bias) {
  constexpr int d = 128, half = 64;
  float x[d];
#pragma unroll
  for (int j = 0; j < d / 32; ++j) tmem_ld32(taddr + 32 * j, x + 32 * j);
  if (t >= hp.n_tokens) return;                       // after the loads: they are warp-wide
  if (bias != nullptr) {
#pragma unroll
    for (int i = 0; i < d; ++i) x[i] = round_to<bf16>(x[i] + __ldg(bias + h * d + i));   // the same for every thread: a broadcast read
  } else {
#pragma unroll
    for (int i = 0; i < d; ++i) x[i] = round_to<bf16>(x[i]);
  }
  const int kind = h < hp.nq ? 0 : (h < hp.nq + hp.nkv ? 1 : 2);     // 0 q, 1 k, 2 v
  const int pos = hp.tok_pos[t];
  bf16* dst;
  if (kind == 0) {
    dst = (bf16*)hp.q_out + ((size_t)t * hp.nq + h) * d;
  } else {
    const int hk = kind == 1 ? h - hp.nq : h - hp.nq - hp.nkv;
    const int page = hp.page_ids[hp.page_start[hp.tok_seq[t]] + page_slot_of(pos, hp.page_size, hp.ring_pages)];
    bf16* pool = (bf16*)(kind == 1 ? hp.k_pool : hp.v_pool);
    dst = pool + (((size_t)page * hp.nkv + hk) * hp.page_size + (pos % hp.page_size)) * d;
  }
  if (kind != 2) {
    const float* w = kind == 0 ? hp.q_norm_w : hp.k_norm_w;
    if (w != nullptr) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < d; ++i) ss += x[i] * x[i];
      const float inv = rsqrtf(ss / (float)d + hp.eps);
#pragma unroll
      for (int i = 0; i < d; i += 4) {
        const float4 ww = *(const float4*)(w + i);
        x[i] = round_to<bf16>(ww.x * round_to<bf16>(x[i] * inv));
        x[i + 1] = round_to<bf16>(ww.y * round_to<bf16>(x[i + 1] * inv));
        x[i + 2] = round_to<bf16>(ww.z * round_to<bf16>(x[i + 2] * inv));
        x[i + 3] = round_to<bf16>(ww.w * round_to<bf16>(x[i + 3] * inv));
      }
    }
    if (hp.cos_t != nullptr) {
      const float4* cs = (const float4*)(hp.cos_t + (size_t)t * half);
      const float4* sn = (const float4*)(hp.sin_t + (size_t)t * half);
#pragma unroll
      for (int i = 0; i < half; i += 4) {
        const float4 c = cs[i / 4], s = sn[i / 4];
        const float cc[4] = {c.x, c.y, c.z, c.w}, ssn[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float lo = x[i + e], hi = x[i + e + half];
          x[i + e] = lo * cc[e] - hi * ssn[e];
          x[i + e + half] = hi * cc[e] + lo * ssn[e];
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < d; i += 8) {
    uint32_t w4[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      __nv_bfloat162 pr = __floats2bfloat162_rn(x[i + 2 * e], x[i + 2 * e + 1]);
      w4[e] = *(uint32_t*)&pr;
    }
    *(uint4*)(dst + i) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
  }
}

// Tile t of the walk: token tiles vary fastest inside groups of TILE_GROUP token tiles, so that the CTAs that run
// side by side share a few weight tiles and a bounded set of activation rows (both stay in L2 however many tokens
// there are).
#define TILE_GROUP 16
__device__ __forceinline__ void tile_of(int t, int m_tiles, int n_tiles, int& m, int& n) {
  const int per_group = TILE_GROUP * n_tiles;
  const int g = t / per_group, r = t - g * per_group;
  const int rows = min(TILE_GROUP, m_tiles - g * TILE_GROUP);
  m = g * TILE_GROUP + r % rows;
  n = r / rows;
}

// The idx-th piece of work of a pair: a tile and a range of its k-blocks.
//
// Walking whole tiles, 128 tiles on 74 pairs take two rounds of which the second is a quarter empty (the down
// projection of a 2,048-token prompt; 160 tiles take three rounds at the sizes of Qwen3-14B).  With `parts` > 1
// every tile's k-blocks are cut into that many equal ranges and the pairs walk the (part, tile) units instead,
// all tiles' first parts before all second parts, so that the pairs that run side by side still stream the same
// k-blocks of a few weight tiles and activation rows through L2.  A tile is then finished by `parts` adds into
// the fp32 residual (the reduce-add epilogue needs no fix-up pass), by different pairs at different times.  The
// adds are ordered, so that the sum does not depend on timing: part q adds after a counter says that part q - 1's
// add of the same token rows is complete, and then raises it (the last part puts it back to zero).  A unit only
// ever waits for a unit that comes earlier in the walk, and a pair takes its units in the walk's order: nobody
// waits for somebody who waits for him.
struct Segment { int tile, kb0, kb1, part; bool last; };
__device__ __forceinline__ bool segment_of(const PrefillGemmArgs& a, int pair, int n_pairs, int total_tiles, int total_kb,
                                           int idx, Segment& sg) {
  const int parts = a.parts < 1 ? 1 : a.parts;
  const long unit = (long)idx * n_pairs + pair;
  if (unit >= (long)total_tiles * parts) return false;
  sg.part = (int)(unit / total_tiles);
  sg.tile = (int)(unit - (long)sg.part * total_tiles);
  sg.kb0 = (int)((long)total_kb * sg.part / parts);
  sg.kb1 = (int)((long)total_kb * (sg.part + 1) / parts);
  sg.last = sg.part == parts - 1;
  return true;
}

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_prefill_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                         const __grid_constant__ CUtensorMap map_out, const PrefillGemmArgs a) {
  constexpr bool GATE = EPI == EPI_SWIGLU;
  constexpr int OUT_PER_TILE = GATE ? BN / 2 : BN;      // output features a tile covers
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t bars[2 * STAGES + 4];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int epilogue_ok;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int total_tiles = a.m_tiles * a.n_tiles;        // m_tiles here: tiles of 256 tokens
  const int total_kb = (a.K + BK - 1) / BK;
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = full0 + 8 * STAGES, acc_full0 = empty0 + 8 * STAGES,
                 acc_empty0 = acc_full0 + 16;
  const uint32_t leader_full0 = map_to_rank(full0, 0), leader_acc_empty0 = map_to_rank(acc_empty0, 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 2); mbar_init(empty0 + 8 * s, 1); }   // two producers
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full0 + 8 * b, 1); mbar_init(acc_empty0 + 8 * b, 8); }     // 4 + 4 epilogue warps
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(2 * BN));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();               // both CTAs' barriers exist before anybody signals across
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abort_ptr = &abort_flag;
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      pdl_wait();                     // the activations come from the kernel before
      int it = 0;
      bool ok = true;
      Segment sg;
      for (int idx = 0; ok && segment_of(a, pair, n_pairs, total_tiles, total_kb, idx, sg); ++idx) {
        int tm, tn;
        tile_of(sg.tile, a.m_tiles, a.n_tiles, tm, tn);
        const int tok0 = tm * (2 * BM) + (int)rank * BM, n0 = tn * OUT_PER_TILE;
        // this CTA's weight rows: its half of the 256 columns (for the gate: gate rows in the leader, up rows in the peer)
        const int w_row = GATE ? n0 + (int)rank * a.up_offset : n0 + (int)rank * (BN / 2);
        for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
          const int s = it % STAGES;
          if (it >= STAGES && !mbar_wait(empty0 + 8 * s, (((uint32_t)(it / STAGES) & 1u) ^ 1u), abort_ptr)) { ok = false; break; }
          const uint32_t dst = smem_u32(smem + (size_t)s * STAGE_BYTES);
          mbar_expect_tx_cluster(leader_full0 + 8 * s, STAGE_BYTES);
          tma_load_2d_pair(dst, &map_x, kb * BK, tok0, leader_full0 + 8 * s);
          tma_load_2d_pair(dst + A_BYTES, &map_w, kb * BK, w_row, leader_full0 + 8 * s);
        }
      }
      if (!ok) atomicCAS(a.status, 0, ERR_PRODUCER);
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = instr_desc_bf16(2 * BM, BN);
      int it = 0, local = 0;
      bool ok = true;
      Segment sg;
      for (; ok && segment_of(a, pair, n_pairs, total_tiles, total_kb, local, sg); ++local) {
        const int buf = local & 1;
        if (local >= 2 && !mbar_wait(acc_empty0 + 8 * buf, (((uint32_t)(local >> 1) & 1u) ^ 1u), abort_ptr)) { ok = false; break; }
        tc_fence_after();
        for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(full0 + 8 * s, (uint32_t)(it / STAGES) & 1u, abort_ptr)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + (size_t)s * STAGE_BYTES);
          const uint64_t da = smem_desc_k_sw128(sa), db = smem_desc_k_sw128(sa + A_BYTES);
#pragma unroll
          for (int j = 0; j < BK / 16; ++j)
            umma_pair_bf16(tmem_base + buf * BN, da + 2 * j, db + 2 * j, idesc, (kb > sg.kb0 || j > 0) ? 1u : 0u);
          umma_commit_pair(empty0 + 8 * s);         // both CTAs may refill the stage
        }
        if (ok) umma_commit_pair(acc_full0 + 8 * buf);
      }
      if (!ok) atomicCAS(a.status, 0, ERR_MMA);
    }
  } else {
    // epilogue warps 2..5 of each CTA: its 128 token rows of the tile
    const int lane_group = warp & 3, row = lane_group * 32 + lane;
    constexpr bool OUT32 = EPI == EPI_STORE_F32 || EPI == EPI_RESIDUAL;
    constexpr int COLS_PER_OP = OUT32 ? 32 : 64;
    uint8_t* stage_out = smem + STAGES * STAGE_BYTES;
    int local = 0, op = 0;
    bool ok = true;
    Segment sg;
    for (; ok && segment_of(a, pair, n_pairs, total_tiles, total_kb, local, sg); ++local) {
      const int buf = local & 1;
      int tm, tn;
      tile_of(sg.tile, a.m_tiles, a.n_tiles, tm, tn);
      const int tok0 = tm * (2 * BM) + (int)rank * BM, n0 = tn * OUT_PER_TILE;
      if (warp == 2) {
        bool got = mbar_wait(acc_full0 + 8 * buf, (uint32_t)(local >> 1) & 1u, abort_ptr);
        if (got && EPI == EPI_RESIDUAL && sg.part > 0 && lane == 0) {
          // a later part of a tile: add once the part before has added to these token rows (it ran a round
          // earlier as a rule, so this seldom waits; the wait is bounded like every other)
          volatile int* flag = a.flags + 2 * sg.tile + (int)rank;
          const long long start = clock64();
          while (*flag != sg.part) {
            if (*abort_ptr || clock64() - start > WAIT_CYCLES) { *abort_ptr = 1; got = false; break; }
            __nanosleep(64);
          }
          if (got) { __threadfence(); if (sg.last) *flag = 0; }      // the last part leaves it zero for the next launch
        }
        got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
        if (lane == 0) epilogue_ok = got ? 1 : 0;
      }
      epilogue_sync();
      ok = epilogue_ok != 0;
      epilogue_sync();
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(lane_group * 32) << 16) + buf * BN;
      if (EPI == EPI_HEAD_PREP) {
        // a tile's 256 columns are two heads; a thread finishes its token's row of each
#pragma unroll 1
        for (int hh = 0; hh < BN / 128; ++hh)
          if (n0 + 128 * hh < a.N) head_prep_row(a.hp, tok0 + row, (n0 >> 7) + hh, taddr + 128 * hh, a.bias);
      } else
#pragma unroll 1
      for (int c = 0; c < OUT_PER_TILE; c += COLS_PER_OP, ++op) {
        if (n0 + c >= a.N) break;
        uint8_t* tile_out = stage_out + (op & 1) * 16384;
        uint8_t* mine = tile_out + row * 128;
        epilogue_sync();
#pragma unroll
        for (int part = 0; part < COLS_PER_OP / 32; ++part) {
          float v[32], u[32];
          tmem_ld32(taddr + c + 32 * part, v);
          if (GATE) tmem_ld32(taddr + BN / 2 + c + 32 * part, u);
          if (a.bias != nullptr && sg.part == 0) {
            // a column is a feature: the same 32 biases for every thread (a broadcast read); columns beyond
            // the matrix are clipped by the TMA store, their bias is taken as zero; a tile's first part adds it
            const int nb = n0 + c + 32 * part;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const bool in = nb + j < a.N;
              v[j] += in ? __ldg(a.bias + nb + j) : 0.f;
              if (GATE) u[j] += in ? __ldg(a.bias + a.up_offset + nb + j) : 0.f;
            }
          }
          if (OUT32) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
              *(float4*)(mine + ((q ^ (row & 7)) << 4)) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
          } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint32_t w[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int e = 8 * q + 2 * i;
                const float lo = GATE ? silu_f(v[e]) * u[e] : v[e];
                const float hi = GATE ? silu_f(v[e + 1]) * u[e + 1] : v[e + 1];
                __nv_bfloat162 pr = __floats2bfloat162_rn(lo, hi);
                w[i] = *(uint32_t*)&pr;
              }
              *(uint4*)(mine + (((4 * part + q) ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        epilogue_sync();
        if (threadIdx.x == 64) {
          if (EPI == EPI_RESIDUAL) tma_reduce_add_2d(&map_out, smem_u32(tile_out), n0 + c, tok0);
          else tma_store_2d(&map_out, smem_u32(tile_out), n0 + c, tok0);
          bulk_commit();
          bulk_wait_read<1>();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_acc_empty0 + 8 * buf);
      if (EPI == EPI_RESIDUAL && !sg.last && threadIdx.x == 64) {
        // not the tile's last part: once this CTA's adds have completed, let the next part add
        bulk_wait_all();
        __threadfence();
        atomicExch(a.flags + 2 * sg.tile + (int)rank, sg.part + 1);
      }
    }
    if (threadIdx.x == 64) bulk_wait_all();
    if (!ok && lane == 0) atomicCAS(a.status, 0, ERR_EPILOGUE);
    tc_fence_before();
  }
  __syncthreads();
  cluster_sync_all();               // nobody leaves while its barriers or tensor memory may still be used by the peer
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN));
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

// A [rows, K] row-major bf16 matrix cut into boxes of box_rows x 64 with the 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, long rows, int K, int box_rows) {
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

// The output [tokens, N] (rows ldo elements apart) cut into boxes of 128 rows x 128 bytes with the 128-byte swizzle.
static int make_out_map(CUtensorMap* map, void* base, int tokens, int N, int ldo, bool f32) {
  EncodeTiledFn fn = encode_tiled();
  if (fn == nullptr) return ODI_ERR_UNSUPPORTED;
  const int elem_bytes = f32 ? 4 : 2;
  cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)tokens};
  cuuint64_t strides[1] = {(cuuint64_t)ldo * elem_bytes};
  cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), BM};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box,
                  elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : ODI_ERR_ARGUMENT;
}

template <int EPI>
static int launch(const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& mo, const PrefillGemmArgs& a, int sms,
                       cudaStream_t stream) {
  constexpr int SMEM = STAGES * STAGE_BYTES + 2 * 16384 + 1024;
  auto kernel = gemm_prefill_kernel<EPI>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = a.m_tiles * a.n_tiles;
  const int pairs = tiles < sms / 2 ? tiles : sms / 2;
  odi_rc = launch_pdl((kernel), dim3(2 * pairs), dim3(THREADS), SMEM, stream, mx, mw, mo, a);
  return launch_status();
}

// x [tokens, K] bf16, w [w_rows, K] bf16 (for EPI_SWIGLU the gate rows followed by the up rows,
// n_out = w_rows / 2), out [tokens, ldo] with rows that start on 16-byte boundaries; status: an int that
// receives an error code if a wait gives up.
// EPI_HEAD_PREP: out is not used; head_prep describes where the heads go (heads of 128, whole-head rotation or
// none, keys and values written).
// bias: null, or fp32 [w_rows] (16-byte aligned), added to the product.
// flags: n_flags ints, zero on entry and left zero (two per tile are used when the work is balanced).
extern "C" int odi_gemm_prefill_bf16(const void* x, const void* w, void* out, int tokens, int n_out, int K, int w_rows,
                                     int ldo, int epi, const HeadPrepArgs* head_prep, const float* bias, int* status,
                                     int* flags, int n_flags, int balance, cudaStream_t stream) {
  if (tokens <= 0 || n_out <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || status == nullptr) return ODI_ERR_UNSUPPORTED;
  const bool gate = epi == EPI_SWIGLU, heads = epi == EPI_HEAD_PREP;
  if (gate ? w_rows != 2 * n_out : w_rows != n_out) return ODI_ERR_ARGUMENT;
  const bool f32 = epi == EPI_STORE_F32 || epi == EPI_RESIDUAL;
  if (!heads && (((uintptr_t)out & 15) || ((long)ldo * (f32 ? 4 : 2)) % 16 != 0)) return ODI_ERR_UNSUPPORTED;
  if ((uintptr_t)bias & 15) return ODI_ERR_UNSUPPORTED;
  if (heads) {
    if (head_prep == nullptr) return ODI_ERR_ARGUMENT;
    const HeadPrepArgs& hp = *head_prep;
    if (hp.d != 128 || n_out != (hp.nq + 2 * hp.nkv) * 128 || !hp.write_kv || hp.n_tokens != tokens ||
        (hp.cos_t != nullptr && hp.rot_dim != hp.d) || ((uintptr_t)hp.q_out & 15) || ((uintptr_t)hp.k_pool & 15) ||
        ((uintptr_t)hp.v_pool & 15) || ((uintptr_t)hp.cos_t & 15) || ((uintptr_t)hp.sin_t & 15) ||
        ((uintptr_t)hp.q_norm_w & 15) || ((uintptr_t)hp.k_norm_w & 15))
      return ODI_ERR_UNSUPPORTED;
  }
  static int sms = 0;
  if (sms == 0) {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) return (int)e;
  }
  CUtensorMap mx, mw, mo;
  int rc = make_map(&mx, x, tokens, K, BM);
  if (rc == 0) rc = make_map(&mw, w, w_rows, K, BN / 2);
  if (rc == 0 && !heads) rc = make_out_map(&mo, out, tokens, n_out, ldo, f32);
  if (rc != 0) return rc;
  if (heads) mo = mx;               // not used by that epilogue
  PrefillGemmArgs a;
  a.out = out; a.status = status; a.tokens = tokens; a.N = n_out; a.K = K; a.ldo = ldo;
  a.up_offset = gate ? n_out : 0;
  a.bias = bias;
  a.hp = heads ? *head_prep : HeadPrepArgs{};
  const int per_tile = gate ? BN / 2 : BN;
  a.m_tiles = (tokens + 2 * BM - 1) / (2 * BM);
  a.n_tiles = (n_out + per_tile - 1) / per_tile;
  if ((long)a.m_tiles * a.n_tiles > 0x7fffffffL) return ODI_ERR_UNSUPPORTED;
  // Parts per tile (see segment_of), for the residual epilogue: the count up to 4 that makes the walk shortest, as
  // long as a part keeps at least 32 k-blocks (its epilogue hides under the next unit's products) and the walk gets
  // at least 15 % shorter; balance: 0 whole tiles always, 1 the choice described, 2..4 that many parts whatever the
  // gain.  Measured on B200, 2,048 tokens, TFLOP/s whole / in parts: 5,120 x 17,408 (160 tiles, three rounds whole,
  // 2.25 in quarters) 1,285 / 1,380; 5,120 x 8,192 (halves: 2.5 rounds) 1,264 / 1,308; 4,096 x 12,288 (128 tiles,
  // two rounds whole, 1.75 in quarters) 1,378 / 1,366: there the whole-tile walk already runs at the rate the power
  // cap sustains (its idle SMs let the busy ones clock higher), so a shorter walk gains nothing and the extra
  // epilogues cost a little; hence the threshold.
  {
    const long tiles = (long)a.m_tiles * a.n_tiles;
    const int pairs = tiles < sms / 2 ? (int)tiles : sms / 2;
    const int total_kb = (K + BK - 1) / BK;
    int parts = 1;
    if (epi == EPI_RESIDUAL && flags != nullptr && 2 * tiles <= n_flags && balance > 0) {
      if (balance >= 2) {
        parts = balance > 4 ? 4 : balance;
      } else {
        const double whole = (double)((tiles + pairs - 1) / pairs);
        double best = whole;
        for (int p = 2; p <= 4 && total_kb / p >= 32; ++p) {
          const double rounds = (double)((tiles * p + pairs - 1) / pairs) / p;
          if (rounds < best * 0.97 && rounds <= whole * 0.85) { best = rounds; parts = p; }
        }
      }
      if (parts > total_kb) parts = total_kb;
    }
    a.parts = parts;
    a.flags = flags;
  }
  switch (epi) {
    case EPI_STORE_BF16: return launch<EPI_STORE_BF16>(mx, mw, mo, a, sms, stream);
    case EPI_STORE_F32: return launch<EPI_STORE_F32>(mx, mw, mo, a, sms, stream);
    case EPI_RESIDUAL: return launch<EPI_RESIDUAL>(mx, mw, mo, a, sms, stream);
    case EPI_SWIGLU: return launch<EPI_SWIGLU>(mx, mw, mo, a, sms, stream);
    case EPI_HEAD_PREP: return launch<EPI_HEAD_PREP>(mx, mw, mo, a, sms, stream);
  }
  return ODI_ERR_ARGUMENT;
}
