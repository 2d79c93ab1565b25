// bf16 causal grouped-query attention over the paged cache on the tensor cores
// (mma.sync m16n8k16, fp32 accumulation, fp32 running-maximum softmax), in two forms:
//
//  * attention_prefill: a block of 4 warps owns 64 consecutive query tokens of one query
//    head of one sequence (16 rows per warp) and walks the sequence's key pages up to the
//    diagonal; works for any q_len >= 1 on top of any cached length.
//  * attention_decode: one query token per sequence.  A block owns one (sequence, kv head,
//    key split); the rows of its MMA are the query heads that share the kv head (up to 16
//    per block), its 4 warps take 16 keys each of every 64-key page and their partial
//    results are merged in shared memory.  With several splits the block writes its merged
//    (acc[d], max, sum) to global memory and the combine kernel below adds the splits of a
//    (token, head) in order.  Either every sequence is cut into `splits` equal ranges, or every
//    block takes the same number of tiles (planned by the host), so that a long sequence has
//    more blocks than a short one and all blocks end together; the host may then also list the
//    (sequence, split) blocks that have keys, and the grid holds no others in front of them.  Two
//    other ways to merge are kept as options and measured slower on B200: 2..8 splits as a
//    thread-block cluster that adds the partials in rank order through distributed shared memory,
//    and the block that finishes a (sequence, kv head) last (an atomic ticket) merging them.
//
// Key/value pages (64 positions x head_dim, contiguous) reach shared memory in one of two ways.  For head
// sizes 64 and 128 the decode block has a fifth warp whose one thread issues TMA copies into a ring of
// four slots with full/empty mbarriers (attention_decode_tma_kernel: 128-byte swizzle, bounded waits).
// Otherwise, and in the prefill form, the warps copy with cp.async, double or triple buffered, one block
// barrier per tile, into rows padded by 16 bytes so that ldmatrix reads are free of bank conflicts for
// every head size that is a multiple of 16.
//
// Compile with -DODI_HEAD_DIM=<d>, d a multiple of 16 up to 256.  No window, no ring:
// layers that need those use attention_simt.cu.
#include "common.cuh"

#ifndef ODI_HEAD_DIM
#error "compile with -DODI_HEAD_DIM=<head size>"
#endif
#define D ODI_HEAD_DIM
#if (D % 16) != 0 || D > 256
#error "head size must be a multiple of 16, at most 256"
#endif

#define KT 64                      // keys per tile = positions per page
#define ROWB (2 * D + 16)          // bytes per shared-memory row
#define TILE_BYTES (KT * ROWB)
#define KSTEPS (D / 16)
#define DTILES (D / 8)
#define LOG2E 1.4426950408889634f

struct MmaAttnArgs {
  const bf16* q;          // [n_tokens, nq, D]
  const bf16* k_pool;     // [pages, nkv, 64, D]
  const bf16* v_pool;
  bf16* out;              // [n_tokens, nq * D]
  float* partial;         // [n_tokens, nq, splits, D + 2]
  const int* cu_q;
  const int* past;
  const int* page_start;
  const int* page_ids;
  int n_seqs, nq, nkv, splits, head_chunks;
  float scale;
  int clustered;          // decode: the splits of a (sequence, kv head) form a cluster and merge in shared memory
  int* tickets;           // decode with global partials: one counter per (sequence, block row), zero before and
                          // after; the block that finishes a row of splits last merges them (null: a combine kernel does)
  const int* tiles_per_split;   // decode with global partials and the combine kernel: when not null, one int on the
                          // device: every block takes that many tiles of 64 keys, so a sequence of n tiles uses
                          // its first ceil(n / that) splits and its other blocks leave at once (`splits` then only
                          // bounds the count); null: every sequence is cut into `splits` equal ranges
  long pool_rows;         // rows of D in each pool (pages * nkv * 64): the TMA-fed decode kernel maps the pools with it
  int* status;            // error word of the TMA-fed decode kernel's bounded waits (0 = fine); null: that kernel is not used
  int items;              // decode with tiles_per_split: when > 0, tiles_per_split[1] is a count n <= items and
                          // tiles_per_split[2 .. 2 + n) the host's list of the blocks that have keys, one entry per
                          // (sequence, split): sequence << 8 | 128 if it is the sequence's last split | split.  The grid
                          // is then `items` wide and has no block without work among those with work.
  int skip_combine;       // decode with global partials: leave them unmerged (the caller's next kernel merges them)
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
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
__device__ __forceinline__ float ld_peer_f32(const float* local, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_addr(local)), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&v;
}

// Copy one page tile (64 rows of D bf16, contiguous in global memory) into padded rows.
__device__ __forceinline__ void load_tile(uint8_t* dst, const bf16* src, int tid, int nthreads) {
  constexpr int CHUNKS = D / 8;    // 16-byte chunks per row
  const uint32_t base = smem_addr(dst);
  for (int i = tid; i < KT * CHUNKS; i += nthreads) {
    const int r = i / CHUNKS, c = i % CHUNKS;
    cp_async16(base + r * ROWB + c * 16, src + (size_t)r * D + c * 8);
  }
}

// Query rows as A fragments.  Row r of the 16-row MMA tile reads q_row(r) (null: a row of zeros).
// a[ks][0]: row lane/4,     cols ks*16 + (lane%4)*2 + {0,1}     a[ks][1]: row lane/4 + 8, same cols
// a[ks][2]: row lane/4,     cols + 8                             a[ks][3]: row lane/4 + 8, cols + 8
__device__ __forceinline__ void load_q_frags(uint32_t (*a)[4], const bf16* row_lo, const bf16* row_hi, int lane) {
  const int c = (lane & 3) * 2;
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    a[ks][0] = row_lo ? *(const uint32_t*)(row_lo + ks * 16 + c) : 0u;
    a[ks][1] = row_hi ? *(const uint32_t*)(row_hi + ks * 16 + c) : 0u;
    a[ks][2] = row_lo ? *(const uint32_t*)(row_lo + ks * 16 + 8 + c) : 0u;
    a[ks][3] = row_hi ? *(const uint32_t*)(row_hi + ks * 16 + 8 + c) : 0u;
  }
}

// ------------------------------------------------------------------------------ prefill

#define PF_WARPS 4
#define PF_STAGES 2

__global__ void __launch_bounds__(PF_WARPS * 32)
attention_prefill_kernel(MmaAttnArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // heads along x, sequences along y, query tiles along z from the last (the most keys) to the first:
  // blocks are handed out x-fastest, so the long tiles start first and the short ones fill the tail
  const int seq = blockIdx.y, head = blockIdx.x, hk = head / (a.nq / a.nkv);
  const int q_begin = a.cu_q[seq], q_len = a.cu_q[seq + 1] - q_begin;
  const int t0 = (gridDim.z - 1 - blockIdx.z) * 64;
  if (t0 >= q_len) return;
  const int past = a.past[seq];
  const int nt = min(64, q_len - t0);
  const int n_tiles = (past + t0 + nt + KT - 1) / KT;       // keys 0 .. past + t0 + nt - 1
  const int* pages = a.page_ids + a.page_start[seq];

  // this warp's rows: tokens t0 + warp*16 + {lane/4, lane/4 + 8}
  const int r_lo = warp * 16 + (lane >> 2), r_hi = r_lo + 8;
  const bf16* q_lo = r_lo < nt ? a.q + ((size_t)(q_begin + t0 + r_lo) * a.nq + head) * D : nullptr;
  const bf16* q_hi = r_hi < nt ? a.q + ((size_t)(q_begin + t0 + r_hi) * a.nq + head) * D : nullptr;
  uint32_t qf[KSTEPS][4];
  load_q_frags(qf, q_lo, q_hi, lane);
  const int pos_lo = past + t0 + r_lo, pos_hi = past + t0 + r_hi;

  float o[DTILES][4];
#pragma unroll
  for (int i = 0; i < DTILES; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  const float sl2 = a.scale * LOG2E;

  auto issue = [&](int tile) {
    uint8_t* st = smem + (size_t)(tile % PF_STAGES) * 2 * TILE_BYTES;
    const size_t base = ((size_t)pages[tile] * a.nkv + hk) * KT * D;
    load_tile(st, a.k_pool + base, tid, PF_WARPS * 32);
    load_tile(st + TILE_BYTES, a.v_pool + base, tid, PF_WARPS * 32);
    cp_async_commit();
  };
  issue(0);
  for (int tile = 0; tile < n_tiles; ++tile) {
    if (tile + 1 < n_tiles) { issue(tile + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const uint8_t* ks_base = smem + (size_t)(tile % PF_STAGES) * 2 * TILE_BYTES;
    const uint32_t k_smem = smem_addr(ks_base), v_smem = k_smem + TILE_BYTES;
    const int kbase = tile * KT;
    // a warp whose rows all lie before this tile has nothing to add (only on the diagonal tiles)
    const bool active = kbase <= past + t0 + warp * 16 + 15;
    if (active) {
      float s[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
        for (int np = 0; np < 4; ++np) {     // pairs of 8-key tiles
          // matrices: (keys np*16 + 0..7, d ks*16 + 0..7), (same keys, d + 8), (keys + 8, d), (keys + 8, d + 8)
          const int m = lane >> 3, r = lane & 7;
          const int key = np * 16 + (m >> 1) * 8 + r, dd = ks * 16 + (m & 1) * 8;
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(k_smem + key * ROWB + dd * 2, b0, b1, b2, b3);
          mma_bf16(s[np * 2], qf[ks], b0, b1);
          mma_bf16(s[np * 2 + 1], qf[ks], b2, b3);
        }
      }
      // mask, scale into the log2 domain, running maximum
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int kj = kbase + i * 8 + (lane & 3) * 2;
        s[i][0] = (kj <= pos_lo) ? s[i][0] * sl2 : -INFINITY;
        s[i][1] = (kj + 1 <= pos_lo) ? s[i][1] * sl2 : -INFINITY;
        s[i][2] = (kj <= pos_hi) ? s[i][2] * sl2 : -INFINITY;
        s[i][3] = (kj + 1 <= pos_hi) ? s[i][3] * sl2 : -INFINITY;
        mx_lo = fmaxf(mx_lo, fmaxf(s[i][0], s[i][1]));
        mx_hi = fmaxf(mx_hi, fmaxf(s[i][2], s[i][3]));
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
      // rows with nothing visible yet keep a zero accumulator; avoid (-inf) - (-inf)
      const float ref_lo = mn_lo == -INFINITY ? 0.f : mn_lo, ref_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
      const float al_lo = exp2f(m_lo - ref_lo), al_hi = exp2f(m_hi - ref_hi);
      m_lo = mn_lo; m_hi = mn_hi;
      float sum_lo = 0.f, sum_hi = 0.f;
      uint32_t pf[4][4];                  // P as A fragments for the 4 key steps of 16
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float p0 = exp2f(s[i][0] - ref_lo), p1 = exp2f(s[i][1] - ref_lo);
        const float p2 = exp2f(s[i][2] - ref_hi), p3 = exp2f(s[i][3] - ref_hi);
        sum_lo += p0 + p1; sum_hi += p2 + p3;
        pf[i >> 1][(i & 1) * 2] = pack_bf16(p0, p1);
        pf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
      l_lo = l_lo * al_lo + sum_lo; l_hi = l_hi * al_hi + sum_hi;
#pragma unroll
      for (int i = 0; i < DTILES; ++i) { o[i][0] *= al_lo; o[i][1] *= al_lo; o[i][2] *= al_hi; o[i][3] *= al_hi; }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {      // 16 keys per step
#pragma unroll
        for (int dp = 0; dp < DTILES / 2; ++dp) {
          // matrices: (keys kk*16 + 0..7, d dp*16 + 0..7), (keys + 8, same d), (keys, d + 8), (keys + 8, d + 8)
          const int m = lane >> 3, r = lane & 7;
          const int key = kk * 16 + (m & 1) * 8 + r, dd = dp * 16 + (m >> 1) * 8;
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(v_smem + key * ROWB + dd * 2, b0, b1, b2, b3);
          mma_bf16(o[dp * 2], pf[kk], b0, b1);
          mma_bf16(o[dp * 2 + 1], pf[kk], b2, b3);
        }
      }
    }
    __syncthreads();    // the stage may be overwritten by the load after next
  }
  // the row sums live spread over the 4 lanes of a quad
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  const float inv_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
  const int c = (lane & 3) * 2;
  if (r_lo < nt) {
    bf16* dst = a.out + ((size_t)(q_begin + t0 + r_lo) * a.nq + head) * D;
#pragma unroll
    for (int i = 0; i < DTILES; ++i) *(uint32_t*)(dst + i * 8 + c) = pack_bf16(o[i][0] * inv_lo, o[i][1] * inv_lo);
  }
  if (r_hi < nt) {
    bf16* dst = a.out + ((size_t)(q_begin + t0 + r_hi) * a.nq + head) * D;
#pragma unroll
    for (int i = 0; i < DTILES; ++i) *(uint32_t*)(dst + i * 8 + c) = pack_bf16(o[i][2] * inv_hi, o[i][3] * inv_hi);
  }
}

// ------------------------------------------------------------------------------ decode

// Merge the split partials of one (token, head) row: out = sum_s e^(m_s - M) acc_s / sum_s e^(m_s - M) l_s,
// the splits in order.  `first`, `step`: which elements of the row this thread writes.
// No load sits behind a branch, so the loads of a pass over the splits are in flight together, four splits
// at a time: the merge costs a few round trips to L2, not one per split.  (Unrolled by eight, the common
// case of four splits ran in the remainder loop, one load after another: 19.1 against 17.4 us at 8 x 2048.)
__device__ __forceinline__ void combine_row(const float* p, bf16* out_row, int splits, int first, int step) {
  float M = -INFINITY;
#pragma unroll 4
  for (int s = 0; s < splits; ++s) M = fmaxf(M, __ldcg(p + s * (D + 2) + D));
  float denom = 0.f;
#pragma unroll 4
  for (int s = 0; s < splits; ++s) {
    const float ms = __ldcg(p + s * (D + 2) + D), ls = __ldcg(p + s * (D + 2) + D + 1);
    denom += ms != -INFINITY ? expf(ms - M) * ls : 0.f;
  }
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
  for (int dd = first; dd < D; dd += step) {
    float v = 0.f;
#pragma unroll 4
    for (int s = 0; s < splits; ++s) {
      const float ms = __ldcg(p + s * (D + 2) + D), x = __ldcg(p + s * (D + 2) + dd);
      v += ms != -INFINITY ? expf(ms - M) * x : 0.f;      // an empty split (max -inf) adds nothing, whatever it holds
    }
    out_row[dd] = __float2bfloat16_rn(v * inv);
  }
}


#define DC_WARPS 4
#ifndef DC_STAGES
#define DC_STAGES (D <= 128 ? 3 : 2)
#endif

// Tiles of 64 keys that one block of a sequence of n_tiles takes.  *wanted is written by the host before
// the launch (no kernel writes it); whatever it holds, `splits` blocks cover the sequence.
__device__ __forceinline__ int tiles_of_a_split(const int* wanted, int splits, int n_tiles) {
  const int even = (n_tiles + splits - 1) / splits;
  return wanted != nullptr ? max(*wanted, even) : even;
}

// Which (sequence, split) a decode block works on; false if it has nothing to do.  Without a list the grid has
// one block per sequence and split up to the bound, and a short sequence's surplus blocks leave at once.  Those
// blocks are not free: each takes a place on an SM for about a microsecond, and a place beside a block that
// streams keys took only about three of them before it stayed empty until that block ended (16 sequences of 128
// to 4,096 keys, 8 kv heads, 15 tiles a block: blocks of the last splits started up to 23 us late behind them, 32 us
// for the whole kernel against 27 us).  With the host's list every block in front of the grid has keys.
#define DC_ERR_PLAN 33
__device__ __forceinline__ bool decode_block_item(const MmaAttnArgs& a, int& seq, int& split, bool& last_listed) {
  last_listed = false;
  if (a.items > 0) {
    if ((int)blockIdx.x >= a.tiles_per_split[1]) return false;
    const int packed = a.tiles_per_split[2 + blockIdx.x];
    seq = packed >> 8;
    split = packed & 127;
    last_listed = (packed & 128) != 0;
    return true;
  }
  // launched sequence by sequence for a cluster (its members must be neighbours in x), split by split otherwise
  seq = a.clustered ? blockIdx.z : blockIdx.x;
  split = a.clustered ? blockIdx.x : blockIdx.z;
  return true;
}
// The host's list must cover what the device's lengths ask for: a sequence whose last listed block ends before
// its keys do would lose keys, so that block reports it instead (the step's status word; the host raises).
__device__ __forceinline__ void decode_check_plan(const MmaAttnArgs& a, bool last_listed, int tile_end, int n_tiles) {
  if (last_listed && tile_end < n_tiles && a.status != nullptr && threadIdx.x == 0) atomicCAS(a.status, 0, DC_ERR_PLAN);
}

// The end of a decode block: the four warps (each saw a quarter of the keys of every tile) merge their running
// (acc, max, sum) through shared memory, and the block's result goes out: the final bf16 rows when the block saw
// the whole sequence, its partial (in the natural-log domain of the combine kernel) otherwise, or stays in shared
// memory for a cluster.  `smem` must be free of tiles: every copy has landed and every warp has left the last tile.
__device__ __forceinline__ void decode_merge_warps(const MmaAttnArgs& a, uint8_t* smem, float (&o)[DTILES][4],
                                                   float m_lo, float m_hi, float l_lo, float l_hi, int warp, int lane,
                                                   int tok, int head0, int heads_here, int split) {
  const int r_lo = lane >> 2, r_hi = r_lo + 8;
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

  // Merge the four warps (each saw a quarter of the keys): [warp][row][D + 2] floats in shared memory.
  float* mg = (float*)smem;
  constexpr int RS = D + 2;
  asm volatile("bar.sync 1, 128;" ::: "memory");      // the four compute warps
  {
    const int c = (lane & 3) * 2;
    float* lo = mg + ((size_t)warp * 16 + r_lo) * RS;
    float* hi = mg + ((size_t)warp * 16 + r_hi) * RS;
#pragma unroll
    for (int i = 0; i < DTILES; ++i) {
      lo[i * 8 + c] = o[i][0]; lo[i * 8 + c + 1] = o[i][1];
      hi[i * 8 + c] = o[i][2]; hi[i * 8 + c + 1] = o[i][3];
    }
    if ((lane & 3) == 0) { lo[D] = m_lo; lo[D + 1] = l_lo; hi[D] = m_hi; hi[D + 1] = l_hi; }
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");      // the four compute warps
  for (int row = warp; row < heads_here; row += DC_WARPS) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DC_WARPS; ++w) M = fmaxf(M, mg[((size_t)w * 16 + row) * RS + D]);
    float wgt[DC_WARPS], L = 0.f;
#pragma unroll
    for (int w = 0; w < DC_WARPS; ++w) {
      const float mw = mg[((size_t)w * 16 + row) * RS + D];
      wgt[w] = mw == -INFINITY ? 0.f : exp2f(mw - M);
      L += wgt[w] * mg[((size_t)w * 16 + row) * RS + D + 1];
    }
    const int head = head0 + row;
    if (a.clustered) {
      // this split's merged partial stays in shared memory, behind the four warps' area
      float* fin = mg + (size_t)DC_WARPS * 16 * RS + (size_t)row * RS;
      for (int dd = lane; dd < D; dd += 32) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < DC_WARPS; ++w) v += wgt[w] * mg[((size_t)w * 16 + row) * RS + dd];
        fin[dd] = v;
      }
      if (lane == 0) { fin[D] = M; fin[D + 1] = L; }
    } else if (a.splits == 1) {
      const float inv = L > 0.f ? 1.f / L : 0.f;
      bf16* dst = a.out + ((size_t)tok * a.nq + head) * D;
      for (int dd = lane; dd < D; dd += 32) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < DC_WARPS; ++w) v += wgt[w] * mg[((size_t)w * 16 + row) * RS + dd];
        dst[dd] = __float2bfloat16_rn(v * inv);
      }
    } else {
      // partial in the natural-log domain of the combine kernel: max * ln 2
      float* dst = a.partial + (((size_t)tok * a.nq + head) * a.splits + split) * RS;
      for (int dd = lane; dd < D; dd += 32) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < DC_WARPS; ++w) v += wgt[w] * mg[((size_t)w * 16 + row) * RS + dd];
        dst[dd] = v;
      }
      if (lane == 0) { dst[D] = M == -INFINITY ? -INFINITY : M * 0.6931471805599453f; dst[D + 1] = L; }
    }
  }
}

__global__ void __launch_bounds__(DC_WARPS * 32)
attention_decode_kernel(MmaAttnArgs a) {
  pdl_launch_dependents();
  // What follows up to pdl_wait() reads only what no kernel of this step writes: the step's index
  // arrays and the cache pages that earlier steps filled.  The page that holds the query's own
  // position is written by the kernel before this one, so it is never requested ahead of the wait.
  extern __shared__ __align__(16) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int seq, split;
  bool last_listed;
  if (!decode_block_item(a, seq, split, last_listed)) return;
  const int hk = blockIdx.y / a.head_chunks, chunk = blockIdx.y % a.head_chunks;
  const int g = a.nq / a.nkv;
  const int heads_here = min(16, g - chunk * 16);
  const int head0 = hk * g + chunk * 16;
  const int tok = a.cu_q[seq];
  const int pos = a.past[seq];                     // the query's position; keys 0 .. pos are visible
  const int n_tiles = pos / KT + 1;
  const int per_split = tiles_of_a_split(a.tiles_per_split, a.splits, n_tiles);
  const int tile_begin = split * per_split, tile_end = min(n_tiles, tile_begin + per_split);
  if (a.tiles_per_split != nullptr && split > 0 && tile_begin >= n_tiles) return;   // a shorter sequence needs fewer blocks
  decode_check_plan(a, last_listed, tile_end, n_tiles);
  const int* pages = a.page_ids + a.page_start[seq];

  auto issue = [&](int tile) {
    uint8_t* st = smem + (size_t)((tile - tile_begin) % DC_STAGES) * 2 * TILE_BYTES;
    const size_t base = ((size_t)pages[tile] * a.nkv + hk) * KT * D;
    load_tile(st, a.k_pool + base, tid, DC_WARPS * 32);
    load_tile(st + TILE_BYTES, a.v_pool + base, tid, DC_WARPS * 32);
  };
  // prologue: DC_STAGES - 1 tiles in flight (empty groups keep the group count uniform)
  bool early[DC_STAGES - 1];
#pragma unroll
  for (int i = 0; i < DC_STAGES - 1; ++i) {
    early[i] = tile_begin + i < tile_end && tile_begin + i < n_tiles - 1;   // not the page of the query itself
    if (early[i]) issue(tile_begin + i);
  }
  pdl_wait();
#pragma unroll
  for (int i = 0; i < DC_STAGES - 1; ++i) {
    if (!early[i] && tile_begin + i < tile_end) issue(tile_begin + i);
    cp_async_commit();
  }

  // rows of the MMA tile are query heads
  const int r_lo = lane >> 2, r_hi = r_lo + 8;
  const bf16* q_lo = r_lo < heads_here ? a.q + ((size_t)tok * a.nq + head0 + r_lo) * D : nullptr;
  const bf16* q_hi = r_hi < heads_here ? a.q + ((size_t)tok * a.nq + head0 + r_hi) * D : nullptr;
  uint32_t qf[KSTEPS][4];
  load_q_frags(qf, q_lo, q_hi, lane);

  float o[DTILES][4];
#pragma unroll
  for (int i = 0; i < DTILES; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  const float sl2 = a.scale * LOG2E;

  for (int tile = tile_begin; tile < tile_end; ++tile) {
    // One barrier per tile: after it this tile's copies are visible to all warps and all warps have left
    // the tile before, whose stage the next request overwrites.
    cp_async_wait<DC_STAGES - 2>();
    __syncthreads();
    if (tile + DC_STAGES - 1 < tile_end) issue(tile + DC_STAGES - 1);
    cp_async_commit();
    const uint8_t* st = smem + (size_t)((tile - tile_begin) % DC_STAGES) * 2 * TILE_BYTES;
    const uint32_t k_smem = smem_addr(st), v_smem = k_smem + TILE_BYTES;
    const int kbase = tile * KT + warp * 16;        // this warp's 16 keys
    if (kbase <= pos) {
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        const int m = lane >> 3, r = lane & 7;
        const int key = warp * 16 + (m >> 1) * 8 + r, dd = ks * 16 + (m & 1) * 8;
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(k_smem + key * ROWB + dd * 2, b0, b1, b2, b3);
        mma_bf16(s[0], qf[ks], b0, b1);
        mma_bf16(s[1], qf[ks], b2, b3);
      }
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int kj = kbase + i * 8 + (lane & 3) * 2;
        s[i][0] = (kj <= pos) ? s[i][0] * sl2 : -INFINITY;
        s[i][1] = (kj + 1 <= pos) ? s[i][1] * sl2 : -INFINITY;
        s[i][2] = (kj <= pos) ? s[i][2] * sl2 : -INFINITY;
        s[i][3] = (kj + 1 <= pos) ? s[i][3] * sl2 : -INFINITY;
        mx_lo = fmaxf(mx_lo, fmaxf(s[i][0], s[i][1]));
        mx_hi = fmaxf(mx_hi, fmaxf(s[i][2], s[i][3]));
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);   // finite: key kbase is visible
      const float al_lo = exp2f(m_lo - mn_lo), al_hi = exp2f(m_hi - mn_hi);
      m_lo = mn_lo; m_hi = mn_hi;
      uint32_t pf[4];
      float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float p0 = exp2f(s[i][0] - mn_lo), p1 = exp2f(s[i][1] - mn_lo);
        const float p2 = exp2f(s[i][2] - mn_hi), p3 = exp2f(s[i][3] - mn_hi);
        sum_lo += p0 + p1; sum_hi += p2 + p3;
        pf[i * 2] = pack_bf16(p0, p1);
        pf[i * 2 + 1] = pack_bf16(p2, p3);
      }
      l_lo = l_lo * al_lo + sum_lo; l_hi = l_hi * al_hi + sum_hi;
#pragma unroll
      for (int i = 0; i < DTILES; ++i) { o[i][0] *= al_lo; o[i][1] *= al_lo; o[i][2] *= al_hi; o[i][3] *= al_hi; }
#pragma unroll
      for (int dp = 0; dp < DTILES / 2; ++dp) {
        const int m = lane >> 3, r = lane & 7;
        const int key = warp * 16 + (m & 1) * 8 + r, dd = dp * 16 + (m >> 1) * 8;
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(v_smem + key * ROWB + dd * 2, b0, b1, b2, b3);
        mma_bf16(o[dp * 2], pf, b0, b1);
        mma_bf16(o[dp * 2 + 1], pf, b2, b3);
      }
    }
  }
  cp_async_wait<0>();
  decode_merge_warps(a, smem, o, m_lo, m_hi, l_lo, l_hi, warp, lane, tok, head0, heads_here, split);
  float* mg = (float*)smem;
  constexpr int RS = D + 2;
  if (a.splits > 1 && !a.clustered && a.tickets != nullptr) {
    // Whoever publishes the last partial of this (sequence, block row) merges them: nobody waits, and the
    // merge reads the splits in order, so the result does not depend on who came last.
    __shared__ int last_block;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      int* ticket = a.tickets + (size_t)seq * gridDim.y + blockIdx.y;
      last_block = atomicAdd(ticket, 1) == a.splits - 1;
      if (last_block) *ticket = 0;                 // ready for the next launch
    }
    __syncthreads();
    if (last_block) {
      __threadfence();
      for (int row = warp; row < heads_here; row += DC_WARPS) {
        const size_t r = (size_t)tok * a.nq + head0 + row;
        combine_row(a.partial + r * a.splits * RS, a.out + r * D, a.splits, lane, 32);
      }
    }
  }
  if (a.clustered) {
    // every thread of every block of the cluster takes part in both barriers
    __syncwarp();
    cluster_sync_all();
    const float* fin = mg + (size_t)DC_WARPS * 16 * RS;
    const uint32_t rank = cluster_rank();
    for (int row = (int)rank + a.splits * warp; row < heads_here; row += a.splits * DC_WARPS) {
      const float* mine = fin + (size_t)row * RS;
      float M = -INFINITY;
      for (int p = 0; p < a.splits; ++p) M = fmaxf(M, ld_peer_f32(mine + D, (uint32_t)p));
      float L = 0.f;
      for (int p = 0; p < a.splits; ++p) {            // rank order: a fixed sum
        const float mp = ld_peer_f32(mine + D, (uint32_t)p);
        if (mp != -INFINITY) L += exp2f(mp - M) * ld_peer_f32(mine + D + 1, (uint32_t)p);
      }
      const float inv = L > 0.f ? 1.f / L : 0.f;
      bf16* dst = a.out + ((size_t)tok * a.nq + head0 + row) * D;
      for (int dd = lane; dd < D; dd += 32) {
        float v = 0.f;
        for (int p = 0; p < a.splits; ++p) {
          const float mp = ld_peer_f32(mine + D, (uint32_t)p);
          if (mp != -INFINITY) v += exp2f(mp - M) * ld_peer_f32(mine + dd, (uint32_t)p);
        }
        dst[dd] = __float2bfloat16_rn(v * inv);
      }
    }
    __syncwarp();
    cluster_sync_all();     // nobody leaves while its shared memory may still be read
  }
}

// ------------------------------------------------------------------------------ decode, TMA-fed
//
// The same split-key decode block with its key/value tiles brought by the tensor-memory accelerator instead of by
// the compute warps: a fifth warp's one thread issues cp.async.bulk.tensor loads (boxes of 64 positions x 64 lanes
// of the head, 128-byte swizzle, no multicast) into a ring of TD_SLOTS slots, a slot being the 64 x D keys or the
// 64 x D values of one page; each slot has a `full` barrier (the copy's bytes) and an `empty` barrier (the four
// compute warps, each when it has read the slot).  Against the cp.async form: a key slot is free again as soon as
// the scores exist, the warps meet at no block barrier per tile, and the compute warps issue no copies.  Four
// slots (64 KB, three of them in flight) measured best on whole decode steps at Qwen3-8B sizes: 3 / 4 / 5 / 6 slots
// gave 3.437 / 3.425 / 3.435 / 3.442 ms a step at 8 x 2,048 keys, 9.2 / 9.1 / - / 9.6 ms at 32 x 8,192 and 9.0 / 8.8 /
// - / 9.0 ms at 8 x 32,768 (a smaller block leaves the kernels before and after it room on the SM to move in and
// out), although the kernel alone streams a little faster with six.  Three blocks an SM (128 registers, no spills,
// 65 KB each) were slower everywhere (batch 64: 8,616 against 9,112 tokens/s).  Pages that earlier steps filled are
// requested before the
// dependency wait; the page of the query's own position after it.  Every wait is bounded (about two seconds), after
// which the block records who gave up in `status`, skips its work and leaves.  Head sizes 64 and 128.
#if D == 64 || D == 128
#include <cuda.h>

#ifndef TD_SLOTS
#define TD_SLOTS 4
#endif
#define TD_BOXES (D / 64)                 // boxes of 64 lanes (128 bytes) per row of the head
#define TD_BOX_BYTES (KT * 128)           // 64 rows of 128 bytes
#define TD_SLOT_BYTES (TD_BOXES * TD_BOX_BYTES)
#define TD_THREADS (DC_WARPS * 32 + 32)
#define TD_WAIT_CYCLES 4000000000ll
#define TD_ERR_PRODUCER 31
#define TD_ERR_CONSUMER 32

__device__ __forceinline__ void td_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void td_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void td_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool td_mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait; false when it gave up (it then records `code`) or when somebody else already has.
__device__ __forceinline__ bool td_mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  const long long start = clock64();
  for (uint32_t i = 0;; ++i) {
    if (td_mbar_test(bar, parity)) return true;
    if ((i & 0xf) == 0xf) {
      if (*abort_flag) return false;
      if (clock64() - start > TD_WAIT_CYCLES) break;
    }
  }
  atomicCAS(status, 0, code);
  __threadfence_block();
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void td_tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// Address of the 16-byte chunk `chunk` (8 lanes of the head) of row `row` in a slot written by TMA with the
// 128-byte swizzle: boxes of 64 lanes, rows of 128 bytes, the chunk index within a row XOR the row's low bits.
__device__ __forceinline__ uint32_t td_chunk_addr(uint32_t slot, int row, int chunk) {
  return slot + (uint32_t)(chunk >> 3) * TD_BOX_BYTES + (uint32_t)row * 128u + (uint32_t)(((chunk & 7) ^ (row & 7)) << 4);
}

__global__ void __launch_bounds__(TD_THREADS)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            MmaAttnArgs a) {
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t bars[2 * TD_SLOTS];
  __shared__ int abort_flag;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int seq, split;
  bool last_listed;
  if (!decode_block_item(a, seq, split, last_listed)) return;
  const int hk = blockIdx.y / a.head_chunks, chunk = blockIdx.y % a.head_chunks;
  const int g = a.nq / a.nkv;
  const int heads_here = min(16, g - chunk * 16);
  const int head0 = hk * g + chunk * 16;
  const int tok = a.cu_q[seq];
  const int pos = a.past[seq];                     // the query's position; keys 0 .. pos are visible
  const int n_tiles = pos / KT + 1;
  const int per_split = tiles_of_a_split(a.tiles_per_split, a.splits, n_tiles);
  const int tile_begin = split * per_split, tile_end = min(n_tiles, tile_begin + per_split);
  if (a.tiles_per_split != nullptr && split > 0 && tile_begin >= n_tiles) return;   // a shorter sequence needs fewer blocks
  decode_check_plan(a, last_listed, tile_end, n_tiles);
  const int* pages = a.page_ids + a.page_start[seq];
  const int my_tiles = max(tile_end - tile_begin, 0);
  const uint32_t full0 = smem_addr(&bars[0]), empty0 = smem_addr(&bars[TD_SLOTS]);
  const uint32_t ring = smem_addr(smem);
  if (tid == 0) {
    for (int s = 0; s < TD_SLOTS; ++s) { td_mbar_init(full0 + 8 * s, 1); td_mbar_init(empty0 + 8 * s, DC_WARPS); }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  volatile int* abort_ptr = &abort_flag;

  float o[DTILES][4];
#pragma unroll
  for (int i = 0; i < DTILES; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

  if (warp == DC_WARPS) {
    // producer: item 2 t is the key slot of the block's t-th tile, item 2 t + 1 its value slot.  The warp reads
    // the page numbers of 32 tiles at a time in one round trip; one thread issues the copies.
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    }
    bool waited = false, ok = true;
    for (int base = 0; base < my_tiles && ok; base += 32) {
      const int my_page = base + lane < my_tiles ? pages[tile_begin + base + lane] : 0;
      const int here = min(32, my_tiles - base);
      for (int j = 0; j < here && ok; ++j) {
        const int page = __shfl_sync(0xffffffffu, my_page, j);
        if (lane == 0) {
          const int tile = tile_begin + base + j;
          if (tile == n_tiles - 1 && !waited) { pdl_wait(); waited = true; }     // the page written in this step
          const int row = (page * a.nkv + hk) * KT;
#pragma unroll
          for (int kv = 0; kv < 2; ++kv) {
            const int item = 2 * (base + j) + kv, s = item % TD_SLOTS;
            if (item >= TD_SLOTS &&
                !td_mbar_wait(empty0 + 8 * s, ((uint32_t)(item / TD_SLOTS) & 1u) ^ 1u, abort_ptr, a.status, TD_ERR_PRODUCER)) {
              ok = false;
              break;
            }
            const uint32_t dst = ring + (uint32_t)s * TD_SLOT_BYTES;
            td_mbar_expect_tx(full0 + 8 * s, TD_SLOT_BYTES);
#pragma unroll
            for (int b = 0; b < TD_BOXES; ++b)
              td_tma_load_2d(dst + b * TD_BOX_BYTES, kv ? &map_v : &map_k, 64 * b, row, full0 + 8 * s);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      }
    }
  } else {
    pdl_wait();                                     // the query comes from the kernel before
    const int r_lo = lane >> 2, r_hi = r_lo + 8;    // rows of the MMA tile are query heads
    const bf16* q_lo = r_lo < heads_here ? a.q + ((size_t)tok * a.nq + head0 + r_lo) * D : nullptr;
    const bf16* q_hi = r_hi < heads_here ? a.q + ((size_t)tok * a.nq + head0 + r_hi) * D : nullptr;
    uint32_t qf[KSTEPS][4];
    load_q_frags(qf, q_lo, q_hi, lane);
    const float sl2 = a.scale * LOG2E;
    bool ok = true;
    for (int t = 0; t < my_tiles && ok; ++t) {
      const int tile = tile_begin + t;
      const int ik = 2 * t, iv = 2 * t + 1;
      const int sk = ik % TD_SLOTS, sv = iv % TD_SLOTS;
      const int kbase = tile * KT + warp * 16;      // this warp's 16 keys
      const bool mine = kbase <= pos;               // some of them are visible
      uint32_t pf[4];
      if (!td_mbar_wait(full0 + 8 * sk, (uint32_t)(ik / TD_SLOTS) & 1u, abort_ptr, a.status, TD_ERR_CONSUMER)) { ok = false; break; }
      if (mine) {
        const uint32_t k_slot = ring + (uint32_t)sk * TD_SLOT_BYTES;
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
          const int m = lane >> 3, r = lane & 7;
          const int key = warp * 16 + (m >> 1) * 8 + r, ch = ks * 2 + (m & 1);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(td_chunk_addr(k_slot, key, ch), b0, b1, b2, b3);
          mma_bf16(s[0], qf[ks], b0, b1);
          mma_bf16(s[1], qf[ks], b2, b3);
        }
        __syncwarp();
        if (lane == 0) td_mbar_arrive(empty0 + 8 * sk);          // the scores exist: the key slot may be refilled
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int kj = kbase + i * 8 + (lane & 3) * 2;
          s[i][0] = (kj <= pos) ? s[i][0] * sl2 : -INFINITY;
          s[i][1] = (kj + 1 <= pos) ? s[i][1] * sl2 : -INFINITY;
          s[i][2] = (kj <= pos) ? s[i][2] * sl2 : -INFINITY;
          s[i][3] = (kj + 1 <= pos) ? s[i][3] * sl2 : -INFINITY;
          mx_lo = fmaxf(mx_lo, fmaxf(s[i][0], s[i][1]));
          mx_hi = fmaxf(mx_hi, fmaxf(s[i][2], s[i][3]));
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);   // finite: key kbase is visible
        const float al_lo = exp2f(m_lo - mn_lo), al_hi = exp2f(m_hi - mn_hi);
        m_lo = mn_lo; m_hi = mn_hi;
        float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float p0 = exp2f(s[i][0] - mn_lo), p1 = exp2f(s[i][1] - mn_lo);
          const float p2 = exp2f(s[i][2] - mn_hi), p3 = exp2f(s[i][3] - mn_hi);
          sum_lo += p0 + p1; sum_hi += p2 + p3;
          pf[i * 2] = pack_bf16(p0, p1);
          pf[i * 2 + 1] = pack_bf16(p2, p3);
        }
        l_lo = l_lo * al_lo + sum_lo; l_hi = l_hi * al_hi + sum_hi;
#pragma unroll
        for (int i = 0; i < DTILES; ++i) { o[i][0] *= al_lo; o[i][1] *= al_lo; o[i][2] *= al_hi; o[i][3] *= al_hi; }
      } else {
        __syncwarp();
        if (lane == 0) td_mbar_arrive(empty0 + 8 * sk);
      }
      if (!td_mbar_wait(full0 + 8 * sv, (uint32_t)(iv / TD_SLOTS) & 1u, abort_ptr, a.status, TD_ERR_CONSUMER)) { ok = false; break; }
      if (mine) {
        const uint32_t v_slot = ring + (uint32_t)sv * TD_SLOT_BYTES;
#pragma unroll
        for (int dp = 0; dp < DTILES / 2; ++dp) {
          const int m = lane >> 3, r = lane & 7;
          const int key = warp * 16 + (m & 1) * 8 + r, ch = dp * 2 + (m >> 1);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(td_chunk_addr(v_slot, key, ch), b0, b1, b2, b3);
          mma_bf16(o[dp * 2], pf, b0, b1);
          mma_bf16(o[dp * 2 + 1], pf, b2, b3);
        }
      }
      __syncwarp();
      if (lane == 0) td_mbar_arrive(empty0 + 8 * sv);
    }
  }
  // Every copy that was requested has landed (each was waited for) unless somebody gave up; then nothing is
  // written.  The ring is free for the merge of the warps.
  __syncthreads();
  if (abort_flag || warp == DC_WARPS) return;
  decode_merge_warps(a, smem, o, m_lo, m_hi, l_lo, l_hi, warp, lane, tok, head0, heads_here, split);
}
#endif

// One block per (token, head).  With `tiles_per_split` a row has the partials of its sequence's first
// ceil(tiles / *tiles_per_split) splits only (one token per sequence: the token's index is the sequence's).
// Up to 32 splits: every thread requests its element of all splits, and the first warp every split's maximum and
// sum, in the same round trip as the position that says how many splits count; the first warp leaves the weights
// in shared memory and every thread adds its elements in split order: one round trip to L2 whatever the number
// of splits (combine_row walks the splits three times, four loads at a time: with the 17 splits of one sequence
// of 2,048 keys that took as long as the attention itself).
__global__ void attention_mma_combine_kernel(const float* __restrict__ partial, bf16* __restrict__ out, int splits,
                                             const int* __restrict__ past, int nq, const int* __restrict__ tiles_per_split) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = blockIdx.x;
  constexpr int RS = D + 2;
  const float* p = partial + row * splits * RS;
  if (splits > 32) {
    int used = splits;
    if (tiles_per_split != nullptr) used = merge_used_splits(tiles_per_split, splits, past[row / nq]);
    combine_row(p, out + row * D, used, threadIdx.x, blockDim.x);
    return;
  }
  // Everything the block reads is requested at once, before any of it is used: this thread's element of every
  // split up to the bound, the splits' statistics (first warp), and the position that says how many splits count.
  // Slots behind the count hold whatever the buffer held; they are loaded and never used.
  float x[32];
  const int dd0 = threadIdx.x;
#pragma unroll
  for (int s = 0; s < 32; ++s) x[s] = (s < splits && dd0 < D) ? __ldcg(p + s * RS + dd0) : 0.f;
  float ms = -INFINITY, ls = 0.f;
  if (threadIdx.x < 32 && (int)threadIdx.x < splits) {
    ms = __ldcg(p + threadIdx.x * RS + D);
    ls = __ldcg(p + threadIdx.x * RS + D + 1);
  }
  int used = splits;
  if (tiles_per_split != nullptr) used = merge_used_splits(tiles_per_split, splits, past[row / nq]);
  __shared__ float weight[32];
  __shared__ float inv_denom;
  if (threadIdx.x < 32) {
    const int s = threadIdx.x;
    if (s >= used) ms = -INFINITY;
    const float M = warp_max(ms);
    // every product and sum below is written as the one instruction it is, so that the output projection's
    // merge prologue (gemm_tcgen05.cu), which does the same sums thread by thread, gives the same bits
    const float w = ms != -INFINITY ? expf(ms - M) : 0.f;       // an empty split (max -inf) adds nothing
    const float wl = ms != -INFINITY ? __fmul_rn(w, ls) : 0.f;
    float denom = 0.f;
    for (int i = 0; i < used; ++i) denom = __fadd_rn(denom, __shfl_sync(0xffffffffu, wl, i));     // in split order
    weight[s] = w;
    if (s == 0) inv_denom = denom > 0.f ? 1.f / denom : 0.f;
  }
  __syncthreads();
  const float inv = inv_denom;
  for (int dd = dd0; dd < D; dd += blockDim.x) {
    if (dd != dd0) {
#pragma unroll
      for (int s = 0; s < 32; ++s) x[s] = s < used ? __ldcg(p + s * RS + dd) : 0.f;
    }
    float v = 0.f;
#pragma unroll
    for (int s = 0; s < 32; ++s)
      if (s < used && weight[s] > 0.f) v = __fmaf_rn(weight[s], x[s], v);      // whatever an empty split's slot holds, it is not read into the sum
    out[row * D + dd] = __float2bfloat16_rn(__fmul_rn(v, inv));
  }
}

extern "C" int odi_attention_mma_head_dim() { return D; }

// Dynamic shared memory of the decode kernel: the ring of K/V stages, or, if larger, the four warps'
// partials plus the block's merged one.  Every launcher of the kernel takes it from here.
static inline int decode_smem_bytes() {
  const int ring = DC_STAGES * 2 * TILE_BYTES;
  const int merge = (DC_WARPS + 1) * 16 * (D + 2) * 4;
  return ring > merge ? ring : merge;
}

#if D == 64 || D == 128
typedef CUresult (*TdEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// A pool as a [rows, D] row-major bf16 matrix cut into boxes of 64 rows x 64 lanes (128 bytes) with the 128-byte swizzle.
static int td_make_map(CUtensorMap* map, const void* base, long rows) {
  static TdEncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (TdEncodeTiledFn)p;
  }
  if (fn == nullptr || ((uintptr_t)base & 15)) return ODI_ERR_UNSUPPORTED;
  cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)D * 2};
  cuuint32_t box[2] = {64, KT};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : ODI_ERR_ARGUMENT;
}

// ODI_DECODE_ATTENTION=cp keeps the cp.async form (for comparisons); anything else, or nothing: the TMA-fed form.
static bool decode_by_tma() {
  static int choice = -1;
  if (choice < 0) {
    const char* e = getenv("ODI_DECODE_ATTENTION");
    choice = (e != nullptr && e[0] == 'c') ? 0 : 1;
  }
  return choice == 1;
}
#endif

// decode != 0 requires q_len == 1 for every sequence (max_q_len == 1).
extern "C" int odi_attention_mma(const MmaAttnArgs* args, int max_q_len, int n_tokens, int decode,
                                 cudaStream_t stream) {
  MmaAttnArgs a = *args;
  if (a.n_seqs <= 0 || n_tokens <= 0) return 0;
  if (a.nq % a.nkv != 0 || a.n_seqs > 65535 || a.splits < 1) return ODI_ERR_UNSUPPORTED;
  const int g = a.nq / a.nkv;
  static bool configured = false;
  const int pf_smem = PF_STAGES * 2 * TILE_BYTES;
  const int dc_smem = decode_smem_bytes();
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pf_smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dc_smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  if (!decode) {
    if (a.splits != 1 || a.nq > 65535) return ODI_ERR_UNSUPPORTED;
    if ((max_q_len + 63) / 64 > 65535) return ODI_ERR_UNSUPPORTED;
    dim3 grid(a.nq, a.n_seqs, (max_q_len + 63) / 64);
    odi_rc = launch_pdl((attention_prefill_kernel), dim3(grid), dim3(PF_WARPS * 32), pf_smem, stream, a);
    return launch_status();
  }
  if (max_q_len != 1) return ODI_ERR_ARGUMENT;
  a.clustered = (a.clustered && a.splits > 1 && a.splits <= 8) ? 1 : 0;
  if (a.splits > 1 && !a.clustered && a.partial == nullptr) return ODI_ERR_ARGUMENT;
  if (a.tiles_per_split != nullptr && (a.clustered || a.tickets != nullptr)) return ODI_ERR_ARGUMENT;
  if (a.items < 0 || (a.items > 0 && a.tiles_per_split == nullptr)) return ODI_ERR_ARGUMENT;
  a.head_chunks = (g + 15) / 16;
  dim3 grid(a.splits, a.nkv * a.head_chunks, a.n_seqs);
  if (!a.clustered) grid = dim3(a.n_seqs, a.nkv * a.head_chunks, a.splits);      // see decode_block_item
  if (a.items > 0) grid = dim3(a.items, a.nkv * a.head_chunks, 1);
  if (grid.y > 65535 || grid.z > 65535) return ODI_ERR_UNSUPPORTED;
  if (a.clustered) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(DC_WARPS * 32);
    cfg.dynamicSmemBytes = dc_smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled();
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = a.splits;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    odi_rc = (int)cudaLaunchKernelEx(&cfg, attention_decode_kernel, a);
    return launch_status();
  }
#if D == 64 || D == 128
  if (a.tickets == nullptr && a.status != nullptr && a.pool_rows > 0 && decode_by_tma()) {
    // the TMA-fed form: the pools as [pool_rows, D] matrices cut into boxes of 64 rows x 64 lanes
    CUtensorMap map_k, map_v;
    int rc = td_make_map(&map_k, a.k_pool, a.pool_rows);
    if (rc == 0) rc = td_make_map(&map_v, a.v_pool, a.pool_rows);
    if (rc != 0) return rc;
    constexpr int TD_SMEM = TD_SLOTS * TD_SLOT_BYTES + 1024;
    static_assert(TD_SLOTS * TD_SLOT_BYTES >= (DC_WARPS + 1) * 16 * (D + 2) * 4, "the merge of the warps reuses the ring");
    static bool td_configured = false;
    if (!td_configured) {
      cudaError_t e = cudaFuncSetAttribute(attention_decode_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TD_SMEM);
      if (e != cudaSuccess) return (int)e;
      td_configured = true;
    }
    odi_rc = launch_pdl((attention_decode_tma_kernel), dim3(grid), dim3(TD_THREADS), TD_SMEM, stream, map_k, map_v, a);
  } else
#endif
  odi_rc = launch_pdl((attention_decode_kernel), dim3(grid), dim3(DC_WARPS * 32), dc_smem, stream, a);
  int rc = launch_status();
  if (rc != 0 || a.splits == 1 || a.tickets != nullptr || a.skip_combine) return rc;
  const int combine_threads = D >= 128 ? 128 : 64;
  odi_rc = launch_pdl((attention_mma_combine_kernel), dim3(n_tokens * a.nq), dim3(combine_threads), 0, stream,
                      (const float*)a.partial, a.out, a.splits, a.past, a.nq, a.tiles_per_split);
  return launch_status();
}

// The combine kernel alone, for partials that a decode launch with skip_combine left unmerged.
extern "C" int odi_attention_mma_combine(const float* partial, bf16* out, int n_tokens, int nq, int splits,
                                         const int* past, const int* tiles_per_split, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (partial == nullptr || out == nullptr || past == nullptr || nq < 1 || splits < 1) return ODI_ERR_ARGUMENT;
  const int combine_threads = D >= 128 ? 128 : 64;
  odi_rc = launch_pdl((attention_mma_combine_kernel), dim3(n_tokens * nq), dim3(combine_threads), 0, stream,
                      partial, out, splits, past, nq, tiles_per_split);
  return launch_status();
}

// ------------------------------------------------------------------------------ allocation-free entry point
//
// See attention_noalloc.h for who this is for and the rules of use.  The decode and combine
// kernels above are used unchanged; only the scratch for the split partials differs: it is
// the fixed array below instead of a caller-provided buffer.
#include <stdio.h>

#include <atomic>

#include "attention_noalloc.h"

static __device__ __align__(256) float odi_noalloc_scratch[ODI_NOALLOC_SCRATCH_FLOATS];

#define ODI_NOALLOC_MAX_DEVICES 64
// Device address of the array on each device; null until that device's set-up has completed.  Threads may make
// their first calls side by side: whoever finishes the set-up publishes the address with release order, a
// reader that sees it (acquire) also sees the set-up done; two threads that both find null both do the
// set-up, which gives the same address and sets the same attribute.
static std::atomic<float*> noalloc_scratch_address[ODI_NOALLOC_MAX_DEVICES];
static thread_local char noalloc_error_text[256] = "";

extern "C" long odi_attention_decode_noalloc_need(int n_tokens, int nq, int splits) {
  return (long)n_tokens * nq * splits * (D + 2);
}

extern "C" long odi_attention_decode_noalloc_capacity() { return ODI_NOALLOC_SCRATCH_FLOATS; }

extern "C" const char* odi_attention_decode_noalloc_error() { return noalloc_error_text; }

extern "C" int odi_attention_decode_noalloc(const MmaAttnArgs* args, int n_tokens, cudaStream_t stream) {
  noalloc_error_text[0] = 0;
  if (args == nullptr) {
    snprintf(noalloc_error_text, sizeof(noalloc_error_text), "args is null");
    return ODI_ERR_ARGUMENT;
  }
  MmaAttnArgs a = *args;
  if (a.n_seqs <= 0 || n_tokens <= 0) return 0;
  if (a.q == nullptr || a.k_pool == nullptr || a.v_pool == nullptr || a.out == nullptr || a.cu_q == nullptr ||
      a.past == nullptr || a.page_start == nullptr || a.page_ids == nullptr) {
    snprintf(noalloc_error_text, sizeof(noalloc_error_text),
             "q, k_pool, v_pool, out, cu_q, past, page_start and page_ids must all be device pointers, one is null");
    return ODI_ERR_ARGUMENT;
  }
  if (a.nq % a.nkv != 0 || a.n_seqs > 65535 || a.splits < 1 || n_tokens != a.n_seqs) {
    snprintf(noalloc_error_text, sizeof(noalloc_error_text),
             "decode attention needs one token per sequence (n_tokens=%d, n_seqs=%d), nq a multiple of nkv, splits >= 1",
             n_tokens, a.n_seqs);
    return ODI_ERR_ARGUMENT;
  }
  const long need = odi_attention_decode_noalloc_need(n_tokens, a.nq, a.splits);
  if (need > ODI_NOALLOC_SCRATCH_FLOATS) {
    snprintf(noalloc_error_text, sizeof(noalloc_error_text),
             "the built-in scratch holds %d floats, this call needs %ld (n_tokens=%d * nq=%d * splits=%d * (head_dim=%d + 2)): "
             "use fewer splits or the entry point that takes a buffer",
             ODI_NOALLOC_SCRATCH_FLOATS, need, n_tokens, a.nq, a.splits, D);
    return ODI_ERR_SCRATCH_LIMIT;
  }
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  if (device < 0 || device >= ODI_NOALLOC_MAX_DEVICES) return ODI_ERR_UNSUPPORTED;
  const int dc_smem = decode_smem_bytes();
  float* address = noalloc_scratch_address[device].load(std::memory_order_acquire);
  if (address == nullptr) {
    // Set-up, once per device with that device current: the array's name is a host-side
    // handle; the address a kernel can use comes from cudaGetSymbolAddress.
    e = cudaGetSymbolAddress((void**)&address, odi_noalloc_scratch);
    if (e != cudaSuccess || address == nullptr) {
      snprintf(noalloc_error_text, sizeof(noalloc_error_text), "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return e != cudaSuccess ? (int)e : ODI_ERR_ARGUMENT;
    }
    e = cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dc_smem);
    if (e != cudaSuccess) return (int)e;
    noalloc_scratch_address[device].store(address, std::memory_order_release);
  }
  a.partial = address;
  a.clustered = 0;      // this entry point is the global-partial form
  a.tickets = nullptr;  // ... with the combine kernel
  a.tiles_per_split = nullptr;   // ... and every sequence cut into `splits` equal ranges
  a.items = 0;
  a.skip_combine = 0;
  a.head_chunks = (a.nq / a.nkv + 15) / 16;
  dim3 grid(a.n_seqs, a.nkv * a.head_chunks, a.splits);
  if (grid.y > 65535 || grid.z > 65535) return ODI_ERR_UNSUPPORTED;
  odi_rc = launch_pdl((attention_decode_kernel), dim3(grid), dim3(DC_WARPS * 32), dc_smem, stream, a);
  int rc = launch_status();
  if (rc != 0 || a.splits == 1) return rc;
  const int combine_threads = D >= 128 ? 128 : 64;
  odi_rc = launch_pdl((attention_mma_combine_kernel), dim3(n_tokens * a.nq), dim3(combine_threads), 0, stream,
                      (const float*)a.partial, a.out, a.splits, a.past, a.nq, (const int*)nullptr);
  return launch_status();
}
