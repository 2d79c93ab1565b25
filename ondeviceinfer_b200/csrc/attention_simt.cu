// Causal grouped-query attention over paged cache slots on the CUDA cores, for any
// mixture of sequences: whole prompts, single decoded tokens, or chunks of a few tokens.
// It is the attention of the float32 path and the fallback of the bf16 path (windows,
// head sizes the tensor-core kernels do not take).
//
// Compile with -DODI_HEAD_DIM=<d>, d a multiple of 16 up to 512.
//
// Work item (one block of 4 warps): one sequence, one key/value head, a tile of query
// rows -- `bq` consecutive tokens times up to 16 of the head's query heads -- and, when
// the key range is split, one split.  Keys are streamed 32 at a time through shared
// memory (converted to fp32); each warp owns 4 rows; lane j scores key j of the tile;
// the softmax is the running-maximum form in fp32; the output accumulates in fp32.
// Key j is visible to the query at position p iff j <= p and (window == 0 or j > p - window).
//
// With splits > 1 every split writes an un-normalised partial (acc[d], max, sum) and
// attention_combine merges them in split order.
#include "common.cuh"

#ifndef ODI_HEAD_DIM
#error "compile with -DODI_HEAD_DIM=<head size>"
#endif

#define D ODI_HEAD_DIM
#define KT 32                 // keys per tile
#define NWARPS 4
#define RW 4                  // rows per warp
#define ROWS (NWARPS * RW)    // rows per block
#define NACC ((D + 31) / 32)  // output registers per row per lane
#define KSTR (D + 4)          // padded row stride of the key tile (floats)

struct AttnArgs {
  const void* q;        // [n_tokens, nq, D]
  const void* k_pool;   // [pages, nkv, page_size, D]
  const void* v_pool;
  void* out;            // [n_tokens, nq * D]
  float* partial;       // [n_tokens, nq, splits, D + 2] when splits > 1
  const int* cu_q;      // [n_seqs + 1] first packed token of each sequence
  const int* past;      // [n_seqs] keys cached before this step
  const int* page_start;
  const int* page_ids;
  int n_seqs, nq, nkv, page_size, ring_pages, window, splits, bq, head_chunks;
  float scale;
};

template <typename T>
__global__ void __launch_bounds__(NWARPS * 32)
attention_simt_kernel(AttnArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float smem[];
  float* Ks = smem;                    // [KT][KSTR]
  float* Vs = Ks + KT * KSTR;          // [KT][D]
  float* Qs = Vs + KT * D;             // [ROWS][D]
  float* Ps = Qs + ROWS * D;           // [ROWS][KT]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int seq = blockIdx.z;
  const int hk = blockIdx.y / a.head_chunks, chunk = blockIdx.y % a.head_chunks;
  const int qtile = blockIdx.x / a.splits, split = blockIdx.x % a.splits;
  const int g = a.nq / a.nkv;
  const int hpb = min(g - chunk * 16, 16);  // query heads of this block
  const int q_begin = a.cu_q[seq], q_len = a.cu_q[seq + 1] - q_begin;
  const int t0 = qtile * a.bq;
  if (t0 >= q_len) return;
  const int nt = min(a.bq, q_len - t0);     // tokens of this tile
  const int nrows = nt * hpb;
  const int past = a.past[seq];
  const int pos_lo = past + t0, pos_hi = past + t0 + nt - 1;

  // Key range seen by any row of the tile, cut into tiles of KT, then into splits.
  int k_lo = a.window > 0 ? max(0, pos_lo - a.window + 1) : 0;
  k_lo = (k_lo / KT) * KT;
  const int n_tiles = (pos_hi + 1 - k_lo + KT - 1) / KT;
  const int per_split = (n_tiles + a.splits - 1) / a.splits;
  const int tile_begin = split * per_split, tile_end = min(n_tiles, tile_begin + per_split);

  // Stage the query rows (fp32).  Row r: token t0 + r / hpb, head chunk*16 + r % hpb.
  for (int i = tid; i < ROWS * D; i += NWARPS * 32) {
    const int r = i / D, dd = i % D;
    float v = 0.f;
    if (r < nrows) {
      const int tok = q_begin + t0 + r / hpb;
      const int h = hk * g + chunk * 16 + r % hpb;
      v = to_f<T>(((const T*)a.q)[((size_t)tok * a.nq + h) * D + dd]);
    }
    Qs[i] = v;
  }

  float m[RW], l[RW], acc[RW][NACC];
  int rpos[RW];
#pragma unroll
  for (int r = 0; r < RW; ++r) {
    m[r] = -INFINITY; l[r] = 0.f;
    const int row = warp * RW + r;
    rpos[r] = row < nrows ? past + t0 + row / hpb : -1;
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[r][i] = 0.f;
  }

  const int* pages = a.page_ids + a.page_start[seq];
  for (int tile = tile_begin; tile < tile_end; ++tile) {
    const int kbase = k_lo + tile * KT;
    __syncthreads();  // previous tile fully consumed (also orders the Qs writes)
    // All KT keys of a tile lie in one page (page_size is a multiple of KT).
    const int page = pages[page_slot_of(kbase, a.page_size, a.ring_pages)];
    const size_t base = (((size_t)page * a.nkv + hk) * a.page_size + (kbase % a.page_size)) * D;
    const T* kp = (const T*)a.k_pool + base;
    const T* vp = (const T*)a.v_pool + base;
    const int nkeys = min(KT, pos_hi + 1 - kbase);
    for (int i = tid; i < KT * D; i += NWARPS * 32) {
      const int j = i / D, dd = i % D;
      float kv = 0.f, vv = 0.f;
      if (j < nkeys) { kv = to_f<T>(kp[i]); vv = to_f<T>(vp[i]); }
      Ks[j * KSTR + dd] = kv;
      Vs[i] = vv;
    }
    __syncthreads();

    // scores: lane = key
    float s[RW];
#pragma unroll
    for (int r = 0; r < RW; ++r) s[r] = 0.f;
    const float* krow = Ks + lane * KSTR;
    const float* qrow = Qs + (warp * RW) * D;
#pragma unroll 4
    for (int dd = 0; dd < D; dd += 4) {
      const float4 kv = *(const float4*)(krow + dd);
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        const float4 qv = *(const float4*)(qrow + r * D + dd);
        s[r] = fmaf(qv.x, kv.x, s[r]); s[r] = fmaf(qv.y, kv.y, s[r]);
        s[r] = fmaf(qv.z, kv.z, s[r]); s[r] = fmaf(qv.w, kv.w, s[r]);
      }
    }
    const int kj = kbase + lane;
    float* prow = Ps + (warp * RW) * KT;
#pragma unroll
    for (int r = 0; r < RW; ++r) {
      const bool vis = rpos[r] >= 0 && kj <= rpos[r] && (a.window == 0 || kj > rpos[r] - a.window);
      const float sc = vis ? s[r] * a.scale : -INFINITY;
      const float mx = warp_max(sc);
      const float m_new = fmaxf(m[r], mx);
      float p = 0.f, alpha = 1.f;
      if (m_new != -INFINITY) {
        p = vis ? expf(sc - m_new) : 0.f;
        alpha = expf(m[r] - m_new);  // m = -inf gives 0
      }
      l[r] = l[r] * alpha + warp_sum(p);
      m[r] = m_new;
#pragma unroll
      for (int i = 0; i < NACC; ++i) acc[r][i] *= alpha;
      prow[r * KT + lane] = p;
    }
    __syncwarp();
    // output: lane = element of the head
#pragma unroll 4
    for (int j = 0; j < KT; ++j) {
      float vv[NACC];
#pragma unroll
      for (int i = 0; i < NACC; ++i) {
        const int dd = lane + 32 * i;
        vv[i] = dd < D ? Vs[j * D + dd] : 0.f;
      }
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        const float p = prow[r * KT + j];
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[r][i] = fmaf(p, vv[i], acc[r][i]);
      }
    }
    __syncwarp();
  }

#pragma unroll
  for (int r = 0; r < RW; ++r) {
    const int row = warp * RW + r;
    if (row >= nrows) continue;
    const int tok = q_begin + t0 + row / hpb;
    const int h = hk * g + chunk * 16 + row % hpb;
    if (a.splits == 1) {
      const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
      T* o = (T*)a.out + ((size_t)tok * a.nq + h) * D;
#pragma unroll
      for (int i = 0; i < NACC; ++i) {
        const int dd = lane + 32 * i;
        if (dd < D) o[dd] = from_f<T>(acc[r][i] * inv);
      }
    } else {
      float* o = a.partial + (((size_t)tok * a.nq + h) * a.splits + split) * (D + 2);
#pragma unroll
      for (int i = 0; i < NACC; ++i) {
        const int dd = lane + 32 * i;
        if (dd < D) o[dd] = acc[r][i];
      }
      if (lane == 0) { o[D] = m[r]; o[D + 1] = l[r]; }
    }
  }
}

// Merge the partials of one (token, head): out = sum_s e^(m_s - M) acc_s / sum_s e^(m_s - M) l_s.
template <typename T>
__global__ void attention_combine_kernel(const float* __restrict__ partial, T* __restrict__ out, int splits) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = blockIdx.x;  // token * nq + head
  const float* p = partial + row * splits * (D + 2);
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, p[s * (D + 2) + D]);
  float denom = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = p[s * (D + 2) + D];
    if (ms != -INFINITY) denom += expf(ms - M) * p[s * (D + 2) + D + 1];
  }
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
  for (int dd = threadIdx.x; dd < D; dd += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = p[s * (D + 2) + D];
      if (ms != -INFINITY) v += expf(ms - M) * p[s * (D + 2) + dd];
    }
    out[row * D + dd] = from_f<T>(v * inv);
  }
}

extern "C" int odi_attention_simt_head_dim() { return D; }

// max_q_len: the longest q_len of the batch (sizes the grid); n_tokens: packed tokens.
extern "C" int odi_attention_simt(const AttnArgs* args, int max_q_len, int n_tokens, int dtype,
                                  cudaStream_t stream) {
  AttnArgs a = *args;
  if (a.n_seqs <= 0 || n_tokens <= 0) return 0;
  if (a.nq % a.nkv != 0 || a.page_size % KT != 0 || a.splits < 1 || a.n_seqs > 65535)
    return ODI_ERR_UNSUPPORTED;
  const int g = a.nq / a.nkv;
  const int hpb = g < 16 ? g : 16;
  a.head_chunks = (g + 15) / 16;
  a.bq = ROWS / hpb > 0 ? ROWS / hpb : 1;
  if (a.splits > 1 && a.partial == nullptr) return ODI_ERR_ARGUMENT;
  const int q_tiles = (max_q_len + a.bq - 1) / a.bq;
  dim3 grid(q_tiles * a.splits, a.nkv * a.head_chunks, a.n_seqs);
  if (grid.y > 65535) return ODI_ERR_UNSUPPORTED;
  const size_t smem = sizeof(float) * (KT * KSTR + KT * D + ROWS * D + ROWS * KT);
  // The shared-memory opt-in is a property of the function, set once per process.
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_simt_kernel<float>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_simt_kernel<bf16>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  if (dtype == 0) odi_rc = launch_pdl((attention_simt_kernel<float>), dim3(grid), dim3(NWARPS * 32), smem, stream, a);
  else odi_rc = launch_pdl((attention_simt_kernel<bf16>), dim3(grid), dim3(NWARPS * 32), smem, stream, a);
  int rc = launch_status();
  if (rc != 0 || a.splits == 1) return rc;
  const int rows = n_tokens * a.nq;
  const int threads = D >= 128 ? 128 : (D >= 64 ? 64 : 32);
  if (dtype == 0) odi_rc = launch_pdl((attention_combine_kernel<float>), dim3(rows), dim3(threads), 0, stream, a.partial, (float*)a.out, a.splits);
  else odi_rc = launch_pdl((attention_combine_kernel<bf16>), dim3(rows), dim3(threads), 0, stream, a.partial, (bf16*)a.out, a.splits);
  return launch_status();
}
