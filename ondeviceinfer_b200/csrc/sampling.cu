// On-device sampling from fp32 logits: greedy argmax, or temperature sampling by the
// inverse CDF of softmax(logits / T) in vocabulary order.
//
// The uniform number of a draw is a pure function of (seed, stream, step): 24 bits of
// a 64-bit mix, so a sequence's tokens do not depend on what else is in the batch and a
// host implementation can restate it exactly:
//   x = seed*0x9E3779B97F4A7C15 + stream*0xBF58476D1CE4E5B9 + step*0x94D049BB133111EB
//       + 0x2545F4914F6CDD1D                      (mod 2^64)
//   x ^= x >> 30; x *= 0xBF58476D1CE4E5B9; x ^= x >> 27; x *= 0x94D049BB133111EB; x ^= x >> 31
//   u = (x >> 40) / 2^24
//
// A row is cut into chunks of 2,048 logits, one CTA each, so that a vocabulary of 150,000
// streams through many SMs at once.  Every CTA leaves its chunk's maximum (lowest index on
// ties) and, for temperature sampling, the chunk's weight sum(exp((x - chunk max) / T)); the
// CTA that finishes a row last (an atomic ticket per row) merges the chunks in vocabulary
// order, finds the chunk in which u * total falls and walks that chunk alone.  The merge
// order is fixed, so a row's token does not depend on which CTA came last.
//
// For a decode loop that stays on the device the kernel can also advance the step's
// counters: with `advance` arrays given, row i adds active[i] (0 or 1) to its position,
// cached length and step number after it has drawn its token, so the next step finds
// its inputs in place.
#include "common.cuh"

#define SAMPLE_THREADS 256
#define SAMPLE_PER_THREAD 8
#define SAMPLE_CHUNK (SAMPLE_THREADS * SAMPLE_PER_THREAD)

__device__ __forceinline__ float uniform_draw(unsigned long long seed, unsigned long long stream,
                                              unsigned long long step) {
  unsigned long long x = seed * 0x9E3779B97F4A7C15ull + stream * 0xBF58476D1CE4E5B9ull +
                         step * 0x94D049BB133111EBull + 0x2545F4914F6CDD1Dull;
  x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27; x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return (float)(x >> 40) * (1.0f / 16777216.0f);
}

struct ChunkPartial { float max; int arg; float weight; int pad; };

// The larger of two (value, index) pairs, the lower index on ties; reduced over the block.
__device__ __forceinline__ void block_argmax(float& v, int& i, float* s_val, int* s_idx) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
  __syncthreads();          // the arrays may still be read from an earlier use
  if (lane == 0) { s_val[warp] = v; s_idx[warp] = i; }
  __syncthreads();
  v = s_val[0]; i = s_idx[0];
#pragma unroll
  for (int w = 1; w < SAMPLE_THREADS / 32; ++w)
    if (s_val[w] > v || (s_val[w] == v && s_idx[w] < i)) { v = s_val[w]; i = s_idx[w]; }
}

// Exclusive and inclusive prefix sums of one value per thread in thread order, and the block's total: a
// shuffle scan inside each warp, then the warps' totals in order.  The association is fixed.
__device__ __forceinline__ void block_scan(float v, float& exclusive, float& inclusive, float& total, float* s_warp) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  __syncthreads();          // s_warp may still be read from an earlier use
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  float offset = 0.f, sum = 0.f;
#pragma unroll
  for (int w = 0; w < SAMPLE_THREADS / 32; ++w) {
    if (w == warp) offset = sum;
    sum += s_warp[w];
  }
  const float prev = __shfl_up_sync(0xffffffffu, incl, 1);
  exclusive = offset + (lane > 0 ? prev : 0.f);
  inclusive = offset + incl;     // the next thread's `exclusive`, bit for bit
  total = sum;
}

// streams / steps may be null when temperature == 0.  partials: [rows, n_chunks]; tickets: one
// per row, zero before the launch and zero again after it.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int* __restrict__ out, int V, int ld, float temperature,
              unsigned long long seed, const int* __restrict__ streams, int* steps,
              int* advance_pos, int* advance_past, const int* __restrict__ active,
              ChunkPartial* partials, int* tickets) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float s_val[SAMPLE_THREADS];
  __shared__ int s_idx[SAMPLE_THREADS];
  __shared__ float s_prefix[SAMPLE_THREADS + 1];
  __shared__ int s_last;
  const int chunk = blockIdx.x, n_chunks = gridDim.x, row = blockIdx.y, tid = threadIdx.x;
  const float* lg = logits + (size_t)row * ld;
  const float inv_t = temperature > 0.f ? 1.f / temperature : 0.f;

  // ---- this chunk: maximum and weight (coalesced; the order inside a chunk does not matter here)
  float x[SAMPLE_PER_THREAD];
  float best = -INFINITY; int best_i = V;
#pragma unroll
  for (int k = 0; k < SAMPLE_PER_THREAD; ++k) {
    const int i = chunk * SAMPLE_CHUNK + k * SAMPLE_THREADS + tid;
    x[k] = i < V ? lg[i] : -INFINITY;
    if (x[k] > best) { best = x[k]; best_i = i; }
  }
  block_argmax(best, best_i, s_val, s_idx);
  float weight = 0.f;
  if (temperature > 0.f) {
    float local = 0.f;
#pragma unroll
    for (int k = 0; k < SAMPLE_PER_THREAD; ++k) local += expf((x[k] - best) * inv_t);   // exp(-inf) = 0 past the end
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
    __syncthreads();
    if ((tid & 31) == 0) s_val[tid >> 5] = local;
    __syncthreads();
    for (int w = 0; w < SAMPLE_THREADS / 32; ++w) weight += s_val[w];
  }
  if (tid == 0) {
    ChunkPartial p; p.max = best; p.arg = best_i; p.weight = weight; p.pad = 0;
    partials[(size_t)row * n_chunks + chunk] = p;
    __threadfence();
    s_last = atomicAdd(&tickets[row], 1) == n_chunks - 1;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const ChunkPartial* mine = partials + (size_t)row * n_chunks;

  // ---- the row's last CTA: merge the chunks
  float mx = -INFINITY; int arg = V;
  for (int c = tid; c < n_chunks; c += SAMPLE_THREADS) {
    const float v = mine[c].max; const int i = mine[c].arg;
    if (v > mx || (v == mx && i < arg)) { mx = v; arg = i; }
  }
  block_argmax(mx, arg, s_val, s_idx);
  int pick = arg < V ? arg : 0;
  if (temperature > 0.f) {
    const int step_now = steps[row];
    // The chunks' weights against the row's maximum, summed in vocabulary order (a block scan: the
    // same association every time), then the chunk in which the target falls.
    float total = 0.f;
    for (int base = 0; base < n_chunks; base += SAMPLE_THREADS) {
      const int c = base + tid;
      const float w = c < n_chunks ? mine[c].weight * expf((mine[c].max - mx) * inv_t) : 0.f;
      float excl, incl, tile_total;
      block_scan(w, excl, incl, tile_total, s_val);
      total += tile_total;
    }
    const float target = uniform_draw(seed, (unsigned long long)streams[row], (unsigned long long)step_now) * total;
    if (tid == 0) s_idx[0] = -1;
    float carried = 0.f, last_excl = 0.f;
    for (int base = 0; base < n_chunks; base += SAMPLE_THREADS) {
      const int c = base + tid;
      const float w = c < n_chunks ? mine[c].weight * expf((mine[c].max - mx) * inv_t) : 0.f;
      float excl, incl, tile_total;
      block_scan(w, excl, incl, tile_total, s_val);      // its barriers also order the write of s_idx[0] above
      excl += carried; incl += carried;
      if (c < n_chunks && excl <= target && target < incl) { s_idx[0] = c; s_prefix[0] = excl; }
      if (c == n_chunks - 1) last_excl = excl;
      carried += tile_total;
    }
    __syncthreads();
    // rounding may leave the target beyond the last weight: the last chunk then
    if (s_idx[0] < 0 && (n_chunks - 1) % SAMPLE_THREADS == tid) { s_idx[0] = n_chunks - 1; s_prefix[0] = last_excl; }
    __syncthreads();
    const float run0 = s_prefix[0];
    const int at = s_idx[0];
    __syncthreads();
    // Each thread owns a contiguous piece of that chunk, so that prefix sums follow vocabulary order.
    const int lo = min(V, at * SAMPLE_CHUNK + tid * SAMPLE_PER_THREAD), hi = min(V, lo + SAMPLE_PER_THREAD);
    float local = 0.f;
    for (int i = lo; i < hi; ++i) local += expf((lg[i] - mx) * inv_t);
    float before, after, chunk_total;
    block_scan(local, before, after, chunk_total, s_val);
    before += run0; after += run0;
    // when rounding leaves the target beyond the chunk's last weight: the chunk's last index
    if (tid == 0) s_idx[0] = min(V, (at + 1) * SAMPLE_CHUNK) - 1;
    __syncthreads();
    // The first index whose cumulative weight exceeds the target lies in exactly one piece.
    if ((before <= target || tid == 0) && target < after && lo < hi) {
      float run = before; int found = hi - 1;
      for (int i = lo; i < hi; ++i) {
        run += expf((lg[i] - mx) * inv_t);
        if (run > target) { found = i; break; }
      }
      s_idx[0] = found;
    }
    __syncthreads();
    pick = s_idx[0];
  }
  if (tid == 0) {
    out[row] = pick;
    tickets[row] = 0;
    if (active != nullptr) {
      const int a = active[row];
      advance_pos[row] += a; advance_past[row] += a;
      if (steps != nullptr) steps[row] += a;
    }
  }
}

extern "C" int odi_sample_chunks(int V) { return (V + SAMPLE_CHUNK - 1) / SAMPLE_CHUNK; }

// partials: n * odi_sample_chunks(V) entries of 16 bytes; tickets: n ints, zero (left zero).
extern "C" int odi_sample(const float* logits, int* out, int n, int V, int ld, float temperature,
                          unsigned long long seed, const int* streams, int* steps, int* advance_pos,
                          int* advance_past, const int* active, void* partials, int* tickets, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (V <= 0 || partials == nullptr || tickets == nullptr) return ODI_ERR_ARGUMENT;
  if (temperature > 0.f && (streams == nullptr || steps == nullptr)) return ODI_ERR_ARGUMENT;
  if (active != nullptr && (advance_pos == nullptr || advance_past == nullptr)) return ODI_ERR_ARGUMENT;
  if (n > 65535) return ODI_ERR_ARGUMENT;
  odi_rc = launch_pdl((sample_kernel), dim3(odi_sample_chunks(V), n), dim3(SAMPLE_THREADS), 0, stream, logits, out, V, ld,
                      temperature, seed, streams, steps, advance_pos, advance_past, active, (ChunkPartial*)partials, tickets);
  return launch_status();
}
