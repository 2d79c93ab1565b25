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
// One block of 256 threads per row.  Ties of the maximum go to the lowest index.
//
// For a decode loop that stays on the device the kernel can also advance the step's
// counters: with `advance` arrays given, row i adds active[i] (0 or 1) to its position,
// cached length and step number after it has drawn its token, so the next step finds
// its inputs in place.
#include "common.cuh"

#define SAMPLE_THREADS 256

__device__ __forceinline__ float uniform_draw(unsigned long long seed, unsigned long long stream,
                                              unsigned long long step) {
  unsigned long long x = seed * 0x9E3779B97F4A7C15ull + stream * 0xBF58476D1CE4E5B9ull +
                         step * 0x94D049BB133111EBull + 0x2545F4914F6CDD1Dull;
  x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27; x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return (float)(x >> 40) * (1.0f / 16777216.0f);
}

// streams / steps may be null when temperature == 0.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int* __restrict__ out, int V, int ld, float temperature,
              unsigned long long seed, const int* __restrict__ streams, int* steps,
              int* advance_pos, int* advance_past, const int* __restrict__ active) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float s_val[SAMPLE_THREADS];
  __shared__ int s_idx[SAMPLE_THREADS];
  __shared__ float s_prefix[SAMPLE_THREADS + 1];
  const int row = blockIdx.x, tid = threadIdx.x;
  const float* lg = logits + (size_t)row * ld;
  // Each thread owns one contiguous segment, so prefix sums follow vocabulary order.
  const int seg = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int lo = min(V, tid * seg), hi = min(V, lo + seg);

  float best = -INFINITY; int best_i = V;
  for (int i = lo; i < hi; ++i) { const float v = lg[i]; if (v > best) { best = v; best_i = i; } }
  s_val[tid] = best; s_idx[tid] = best_i;
  __syncthreads();
  for (int o = SAMPLE_THREADS / 2; o > 0; o >>= 1) {
    if (tid < o) {
      const float v = s_val[tid + o]; const int i = s_idx[tid + o];
      if (v > s_val[tid] || (v == s_val[tid] && i < s_idx[tid])) { s_val[tid] = v; s_idx[tid] = i; }
    }
    __syncthreads();
  }
  const float mx = s_val[0];
  const int arg = s_idx[0];
  if (temperature <= 0.f) {
    if (tid == 0) {
      out[row] = arg < V ? arg : 0;
      if (active != nullptr) {
        const int a = active[row];
        advance_pos[row] += a; advance_past[row] += a;
        if (steps != nullptr) steps[row] += a;
      }
    }
    return;
  }
  __syncthreads();

  const float inv_t = 1.f / temperature;
  float local = 0.f;
  for (int i = lo; i < hi; ++i) local += expf((lg[i] - mx) * inv_t);
  s_val[tid] = local;
  __syncthreads();
  if (tid == 0) {
    float run = 0.f;
    for (int t = 0; t < SAMPLE_THREADS; ++t) { s_prefix[t] = run; run += s_val[t]; }
    s_prefix[SAMPLE_THREADS] = run;
    s_idx[0] = V - 1;  // default when rounding leaves the target beyond the last weight
  }
  __syncthreads();
  const float total = s_prefix[SAMPLE_THREADS];
  const int step_now = steps[row];   // read by every thread before thread 0 may advance it
  __syncthreads();
  const float target = uniform_draw(seed, (unsigned long long)streams[row], (unsigned long long)step_now) * total;
  // The first index whose cumulative weight exceeds the target lies in exactly one segment.
  const float before = s_prefix[tid], after = s_prefix[tid + 1];
  if (before <= target && target < after && lo < hi) {
    float run = before; int pick = hi - 1;
    for (int i = lo; i < hi; ++i) {
      run += expf((lg[i] - mx) * inv_t);
      if (run > target) { pick = i; break; }
    }
    s_idx[0] = pick;
  }
  __syncthreads();
  if (tid == 0) {
    out[row] = s_idx[0];
    if (active != nullptr) {
      const int a = active[row];
      advance_pos[row] += a; advance_past[row] += a; steps[row] += a;
    }
  }
}

extern "C" int odi_sample(const float* logits, int* out, int n, int V, int ld, float temperature,
                          unsigned long long seed, const int* streams, int* steps, int* advance_pos,
                          int* advance_past, const int* active, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (temperature > 0.f && (streams == nullptr || steps == nullptr)) return ODI_ERR_ARGUMENT;
  if (active != nullptr && (advance_pos == nullptr || advance_past == nullptr)) return ODI_ERR_ARGUMENT;
  odi_rc = launch_pdl((sample_kernel), dim3(n), dim3(SAMPLE_THREADS), 0, stream, logits, out, V, ld, temperature, seed,
                      streams, steps, advance_pos, advance_past, active);
  return launch_status();
}
