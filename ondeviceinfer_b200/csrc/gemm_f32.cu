// True 32-bit matrix product for the float32 path: C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]) (+ R).
//
// Plain FMA on the CUDA cores: no tensor cores, no TF32, no split of the K loop.  Each
// output element is accumulated over k = 0..K-1 in that order whatever M is, so a row's
// result does not depend on how many other rows are in the batch.
//
// 64x64 output tile per block of 256 threads, 4x4 outputs per thread, K in slices of 16
// staged through shared memory (stored k-major so the inner loop reads float4s).
// Any M, N, K >= 1; rows of A and W are read with float4 when K, lda, ldw are multiples
// of 4 and the bases 16-byte aligned, else element by element.
#include "common.cuh"

#define TM 64
#define TN 64
#define TK 16

template <bool VEC>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, float* C,
                const float* R, const float* __restrict__ bias, int M, int N, int K, int lda, int ldw, int ldc, int ldr) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ __align__(16) float As[TK][TM + 4];
  __shared__ __align__(16) float Ws[TK][TN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads; thread owns rows ty*4.., cols tx*4..
  const int lr = tid >> 2, lk = (tid & 3) * 4;  // loader: row lr of the tile, k offset lk
  float acc[4][4] = {};

  for (int k0 = 0; k0 < K; k0 += TK) {
    float a[4] = {0.f, 0.f, 0.f, 0.f}, w[4] = {0.f, 0.f, 0.f, 0.f};
    const int gm = m0 + lr, gn = n0 + lr, gk = k0 + lk;
    if (VEC) {
      if (gm < M && gk < K) { float4 v = *(const float4*)(A + (size_t)gm * lda + gk); a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w; }
      if (gn < N && gk < K) { float4 v = *(const float4*)(W + (size_t)gn * ldw + gk); w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w; }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (gm < M && gk + i < K) a[i] = A[(size_t)gm * lda + gk + i];
        if (gn < N && gk + i < K) w[i] = W[(size_t)gn * ldw + gk + i];
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) { As[lk + i][lr] = a[i]; Ws[lk + i][lr] = w[i]; }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      const float4 av = *(const float4*)&As[k][ty * 4];
      const float4 wv = *(const float4*)&Ws[k][tx * 4];
      const float ar[4] = {av.x, av.y, av.z, av.w};
      const float wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias != nullptr) v += bias[n];
      if (R != nullptr) v += R[(size_t)m * ldr + n];
      C[(size_t)m * ldc + n] = v;
    }
  }
}

// R may be null (no residual) or alias C (in-place add: each element is read and then
// written by the same thread).  bias may be null; it is added to the product before the residual.
extern "C" int odi_gemm_f32(const float* A, const float* W, float* C, const float* R, const float* bias, int M, int N,
                            int K, int lda, int ldw, int ldc, int ldr, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return ODI_ERR_ARGUMENT;
  dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
  if (grid.y > 65535) return ODI_ERR_UNSUPPORTED;
  const bool vec = (K % 4 == 0) && (lda % 4 == 0) && (ldw % 4 == 0) &&
                   ((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0);
  if (vec) odi_rc = launch_pdl((gemm_f32_kernel<true>), dim3(grid), dim3(256), 0, stream, A, W, C, R, bias, M, N, K, lda, ldw, ldc, ldr);
  else odi_rc = launch_pdl((gemm_f32_kernel<false>), dim3(grid), dim3(256), 0, stream, A, W, C, R, bias, M, N, K, lda, ldw, ldc, ldr);
  return launch_status();
}
