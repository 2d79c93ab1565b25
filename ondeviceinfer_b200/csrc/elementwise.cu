// Memory-bound kernels of a decoder step: embedding gather, RMSNorm, the fused
// per-head Q/K norm + rotary embedding + key/value cache write, the gated activation
// and the residual add.  Each is written for both element types (dtype 0 = float,
// 1 = bf16); statistics, angles and the residual stream are fp32 in both.
#include "common.cuh"

// ---------------------------------------------------------------------------------
// Embedding: hidden[t, :] = table[ids[t], :], widened to the fp32 residual stream.
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ hidden, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const T* row = table + (size_t)ids[t] * H;
  float* out = hidden + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = to_f<T>(row[i]);
}

extern "C" int odi_embed(const void* table, const int* ids, float* hidden, int n, int H, int dtype,
                         cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
  if (dtype == 0) odi_rc = launch_pdl((embed_kernel<float>), dim3(n), dim3(threads), 0, stream, (const float*)table, ids, hidden, H);
  else odi_rc = launch_pdl((embed_kernel<bf16>), dim3(n), dim3(threads), 0, stream, (const bf16*)table, ids, hidden, H);
  return launch_status();
}

// ---------------------------------------------------------------------------------
// RMSNorm over fp32 rows: y = x * rsqrt(mean(x^2) + eps) rounded to T, then
// out = weight * y rounded to T (the order of the reference: normalise in fp32, cast,
// scale).  `rows` (optional) gathers input rows, so the final norm runs only on the
// positions whose logits are wanted.
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                               T* __restrict__ out, const int* __restrict__ rows, int H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) { float v = xr[i]; ss += v * v; }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
  T* o = out + (size_t)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float y = round_to<T>(xr[i] * inv);
    o[i] = from_f<T>(w[i] * y);
  }
}

template <typename T> struct Pack4;
template <> struct Pack4<float> {
  static __device__ __forceinline__ void store(float* p, float a, float b, float c, float d) {
    *(float4*)p = make_float4(a, b, c, d);
  }
};
template <> struct Pack4<bf16> {
  static __device__ __forceinline__ void store(bf16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    *(uint2*)p = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
  }
};

template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) { return *(const float4*)p; }
template <> __device__ __forceinline__ float4 load4<bf16>(const bf16* p) {
  const uint2 raw = *(const uint2*)p;
  const float2 lo = __bfloat1622float2(*(const __nv_bfloat162*)&raw.x), hi = __bfloat1622float2(*(const __nv_bfloat162*)&raw.y);
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}

// H a multiple of 4 and at most 4 * NV * blockDim.x: one read of the row, kept in registers.
// add != null (then rows == null): the row becomes x + add first, is written back to x, and that sum is normed:
// the residual add of a product that a library computed, fused with the norm that follows it.
template <typename T, int NV>
__global__ void rmsnorm_vec_kernel(float* __restrict__ x, const float* __restrict__ w,
                                   T* __restrict__ out, const int* __restrict__ rows, const T* __restrict__ add,
                                   int H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  float4* xr = (float4*)(x + (size_t)(rows ? rows[r] : r) * H);
  const int nvec = H >> 2;
  float4 v[NV];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    v[j] = i < nvec ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    if (add != nullptr && i < nvec) {
      const float4 y = load4<T>(add + (size_t)r * H + 4 * i);
      v[j].x += y.x; v[j].y += y.y; v[j].z += y.z; v[j].w += y.w;
      xr[i] = v[j];
    }
    ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
  T* o = out + (size_t)r * H;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i < nvec) {
      const float4 ww = ((const float4*)w)[i];
      Pack4<T>::store(o + 4 * i, ww.x * round_to<T>(v[j].x * inv), ww.y * round_to<T>(v[j].y * inv),
                      ww.z * round_to<T>(v[j].z * inv), ww.w * round_to<T>(v[j].w * inv));
    }
  }
}

// add: null, or [n, H] in the dtype of out: x += add in place before the norm (vector form only: the caller asks
// odi_rmsnorm_adds first).
extern "C" int odi_rmsnorm_adds(const float* x, const float* w, const void* out, const void* add, int H) {
  return H % 4 == 0 && H <= 4 * 4 * 512 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) &&
         ((uintptr_t)out % 16 == 0) && ((uintptr_t)add % 8 == 0);
}

extern "C" int odi_rmsnorm(float* x, const float* w, void* out, const int* rows, const void* add, int n, int H,
                           float eps, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  const bool aligned = H % 4 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) && ((uintptr_t)out % 16 == 0);
  if (add != nullptr && (rows != nullptr || !odi_rmsnorm_adds(x, w, out, add, H))) return ODI_ERR_UNSUPPORTED;
  if (aligned && H <= 4 * 4 * 512) {
    const int nvec = H / 4;
    const int threads = nvec >= 1024 ? 512 : (nvec >= 256 ? 256 : 128);
    const int nv = (nvec + threads - 1) / threads;   // 1..4
#define ODI_NORM(T, NV) rmsnorm_vec_kernel<T, NV><<<n, threads, 0, stream>>>(x, w, (T*)out, rows, (const T*)add, H, eps)
    if (dtype == 0) { if (nv <= 1) ODI_NORM(float, 1); else if (nv <= 2) ODI_NORM(float, 2); else ODI_NORM(float, 4); }
    else { if (nv <= 1) ODI_NORM(bf16, 1); else if (nv <= 2) ODI_NORM(bf16, 2); else ODI_NORM(bf16, 4); }
#undef ODI_NORM
    return launch_status();
  }
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  if (dtype == 0) odi_rc = launch_pdl((rmsnorm_kernel<float>), dim3(n), dim3(threads), 0, stream, (const float*)x, w, (float*)out, rows, H, eps);
  else odi_rc = launch_pdl((rmsnorm_kernel<bf16>), dim3(n), dim3(threads), 0, stream, (const float*)x, w, (bf16*)out, rows, H, eps);
  return launch_status();
}

// ---------------------------------------------------------------------------------
// Fused head preparation.  Input: packed projections qkv[t, (nq + 2 nkv) * d] (query
// heads, then key heads, then value heads).  One warp per (token, head):
//   query / key heads: optional RMSNorm over d with one [d] weight for all heads,
//                      optional half-split rotary embedding with the step's fp32
//                      cos/sin tables [token, rot_dim / 2];
//   query heads go to q_out[t, h, :]; key and value heads go to the cache page that
//   holds the token's position (value heads are copied as they are).
// Cache layout: pool[page][kv_head][row][d], row = position % page_size.
// write_kv == 0 skips the key/value heads (a layer that reads another layer's cache).
// ---------------------------------------------------------------------------------
template <typename T, int MAXP>
__global__ void head_prep_kernel(HeadPrepArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int heads = a.nq + (a.write_kv ? 2 * a.nkv : 0);
  const long item = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long)a.n_tokens * heads) return;
  const int t = (int)(item / heads), h = (int)(item % heads);
  const int d = a.d, half = a.rot_dim >> 1;
  const T* src = (const T*)a.qkv + (size_t)t * (a.nq + 2 * a.nkv) * d + (size_t)h * d;
  const int kind = h < a.nq ? 0 : (h < a.nq + a.nkv ? 1 : 2);  // 0 q, 1 k, 2 v
  const int pos = a.tok_pos[t];

  T* dst;
  if (kind == 0) {
    dst = (T*)a.q_out + ((size_t)t * a.nq + h) * d;
  } else {
    const int hk = kind == 1 ? h - a.nq : h - a.nq - a.nkv;
    const int s = a.tok_seq[t];
    const int page = a.page_ids[a.page_start[s] + page_slot_of(pos, a.page_size, a.ring_pages)];
    T* pool = (T*)(kind == 1 ? a.k_pool : a.v_pool);
    dst = pool + (((size_t)page * a.nkv + hk) * a.page_size + (pos % a.page_size)) * d;
  }
  if (kind == 2) {
    for (int i = lane; i < d; i += 32) dst[i] = src[i];
    return;
  }
  // Element i of the head lives in lane i % 32, register i / 32.
  float x[MAXP];
  float ss = 0.f;
#pragma unroll
  for (int r = 0; r < MAXP; ++r) {
    const int i = lane + 32 * r;
    x[r] = i < d ? to_f<T>(src[i]) : 0.f;
    ss += x[r] * x[r];
  }
  const float* w = kind == 0 ? a.q_norm_w : a.k_norm_w;
  if (w != nullptr) {
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)d + a.eps);
#pragma unroll
    for (int r = 0; r < MAXP; ++r) {
      const int i = lane + 32 * r;
      if (i < d) x[r] = round_to<T>(w[i] * round_to<T>(x[r] * inv));
    }
  }
  if (a.cos_t != nullptr) {
    // Pair (i, i + half) for i < half.  The partner of element i sits in another lane
    // and register unless half is a multiple of 32, so go through shared memory.
    __shared__ float stage[4][32 * MAXP];
    float* st = stage[threadIdx.x >> 5];
#pragma unroll
    for (int r = 0; r < MAXP; ++r) st[lane + 32 * r] = x[r];
    __syncwarp();
#pragma unroll
    for (int r = 0; r < MAXP; ++r) {
      const int i = lane + 32 * r;
      if (i < a.rot_dim) {
        const int f = i < half ? i : i - half;
        const float cs = a.cos_t[(size_t)t * half + f], sn = a.sin_t[(size_t)t * half + f];
        const float other = i < half ? -st[i + half] : st[i - half];
        x[r] = x[r] * cs + other * sn;
      }
    }
  }
#pragma unroll
  for (int r = 0; r < MAXP; ++r) {
    const int i = lane + 32 * r;
    if (i < d) dst[i] = from_f<T>(x[r]);
  }
}

// Fast form for head sizes that are a multiple of 32 with the whole head rotated (or none of
// it): lane i holds the VEC = d / 32 contiguous elements [VEC * i, VEC * i + VEC), read and written
// as one vector; the rotation partner of an element (d / 2 further) sits in lane i + 16 at the
// same register, reached by a shuffle.  Same arithmetic as head_prep_kernel.
template <int VEC>
__global__ void head_prep_vec_kernel(HeadPrepArgs a, int heads_per_warp) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int heads = a.nq + (a.write_kv ? 2 * a.nkv : 0);
  const int groups = (heads + heads_per_warp - 1) / heads_per_warp;      // warps per token
  const long item = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long)a.n_tokens * groups) return;
  const int t = (int)(item / groups), h_begin = (int)(item % groups) * heads_per_warp;
  const int h_end = min(heads, h_begin + heads_per_warp);
  const int d = a.d, half = d >> 1;
  const int pos = a.tok_pos[t];
  // what does not depend on the head is read once per token: the rotation table entries of this
  // lane's elements, the norm weights, the token's cache page
  float cs[VEC], sn[VEC], wq[VEC], wk[VEC];
#pragma unroll
  for (int r = 0; r < VEC; ++r) {
    const int i = VEC * lane + r, f = i < half ? i : i - half;
    cs[r] = a.cos_t ? a.cos_t[(size_t)t * half + f] : 1.f;
    sn[r] = a.cos_t ? a.sin_t[(size_t)t * half + f] : 0.f;
    wq[r] = a.q_norm_w ? a.q_norm_w[i] : 1.f;
    wk[r] = a.k_norm_w ? a.k_norm_w[i] : 1.f;
  }
  int page = 0;
  if (a.write_kv && h_end > a.nq)
    page = a.page_ids[a.page_start[a.tok_seq[t]] + page_slot_of(pos, a.page_size, a.ring_pages)];
  const bf16* token_src = (const bf16*)a.qkv + (size_t)t * (a.nq + 2 * a.nkv) * d + VEC * lane;
  for (int h = h_begin; h < h_end; ++h) {
    const bf16* src = token_src + (size_t)h * d;
    const int kind = h < a.nq ? 0 : (h < a.nq + a.nkv ? 1 : 2);
    bf16* dst;
    if (kind == 0) {
      dst = (bf16*)a.q_out + ((size_t)t * a.nq + h) * d;
    } else {
      const int hk = kind == 1 ? h - a.nq : h - a.nq - a.nkv;
      bf16* pool = (bf16*)(kind == 1 ? a.k_pool : a.v_pool);
      dst = pool + (((size_t)page * a.nkv + hk) * a.page_size + (pos % a.page_size)) * d;
    }
    dst += VEC * lane;
    bf16 raw[VEC];
    if (VEC == 1) raw[0] = src[0];
    else if (VEC == 2) *(uint32_t*)raw = *(const uint32_t*)src;
    else if (VEC == 4) *(uint2*)raw = *(const uint2*)src;
    else *(uint4*)raw = *(const uint4*)src;
    if (kind != 2) {
      float x[VEC];
      float ss = 0.f;
#pragma unroll
      for (int r = 0; r < VEC; ++r) { x[r] = __bfloat162float(raw[r]); ss += x[r] * x[r]; }
      if ((kind == 0 ? a.q_norm_w : a.k_norm_w) != nullptr) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)d + a.eps);
#pragma unroll
        for (int r = 0; r < VEC; ++r) x[r] = round_to<bf16>((kind == 0 ? wq[r] : wk[r]) * round_to<bf16>(x[r] * inv));
      }
      if (a.cos_t != nullptr) {
#pragma unroll
        for (int r = 0; r < VEC; ++r) {
          const float partner = __shfl_xor_sync(0xffffffffu, x[r], 16);
          x[r] = x[r] * cs[r] + ((VEC * lane + r) < half ? -partner : partner) * sn[r];
        }
      }
#pragma unroll
      for (int r = 0; r < VEC; ++r) raw[r] = __float2bfloat16_rn(x[r]);
    }
    if (VEC == 1) dst[0] = raw[0];
    else if (VEC == 2) *(uint32_t*)dst = *(uint32_t*)raw;
    else if (VEC == 4) *(uint2*)dst = *(uint2*)raw;
    else *(uint4*)dst = *(uint4*)raw;
  }
}

extern "C" int odi_head_prep(const HeadPrepArgs* args, int dtype, cudaStream_t stream) {
  HeadPrepArgs a = *args;
  if (a.n_tokens <= 0) return 0;
  if (a.d > 512 || a.d <= 0 || (a.rot_dim & 1) || a.rot_dim > a.d) return ODI_ERR_UNSUPPORTED;
  const int heads = a.nq + (a.write_kv ? 2 * a.nkv : 0);
  const long items = (long)a.n_tokens * heads;
  const int blocks = (int)((items + 3) / 4);
  if (dtype == 1 && a.d % 32 == 0 && a.d <= 256 && (a.cos_t == nullptr || a.rot_dim == a.d) &&
      ((uintptr_t)a.qkv % 16 == 0) && ((uintptr_t)a.q_out % 16 == 0)) {
    // few tokens (decode): a warp per (token, head) for parallelism; many tokens (prefill): a warp
    // takes a quarter of a token's heads, so the per-token table entries are read once for all of them
    const int hpw = a.n_tokens >= 256 ? (heads + 3) / 4 : 1;
    const long warps = (long)a.n_tokens * ((heads + hpw - 1) / hpw);
    const int vblocks = (int)((warps + 3) / 4);
    switch (a.d / 32) {
      case 1: odi_rc = launch_pdl((head_prep_vec_kernel<1>), dim3(vblocks), dim3(128), 0, stream, a, hpw); return launch_status();
      case 2: odi_rc = launch_pdl((head_prep_vec_kernel<2>), dim3(vblocks), dim3(128), 0, stream, a, hpw); return launch_status();
      case 4: odi_rc = launch_pdl((head_prep_vec_kernel<4>), dim3(vblocks), dim3(128), 0, stream, a, hpw); return launch_status();
      case 8: odi_rc = launch_pdl((head_prep_vec_kernel<8>), dim3(vblocks), dim3(128), 0, stream, a, hpw); return launch_status();
      default: break;
    }
  }
#define ODI_LAUNCH(T, P) head_prep_kernel<T, P><<<blocks, 128, 0, stream>>>(a)
  if (dtype == 0) {
    if (a.d <= 128) ODI_LAUNCH(float, 4); else if (a.d <= 256) ODI_LAUNCH(float, 8); else ODI_LAUNCH(float, 16);
  } else {
    if (a.d <= 128) ODI_LAUNCH(bf16, 4); else if (a.d <= 256) ODI_LAUNCH(bf16, 8); else ODI_LAUNCH(bf16, 16);
  }
#undef ODI_LAUNCH
  return launch_status();
}

// ---------------------------------------------------------------------------------
// Gated activation on concatenated projections gu[t, 0:I] = gate, gu[t, I:2I] = up:
// out[t, i] = silu(gate) * up, computed in fp32 and rounded once.
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, long n, int I) {
  pdl_launch_dependents();
  pdl_wait();
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n * I) return;
  const long t = idx / I;
  const int i = (int)(idx % I);
  const float g = to_f<T>(gu[t * 2 * I + i]);
  const float u = to_f<T>(gu[t * 2 * I + I + i]);
  out[idx] = from_f<T>(g / (1.f + expf(-g)) * u);
}

// bf16, I a multiple of 8: each thread handles 8 consecutive elements with 16-byte accesses.
__global__ void silu_mul_vec_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, long n, int I) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = I >> 3;
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n * per_row) return;
  const long t = idx / per_row;
  const int i = (int)(idx % per_row) * 8;
  const uint4 gv = *(const uint4*)(gu + t * 2 * I + i);
  const uint4 uv = *(const uint4*)(gu + t * 2 * I + I + i);
  const __nv_bfloat162* g2 = (const __nv_bfloat162*)&gv;
  const __nv_bfloat162* u2 = (const __nv_bfloat162*)&uv;
  uint4 ov;
  __nv_bfloat162* o2 = (__nv_bfloat162*)&ov;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    // fast exponential and division: their error (a few ulp of fp32) is far below the bf16 rounding of the result
    const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
    o2[j] = __floats2bfloat162_rn(__fdividef(g.x, 1.f + __expf(-g.x)) * u.x, __fdividef(g.y, 1.f + __expf(-g.y)) * u.y);
  }
  *(uint4*)(out + t * I + i) = ov;
}

extern "C" int odi_silu_mul(const void* gu, void* out, int n, int I, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (dtype == 1 && I % 8 == 0 && ((uintptr_t)gu % 16 == 0) && ((uintptr_t)out % 16 == 0)) {
    const long work = (long)n * (I / 8);
    odi_rc = launch_pdl((silu_mul_vec_kernel), dim3((int)((work + 255) / 256)), dim3(256), 0, stream, (const bf16*)gu, (bf16*)out, n, I);
    return launch_status();
  }
  const long total = (long)n * I;
  const int blocks = (int)((total + 255) / 256);
  if (dtype == 0) odi_rc = launch_pdl((silu_mul_kernel<float>), dim3(blocks), dim3(256), 0, stream, (const float*)gu, (float*)out, n, I);
  else odi_rc = launch_pdl((silu_mul_kernel<bf16>), dim3(blocks), dim3(256), 0, stream, (const bf16*)gu, (bf16*)out, n, I);
  return launch_status();
}

// ---------------------------------------------------------------------------------
// Residual add into the fp32 stream: hidden += y.
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void residual_add_kernel(float* __restrict__ hidden, const T* __restrict__ y, long n) {
  pdl_launch_dependents();
  pdl_wait();
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < n) hidden[idx] += to_f<T>(y[idx]);
}

__global__ void residual_add_vec_kernel(float* __restrict__ hidden, const bf16* __restrict__ y, long n8) {
  pdl_launch_dependents();
  pdl_wait();
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n8) return;
  const uint4 yv = ((const uint4*)y)[idx];
  const __nv_bfloat162* y2 = (const __nv_bfloat162*)&yv;
  float4* h = (float4*)hidden + 2 * idx;
  float4 a = h[0], b = h[1];
  const float2 y0 = __bfloat1622float2(y2[0]), y1 = __bfloat1622float2(y2[1]);
  const float2 y2f = __bfloat1622float2(y2[2]), y3 = __bfloat1622float2(y2[3]);
  a.x += y0.x; a.y += y0.y; a.z += y1.x; a.w += y1.y;
  b.x += y2f.x; b.y += y2f.y; b.z += y3.x; b.w += y3.y;
  h[0] = a; h[1] = b;
}

extern "C" int odi_residual_add(float* hidden, const void* y, long n, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (dtype == 1 && n % 8 == 0 && ((uintptr_t)hidden % 16 == 0) && ((uintptr_t)y % 16 == 0)) {
    const long n8 = n / 8;
    odi_rc = launch_pdl((residual_add_vec_kernel), dim3((int)((n8 + 255) / 256)), dim3(256), 0, stream, hidden, (const bf16*)y, n8);
    return launch_status();
  }
  const int blocks = (int)((n + 255) / 256);
  if (dtype == 0) odi_rc = launch_pdl((residual_add_kernel<float>), dim3(blocks), dim3(256), 0, stream, hidden, (const float*)y, n);
  else odi_rc = launch_pdl((residual_add_kernel<bf16>), dim3(blocks), dim3(256), 0, stream, hidden, (const bf16*)y, n);
  return launch_status();
}

// ---------------------------------------------------------------------------------
// Widen rows to fp32 (logits of a bf16 matrix product returned as fp32).
// ---------------------------------------------------------------------------------
__global__ void widen_kernel(const bf16* __restrict__ x, float* __restrict__ out, long n) {
  pdl_launch_dependents();
  pdl_wait();
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < n) out[idx] = __bfloat162float(x[idx]);
}

extern "C" int odi_widen(const void* x, float* out, long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  odi_rc = launch_pdl((widen_kernel), dim3((int)((n + 255) / 256)), dim3(256), 0, stream, (const bf16*)x, out, n);
  return launch_status();
}

// ---------------------------------------------------------------------------------
// y[t, n] += bias[n] in place, one rounding to the dtype of y (after a product that the vendor
// library computed: the tensor-core kernels of this library add their bias themselves).
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void bias_add_kernel(T* __restrict__ y, const float* __restrict__ bias, long rows, int N) {
  pdl_launch_dependents();
  pdl_wait();
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < rows * N) y[idx] = from_f<T>(to_f<T>(y[idx]) + bias[idx % N]);
}

extern "C" int odi_bias_add(void* y, const float* bias, long rows, int N, int dtype, cudaStream_t stream) {
  if (rows <= 0 || N <= 0) return 0;
  const long n = rows * N;
  if ((n + 255) / 256 > 0x7fffffffL) return ODI_ERR_UNSUPPORTED;
  const dim3 grid((unsigned)((n + 255) / 256));
  if (dtype == 0) odi_rc = launch_pdl((bias_add_kernel<float>), grid, dim3(256), 0, stream, (float*)y, bias, rows, N);
  else odi_rc = launch_pdl((bias_add_kernel<bf16>), grid, dim3(256), 0, stream, (bf16*)y, bias, rows, N);
  return launch_status();
}

// ---------------------------------------------------------------------------------
// Rotary tables of a step: cos/sin[t, i] of position[t] * inv_freq[i], evaluated in
// fp32 with the full-range sincosf.  One table serves every layer of the step.
// ---------------------------------------------------------------------------------
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, const int* __restrict__ tok_pos,
                                  float* __restrict__ cos_t, float* __restrict__ sin_t, int n, int half) {
  pdl_launch_dependents();
  pdl_wait();
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long)n * half) return;
  const int t = (int)(idx / half), i = (int)(idx % half);
  float sn, cs;
  sincosf((float)tok_pos[t] * inv_freq[i], &sn, &cs);
  cos_t[idx] = cs;
  sin_t[idx] = sn;
}

extern "C" int odi_rope_table(const float* inv_freq, const int* tok_pos, float* cos_t, float* sin_t, int n,
                              int half, cudaStream_t stream) {
  if (n <= 0 || half <= 0) return 0;
  const long total = (long)n * half;
  odi_rc = launch_pdl((rope_table_kernel), dim3((int)((total + 255) / 256)), dim3(256), 0, stream, inv_freq, tok_pos, cos_t, sin_t, n, half);
  return launch_status();
}
