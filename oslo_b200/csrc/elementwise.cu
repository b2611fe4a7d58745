// Memory-bound kernels: LayerNorm, bias+GeLU, bias+dropout+residual, rotary, softmax on scores,
// cross-entropy pieces, AdamW, n-gram blocking. All use 16-byte vector accesses on the contiguous
// dim, fp32 math, and run on the caller's stream.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include "oslo_kernels.h"
#include "ptx.cuh"

namespace oslo {

template <typename T> struct Cvt;
template <> struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float to(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Cvt<__half> {
  static __device__ __forceinline__ float to(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from(float v) { return __float2half_rn(v); }
};
template <> struct Cvt<float> {
  static __device__ __forceinline__ float to(float v) { return v; }
  static __device__ __forceinline__ float from(float v) { return v; }
};

// VEC elements = 16 bytes
template <typename T> struct VecOf { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float* f) {
  constexpr int N = VecOf<T>::N;
  uint4 raw = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < N; ++i) f[i] = Cvt<T>::to(e[i]);
}
template <typename T>
__device__ __forceinline__ void store_vec(T* p, const float* f) {
  constexpr int N = VecOf<T>::N;
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < N; ++i) e[i] = Cvt<T>::from(f[i]);
  *reinterpret_cast<uint4*>(p) = raw;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = (threadIdx.x < THREADS / 32) ? sh[threadIdx.x] : 0.f;
  if (w == 0) r = warp_sum(r);
  if (threadIdx.x == 0) sh[0] = r;
  __syncthreads();
  return sh[0];
}
template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* sh) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = (threadIdx.x < THREADS / 32) ? sh[threadIdx.x] : -CUDART_INF_F;
  if (w == 0) r = warp_max(r);
  if (threadIdx.x == 0) sh[0] = r;
  __syncthreads();
  return sh[0];
}

__device__ __forceinline__ float gelu_f(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanhf(u));
}
__device__ __forceinline__ float dgelu_f(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  const float t = tanhf(u);
  return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * 0.7978845608028654f * (1.0f + 0.134145f * x * x);
}

// ---------------------------------------------------------------------- LayerNorm
constexpr int LN_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(LN_THREADS) layernorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                                   const T* __restrict__ b, T* __restrict__ y,
                                                                   float* __restrict__ mean, float* __restrict__ rstd,
                                                                   int rows, int cols, float eps) {
  constexpr int V = VecOf<T>::N;
  __shared__ float sh[LN_THREADS / 32];
  const int row = blockIdx.x;
  const T* xr = x + static_cast<size_t>(row) * cols;
  T* yr = y + static_cast<size_t>(row) * cols;
  const int nvec = cols / V;
  float s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += LN_THREADS) {
    float f[V];
    load_vec(xr + i * V, f);
#pragma unroll
    for (int j = 0; j < V; ++j) s += f[j];
  }
  for (int i = nvec * V + threadIdx.x; i < cols; i += LN_THREADS) s += Cvt<T>::to(xr[i]);
  const float mu = block_sum<LN_THREADS>(s, sh) / cols;
  float q = 0.f;
  for (int i = threadIdx.x; i < nvec; i += LN_THREADS) {
    float f[V];
    load_vec(xr + i * V, f);
#pragma unroll
    for (int j = 0; j < V; ++j) { const float d = f[j] - mu; q += d * d; }
  }
  for (int i = nvec * V + threadIdx.x; i < cols; i += LN_THREADS) { const float d = Cvt<T>::to(xr[i]) - mu; q += d * d; }
  const float rs = rsqrtf(block_sum<LN_THREADS>(q, sh) / cols + eps);
  if (threadIdx.x == 0) { mean[row] = mu; rstd[row] = rs; }
  for (int i = threadIdx.x; i < nvec; i += LN_THREADS) {
    float f[V], g[V], h[V];
    load_vec(xr + i * V, f);
    load_vec(w + i * V, g);
    if (b) load_vec(b + i * V, h);
#pragma unroll
    for (int j = 0; j < V; ++j) f[j] = (f[j] - mu) * rs * g[j] + (b ? h[j] : 0.f);
    store_vec(yr + i * V, f);
  }
  for (int i = nvec * V + threadIdx.x; i < cols; i += LN_THREADS)
    yr[i] = Cvt<T>::from((Cvt<T>::to(xr[i]) - mu) * rs * Cvt<T>::to(w[i]) + (b ? Cvt<T>::to(b[i]) : 0.f));
}

// Each CTA walks rows blockIdx.x, +gridDim.x, ...; thread t owns the same columns in every row, so the
// weight/bias gradient partials stay in registers (up to LN_MAXV vectors per thread) until the end.
constexpr int LN_MAXV = 4;
template <typename T>
__global__ void __launch_bounds__(LN_THREADS) layernorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                                   const T* __restrict__ w,
                                                                   const float* __restrict__ mean,
                                                                   const float* __restrict__ rstd, T* __restrict__ dx,
                                                                   float* __restrict__ dw_part,
                                                                   float* __restrict__ db_part, int rows, int cols) {
  constexpr int V = VecOf<T>::N;
  __shared__ float sh[LN_THREADS / 32];
  const int nvec = cols / V;  // host guarantees cols % V == 0 and nvec <= LN_THREADS * LN_MAXV
  float dwacc[LN_MAXV][V], dbacc[LN_MAXV][V], wv[LN_MAXV][V];
#pragma unroll
  for (int k = 0; k < LN_MAXV; ++k) {
    const int i = threadIdx.x + k * LN_THREADS;
#pragma unroll
    for (int j = 0; j < V; ++j) { dwacc[k][j] = 0.f; dbacc[k][j] = 0.f; wv[k][j] = 0.f; }
    if (i < nvec) load_vec(w + i * V, wv[k]);
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + static_cast<size_t>(row) * cols;
    const T* gr = dy + static_cast<size_t>(row) * cols;
    T* dr = dx + static_cast<size_t>(row) * cols;
    const float mu = mean[row], rs = rstd[row];
    float xh[LN_MAXV][V], gw[LN_MAXV][V];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < LN_MAXV; ++k) {
      const int i = threadIdx.x + k * LN_THREADS;
      if (i < nvec) {
        float g[V];
        load_vec(xr + i * V, xh[k]);
        load_vec(gr + i * V, g);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          xh[k][j] = (xh[k][j] - mu) * rs;
          dwacc[k][j] += g[j] * xh[k][j];
          dbacc[k][j] += g[j];
          gw[k][j] = g[j] * wv[k][j];
          s1 += gw[k][j];
          s2 += gw[k][j] * xh[k][j];
        }
      }
    }
    s1 = block_sum<LN_THREADS>(s1, sh) / cols;
    s2 = block_sum<LN_THREADS>(s2, sh) / cols;
#pragma unroll
    for (int k = 0; k < LN_MAXV; ++k) {
      const int i = threadIdx.x + k * LN_THREADS;
      if (i < nvec) {
        float o[V];
#pragma unroll
        for (int j = 0; j < V; ++j) o[j] = rs * (gw[k][j] - s1 - xh[k][j] * s2);
        store_vec(dr + i * V, o);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < LN_MAXV; ++k) {
    const int i = threadIdx.x + k * LN_THREADS;
    if (i < nvec) {
      float* dwp = dw_part + static_cast<size_t>(blockIdx.x) * cols + i * V;
      float* dbp = db_part + static_cast<size_t>(blockIdx.x) * cols + i * V;
#pragma unroll
      for (int j = 0; j < V; ++j) { dwp[j] = dwacc[k][j]; dbp[j] = dbacc[k][j]; }
    }
  }
}

// out[c] = sum_p part[p, c]; optional second pair for LayerNorm's (dw, db)
template <typename T>
__global__ void reduce_parts_kernel(const float* __restrict__ pa, const float* __restrict__ pb, T* __restrict__ oa,
                                    T* __restrict__ ob, int parts, int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float a = 0.f, b = 0.f;
  for (int p = 0; p < parts; ++p) {
    a += pa[static_cast<size_t>(p) * cols + c];
    if (pb) b += pb[static_cast<size_t>(p) * cols + c];
  }
  oa[c] = Cvt<T>::from(a);
  if (pb && ob) ob[c] = Cvt<T>::from(b);
}

template <typename T>
__global__ void colsum_kernel(const T* __restrict__ x, float* __restrict__ part, int rows, int cols) {
  // grid (col blocks, parts); each thread owns one column and strides over the rows of its part
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int r = blockIdx.y; r < rows; r += gridDim.y) s += Cvt<T>::to(x[static_cast<size_t>(r) * cols + c]);
  part[static_cast<size_t>(blockIdx.y) * cols + c] = s;
}

// 16-bit inputs, cols % 8 == 0, 16-byte aligned rows: each thread owns 8 adjacent columns (one 16-byte load per row)
// and keeps four rows in flight
template <typename T>
__global__ void __launch_bounds__(128) colsum_vec8_kernel(const T* __restrict__ x, float* __restrict__ part, int rows,
                                                          int cols) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= cols) return;
  float s[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) s[j] = 0.f;
  const int step = gridDim.y;
  int r = blockIdx.y;
  for (; r + 3 * step < rows; r += 4 * step) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(r + u * step) * cols + c);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const T* e = reinterpret_cast<const T*>(&v[u]);
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j] += Cvt<T>::to(e[j]);
    }
  }
  for (; r < rows; r += step) {
    const uint4 v = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * cols + c);
    const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j] += Cvt<T>::to(e[j]);
  }
  float* o = part + static_cast<size_t>(blockIdx.y) * cols + c;
  *reinterpret_cast<float4*>(o) = make_float4(s[0], s[1], s[2], s[3]);
  *reinterpret_cast<float4*>(o + 4) = make_float4(s[4], s[5], s[6], s[7]);
}

// rotary applied in place to the first `rd` dims of every head of x [tokens, H, D]; one thread rotates the four
// pairs of one 16-byte vector, the other D - rd dims are never touched (rd % 8 == 0, D % 8 == 0)
template <typename T>
__global__ void rotary_inplace_kernel(T* __restrict__ x, const long long* __restrict__ pos, long long tokens, int H,
                                      int D, int rd, float log2_base, int inverse) {
  const int vec_per_head = rd / 8;
  const long long total = tokens * H * vec_per_head;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int vi = static_cast<int>(i % vec_per_head);
    const long long th = i / vec_per_head;   // token * H + head
    const long long tok = th / H;
    T* p = x + static_cast<size_t>(th) * D + vi * 8;
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    T* e = reinterpret_cast<T*>(&raw);
    const float ps = static_cast<float>(pos[tok]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int pr = vi * 4 + j;
      const float inv_freq = exp2f(-log2_base * (2.0f * pr) / rd);
      float sn, cs;
      sincosf(ps * inv_freq, &sn, &cs);
      if (inverse) sn = -sn;
      const float a = Cvt<T>::to(e[2 * j]), b = Cvt<T>::to(e[2 * j + 1]);
      e[2 * j] = Cvt<T>::from(a * cs - b * sn);
      e[2 * j + 1] = Cvt<T>::from(b * cs + a * sn);
    }
    *reinterpret_cast<uint4*>(p) = raw;
  }
}

// ---------------------------------------------------------------------- bias + GeLU
template <typename T, bool BWD>
__global__ void bias_gelu_kernel(const T* __restrict__ a, const T* __restrict__ x, const T* __restrict__ bias,
                                 T* __restrict__ out, long long total_vec, int cols) {
  constexpr int V = VecOf<T>::N;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total_vec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = i * V;
    const int c = static_cast<int>(e % cols);
    float xv[V], bv[V], o[V];
    load_vec(x + e, xv);
    if (bias) {
      load_vec(bias + c, bv);
#pragma unroll
      for (int j = 0; j < V; ++j) xv[j] += bv[j];
    }
    if (BWD) {
      float g[V];
      load_vec(a + e, g);
#pragma unroll
      for (int j = 0; j < V; ++j) o[j] = g[j] * dgelu_f(xv[j]);
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) o[j] = gelu_f(xv[j]);
    }
    store_vec(out + e, o);
  }
}

// ---------------------------------------------------------------------- bias + dropout + residual
__device__ __forceinline__ float hash_uniform(unsigned long long seed, unsigned long long idx) {
  unsigned long long z = seed + idx * 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return static_cast<float>(z >> 40) * (1.0f / 16777216.0f);
}
template <typename T>
__global__ void bias_dropout_residual_kernel(const T* __restrict__ x, const T* __restrict__ bias,
                                             const T* __restrict__ res, T* __restrict__ y, long long total_vec,
                                             int cols, float p, unsigned long long seed, int mode) {
  constexpr int V = VecOf<T>::N;
  const float keep_scale = p < 1.f ? 1.f / (1.f - p) : 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total_vec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = i * V;
    float xv[V];
    load_vec(x + e, xv);
    if (mode == 0 && bias) {
      float bv[V];
      load_vec(bias + static_cast<int>(e % cols), bv);
#pragma unroll
      for (int j = 0; j < V; ++j) xv[j] += bv[j];
    }
    if (p > 0.f) {
#pragma unroll
      for (int j = 0; j < V; ++j) xv[j] = hash_uniform(seed, e + j) >= p ? xv[j] * keep_scale : 0.f;
    }
    if (mode == 0 && res) {
      float rv[V];
      load_vec(res + e, rv);
#pragma unroll
      for (int j = 0; j < V; ++j) xv[j] += rv[j];
    }
    store_vec(y + e, xv);
  }
}

// ---------------------------------------------------------------------- rotary (GPT-J, interleaved pairs)
template <typename T>
__global__ void rotary_kernel(const T* __restrict__ x, T* __restrict__ y, const long long* __restrict__ pos, int B,
                              int S, int H, int D, int rd, float log2_base, int inverse) {
  // one thread per (token, head, pair); dims >= rd are copied by the threads with pair index >= rd/2
  const long long total = static_cast<long long>(B) * S * H * (D / 2);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int pr = static_cast<int>(i % (D / 2));
    const long long th = i / (D / 2);       // token * H + head
    const long long tok = th / H;
    const size_t off = static_cast<size_t>(th) * D + 2 * pr;
    float a = Cvt<T>::to(x[off]), b = Cvt<T>::to(x[off + 1]);
    if (2 * pr < rd) {
      const float inv_freq = exp2f(-log2_base * (2.0f * pr) / rd);
      float sn, cs;
      sincosf(static_cast<float>(pos[tok]) * inv_freq, &sn, &cs);
      if (inverse) sn = -sn;
      const float na = a * cs - b * sn;
      const float nb = b * cs + a * sn;
      a = na; b = nb;
    }
    y[off] = Cvt<T>::from(a);
    y[off + 1] = Cvt<T>::from(b);
  }
}

// ---------------------------------------------------------------------- softmax on scores
constexpr int SM_THREADS = 128;
// mode 0: causal (row r of sq keeps cols <= r + (sk - sq)); mode 1: explicit mask (1 = masked -> -10000)
template <typename T>
__global__ void __launch_bounds__(SM_THREADS) softmax_fwd_kernel(const T* __restrict__ x,
                                                                 const uint8_t* __restrict__ mask, T* __restrict__ y,
                                                                 int sq, int sk, int heads, int mask_b, float scale,
                                                                 int mode) {
  __shared__ float sh[SM_THREADS / 32];
  const long long row = blockIdx.x;  // over batches * sq
  const int r = static_cast<int>(row % sq);
  const long long bh = row / sq;
  const T* xr = x + row * sk;
  T* yr = y + row * sk;
  const uint8_t* mr = nullptr;
  if (mode == 1) {
    const long long b = bh / heads;
    mr = mask + ((mask_b == 1 ? 0 : b) * sq + r) * static_cast<long long>(sk);
  }
  const int limit = mode == 0 ? min(sk, r + (sk - sq) + 1) : sk;
  float mx = -CUDART_INF_F;
  for (int c = threadIdx.x; c < limit; c += SM_THREADS) {
    float v = Cvt<T>::to(xr[c]) * scale;
    if (mr && mr[c]) v = -10000.f;
    mx = fmaxf(mx, v);
  }
  mx = block_max<SM_THREADS>(mx, sh);
  float s = 0.f;
  for (int c = threadIdx.x; c < limit; c += SM_THREADS) {
    float v = Cvt<T>::to(xr[c]) * scale;
    if (mr && mr[c]) v = -10000.f;
    s += __expf(v - mx);
  }
  s = block_sum<SM_THREADS>(s, sh);
  const float inv = 1.f / s;
  for (int c = threadIdx.x; c < sk; c += SM_THREADS) {
    float o = 0.f;
    if (c < limit) {
      float v = Cvt<T>::to(xr[c]) * scale;
      if (mr && mr[c]) v = -10000.f;
      o = __expf(v - mx) * inv;
    }
    yr[c] = Cvt<T>::from(o);
  }
}
template <typename T>
__global__ void __launch_bounds__(SM_THREADS) softmax_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy,
                                                                 T* __restrict__ dx, int cols, float scale) {
  __shared__ float sh[SM_THREADS / 32];
  const long long row = blockIdx.x;
  const T* yr = y + row * cols;
  const T* gr = dy + row * cols;
  T* dr = dx + row * cols;
  float s = 0.f;
  for (int c = threadIdx.x; c < cols; c += SM_THREADS) s += Cvt<T>::to(yr[c]) * Cvt<T>::to(gr[c]);
  s = block_sum<SM_THREADS>(s, sh);
  for (int c = threadIdx.x; c < cols; c += SM_THREADS) {
    const float yy = Cvt<T>::to(yr[c]);
    dr[c] = Cvt<T>::from(scale * yy * (Cvt<T>::to(gr[c]) - s));
  }
}

// ---------------------------------------------------------------------- cross-entropy pieces
constexpr int CE_THREADS = 256;
template <typename T>
__global__ void __launch_bounds__(CE_THREADS) ce_stats_kernel(const T* __restrict__ logits,
                                                              const long long* __restrict__ labels,
                                                              float* __restrict__ rowmax, float* __restrict__ sumexp,
                                                              float* __restrict__ target, int cols, int ld,
                                                              long long vocab_start) {
  constexpr int V = VecOf<T>::N;
  __shared__ float sh[CE_THREADS / 32];
  const int row = blockIdx.x;
  const T* lr = logits + static_cast<size_t>(row) * ld;
  float m = -CUDART_INF_F, s = 0.f;  // online (max, sum exp) per thread
  const bool vec_ok = (ld % V == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  const int nvec = vec_ok ? cols / V : 0;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    float f[V];
    load_vec(lr + i * V, f);
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < V; ++j) lm = fmaxf(lm, f[j]);
    const float nm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < V; ++j) acc += __expf(f[j] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  for (int i = nvec * V + threadIdx.x; i < cols; i += CE_THREADS) {
    const float f = Cvt<T>::to(lr[i]);
    const float nm = fmaxf(m, f);
    s = s * __expf(m - nm) + __expf(f - nm);
    m = nm;
  }
  const float gm = block_max<CE_THREADS>(m, sh);
  const float contrib = (m == -CUDART_INF_F) ? 0.f : s * __expf(m - gm);
  const float gs = block_sum<CE_THREADS>(contrib, sh);
  if (threadIdx.x == 0) {
    rowmax[row] = gm;
    sumexp[row] = gs;
    const long long t = labels[row] - vocab_start;
    target[row] = (t >= 0 && t < cols) ? Cvt<T>::to(lr[t]) : 0.f;
  }
}
template <typename T>
__global__ void __launch_bounds__(CE_THREADS) ce_grad_kernel(T* __restrict__ logits,
                                                             const long long* __restrict__ labels,
                                                             const float* __restrict__ lse,
                                                             const float* __restrict__ scale, int cols, int ld,
                                                             long long vocab_start) {
  constexpr int V = VecOf<T>::N;
  const int row = blockIdx.x;
  T* lr = logits + static_cast<size_t>(row) * ld;
  const float l = lse[row], sc = scale[row];
  const long long t = labels[row] - vocab_start;
  const bool vec_ok = (ld % V == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  const int nvec = vec_ok ? cols / V : 0;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    float f[V];
    load_vec(lr + i * V, f);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      float pr = __expf(f[j] - l);
      if (i * V + j == t) pr -= 1.f;
      f[j] = pr * sc;
    }
    store_vec(lr + i * V, f);
  }
  for (int i = nvec * V + threadIdx.x; i < cols; i += CE_THREADS) {
    float pr = __expf(Cvt<T>::to(lr[i]) - l);
    if (i == t) pr -= 1.f;
    lr[i] = Cvt<T>::from(pr * sc);
  }
}

// (max, sum exp, label logit) of a row from its per-128-column-block records [blocks, rows, 3] (written by the LM-head
// GEMM's cross-entropy epilogue): one thread per row, fixed order, so the result does not depend on the tile schedule
__global__ void ce_reduce_stats_kernel(const float* __restrict__ stats, float* __restrict__ rowmax,
                                       float* __restrict__ sumexp, float* __restrict__ target, int rows, int blocks) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  float m = -3.0e38f, s = 0.f, t = 0.f;
  for (int b = 0; b < blocks; ++b) {
    const float* rec = stats + (static_cast<size_t>(b) * rows + row) * 3;
    const float bm = rec[0], bs = rec[1];
    const float nm = fmaxf(m, bm);
    s = s * __expf(m - nm) + bs * __expf(bm - nm);
    m = nm;
    t += rec[2];
  }
  rowmax[row] = m;
  sumexp[row] = s;
  target[row] = t;
}

// ---------------------------------------------------------------------- AdamW / norms
__device__ __forceinline__ void adam_update(float& p, float& m, float& v, float g, float lr, float beta1, float beta2,
                                            float eps, float decay, float inv_bc1, float inv_bc2) {
  m = beta1 * m + (1.f - beta1) * g;
  v = beta2 * v + (1.f - beta2) * g * g;
  p = p * decay - lr * (m * inv_bc1) / (sqrtf(v * inv_bc2) + eps);
}
// Four elements per thread and iteration through 16-byte accesses (p, m, v) and 8-byte accesses (16-bit g and
// p_lp); the launcher only takes this path when every pointer is 16-byte aligned. Elements past the last
// multiple of 4 are handled by the first threads one by one.
template <typename G, typename LP>
__global__ void __launch_bounds__(256) adam_kernel(float* __restrict__ p, const G* __restrict__ g, float* __restrict__ m,
                                                   float* __restrict__ v, LP* __restrict__ p_lp, long long n, float lr,
                                                   float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                                                   float grad_scale, const float* __restrict__ inv_scale_dev, int vec) {
  const float gs = grad_scale * (inv_scale_dev ? *inv_scale_dev : 1.f);
  const float decay = 1.f - lr * wd, inv_bc1 = 1.f / bc1, inv_bc2 = 1.f / bc2;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long n4 = vec ? n / 4 : 0;
  for (long long i = tid; i < n4; i += nthreads) {
    float4 pp = reinterpret_cast<const float4*>(p)[i];
    float4 mm = reinterpret_cast<const float4*>(m)[i];
    float4 vv = reinterpret_cast<const float4*>(v)[i];
    float gg[4];
    if constexpr (sizeof(G) == 4) {
      const float4 t = reinterpret_cast<const float4*>(g)[i];
      gg[0] = t.x; gg[1] = t.y; gg[2] = t.z; gg[3] = t.w;
    } else {
      const uint2 t = reinterpret_cast<const uint2*>(g)[i];
      const G* h = reinterpret_cast<const G*>(&t);
#pragma unroll
      for (int k = 0; k < 4; ++k) gg[k] = Cvt<G>::to(h[k]);
    }
    adam_update(pp.x, mm.x, vv.x, gg[0] * gs, lr, beta1, beta2, eps, decay, inv_bc1, inv_bc2);
    adam_update(pp.y, mm.y, vv.y, gg[1] * gs, lr, beta1, beta2, eps, decay, inv_bc1, inv_bc2);
    adam_update(pp.z, mm.z, vv.z, gg[2] * gs, lr, beta1, beta2, eps, decay, inv_bc1, inv_bc2);
    adam_update(pp.w, mm.w, vv.w, gg[3] * gs, lr, beta1, beta2, eps, decay, inv_bc1, inv_bc2);
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (p_lp) {
      LP o[4] = {Cvt<LP>::from(pp.x), Cvt<LP>::from(pp.y), Cvt<LP>::from(pp.z), Cvt<LP>::from(pp.w)};
      reinterpret_cast<uint2*>(p_lp)[i] = *reinterpret_cast<const uint2*>(o);
    }
  }
  for (long long i = n4 * 4 + tid; i < n; i += nthreads) {
    float pi = p[i], mi = m[i], vi = v[i];
    adam_update(pi, mi, vi, Cvt<G>::to(g[i]) * gs, lr, beta1, beta2, eps, decay, inv_bc1, inv_bc2);
    p[i] = pi; m[i] = mi; v[i] = vi;
    if (p_lp) p_lp[i] = Cvt<LP>::from(pi);
  }
}
// sum of squares: 16-byte loads when `vec` (pointer 16-byte aligned), one atomic per block
template <typename T>
__global__ void __launch_bounds__(256) sumsq_kernel(const T* __restrict__ x, float* __restrict__ out, long long n, int vec) {
  __shared__ float sh[8];
  constexpr int PER = 16 / sizeof(T);
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long nv = vec ? n / PER : 0;
  float s0 = 0.f, s1 = 0.f;
  for (long long i = tid; i < nv; i += 2 * nthreads) {
    const uint4 a = reinterpret_cast<const uint4*>(x)[i];
    const bool two = i + nthreads < nv;
    uint4 b = make_uint4(0, 0, 0, 0);
    if (two) b = reinterpret_cast<const uint4*>(x)[i + nthreads];
    const T* ha = reinterpret_cast<const T*>(&a);
    const T* hb = reinterpret_cast<const T*>(&b);
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const float fa = Cvt<T>::to(ha[k]);
      s0 += fa * fa;
      const float fb = two ? Cvt<T>::to(hb[k]) : 0.f;
      s1 += fb * fb;
    }
  }
  for (long long i = nv * PER + tid; i < n; i += nthreads) {
    const float f = Cvt<T>::to(x[i]);
    s0 += f * f;
  }
  const float s = block_sum<256>(s0 + s1, sh);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

// ---------------------------------------------------------------------- split-K GEMM finalisation
// out[r, c] = T(act(sum_s ws[s, r, c] + bias[c])): sums the k-slice planes of a split-K GEMM in a fixed order
template <typename T>
__global__ void splitk_finalize_kernel(const float* __restrict__ ws, const T* __restrict__ bias, T* __restrict__ out,
                                       long long n, int cols, int split_k, int gelu_from) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < split_k; ++s) v += ws[s * n + i];
    const int c = static_cast<int>(i % cols);
    if (bias) v += Cvt<T>::to(bias[c]);
    if (gelu_from >= 0 && c >= gelu_from) v = gelu_f(v);
    out[i] = Cvt<T>::from(v);
  }
}

// ---------------------------------------------------------------------- n-gram blocking
// thread `c` compares the (n-1)-gram starting at c with the last (n-1) tokens of the row; on a match the
// token that followed it is banned. No shared memory is used, so the row length is unbounded.
__global__ void ngram_ban_kernel(const long long* __restrict__ tokens, float* __restrict__ lprobs, int len, int vocab,
                                 int n, int* err) {
  const int row = blockIdx.x;
  const long long* t = tokens + static_cast<size_t>(row) * len;
  const int starts = len - n + 1;  // candidate n-grams fully inside the row
  for (int c = threadIdx.x; c < starts; c += blockDim.x) {
    bool match = true;
    for (int k = 0; k < n - 1; ++k) {
      if (t[c + k] != t[len - n + 1 + k]) { match = false; break; }
    }
    if (match) {
      const long long banned = t[c + n - 1];
      if (banned >= 0 && banned < vocab) lprobs[static_cast<size_t>(row) * vocab + banned] = -CUDART_INF_F;
      else OSLO_REPORT_BOUNDS(err);   // a generated token outside the vocabulary: nothing to ban, skipped
    }
  }
}

static inline int grid_for(long long work, int threads, int cap = 148 * 16) {
  long long b = (work + threads - 1) / threads;
  if (b < 1) b = 1;
  return static_cast<int>(b < cap ? b : cap);
}
#define RET_LAST() return static_cast<int>(cudaGetLastError())
#define DISPATCH_16(dtype, T, ...)                                   \
  if ((dtype) == OSLO_DT_BF16) { using T = __nv_bfloat16; __VA_ARGS__ } \
  else if ((dtype) == OSLO_DT_FP16) { using T = __half; __VA_ARGS__ }   \
  else if ((dtype) == OSLO_DT_FP32) { using T = float; __VA_ARGS__ }    \
  else return -2;

}  // namespace oslo

using namespace oslo;

extern "C" int oslo_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                                  int rows, int cols, float eps, int dtype, cudaStream_t st) {
  if (rows <= 0) return 0;
  DISPATCH_16(dtype, T, {
    if (cols % VecOf<T>::N) return -3;
    layernorm_fwd_kernel<T><<<rows, LN_THREADS, 0, st>>>((const T*)x, (const T*)w, (const T*)b, (T*)y, mean, rstd,
                                                          rows, cols, eps);
  })
  RET_LAST();
}

extern "C" int oslo_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                                  void* dx, float* dw_part, float* db_part, void* dw, void* db, int rows, int cols,
                                  int parts, int dtype, cudaStream_t st) {
  if (rows <= 0) return 0;
  DISPATCH_16(dtype, T, {
    constexpr int V = VecOf<T>::N;
    if (cols % V || cols / V > LN_THREADS * LN_MAXV) return -3;
    layernorm_bwd_kernel<T><<<parts, LN_THREADS, 0, st>>>((const T*)dy, (const T*)x, (const T*)w, mean, rstd, (T*)dx,
                                                          dw_part, db_part, rows, cols);
    reduce_parts_kernel<T><<<(cols + 255) / 256, 256, 0, st>>>(dw_part, db_part, (T*)dw, (T*)db, parts, cols);
  })
  RET_LAST();
}

extern "C" int oslo_bias_gelu_fwd(const void* x, const void* bias, void* y, long long rows, int cols, int dtype,
                                  cudaStream_t st) {
  DISPATCH_16(dtype, T, {
    constexpr int V = VecOf<T>::N;
    if (cols % V) return -3;
    const long long tv = rows * cols / V;
    if (tv == 0) return 0;
    bias_gelu_kernel<T, false><<<grid_for(tv, 256), 256, 0, st>>>(nullptr, (const T*)x, (const T*)bias, (T*)y, tv, cols);
  })
  RET_LAST();
}
extern "C" int oslo_bias_gelu_bwd(const void* dy, const void* x, const void* bias, void* dx, long long rows, int cols,
                                  int dtype, cudaStream_t st) {
  DISPATCH_16(dtype, T, {
    constexpr int V = VecOf<T>::N;
    if (cols % V) return -3;
    const long long tv = rows * cols / V;
    if (tv == 0) return 0;
    bias_gelu_kernel<T, true><<<grid_for(tv, 256), 256, 0, st>>>((const T*)dy, (const T*)x, (const T*)bias, (T*)dx, tv, cols);
  })
  RET_LAST();
}

extern "C" int oslo_bias_dropout_residual(const void* x, const void* bias, const void* residual, void* y,
                                          long long rows, int cols, float p, unsigned long long seed, int mode,
                                          int dtype, cudaStream_t st) {
  DISPATCH_16(dtype, T, {
    constexpr int V = VecOf<T>::N;
    if (cols % V) return -3;
    const long long tv = rows * cols / V;
    if (tv == 0) return 0;
    bias_dropout_residual_kernel<T><<<grid_for(tv, 256), 256, 0, st>>>((const T*)x, (const T*)bias, (const T*)residual,
                                                                      (T*)y, tv, cols, p, seed, mode);
  })
  RET_LAST();
}

extern "C" int oslo_colsum(const void* x, float* part, float* out, int rows, int cols, int parts, int dtype,
                           cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return 0;
  if (dtype != OSLO_DT_FP32 && cols % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(part) & 15) == 0) {
    dim3 grid((cols / 8 + 127) / 128, parts);
    if (dtype == OSLO_DT_BF16) colsum_vec8_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>((const __nv_bfloat16*)x, part, rows, cols);
    else colsum_vec8_kernel<__half><<<grid, 128, 0, st>>>((const __half*)x, part, rows, cols);
  } else {
    DISPATCH_16(dtype, T, {
      dim3 grid((cols + 127) / 128, parts);
      colsum_kernel<T><<<grid, 128, 0, st>>>((const T*)x, part, rows, cols);
    })
  }
  reduce_parts_kernel<float><<<(cols + 255) / 256, 256, 0, st>>>(part, nullptr, out, nullptr, parts, cols);
  RET_LAST();
}

extern "C" int oslo_rotary(const void* x, void* y, const long long* positions, int B, int S, int H, int D,
                           int rotary_dim, float base, int inverse, int dtype, cudaStream_t st) {
  const long long total = static_cast<long long>(B) * S * H * (D / 2);
  if (total == 0) return 0;
  if (D % 2 || rotary_dim % 2 || rotary_dim > D) return -3;
  DISPATCH_16(dtype, T, {
    rotary_kernel<T><<<grid_for(total, 256), 256, 0, st>>>((const T*)x, (T*)y, positions, B, S, H, D, rotary_dim,
                                                          log2f(base), inverse);
  })
  RET_LAST();
}

// in-place variant: x [B, S, H, D] contiguous, only the first rotary_dim dims of each head are read and written
extern "C" int oslo_rotary_inplace(void* x, const long long* positions, int B, int S, int H, int D, int rotary_dim,
                                   float base, int inverse, int dtype, cudaStream_t st) {
  const long long tokens = static_cast<long long>(B) * S;
  if (tokens == 0 || rotary_dim == 0) return 0;
  if (D % 8 || rotary_dim % 8 || rotary_dim > D || (reinterpret_cast<uintptr_t>(x) & 15)) return -3;
  const long long total = tokens * H * (rotary_dim / 8);
  if (dtype == OSLO_DT_BF16)
    rotary_inplace_kernel<__nv_bfloat16><<<grid_for(total, 256), 256, 0, st>>>((__nv_bfloat16*)x, positions, tokens, H, D,
                                                                               rotary_dim, log2f(base), inverse);
  else if (dtype == OSLO_DT_FP16)
    rotary_inplace_kernel<__half><<<grid_for(total, 256), 256, 0, st>>>((__half*)x, positions, tokens, H, D, rotary_dim,
                                                                        log2f(base), inverse);
  else
    return -2;
  RET_LAST();
}

extern "C" int oslo_causal_softmax_fwd(const void* x, void* y, int batches, int sq, int sk, float scale, int dtype,
                                       cudaStream_t st) {
  const long long rows = static_cast<long long>(batches) * sq;
  if (rows == 0) return 0;
  DISPATCH_16(dtype, T, {
    softmax_fwd_kernel<T><<<static_cast<unsigned>(rows), SM_THREADS, 0, st>>>((const T*)x, nullptr, (T*)y, sq, sk, 1, 1,
                                                                             scale, 0);
  })
  RET_LAST();
}
extern "C" int oslo_masked_softmax_fwd(const void* x, const uint8_t* mask, void* y, int b, int h, int sq, int sk,
                                       int mask_b, float scale, int dtype, cudaStream_t st) {
  const long long rows = static_cast<long long>(b) * h * sq;
  if (rows == 0) return 0;
  DISPATCH_16(dtype, T, {
    softmax_fwd_kernel<T><<<static_cast<unsigned>(rows), SM_THREADS, 0, st>>>((const T*)x, mask, (T*)y, sq, sk, h, mask_b,
                                                                             scale, 1);
  })
  RET_LAST();
}
extern "C" int oslo_softmax_bwd(const void* y, const void* dy, void* dx, long long rows, int cols, float scale,
                                int dtype, cudaStream_t st) {
  if (rows == 0) return 0;
  DISPATCH_16(dtype, T, {
    softmax_bwd_kernel<T><<<static_cast<unsigned>(rows), SM_THREADS, 0, st>>>((const T*)y, (const T*)dy, (T*)dx, cols, scale);
  })
  RET_LAST();
}

extern "C" int oslo_ce_stats(const void* logits, const long long* labels, float* rowmax, float* sumexp, float* target,
                             int rows, int cols, int ld, long long vocab_start, int dtype, cudaStream_t st) {
  if (rows == 0) return 0;
  DISPATCH_16(dtype, T, {
    ce_stats_kernel<T><<<rows, CE_THREADS, 0, st>>>((const T*)logits, labels, rowmax, sumexp, target, cols, ld, vocab_start);
  })
  RET_LAST();
}
extern "C" int oslo_ce_grad(void* logits, const long long* labels, const float* lse, const float* scale, int rows,
                            int cols, int ld, long long vocab_start, int dtype, cudaStream_t st) {
  if (rows == 0) return 0;
  DISPATCH_16(dtype, T, {
    ce_grad_kernel<T><<<rows, CE_THREADS, 0, st>>>((T*)logits, labels, lse, scale, cols, ld, vocab_start);
  })
  RET_LAST();
}

extern "C" int oslo_adam(float* p, const void* g, float* m, float* v, void* p_lp, long long n, float lr, float beta1,
                         float beta2, float eps, float wd, float bc1, float bc2, float grad_scale,
                         const float* inv_scale_dev, int g_dtype, int lp_dtype, cudaStream_t st) {
  if (n == 0) return 0;
  const int grid = grid_for((n + 3) / 4, 256, 148 * 8);
  const auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  const int vec = (al16(p) && al16(g) && al16(m) && al16(v) && al16(p_lp)) ? 1 : 0;
#define ADAM_LAUNCH(G, LP) \
  adam_kernel<G, LP><<<grid, 256, 0, st>>>(p, (const G*)g, m, v, (LP*)p_lp, n, lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale, inv_scale_dev, vec)
  if (g_dtype == OSLO_DT_BF16) {
    if (lp_dtype == OSLO_DT_FP16) ADAM_LAUNCH(__nv_bfloat16, __half); else ADAM_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  } else if (g_dtype == OSLO_DT_FP16) {
    if (lp_dtype == OSLO_DT_BF16) ADAM_LAUNCH(__half, __nv_bfloat16); else ADAM_LAUNCH(__half, __half);
  } else if (g_dtype == OSLO_DT_FP32) {
    if (lp_dtype == OSLO_DT_FP16) ADAM_LAUNCH(float, __half); else ADAM_LAUNCH(float, __nv_bfloat16);
  } else {
    return -2;
  }
#undef ADAM_LAUNCH
  RET_LAST();
}

extern "C" int oslo_sumsq(const void* x, float* out, long long n, int dtype, cudaStream_t st) {
  if (n == 0) return 0;
  const int vec = (reinterpret_cast<uintptr_t>(x) & 15) == 0 ? 1 : 0;
  DISPATCH_16(dtype, T, { sumsq_kernel<T><<<grid_for((n + 7) / 8, 256, 148 * 8), 256, 0, st>>>((const T*)x, out, n, vec); })
  RET_LAST();
}

extern "C" int oslo_ce_reduce_stats(const float* stats, float* rowmax, float* sumexp, float* target, int rows, int blocks,
                                    cudaStream_t st) {
  if (rows <= 0 || blocks <= 0) return 0;
  ce_reduce_stats_kernel<<<(rows + 127) / 128, 128, 0, st>>>(stats, rowmax, sumexp, target, rows, blocks);
  RET_LAST();
}

extern "C" int oslo_ngram_ban(const long long* tokens, float* lprobs, int rows, int len, int vocab, int n,
                              int* err_word, cudaStream_t st) {
  if (rows == 0 || n <= 0 || len + 1 < n) return 0;
  ngram_ban_kernel<<<rows, 256, 0, st>>>(tokens, lprobs, len, vocab, n, err_word);
  RET_LAST();
}

extern "C" int oslo_splitk_finalize(const float* ws, const void* bias, void* out, long long rows, int cols, int split_k,
                                    int gelu_from, int dtype, cudaStream_t st) {
  const long long n = rows * cols;
  if (n == 0) return 0;
  if (dtype == OSLO_DT_BF16)
    splitk_finalize_kernel<__nv_bfloat16><<<grid_for(n, 256), 256, 0, st>>>(ws, (const __nv_bfloat16*)bias, (__nv_bfloat16*)out, n, cols, split_k, gelu_from);
  else if (dtype == OSLO_DT_FP16)
    splitk_finalize_kernel<__half><<<grid_for(n, 256), 256, 0, st>>>(ws, (const __half*)bias, (__half*)out, n, cols, split_k, gelu_from);
  else
    return -2;
  RET_LAST();
}
