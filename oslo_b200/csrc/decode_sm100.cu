// Kernels of the single-token decode step (a handful of rows per call). Everything here is bound by how fast
// weights and the KV cache stream out of HBM and by launch count, not by math, so the kernels are plain
// wide-load CUDA-core code with as many 16-byte loads in flight as the register file allows, and they fuse what
// the eager path runs as separate launches:
//   * gemv_rows_kernel: y[m, n] = act(sum_k [x1 | x2][m, k] * W[n, k] + bias[n]) + res[m, n] for m <= 4 (beyond that the CUDA
//     cores cannot keep up with HBM and the tensor-core split-k path takes over). One block owns four output
//     columns and the whole k range, so there is no second pass; the input may come in two pieces
//     (attention output and MLP activation feeding the merged out_proj / fc_out product of a parallel block).
//   * rotary_append_kernel: GPT-J rotary on q and k of the new token, q to a contiguous buffer, k and v written
//     into the static cache at the position held in device memory.
//
// Reference behaviour covered: one iteration of the token loop of oslo/generation_utils.py:1269-1361 through a
// GPT-J block (oslo/models/gptj/modeling_gptj.py:196-320: rotary at the cache offset, torch.cat cache growth,
// attention, out_proj, MLP, parallel residual).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include "oslo_kernels.h"
#include "ptx.cuh"

namespace oslo {

template <typename T> struct DCvt;
template <> struct DCvt<__nv_bfloat16> {
  static __device__ __forceinline__ float2 to2(uint32_t v) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v)); }
  static __device__ __forceinline__ __nv_bfloat16 from(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float to(__nv_bfloat16 v) { return __bfloat162float(v); }
};
template <> struct DCvt<__half> {
  static __device__ __forceinline__ float2 to2(uint32_t v) { return __half22float2(*reinterpret_cast<const __half2*>(&v)); }
  static __device__ __forceinline__ __half from(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ float to(__half v) { return __half2float(v); }
};

__device__ __forceinline__ uint4 ld_stream_16(const void* p) {   // weights are read once: keep them out of L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ float gelu_tanh_dec(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * x * (1.0f + t);
}

constexpr int GV_COLS = 4;      // output columns per warp
constexpr int GV_THREADS = 256;

// accumulate the k range [k_begin, K) in steps of k_step for GV_COLS weight rows; two chunks per iteration so that
// each lane keeps 2 * GV_COLS 16-byte weight loads in flight
template <typename T, int MR>
__device__ __forceinline__ void gemv_segment(const T* __restrict__ x, int ldx, int K, const T* __restrict__ w, int ldw,
                                             int m_valid, int k_begin, int k_step, float (&acc)[GV_COLS][MR]) {
  for (int k = k_begin; k < K; k += 2 * k_step) {
    const int kb = k + k_step;
    const bool second = kb < K;
    uint4 wv[2][GV_COLS];
#pragma unroll
    for (int c = 0; c < GV_COLS; ++c) {
      wv[0][c] = ld_stream_16(w + static_cast<size_t>(c) * ldw + k);
      wv[1][c] = second ? ld_stream_16(w + static_cast<size_t>(c) * ldw + kb) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (u == 1 && !second) break;
      const int kk = u ? kb : k;
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        if (m < m_valid) {
          const uint4 xv = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(m) * ldx + kk);
          const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
          for (int c = 0; c < GV_COLS; ++c) {
            const uint32_t ww[4] = {wv[u][c].x, wv[u][c].y, wv[u][c].z, wv[u][c].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 a = DCvt<T>::to2(xw[j]);
              const float2 b = DCvt<T>::to2(ww[j]);
              acc[c][m] = fmaf(a.x, b.x, acc[c][m]);
              acc[c][m] = fmaf(a.y, b.y, acc[c][m]);
            }
          }
        }
      }
    }
  }
}

// W is [N, K1 + K2] with row stride ldw (K-major); x1 [m, K1], x2 [m, K2] (x2 may be null); N % 4 == 0, K % 8 == 0.
// One block per group of GV_COLS output columns: its 8 warps interleave over the k range (each lane 8 elements of
// every 2048-element stripe), so consecutive warps read consecutive 512-byte pieces of the same weight rows.
template <typename T, int MR>
__global__ void __launch_bounds__(GV_THREADS) gemv_rows_kernel(const T* __restrict__ x1, int ld1, int K1,
                                                               const T* __restrict__ x2, int ld2, int K2,
                                                               const T* __restrict__ W, int ldw,
                                                               const T* __restrict__ bias,
                                                               const T* __restrict__ res, int ldr, T* __restrict__ out,
                                                               int ldo, int N, int m_valid, int gelu_from) {
  __shared__ float red[GV_THREADS / 32][GV_COLS * MR];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int k_begin = threadIdx.x * 8, k_step = GV_THREADS * 8;
  for (int n0 = blockIdx.x * GV_COLS; n0 < N; n0 += gridDim.x * GV_COLS) {
    float acc[GV_COLS][MR];
#pragma unroll
    for (int c = 0; c < GV_COLS; ++c)
#pragma unroll
      for (int m = 0; m < MR; ++m) acc[c][m] = 0.f;
    const T* w = W + static_cast<size_t>(n0) * ldw;
    gemv_segment<T, MR>(x1, ld1, K1, w, ldw, m_valid, k_begin, k_step, acc);
    if (x2 != nullptr) gemv_segment<T, MR>(x2, ld2, K2, w + K1, ldw, m_valid, k_begin, k_step, acc);
#pragma unroll
    for (int c = 0; c < GV_COLS; ++c)
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        float v = acc[c][m];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0) red[warp][c * MR + m] = v;
      }
    __syncthreads();
    if (threadIdx.x < GV_COLS * MR) {
      const int c = threadIdx.x / MR, m = threadIdx.x % MR;
      float v = 0.f;
#pragma unroll
      for (int wv = 0; wv < GV_THREADS / 32; ++wv) v += red[wv][threadIdx.x];
      if (m < m_valid) {
        const int n = n0 + c;
        if (bias) v += DCvt<T>::to(bias[n]);
        if (gelu_from >= 0 && n >= gelu_from) v = gelu_tanh_dec(v);
        if (res) v += DCvt<T>::to(res[static_cast<size_t>(m) * ldr + n]);
        out[static_cast<size_t>(m) * ldo + n] = DCvt<T>::from(v);
      }
    }
    __syncthreads();
  }
}

// One block per (batch row, head): rotary (pairs (2i, 2i+1) of the first rotary_dim dims, position pos[b]) on q and
// k; q -> q_out [B, H, D]; k, v -> cache[b, h, write_index[0], :]. q/k/v rows are [H * D] slices with row strides.
template <typename T>
__global__ void rotary_append_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                                     long long ldq, long long ldk, long long ldv, T* __restrict__ q_out,
                                     T* __restrict__ kc, T* __restrict__ vc, const int* __restrict__ lengths,
                                     const long long* __restrict__ write_index, int H, int D, int Tmax, int rotary_dim,
                                     float log2_base, int* err) {
  const int b = blockIdx.y, h = blockIdx.x;
  const long long wi = write_index[0];
  if (wi < 0 || wi >= Tmax) {   // never write outside the cache
    OSLO_REPORT_BOUNDS(err);
    return;
  }
  const float pos = static_cast<float>(lengths[b]);
  const T* qp = q + b * ldq + static_cast<long long>(h) * D;
  const T* kp = k + b * ldk + static_cast<long long>(h) * D;
  const T* vp = v + b * ldv + static_cast<long long>(h) * D;
  T* qo = q_out + (static_cast<long long>(b) * H + h) * D;
  T* ko = kc + ((static_cast<long long>(b) * H + h) * Tmax + wi) * D;
  T* vo = vc + ((static_cast<long long>(b) * H + h) * Tmax + wi) * D;
  for (int i = threadIdx.x; i < D / 2; i += blockDim.x) {
    const int d0 = 2 * i;
    float q0 = DCvt<T>::to(qp[d0]), q1 = DCvt<T>::to(qp[d0 + 1]);
    float k0 = DCvt<T>::to(kp[d0]), k1 = DCvt<T>::to(kp[d0 + 1]);
    if (d0 < rotary_dim) {
      const float inv_freq = exp2f(-log2_base * (2.0f * i) / rotary_dim);   // same expression as rotary_kernel
      float sn, cs;
      sincosf(pos * inv_freq, &sn, &cs);
      const float a = q0 * cs - q1 * sn, bq = q1 * cs + q0 * sn;
      q0 = a; q1 = bq;
      const float c = k0 * cs - k1 * sn, dk = k1 * cs + k0 * sn;
      k0 = c; k1 = dk;
    }
    qo[d0] = DCvt<T>::from(q0); qo[d0 + 1] = DCvt<T>::from(q1);
    ko[d0] = DCvt<T>::from(k0); ko[d0 + 1] = DCvt<T>::from(k1);
    vo[d0] = vp[d0]; vo[d0 + 1] = vp[d0 + 1];
  }
}

template <typename T>
static int gemv_launch(const void* x1, int ld1, int K1, const void* x2, int ld2, int K2, const void* W, int ldw,
                       const void* bias, const void* res, int ldr, void* out, int ldo, int M, int N, int gelu_from,
                       int num_sms, cudaStream_t st) {
  int blocks = N / GV_COLS;                   // one block per column group, at most 8 resident blocks per SM's worth
  if (blocks > num_sms * 8) blocks = num_sms * 8;
  if (blocks < 1) blocks = 1;
#define GV_CASE(MR)                                                                                               \
  gemv_rows_kernel<T, MR><<<blocks, GV_THREADS, 0, st>>>((const T*)x1, ld1, K1, (const T*)x2, ld2, K2, (const T*)W, ldw, \
                                                         (const T*)bias, (const T*)res, ldr, (T*)out, ldo, N, M, gelu_from)
  if (M <= 1) GV_CASE(1);
  else if (M <= 2) GV_CASE(2);
  else GV_CASE(4);
#undef GV_CASE
  return static_cast<int>(cudaGetLastError());
}

}  // namespace oslo

extern "C" int oslo_gemv_rows(const void* x1, int ld1, int K1, const void* x2, int ld2, int K2, const void* W, int ldw,
                              const void* bias, const void* res, int ldr, void* out, int ldo, int M, int N,
                              int gelu_from, int dtype, int num_sms, cudaStream_t stream) {
  using namespace oslo;
  if (M <= 0 || N <= 0) return 0;
  if (M > 4 || N % GV_COLS || K1 <= 0 || K1 % 8 || (x2 && (K2 <= 0 || K2 % 8)) || ld1 % 8 || ldw % 8 || (x2 && ld2 % 8))
    return -1;
  const void* ptrs[3] = {x1, x2, W};
  for (const void* p : ptrs)
    if (reinterpret_cast<uintptr_t>(p) & 15) return -4;
  if (dtype == OSLO_DT_BF16)
    return gemv_launch<__nv_bfloat16>(x1, ld1, K1, x2, ld2, x2 ? K2 : 0, W, ldw, bias, res, ldr, out, ldo, M, N, gelu_from, num_sms, stream);
  if (dtype == OSLO_DT_FP16)
    return gemv_launch<__half>(x1, ld1, K1, x2, ld2, x2 ? K2 : 0, W, ldw, bias, res, ldr, out, ldo, M, N, gelu_from, num_sms, stream);
  return -2;
}

extern "C" int oslo_rotary_append(const void* q, const void* k, const void* v, long long ldq, long long ldk,
                                  long long ldv, void* q_out, void* kc, void* vc, const int* lengths,
                                  const long long* write_index, int B, int H, int D, int Tmax, int rotary_dim, float base,
                                  int dtype, int* err_word, cudaStream_t stream) {
  using namespace oslo;
  if (B <= 0 || H <= 0) return 0;
  if (D % 2 || rotary_dim % 2 || rotary_dim > D) return -1;
  dim3 grid(H, B);
  const int threads = D / 2 >= 128 ? 128 : (D / 2 >= 64 ? 64 : 32);
  if (dtype == OSLO_DT_BF16)
    rotary_append_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, ldq, ldk, ldv, (__nv_bfloat16*)q_out,
        (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, lengths, write_index, H, D, Tmax, rotary_dim, log2f(base), err_word);
  else if (dtype == OSLO_DT_FP16)
    rotary_append_kernel<__half><<<grid, threads, 0, stream>>>((const __half*)q, (const __half*)k, (const __half*)v, ldq,
                                                               ldk, ldv, (__half*)q_out, (__half*)kc, (__half*)vc, lengths,
                                                               write_index, H, D, Tmax, rotary_dim, log2f(base), err_word);
  else
    return -2;
  return static_cast<int>(cudaGetLastError());
}
